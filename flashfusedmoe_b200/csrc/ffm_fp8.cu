// Row-wise e4m3 quantisation for the opt-in FP8 forward projections: q[r, :] = x[r, :] / scale[r] rounded to e4m3
// (saturating), scale[r] = max |x[r, :]| / 448 (448 = largest finite e4m3 value). One warp per row, two passes over
// the row (the second one hits L1 / L2), 16-byte loads and 8-byte stores. HBM-bound: reads 2 B and writes 1 B per
// element. The same kernel quantises activations (one scale per token row) and weights (one scale per output
// channel: a row of [E * N, K]).
#include <cuda_fp8.h>

#include "ffm_common.cuh"

namespace ffm {

namespace {

constexpr int Q_THREADS = 256;
constexpr int Q_WARPS = Q_THREADS / 32;

__device__ __forceinline__ uint32_t pack_e4m3x4(float a, float b, float c, float d) {
  const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
  const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
  return lo | (hi << 16);
}

__global__ void __launch_bounds__(Q_THREADS)
quantize_rows_e4m3_kernel(const bf16* __restrict__ x, long long rows, int K, uint8_t* __restrict__ q,
                          float* __restrict__ scale) {
  const int lane = threadIdx.x & 31;
  const int chunks = K >> 3;
  for (long long r = static_cast<long long>(blockIdx.x) * Q_WARPS + (threadIdx.x >> 5); r < rows;
       r += static_cast<long long>(gridDim.x) * Q_WARPS) {
    const uint4* src = reinterpret_cast<const uint4*>(x + r * K);
    float amax = 0.0f;
    for (int c = lane; c < chunks; c += 32) {
      const uint4 v = __ldg(src + c);
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = unpack_bf16x2(w[i]);
        amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y)));
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    // an all-zero row (padding) keeps scale 1 so that nothing divides by zero; its quantised values are zero anyway
    const float s = amax > 0.0f ? amax * (1.0f / 448.0f) : 1.0f;
    const float inv = 1.0f / s;
    if (lane == 0) scale[r] = s;
    uint2* dst = reinterpret_cast<uint2*>(q + r * K);
    for (int c = lane; c < chunks; c += 32) {
      const uint4 v = __ldg(src + c);
      const float2 a = unpack_bf16x2(v.x), b = unpack_bf16x2(v.y), cc = unpack_bf16x2(v.z), d = unpack_bf16x2(v.w);
      dst[c] = make_uint2(pack_e4m3x4(a.x * inv, a.y * inv, b.x * inv, b.y * inv),
                          pack_e4m3x4(cc.x * inv, cc.y * inv, d.x * inv, d.y * inv));
    }
  }
}

// The same conversion with scales chosen by the caller: row r uses scale_in[r / rows_per_scale] (weights: one scale
// per expert = rows_per_scale output channels).
__global__ void __launch_bounds__(Q_THREADS)
quantize_rows_given_scale_kernel(const bf16* __restrict__ x, long long rows, int K, long long rows_per_scale,
                                 const float* __restrict__ scale_in, uint8_t* __restrict__ q) {
  const int lane = threadIdx.x & 31;
  const int chunks = K >> 3;
  for (long long r = static_cast<long long>(blockIdx.x) * Q_WARPS + (threadIdx.x >> 5); r < rows;
       r += static_cast<long long>(gridDim.x) * Q_WARPS) {
    const float inv = 1.0f / __ldg(scale_in + r / rows_per_scale);
    const uint4* src = reinterpret_cast<const uint4*>(x + r * K);
    uint2* dst = reinterpret_cast<uint2*>(q + r * K);
    for (int c = lane; c < chunks; c += 32) {
      const uint4 v = __ldg(src + c);
      const float2 a = unpack_bf16x2(v.x), b = unpack_bf16x2(v.y), cc = unpack_bf16x2(v.z), d = unpack_bf16x2(v.w);
      dst[c] = make_uint2(pack_e4m3x4(a.x * inv, a.y * inv, b.x * inv, b.y * inv),
                          pack_e4m3x4(cc.x * inv, cc.y * inv, d.x * inv, d.y * inv));
    }
  }
}

}  // namespace

}  // namespace ffm

using namespace ffm;

extern "C" int ffm_quantize_rows_e4m3(const void* x, int64_t rows, int K, void* q, float* scale, ffm_stream_t stream) {
  if (!x || !q || !scale) return FFM_ERR_BAD_ARG;
  if (rows < 0 || K <= 0) return FFM_ERR_BAD_ARG;
  if (K % 16 != 0) return FFM_ERR_UNSUPPORTED;
  if (rows == 0) return FFM_OK;
  long long blocks = (rows + Q_WARPS - 1) / Q_WARPS;
  if (blocks > 148LL * 16) blocks = 148LL * 16;
  quantize_rows_e4m3_kernel<<<static_cast<int>(blocks), Q_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const bf16*>(x), rows, K, static_cast<uint8_t*>(q), scale);
  return cudaGetLastError() == cudaSuccess ? FFM_OK : FFM_ERR_LAUNCH;
}

extern "C" int ffm_quantize_rows_given_scale_e4m3(const void* x, int64_t rows, int K, int64_t rows_per_scale,
                                                  const float* scale_in, void* q, ffm_stream_t stream) {
  if (!x || !q || !scale_in) return FFM_ERR_BAD_ARG;
  if (rows < 0 || K <= 0 || rows_per_scale < 1) return FFM_ERR_BAD_ARG;
  if (K % 16 != 0) return FFM_ERR_UNSUPPORTED;
  if (rows == 0) return FFM_OK;
  long long blocks = (rows + Q_WARPS - 1) / Q_WARPS;
  if (blocks > 148LL * 16) blocks = 148LL * 16;
  quantize_rows_given_scale_kernel<<<static_cast<int>(blocks), Q_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const bf16*>(x), rows, K, rows_per_scale, scale_in, static_cast<uint8_t*>(q));
  return cudaGetLastError() == cudaSuccess ? FFM_OK : FFM_ERR_LAUNCH;
}
