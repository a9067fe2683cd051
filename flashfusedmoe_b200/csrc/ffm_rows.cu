// HBM-bound row kernels: permute into grouped rows, weighted combine and its backward, GLU backward.
// One warp per row, 16-byte vector accesses, fp32 arithmetic, bf16 storage.
#include "ffm_common.cuh"

namespace ffm {

namespace {

constexpr int ROW_THREADS = 256;
constexpr int ROW_WARPS = ROW_THREADS / 32;

__global__ void __launch_bounds__(ROW_THREADS)
permute_rows_kernel(const bf16* __restrict__ x, const int32_t* __restrict__ src, long long rows, int top_k, int D,
                    int zero_padding, bf16* __restrict__ grouped) {
  const int lane = threadIdx.x & 31;
  const int chunks = D >> 3;
  for (long long r = static_cast<long long>(blockIdx.x) * ROW_WARPS + (threadIdx.x >> 5); r < rows;
       r += static_cast<long long>(gridDim.x) * ROW_WARPS) {
    const int i = src[r];
    uint4* dst = reinterpret_cast<uint4*>(grouped + r * D);
    if (i < 0) {
      if (zero_padding) {
        for (int c = lane; c < chunks; c += 32) dst[c] = make_uint4(0, 0, 0, 0);
      }
    } else {
      const uint4* s = reinterpret_cast<const uint4*>(x + static_cast<long long>(i / top_k) * D);
      for (int c = lane; c < chunks; c += 32) dst[c] = __ldg(s + c);
    }
  }
}

__device__ __forceinline__ void fma8(float (&acc)[8], const uint4& v, float w) {
  const float2 a = unpack_bf16x2(v.x), b = unpack_bf16x2(v.y), c = unpack_bf16x2(v.z), d = unpack_bf16x2(v.w);
  acc[0] = fmaf(a.x, w, acc[0]);
  acc[1] = fmaf(a.y, w, acc[1]);
  acc[2] = fmaf(b.x, w, acc[2]);
  acc[3] = fmaf(b.y, w, acc[3]);
  acc[4] = fmaf(c.x, w, acc[4]);
  acc[5] = fmaf(c.y, w, acc[5]);
  acc[6] = fmaf(d.x, w, acc[6]);
  acc[7] = fmaf(d.y, w, acc[7]);
}

__device__ __forceinline__ uint4 pack8(const float (&a)[8]) {
  return make_uint4(pack_bf16x2(a[0], a[1]), pack_bf16x2(a[2], a[3]), pack_bf16x2(a[4], a[5]), pack_bf16x2(a[6], a[7]));
}

__global__ void __launch_bounds__(ROW_THREADS)
combine_forward_kernel(const bf16* __restrict__ Y, const int32_t* __restrict__ pos, const float* __restrict__ w,
                       const bf16* __restrict__ addend, long long N, int top_k, int D, bf16* __restrict__ out) {
  const int lane = threadIdx.x & 31;
  const int chunks = D >> 3;
  const int cblocks = (chunks + 31) >> 5;  // a warp handles one token and one block of 32 chunks (256 columns)
  const long long items = N * cblocks;
  for (long long item = static_cast<long long>(blockIdx.x) * ROW_WARPS + (threadIdx.x >> 5); item < items;
       item += static_cast<long long>(gridDim.x) * ROW_WARPS) {
    const long long n = item / cblocks;
    const int c0 = static_cast<int>(item % cblocks) << 5;
    // lane j < k holds slot j's row and weight
    int my_pos = 0;
    float my_w = 0.0f;
    if (lane < top_k) {
      my_pos = pos[n * top_k + lane];
      my_w = (w != nullptr) ? bf16_round(w[n * top_k + lane]) : 1.0f;
    }
    // every lane takes part in the shuffles, lanes past the row end only skip memory
    {
      const int c = c0 + lane;
      const bool active = c < chunks;
      float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      for (int j = 0; j < top_k; ++j) {
        const int pj = __shfl_sync(0xffffffffu, my_pos, j);
        const float wj = __shfl_sync(0xffffffffu, my_w, j);
        if (active) {
          const uint4 v = __ldg(reinterpret_cast<const uint4*>(Y + static_cast<long long>(pj) * D) + c);
          fma8(acc, v, wj);
        }
      }
      if (!active) continue;
      if (addend != nullptr) {
        // the reference adds the shared expert to the already rounded routed output
        const uint4 r = pack8(acc);
        const uint4 a = __ldg(reinterpret_cast<const uint4*>(addend + n * D) + c);
        float s[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        fma8(s, r, 1.0f);
        fma8(s, a, 1.0f);
        reinterpret_cast<uint4*>(out + n * D)[c] = pack8(s);
      } else {
        reinterpret_cast<uint4*>(out + n * D)[c] = pack8(acc);
      }
    }
  }
}

__global__ void __launch_bounds__(ROW_THREADS)
combine_backward_kernel(const bf16* __restrict__ go, const bf16* __restrict__ Y, const float* __restrict__ w,
                        const int32_t* __restrict__ src, long long rows, int top_k, int D, bf16* __restrict__ gYw,
                        float* __restrict__ gw) {
  const int lane = threadIdx.x & 31;
  const int chunks = D >> 3;
  for (long long r = static_cast<long long>(blockIdx.x) * ROW_WARPS + (threadIdx.x >> 5); r < rows;
       r += static_cast<long long>(gridDim.x) * ROW_WARPS) {
    const int i = src[r];
    uint4* dst = reinterpret_cast<uint4*>(gYw + r * D);
    if (i < 0) {
      for (int c = lane; c < chunks; c += 32) dst[c] = make_uint4(0, 0, 0, 0);
      continue;
    }
    const long long n = i / top_k;
    const float wi = (w != nullptr) ? bf16_round(w[i]) : 1.0f;
    const uint4* g = reinterpret_cast<const uint4*>(go + n * D);
    const uint4* y = (Y != nullptr) ? reinterpret_cast<const uint4*>(Y + r * D) : nullptr;
    float dot = 0.0f;
    for (int c = lane; c < chunks; c += 32) {
      const uint4 gv = __ldg(g + c);
      float o[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      fma8(o, gv, wi);
      dst[c] = pack8(o);
      if (y != nullptr) {
        const uint4 yv = __ldg(y + c);
        const float2 g0 = unpack_bf16x2(gv.x), g1 = unpack_bf16x2(gv.y), g2 = unpack_bf16x2(gv.z), g3 = unpack_bf16x2(gv.w);
        const float2 y0 = unpack_bf16x2(yv.x), y1 = unpack_bf16x2(yv.y), y2 = unpack_bf16x2(yv.z), y3 = unpack_bf16x2(yv.w);
        dot = fmaf(g0.x, y0.x, dot);
        dot = fmaf(g0.y, y0.y, dot);
        dot = fmaf(g1.x, y1.x, dot);
        dot = fmaf(g1.y, y1.y, dot);
        dot = fmaf(g2.x, y2.x, dot);
        dot = fmaf(g2.y, y2.y, dot);
        dot = fmaf(g3.x, y3.x, dot);
        dot = fmaf(g3.y, y3.y, dot);
      }
    }
    if (y != nullptr && gw != nullptr) {
      dot = warp_sum(dot);
      if (lane == 0) gw[i] = dot;
    }
  }
}

__global__ void __launch_bounds__(ROW_THREADS)
glu_backward_kernel(const bf16* __restrict__ dAct, const bf16* __restrict__ preact, const int32_t* __restrict__ tile_start,
                    int groups, long long rows, int H, int act, bf16* __restrict__ gU) {
  long long used = rows;
  if (tile_start != nullptr) {
    const long long u = static_cast<long long>(tile_start[groups]) * 128;
    if (u < used) used = u;
  }
  const int chunks = H >> 3;
  const long long total = used * chunks;
  for (long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = idx / chunks;
    const int c = static_cast<int>(idx % chunks);
    const uint4 ga = __ldg(reinterpret_cast<const uint4*>(dAct + r * H) + c);
    const uint4 gg = __ldg(reinterpret_cast<const uint4*>(preact + r * 2 * H) + c);
    const uint4 uu = __ldg(reinterpret_cast<const uint4*>(preact + r * 2 * H + H) + c);
    const uint32_t gav[4] = {ga.x, ga.y, ga.z, ga.w};
    const uint32_t ggv[4] = {gg.x, gg.y, gg.z, gg.w};
    const uint32_t uuv[4] = {uu.x, uu.y, uu.z, uu.w};
    uint32_t dg[4], du[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const float2 a = unpack_bf16x2(gav[q]), g = unpack_bf16x2(ggv[q]), u = unpack_bf16x2(uuv[q]);
      const float2 r0 = glu_bwd(act, a.x, g.x, u.x);
      const float2 r1 = glu_bwd(act, a.y, g.y, u.y);
      dg[q] = pack_bf16x2(r0.x, r1.x);
      du[q] = pack_bf16x2(r0.y, r1.y);
    }
    reinterpret_cast<uint4*>(gU + r * 2 * H)[c] = make_uint4(dg[0], dg[1], dg[2], dg[3]);
    reinterpret_cast<uint4*>(gU + r * 2 * H + H)[c] = make_uint4(du[0], du[1], du[2], du[3]);
  }
}

int grid_for_rows(long long rows) {
  long long blocks = (rows + ROW_WARPS - 1) / ROW_WARPS;
  const long long cap = 148LL * 16;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return static_cast<int>(blocks);
}

}  // namespace

}  // namespace ffm

using namespace ffm;

extern "C" int ffm_permute_rows(const void* x, const int32_t* src, int64_t rows_cap, int top_k, int D,
                                int zero_padding, void* grouped, ffm_stream_t stream) {
  if (!x || !src || !grouped) return FFM_ERR_BAD_ARG;
  if (rows_cap < 0 || top_k < 1 || D <= 0) return FFM_ERR_BAD_ARG;
  if (D % 8 != 0) return FFM_ERR_UNSUPPORTED;
  if (rows_cap == 0) return FFM_OK;
  FFM_PREFER_MAX_SHARED(permute_rows_kernel);
  permute_rows_kernel<<<grid_for_rows(rows_cap), ROW_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const bf16*>(x), src, rows_cap, top_k, D, zero_padding, static_cast<bf16*>(grouped));
  return cudaGetLastError() == cudaSuccess ? FFM_OK : FFM_ERR_LAUNCH;
}

extern "C" int ffm_combine_forward(const void* Y, const int32_t* pos, const float* w, const void* addend, int64_t N,
                                   int top_k, int D, void* out, ffm_stream_t stream) {
  if (!Y || !pos || !out) return FFM_ERR_BAD_ARG;
  if (N < 0 || top_k < 1 || D <= 0) return FFM_ERR_BAD_ARG;
  if (D % 8 != 0 || top_k > 32) return FFM_ERR_UNSUPPORTED;
  if (N == 0) return FFM_OK;
  FFM_PREFER_MAX_SHARED(combine_forward_kernel);
  combine_forward_kernel<<<grid_for_rows(N * ((D / 8 + 31) / 32)), ROW_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const bf16*>(Y), pos, w, static_cast<const bf16*>(addend), N, top_k, D, static_cast<bf16*>(out));
  return cudaGetLastError() == cudaSuccess ? FFM_OK : FFM_ERR_LAUNCH;
}

extern "C" int ffm_combine_backward(const void* go, const void* Y, const float* w, const int32_t* src,
                                    int64_t rows_cap, int top_k, int D, void* gYw, float* gw, ffm_stream_t stream) {
  if (!go || !src || !gYw) return FFM_ERR_BAD_ARG;
  if (rows_cap < 0 || top_k < 1 || D <= 0) return FFM_ERR_BAD_ARG;
  if (D % 8 != 0) return FFM_ERR_UNSUPPORTED;
  if (rows_cap == 0) return FFM_OK;
  FFM_PREFER_MAX_SHARED(combine_backward_kernel);
  combine_backward_kernel<<<grid_for_rows(rows_cap), ROW_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const bf16*>(go), static_cast<const bf16*>(Y), w, src, rows_cap, top_k, D,
      static_cast<bf16*>(gYw), gw);
  return cudaGetLastError() == cudaSuccess ? FFM_OK : FFM_ERR_LAUNCH;
}

extern "C" int ffm_glu_backward(const void* dAct, const void* preact, const int32_t* tile_start, int groups,
                                int64_t rows, int H, int activation, void* gU, ffm_stream_t stream) {
  if (!dAct || !preact || !gU) return FFM_ERR_BAD_ARG;
  if (rows < 0 || H <= 0 || activation < 0 || activation > 3) return FFM_ERR_BAD_ARG;
  if (tile_start != nullptr && groups < 1) return FFM_ERR_BAD_ARG;
  if (H % 8 != 0) return FFM_ERR_UNSUPPORTED;
  if (rows == 0) return FFM_OK;
  long long work = rows * (H / 8);
  long long blocks = (work + ROW_THREADS - 1) / ROW_THREADS;
  const long long cap = 148LL * 32;
  if (blocks > cap) blocks = cap;
  FFM_PREFER_MAX_SHARED(glu_backward_kernel);
  glu_backward_kernel<<<static_cast<int>(blocks), ROW_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const bf16*>(dAct), static_cast<const bf16*>(preact), tile_start, groups, rows, H, activation,
      static_cast<bf16*>(gU));
  return cudaGetLastError() == cudaSuccess ? FFM_OK : FFM_ERR_LAUNCH;
}
