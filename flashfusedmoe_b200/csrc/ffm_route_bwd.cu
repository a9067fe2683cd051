// Routing backward for sm_100a.
//
//   route_bwd_token    one warp per token: gradient of the logits (softmax / sigmoid Jacobian of the top-k
//                      weights, z-loss and aux-loss terms), rounded to bf16 as the reference does before its
//                      two skinny GEMMs, then dH[n, :] (+)= gl[n, :] * gate_w, skipping zero entries.
//   route_bwd_dgate    dGate partial sums over chunks of tokens (fp32), 8 experts x 8 columns per thread.
//   route_bwd_reduce   fixed-order sum of the partials -> bf16 dGate.
// Many experts (E a multiple of 64, D a multiple of 64, at least 1024 tokens): dGate = gl^T hidden is a GEMM with the
// token dimension as K, so it runs on the tensor cores instead (ffm_grouped_gemm_wgrad over DG_SPLITS ranges of the
// tokens, partial products in bf16, summed in fixed order by dgate_sum_splits); the dense CUDA-core reduction costs
// N E D multiply-adds, 285 us at N = 16384, E = 64, D = 2048.
#include "ffm_common.cuh"

namespace ffm {

namespace {

constexpr int RB_THREADS = 256;
constexpr int RB_WARPS = RB_THREADS / 32;
constexpr int MAX_E = 256;
constexpr int DG_THREADS = 128;            // 128 threads x 8 columns = 1024 columns per block
constexpr int DG_COLS = DG_THREADS * 8;
constexpr int DG_EXPERTS = 8;

__device__ __forceinline__ int round_up8(int x) { return (x + 7) & ~7; }

__global__ void __launch_bounds__(RB_THREADS)
route_bwd_token(const float* __restrict__ gw, const float* __restrict__ topk_w, const int32_t* __restrict__ topk_idx,
                const bf16* __restrict__ logits, const float* __restrict__ lse, const float* __restrict__ gaux,
                const float* __restrict__ gz_ptr, const bf16* __restrict__ gate_w, long long N, int D, int E, int top_k, int gating,
                int accumulate, bf16* __restrict__ gl_out, bf16* __restrict__ dH) {
  const int lane = threadIdx.x & 31;
  const int chunks = D >> 3;
  const int groups = (E + 31) >> 5;
  const int ldg_ = round_up8(E);
  const float inv_n = 1.0f / static_cast<float>(N);
  const float gz = (gz_ptr != nullptr) ? __ldg(gz_ptr) : 0.0f;

  for (long long n = static_cast<long long>(blockIdx.x) * RB_WARPS + (threadIdx.x >> 5); n < N;
       n += static_cast<long long>(gridDim.x) * RB_WARPS) {
    // ---- gradient w.r.t. the k selected logits (lanes 0..k-1) ----
    float g = 0.0f, s = 0.0f;
    int idx = -1;
    if (lane < top_k) {
      g = gw[n * top_k + lane];
      s = topk_w[n * top_k + lane];
      idx = topk_idx[n * top_k + lane];
      if (idx < 0 || idx >= E) idx = -1;
    }
    float gtl;
    if (gating == FFM_GATING_SOFTMAX) {
      if (gaux != nullptr && idx >= 0) g += gaux[idx] * inv_n;
      const float sg = warp_sum(g * s);
      gtl = s * (g - sg);
    } else {
      float sc = 0.0f;
      if (idx >= 0) sc = sigmoidf_(__bfloat162float(logits[n * E + idx]));
      const float ssum = warp_sum(sc);
      const float gdw = warp_sum(g * s);
      gtl = (g - gdw) / (ssum + 1e-6f) * sc * (1.0f - sc);
    }
    const float lse_n = (gz != 0.0f) ? lse[n] : 0.0f;

    // ---- dense gradient row: lane owns experts g * 32 + lane ----
    float glv[MAX_E / 32];
#pragma unroll
    for (int q = 0; q < MAX_E / 32; ++q) {
      glv[q] = 0.0f;
      if (q < groups) {
        const int e = q * 32 + lane;
        float v = 0.0f;
        for (int j = 0; j < top_k; ++j) {
          const int ij = __shfl_sync(0xffffffffu, idx, j);
          const float gj = __shfl_sync(0xffffffffu, gtl, j);
          if (ij == e) v += gj;
        }
        if (e < E) {
          const bool need_logit = (gz != 0.0f) || (gating == FFM_GATING_SIGMOID && gaux != nullptr);
          if (need_logit) {
            const float l = __bfloat162float(logits[n * E + e]);
            if (gz != 0.0f) v += gz * 2.0f * lse_n * inv_n * __expf(l - lse_n);
            if (gating == FFM_GATING_SIGMOID && gaux != nullptr) {
              const float sc = sigmoidf_(l);
              v += gaux[e] * sc * (1.0f - sc) * inv_n;
            }
          }
          const bf16 vb = __float2bfloat16_rn(v);
          gl_out[n * ldg_ + e] = vb;
          glv[q] = __bfloat162float(vb);
        } else if (e < ldg_) {
          gl_out[n * ldg_ + e] = __float2bfloat16_rn(0.0f);
        }
      }
    }

    // ---- dH[n, :] (+)= sum_e gl[e] * gate_w[e, :] ----
    for (int c0 = 0; c0 < chunks; c0 += 32) {
      const int c = c0 + lane;
      const bool active = c < chunks;
      float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
      for (int q = 0; q < MAX_E / 32; ++q) {
        if (q < groups) {
          const unsigned nz = __ballot_sync(0xffffffffu, glv[q] != 0.0f);
          unsigned m = nz;
          while (m) {
            const int l = __ffs(m) - 1;
            m &= m - 1;
            const float ge = __shfl_sync(0xffffffffu, glv[q], l);
            if (active) {
              const int e = q * 32 + l;
              const uint4 wv = __ldg(reinterpret_cast<const uint4*>(gate_w + static_cast<long long>(e) * D) + c);
              const float2 a = unpack_bf16x2(wv.x), b = unpack_bf16x2(wv.y), cc = unpack_bf16x2(wv.z), d = unpack_bf16x2(wv.w);
              acc[0] = fmaf(a.x, ge, acc[0]);
              acc[1] = fmaf(a.y, ge, acc[1]);
              acc[2] = fmaf(b.x, ge, acc[2]);
              acc[3] = fmaf(b.y, ge, acc[3]);
              acc[4] = fmaf(cc.x, ge, acc[4]);
              acc[5] = fmaf(cc.y, ge, acc[5]);
              acc[6] = fmaf(d.x, ge, acc[6]);
              acc[7] = fmaf(d.y, ge, acc[7]);
            }
          }
        }
      }
      if (!active) continue;
      uint4* dst = reinterpret_cast<uint4*>(dH + n * D) + c;
      if (accumulate) {
        // the reference rounds the routing term to bf16 (GEMM output) before adding it to dH
        const uint4 old = *dst;
        const float2 o0 = unpack_bf16x2(old.x), o1 = unpack_bf16x2(old.y), o2 = unpack_bf16x2(old.z), o3 = unpack_bf16x2(old.w);
        acc[0] = bf16_round(acc[0]) + o0.x;
        acc[1] = bf16_round(acc[1]) + o0.y;
        acc[2] = bf16_round(acc[2]) + o1.x;
        acc[3] = bf16_round(acc[3]) + o1.y;
        acc[4] = bf16_round(acc[4]) + o2.x;
        acc[5] = bf16_round(acc[5]) + o2.y;
        acc[6] = bf16_round(acc[6]) + o3.x;
        acc[7] = bf16_round(acc[7]) + o3.y;
      }
      *dst = make_uint4(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]), pack_bf16x2(acc[4], acc[5]),
                        pack_bf16x2(acc[6], acc[7]));
    }
  }
}

// grid = (token chunks, column blocks, expert groups of 8)
__global__ void __launch_bounds__(DG_THREADS)
route_bwd_dgate(const bf16* __restrict__ gl, const bf16* __restrict__ hidden, long long N, int D, int E,
                int tokens_per_chunk, float* __restrict__ partial) {
  const int ldg_ = round_up8(E);
  const int col0 = blockIdx.y * DG_COLS + threadIdx.x * 8;
  const int e0 = blockIdx.z * DG_EXPERTS;
  const long long n_begin = static_cast<long long>(blockIdx.x) * tokens_per_chunk;
  long long n_end = n_begin + tokens_per_chunk;
  if (n_end > N) n_end = N;
  const bool col_ok = col0 < D;

  float acc[DG_EXPERTS][8];
#pragma unroll
  for (int e = 0; e < DG_EXPERTS; ++e)
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[e][i] = 0.0f;

  if (col_ok) {
    // four tokens per trip: all gradient rows first, then the hidden rows that are needed, then the FMAs
    for (long long n0 = n_begin; n0 < n_end; n0 += 4) {
      uint4 gv[4], hv[4];
      bool need[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const long long n = n0 + j;
        gv[j] = make_uint4(0, 0, 0, 0);
        if (n < n_end) gv[j] = __ldg(reinterpret_cast<const uint4*>(gl + n * ldg_ + e0));
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        need[j] = (gv[j].x | gv[j].y | gv[j].z | gv[j].w) != 0u;  // skip rows whose eight gradients are +0
        hv[j] = make_uint4(0, 0, 0, 0);
        if (need[j]) hv[j] = __ldg(reinterpret_cast<const uint4*>(hidden + (n0 + j) * D + col0));
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (!need[j]) continue;
        const float2 h0 = unpack_bf16x2(hv[j].x), h1 = unpack_bf16x2(hv[j].y), h2 = unpack_bf16x2(hv[j].z),
                     h3 = unpack_bf16x2(hv[j].w);
        const float h[8] = {h0.x, h0.y, h1.x, h1.y, h2.x, h2.y, h3.x, h3.y};
        const float2 g0 = unpack_bf16x2(gv[j].x), g1 = unpack_bf16x2(gv[j].y), g2 = unpack_bf16x2(gv[j].z),
                     g3 = unpack_bf16x2(gv[j].w);
        const float g[8] = {g0.x, g0.y, g1.x, g1.y, g2.x, g2.y, g3.x, g3.y};
#pragma unroll
        for (int e = 0; e < DG_EXPERTS; ++e)
#pragma unroll
          for (int i = 0; i < 8; ++i) acc[e][i] = fmaf(g[e], h[i], acc[e][i]);
      }
    }
    float* out = partial + (static_cast<long long>(blockIdx.x) * ldg_ + e0) * D + col0;
#pragma unroll
    for (int e = 0; e < DG_EXPERTS; ++e) {
      if (e0 + e < ldg_) {
        float4* o = reinterpret_cast<float4*>(out + static_cast<long long>(e) * D);
        o[0] = make_float4(acc[e][0], acc[e][1], acc[e][2], acc[e][3]);
        o[1] = make_float4(acc[e][4], acc[e][5], acc[e][6], acc[e][7]);
      }
    }
  }
}

// Block = 32 columns x 8 chunk lanes: thread (tx, ty) sums partials ty, ty + 8, ... of output tx, then the eight
// lane sums are added in lane order. Fixed order, 8 x the parallelism of one thread per output.
__global__ void __launch_bounds__(256)
route_bwd_reduce(const float* __restrict__ partial, int chunks_n, int D, int E, bf16* __restrict__ dGate) {
  __shared__ float s_part[8][33];
  const int ldg_ = round_up8(E);
  const int tx = threadIdx.x & 31;
  const int ty = threadIdx.x >> 5;
  const long long total = static_cast<long long>(E) * D;
  for (long long base = static_cast<long long>(blockIdx.x) * 32; base < total;
       base += static_cast<long long>(gridDim.x) * 32) {
    const long long i = base + tx;
    float s = 0.0f;
    if (i < total) {
      const int e = static_cast<int>(i / D);
      const int d = static_cast<int>(i % D);
      const float* src = partial + static_cast<long long>(e) * D + d;
      const long long stride = static_cast<long long>(ldg_) * D;
#pragma unroll 4
      for (int c = ty; c < chunks_n; c += 8) s += src[c * stride];
    }
    s_part[ty][tx] = s;
    __syncthreads();
    if (ty == 0 && i < total) {
      float t = 0.0f;
#pragma unroll
      for (int k = 0; k < 8; ++k) t += s_part[k][tx];
      dGate[i] = __float2bfloat16_rn(t);
    }
    __syncthreads();
  }
}

constexpr int DG_SPLITS = 8;

// tile_start of DG_SPLITS equal ranges (whole tile pairs) over `pairs` pairs of 128-row tiles
__global__ void dgate_split_tiles(int32_t* __restrict__ ts, int pairs) {
  const int s = threadIdx.x;
  if (s <= DG_SPLITS) ts[s] = 2 * static_cast<int>((static_cast<long long>(pairs) * s) / DG_SPLITS);
}

__global__ void __launch_bounds__(256) dgate_sum_splits(const bf16* __restrict__ part, long long total,
                                                        bf16* __restrict__ dGate) {
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float t = 0.0f;
#pragma unroll
    for (int k = 0; k < DG_SPLITS; ++k) t += __bfloat162float(part[k * total + i]);
    dGate[i] = __float2bfloat16_rn(t);
  }
}

bool dgate_on_tensor_cores(long long N, int D, int E) { return E % 64 == 0 && D % 64 == 0 && N >= 1024; }

struct DgatePlan {
  int chunks_n;
  int tokens_per_chunk;
  int col_blocks;
  int e_groups;
};

DgatePlan plan_dgate(long long N, int D, int E) {
  DgatePlan p;
  p.col_blocks = (D + DG_COLS - 1) / DG_COLS;
  p.e_groups = (E + DG_EXPERTS - 1) / DG_EXPERTS;
  long long want = 296 / (static_cast<long long>(p.col_blocks) * p.e_groups);  // about two blocks per SM
  if (want < 1) want = 1;
  long long tpc = (N + want - 1) / want;
  if (tpc < 16) tpc = 16;
  p.tokens_per_chunk = static_cast<int>(tpc);
  p.chunks_n = static_cast<int>((N + tpc - 1) / tpc);
  if (p.chunks_n < 1) p.chunks_n = 1;
  return p;
}

size_t align256(size_t x) { return (x + 255) / 256 * 256; }

}  // namespace

}  // namespace ffm

using namespace ffm;

extern "C" size_t ffm_route_backward_workspace_bytes(int64_t N, int D, int E) {
  if (N < 0 || D <= 0 || E < 1) return 0;
  const int ldg_ = (E + 7) & ~7;
  const size_t gl_bytes = align256(static_cast<size_t>(N > 0 ? N : 1) * ldg_ * 2);
  if (dgate_on_tensor_cores(N, D, E)) {
    return gl_bytes + align256(static_cast<size_t>(DG_SPLITS) * E * D * 2) + 256;  // partials (bf16) + tile_start
  }
  DgatePlan p = plan_dgate(N > 0 ? N : 1, D, E);
  return gl_bytes + align256(static_cast<size_t>(p.chunks_n) * ldg_ * D * 4);
}

extern "C" int ffm_route_backward(const float* gw, const float* topk_w, const int32_t* topk_idx, const void* logits,
                                  const float* lse, const float* gaux, const float* gz, const void* hidden,
                                  const void* gate_w, int64_t N, int D, int E, int top_k, int gating, int accumulate,
                                  void* dH, void* dGate, void* workspace, size_t workspace_bytes, int32_t* status,
                                  ffm_stream_t stream) {
  if (!gw || !topk_w || !topk_idx || !hidden || !gate_w || !dH || !dGate || !workspace || !status) {
    return FFM_ERR_BAD_ARG;
  }
  if (N < 0 || D <= 0 || E < 1 || top_k < 1) return FFM_ERR_BAD_ARG;
  if (gating != FFM_GATING_SOFTMAX && gating != FFM_GATING_SIGMOID) return FFM_ERR_BAD_ARG;
  const bool need_logits = gating == FFM_GATING_SIGMOID || gz != nullptr;
  if (need_logits && (!logits || (gz != nullptr && !lse))) return FFM_ERR_BAD_ARG;
  if (D % 8 != 0 || E > MAX_E || top_k > 32 || top_k > E) return FFM_ERR_UNSUPPORTED;
  if (workspace_bytes < ffm_route_backward_workspace_bytes(N, D, E)) return FFM_ERR_WORKSPACE;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int ldg_ = (E + 7) & ~7;
  bf16* gl = static_cast<bf16*>(workspace);
  float* partial = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) +
                                            align256(static_cast<size_t>(N > 0 ? N : 1) * ldg_ * 2));
  if (N > 0) {
    long long blocks = (N + RB_WARPS - 1) / RB_WARPS;
    if (blocks > 148LL * 16) blocks = 148LL * 16;
    FFM_PREFER_MAX_SHARED(route_bwd_token);
    route_bwd_token<<<static_cast<int>(blocks), RB_THREADS, 0, s>>>(
        gw, topk_w, topk_idx, static_cast<const bf16*>(logits), lse, gaux, gz, static_cast<const bf16*>(gate_w), N, D,
        E, top_k, gating, accumulate, gl, static_cast<bf16*>(dH));
  }
  if (dgate_on_tensor_cores(N, D, E)) {
    // gl is [N, E] contiguous here (E % 8 == 0). dGate[e, :] = sum_n gl[n, e] hidden[n, :]
    uint8_t* base = static_cast<uint8_t*>(workspace) + align256(static_cast<size_t>(N) * ldg_ * 2);
    bf16* part = reinterpret_cast<bf16*>(base);
    int32_t* ts = reinterpret_cast<int32_t*>(base + align256(static_cast<size_t>(DG_SPLITS) * E * D * 2));
    const int pairs = static_cast<int>((N + 255) / 256);
    dgate_split_tiles<<<1, 32, 0, s>>>(ts, pairs);
    const int rc = ffm_grouped_gemm_wgrad(gl, hidden, DG_SPLITS, ts, N, E, D, 1.0f, part, status, stream);
    if (rc != FFM_OK) return rc;
    const long long total = static_cast<long long>(E) * D;
    long long blocks = (total + 255) / 256;
    if (blocks > 148LL * 8) blocks = 148LL * 8;
    dgate_sum_splits<<<static_cast<int>(blocks), 256, 0, s>>>(part, total, static_cast<bf16*>(dGate));
    return cudaGetLastError() == cudaSuccess ? FFM_OK : FFM_ERR_LAUNCH;
  }
  DgatePlan p = plan_dgate(N > 0 ? N : 1, D, E);
  if (N > 0) {
    dim3 grid(p.chunks_n, p.col_blocks, p.e_groups);
    FFM_PREFER_MAX_SHARED(route_bwd_dgate);
    route_bwd_dgate<<<grid, DG_THREADS, 0, s>>>(gl, static_cast<const bf16*>(hidden), N, D, E, p.tokens_per_chunk,
                                                partial);
  }
  {
    long long total = static_cast<long long>(E) * D;
    long long blocks = (total + 31) / 32;
    if (blocks > 148LL * 8) blocks = 148LL * 8;
    FFM_PREFER_MAX_SHARED(route_bwd_reduce);
    route_bwd_reduce<<<static_cast<int>(blocks), 256, 0, s>>>(partial, N > 0 ? p.chunks_n : 0, D, E,
                                                              static_cast<bf16*>(dGate));
  }
  return cudaGetLastError() == cudaSuccess ? FFM_OK : FFM_ERR_LAUNCH;
}
