// Routing forward for sm_100a.
//
//   route_gate_topk   one warp per pair of tokens: gate GEMM (fp32 accumulate, bf16 round), scoring,
//                     iterative-argmax top-k (lowest index wins ties), renormalisation, logsumexp,
//                     per-block expert histogram and probability-mass partial sums.
//   route_scan        one block: per-expert exclusive scan of the block histograms, expert counts,
//                     128-row-aligned segment starts (tile_start) and the loss statistics, all summed in a
//                     fixed order so results do not depend on scheduling.
//   route_rank        stable rank of every routed slot inside its expert segment -> pos[] and src[].
//
// Tokens are assigned to blocks in contiguous chunks, so "block order, then warp order, then slot order"
// equals the (token, slot) order of a stable sort by expert id.
#include <atomic>

#include "ffm_common.cuh"

namespace ffm {

namespace {

constexpr int ROUTE_THREADS = 256;
constexpr int ROUTE_WARPS = ROUTE_THREADS / 32;
constexpr int MAX_E = 256;
constexpr int TPW = 2;  // tokens per warp pass

struct RouteGrid {
  int blocks;
  int tokens_per_block;
};

// Tokens a block of the gate kernel handles per iteration: 8 warps x 2 tokens when a warp owns all experts
// (E <= 32), 16 / NG when the warps of a block share NG groups of 32 experts.
int route_granule(int E) { return E <= 32 ? 16 : (E <= 64 ? 8 : (E <= 128 ? 4 : 2)); }

RouteGrid route_grid(long long N, int granule = 16) {
  // Contiguous token chunks, a multiple of the granule, about four blocks per SM.
  long long target_blocks = 148 * 4;
  long long tpb = (N + target_blocks - 1) / target_blocks;
  tpb = ((tpb + granule - 1) / granule) * granule;
  if (tpb < granule) tpb = granule;
  RouteGrid g;
  g.tokens_per_block = static_cast<int>(tpb);
  g.blocks = static_cast<int>((N + tpb - 1) / tpb);
  if (g.blocks < 1) g.blocks = 1;
  return g;
}

// Sum GW per-lane partial accumulators across the warp; on return lane l holds the total of
// accumulator (l % GW) in a[0].
template <int GW>
__device__ __forceinline__ void transpose_reduce(float (&a)[GW], int lane) {
#pragma unroll
  for (int n = GW; n > 1; n >>= 1) {
    const int o = n >> 1;
    const bool upper = (lane & o) != 0;
#pragma unroll
    for (int i = 0; i < o; ++i) {
      const float lo = a[i], hi = a[i + o];
      const float send = upper ? lo : hi;
      const float keep = upper ? hi : lo;
      a[i] = keep + __shfl_xor_sync(0xffffffffu, send, o);
    }
  }
#pragma unroll
  for (int o = 16; o >= GW; o >>= 1) a[0] += __shfl_xor_sync(0xffffffffu, a[0], o);
}

__device__ __forceinline__ float dot8(const uint4& h, const uint4& w, float acc) {
  const float2 h0 = unpack_bf16x2(h.x), h1 = unpack_bf16x2(h.y), h2 = unpack_bf16x2(h.z), h3 = unpack_bf16x2(h.w);
  const float2 w0 = unpack_bf16x2(w.x), w1 = unpack_bf16x2(w.y), w2 = unpack_bf16x2(w.z), w3 = unpack_bf16x2(w.w);
  acc = fmaf(h0.x, w0.x, acc);
  acc = fmaf(h0.y, w0.y, acc);
  acc = fmaf(h1.x, w1.x, acc);
  acc = fmaf(h1.y, w1.y, acc);
  acc = fmaf(h2.x, w2.x, acc);
  acc = fmaf(h2.y, w2.y, acc);
  acc = fmaf(h3.x, w3.x, acc);
  acc = fmaf(h3.y, w3.y, acc);
  return acc;
}

struct RouteOpts {
  int gating;
  float weight_scale;
  int pre_softmax;  // softmax gating: probabilities over all experts before selection (DeepSeek-V3 style)
  int n_group;      // > 0: group-limited selection over n_group contiguous expert groups
  int topk_group;   // groups kept per token
};

// Warp arg-max of (value, expert) pairs: greater value wins, equal values go to the lower expert index.
__device__ __forceinline__ void warp_argmax(float& best, int& best_e) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
    if (ov > best || (ov == best && oe < best_e)) {
      best = ov;
      best_e = oe;
    }
  }
}

// Scoring, selection, weights and statistics of one token whose bf16-rounded logits are spread over the warp:
// lane holds expert g * 32 + lane for NG > 1 (GW == 32), expert lane % GW for NG == 1 (lanes >= GW replicate).
template <int GW, int NG>
__device__ __forceinline__ void route_token(const float (&logit)[NG], long long n, int lane, int E, int top_k,
                                            const RouteOpts& o, const float* __restrict__ bias,
                                            bf16* __restrict__ logits_out, float* __restrict__ topk_w,
                                            int32_t* __restrict__ topk_idx, float* __restrict__ lse_out,
                                            float (&mass)[NG], int (&cnt)[NG], float& zsum) {
  const bool holder_lane = (NG > 1) || (lane < GW);
  const int lane_e = (NG > 1) ? lane : (lane % GW);

  // logsumexp over all experts (z-loss, and the normaliser of pre-softmax scoring)
  float lmax = -INFINITY;
#pragma unroll
  for (int g = 0; g < NG; ++g) {
    const int e = g * GW + lane_e;
    if (holder_lane && e < E) {
      lmax = fmaxf(lmax, logit[g]);
      if (logits_out != nullptr) logits_out[n * E + e] = __float2bfloat16_rn(logit[g]);
    }
  }
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) lmax = fmaxf(lmax, __shfl_xor_sync(0xffffffffu, lmax, s));
  float esum = 0.0f;
#pragma unroll
  for (int g = 0; g < NG; ++g) {
    const int e = g * GW + lane_e;
    if (holder_lane && e < E) esum += __expf(logit[g] - lmax);
  }
  esum = warp_sum(esum);
  const float lse = lmax + __logf(esum);
  if (lane == 0) {
    lse_out[n] = lse;
    zsum += lse * lse;
  }

  float sel[NG];  // value used for selection
  float val[NG];  // unbiased value that becomes the weight (logit, probability or sigmoid score)
#pragma unroll
  for (int g = 0; g < NG; ++g) {
    const int e = g * GW + lane_e;
    const bool valid = holder_lane && e < E;
    const float lg = logit[g];
    float v;
    if (o.gating == FFM_GATING_SIGMOID) {
      v = sigmoid_rn(lg);
    } else if (o.pre_softmax) {
      v = __expf(lg - lse);
    } else {
      v = lg;
    }
    float sv = v;
    if (bias != nullptr && valid) sv = v + bias[e];
    val[g] = valid ? v : 0.0f;
    sel[g] = valid ? sv : -INFINITY;
  }
  if (o.gating == FFM_GATING_SIGMOID) {
#pragma unroll
    for (int g = 0; g < NG; ++g) mass[g] += val[g];
  }

  // ---- group-limited selection: keep the topk_group groups with the best sum of their top scores ----
  if (o.n_group > 0) {
    const int epg = E / o.n_group;
    const int per_group = top_k / o.topk_group;
    const bool use_sum = per_group > 1 && per_group <= epg;
    const int rounds = use_sum ? per_group : 1;
    float my_gscore = -INFINITY;  // lane gi holds the score of group gi
    for (int gi = 0; gi < o.n_group; ++gi) {
      float tmp[NG];
#pragma unroll
      for (int g = 0; g < NG; ++g) {
        const int e = g * GW + lane_e;
        tmp[g] = (e / epg == gi) ? sel[g] : -INFINITY;
      }
      float score = 0.0f;
      for (int r = 0; r < rounds; ++r) {
        float best = -INFINITY;
        int best_e = 0x7fffffff;
#pragma unroll
        for (int g = 0; g < NG; ++g) {
          if (tmp[g] > best) {
            best = tmp[g];
            best_e = g * GW + lane_e;
          }
        }
        warp_argmax(best, best_e);
        score = (r == 0) ? best : score + best;
#pragma unroll
        for (int g = 0; g < NG; ++g) {
          if (holder_lane && g * GW + lane_e == best_e) tmp[g] = -INFINITY;
        }
      }
      if (lane == gi) my_gscore = score;
    }
    unsigned keep = 0u;
    float gs = (lane < o.n_group) ? my_gscore : -INFINITY;
    for (int r = 0; r < o.topk_group; ++r) {
      float best = gs;
      int best_l = (gs == -INFINITY) ? 0x7fffffff : lane;
      warp_argmax(best, best_l);
      if (best_l < 32) keep |= 1u << best_l;
      if (lane == best_l) gs = -INFINITY;
    }
#pragma unroll
    for (int g = 0; g < NG; ++g) {
      const int e = g * GW + lane_e;
      if (!((keep >> ((e / epg) & 31)) & 1u)) sel[g] = -INFINITY;
    }
  }

  // ---- top-k by iterative argmax, lowest index wins ties ----
  float my_val = 0.0f;
  int my_idx = 0;
  for (int j = 0; j < top_k; ++j) {
    float best = -INFINITY;
    int best_e = 0x7fffffff;
#pragma unroll
    for (int g = 0; g < NG; ++g) {
      if (sel[g] > best) {
        best = sel[g];
        best_e = g * GW + lane_e;
      }
    }
    warp_argmax(best, best_e);
    // the holder of best_e publishes the unbiased value and retires the expert
    float v_pub = 0.0f;
#pragma unroll
    for (int g = 0; g < NG; ++g) {
      if (holder_lane && g * GW + lane_e == best_e) {
        v_pub = val[g];
        sel[g] = -INFINITY;
      }
    }
    v_pub = __shfl_sync(0xffffffffu, v_pub, best_e & 31);
    if (lane == j) {
      my_val = v_pub;
      my_idx = best_e;
    }
  }

  // ---- weights over the k selected values (lanes 0..k-1) ----
  float w;
  if (o.gating == FFM_GATING_SOFTMAX && !o.pre_softmax) {
    float m = (lane < top_k) ? my_val : -INFINITY;
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, s));
    const float ex = (lane < top_k) ? __expf(my_val - m) : 0.0f;
    const float den = warp_sum(ex);
    w = ex / den;
  } else {
    const float sc = (lane < top_k) ? my_val : 0.0f;
    const float den = warp_sum(sc) + 1e-6f;
    w = sc / den;
  }
  w *= o.weight_scale;
  if (lane < top_k) {
    topk_w[n * top_k + lane] = w;
    topk_idx[n * top_k + lane] = my_idx;
  }
  // ---- per-warp statistics: lane (e % 32) owns expert e ----
  for (int j = 0; j < top_k; ++j) {
    const int ej = __shfl_sync(0xffffffffu, my_idx, j);
    const float wj = __shfl_sync(0xffffffffu, w, j);
    const int own_lane = (NG > 1) ? (ej & 31) : ej;
#pragma unroll
    for (int g = 0; g < NG; ++g) {
      if (lane == own_lane && g == ((NG > 1) ? (ej >> 5) : 0)) {
        cnt[g] += 1;
        if (o.gating == FFM_GATING_SOFTMAX) mass[g] += wj;
      }
    }
  }
}

// Expert e = g * 32 + lane for NG > 1 (GW == 32); e = lane % GW for NG == 1.
template <int GW, int NG>
__global__ void __launch_bounds__(ROUTE_THREADS, (GW <= 8 ? 4 : (GW <= 16 ? 2 : 1)))
route_gate_topk(const bf16* __restrict__ hidden, const bf16* __restrict__ gate_w, const float* __restrict__ bias,
                long long N, int D, int E, int top_k, RouteOpts opts, int tokens_per_block,
                bf16* __restrict__ logits_out, float* __restrict__ topk_w, int32_t* __restrict__ topk_idx,
                float* __restrict__ lse_out, int32_t* __restrict__ block_hist, float* __restrict__ block_mass,
                float* __restrict__ block_z, int gate_in_smem) {
  // sized for the experts this instantiation can see, so that the few-expert variants fit beside a resident GEMM
  __shared__ float s_mass[ROUTE_WARPS][GW * NG];
  __shared__ int s_cnt[ROUTE_WARPS][GW * NG];
  __shared__ float s_z[ROUTE_WARPS];

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const long long tok_begin = static_cast<long long>(blockIdx.x) * tokens_per_block;
  long long tok_end = tok_begin + tokens_per_block;
  if (tok_end > N) tok_end = N;
  const int chunks = D >> 3;  // 16-byte chunks per row

  // Few experts (a warp owns them all): the block copies the gate matrix into shared memory once and every token's
  // dot products read it from there. Read from global memory instead, each lane re-loads E 16-byte chunks per chunk
  // of the token, far more loads than the 64 registers of this occupancy can keep in flight, and the kernel ran at
  // an eighth of HBM speed.
  extern __shared__ uint4 s_gate[];
  if (NG == 1 && gate_in_smem) {
    const uint4* gsrc = reinterpret_cast<const uint4*>(gate_w);
    for (int i = threadIdx.x; i < E * chunks; i += ROUTE_THREADS) s_gate[i] = __ldg(gsrc + i);
    __syncthreads();
  }

  float mass[NG];
  int cnt[NG];
#pragma unroll
  for (int g = 0; g < NG; ++g) {
    mass[g] = 0.0f;
    cnt[g] = 0;
  }
  float zsum = 0.0f;

  if constexpr (NG > 1) {
    // Many experts: the warps of a block share the gate GEMM of a few token pairs. Warp w computes the 32 experts
    // of group (w % NG) for pair (w / NG) and leaves the logits in shared memory; then warp t routes token t of the
    // iteration. 8 / NG pairs per iteration keep every warp busy in the GEMM phase for any NG in {2, 4, 8}.
    constexpr int PAIRS = ROUTE_WARPS / NG;
    __shared__ float s_logit[2 * PAIRS][NG * 32];
    const int my_pair = warp / NG;
    const int my_group = warp % NG;
    for (long long it0 = tok_begin; it0 < tok_end; it0 += 2 * PAIRS) {
      const long long t0 = it0 + 2 * my_pair;
      if (t0 < tok_end) {
        const bool has1 = (t0 + 1) < tok_end;
        const uint4* h0p = reinterpret_cast<const uint4*>(hidden + t0 * D);
        const uint4* h1p = reinterpret_cast<const uint4*>(hidden + (has1 ? t0 + 1 : t0) * D);
        float acc0[32], acc1[32];
#pragma unroll
        for (int e = 0; e < 32; ++e) {
          acc0[e] = 0.0f;
          acc1[e] = 0.0f;
        }
        for (int c = lane; c < chunks; c += 32) {
          const uint4 a0 = __ldg(h0p + c);
          const uint4 a1 = __ldg(h1p + c);
#pragma unroll
          for (int e = 0; e < 32; ++e) {
            const int ee = my_group * 32 + e;
            if (ee < E) {
              const uint4 w = __ldg(reinterpret_cast<const uint4*>(gate_w + static_cast<long long>(ee) * D) + c);
              acc0[e] = dot8(a0, w, acc0[e]);
              acc1[e] = dot8(a1, w, acc1[e]);
            }
          }
        }
        transpose_reduce<32>(acc0, lane);
        transpose_reduce<32>(acc1, lane);
        s_logit[2 * my_pair][my_group * 32 + lane] = bf16_round(acc0[0]);
        s_logit[2 * my_pair + 1][my_group * 32 + lane] = bf16_round(acc1[0]);
      }
      __syncthreads();
      if (warp < 2 * PAIRS && it0 + warp < tok_end) {
        float logit[NG];
#pragma unroll
        for (int g = 0; g < NG; ++g) logit[g] = s_logit[warp][g * 32 + lane];
        route_token<GW, NG>(logit, it0 + warp, lane, E, top_k, opts, bias, logits_out, topk_w, topk_idx, lse_out, mass,
                            cnt, zsum);
      }
      __syncthreads();
    }
  } else {
    for (long long t0 = tok_begin + warp * TPW; t0 < tok_end; t0 += ROUTE_WARPS * TPW) {
      const bool has1 = (t0 + 1) < tok_end;
      const uint4* h0p = reinterpret_cast<const uint4*>(hidden + t0 * D);
      const uint4* h1p = reinterpret_cast<const uint4*>(hidden + (has1 ? t0 + 1 : t0) * D);

      // ---- gate GEMM: logit[tk][g] for expert g * 32 + lane (or lane % GW) ----
      float logit0[NG], logit1[NG];
  #pragma unroll
      for (int g = 0; g < NG; ++g) {
        float acc0[GW], acc1[GW];
  #pragma unroll
        for (int e = 0; e < GW; ++e) {
          acc0[e] = 0.0f;
          acc1[e] = 0.0f;
        }
        // unrolled so that the loads of several chunks are in flight together (the kernel is latency-bound)
  #pragma unroll(GW <= 16 ? 4 : 1)
        for (int c = lane; c < chunks; c += 32) {
          const uint4 a0 = __ldg(h0p + c);
          const uint4 a1 = __ldg(h1p + c);
  #pragma unroll
          for (int e = 0; e < GW; ++e) {
            const int ee = g * GW + e;
            if (ee < E) {
              const uint4 w = gate_in_smem
                                  ? s_gate[ee * chunks + c]
                                  : __ldg(reinterpret_cast<const uint4*>(gate_w + static_cast<long long>(ee) * D) + c);
              acc0[e] = dot8(a0, w, acc0[e]);
              acc1[e] = dot8(a1, w, acc1[e]);
            }
          }
        }
        transpose_reduce<GW>(acc0, lane);
        transpose_reduce<GW>(acc1, lane);
        logit0[g] = bf16_round(acc0[0]);
        logit1[g] = bf16_round(acc1[0]);
      }

      route_token<GW, NG>(logit0, t0, lane, E, top_k, opts, bias, logits_out, topk_w, topk_idx, lse_out, mass, cnt, zsum);
      if (has1) {
        route_token<GW, NG>(logit1, t0 + 1, lane, E, top_k, opts, bias, logits_out, topk_w, topk_idx, lse_out, mass, cnt,
                            zsum);
      }
    }
  }

  // ---- block reduction in fixed warp order ----
#pragma unroll
  for (int g = 0; g < NG; ++g) {
    const int e = g * GW + (NG > 1 ? lane : (lane % GW));
    const bool holder_lane = (NG > 1) || (lane < GW);
    if (holder_lane && e < E) {
      s_mass[warp][e] = mass[g];
      s_cnt[warp][e] = cnt[g];
    }
  }
  if (lane == 0) s_z[warp] = zsum;
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += ROUTE_THREADS) {
    float m = 0.0f;
    int c = 0;
    for (int w = 0; w < ROUTE_WARPS; ++w) {
      m += s_mass[w][e];
      c += s_cnt[w][e];
    }
    block_mass[static_cast<long long>(blockIdx.x) * E + e] = m;
    block_hist[static_cast<long long>(blockIdx.x) * E + e] = c;
  }
  if (threadIdx.x == 0) {
    float z = 0.0f;
    for (int w = 0; w < ROUTE_WARPS; ++w) z += s_z[w];
    block_z[blockIdx.x] = z;
  }
}

// Scoring / top-k / statistics from logits that a GEMM already wrote (bf16 [N, E]): one warp per token, lane holds
// experts g * 32 + lane. Used when the gate GEMM runs on the tensor cores (many experts), where a CUDA-core dot
// product per (token, expert) would dominate the routing time.
template <int NG>
__global__ void __launch_bounds__(ROUTE_THREADS)
route_from_logits(const bf16* __restrict__ logits, const float* __restrict__ bias, long long N, int E, int top_k,
                  RouteOpts opts, int tokens_per_block, float* __restrict__ topk_w, int32_t* __restrict__ topk_idx,
                  float* __restrict__ lse_out, int32_t* __restrict__ block_hist, float* __restrict__ block_mass,
                  float* __restrict__ block_z) {
  __shared__ float s_mass[ROUTE_WARPS][MAX_E];
  __shared__ int s_cnt[ROUTE_WARPS][MAX_E];
  __shared__ float s_z[ROUTE_WARPS];
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const long long tok_begin = static_cast<long long>(blockIdx.x) * tokens_per_block;
  long long tok_end = tok_begin + tokens_per_block;
  if (tok_end > N) tok_end = N;
  float mass[NG];
  int cnt[NG];
#pragma unroll
  for (int g = 0; g < NG; ++g) {
    mass[g] = 0.0f;
    cnt[g] = 0;
  }
  float zsum = 0.0f;
  for (long long n = tok_begin + warp; n < tok_end; n += ROUTE_WARPS) {
    float logit[NG];
#pragma unroll
    for (int g = 0; g < NG; ++g) {
      const int e = g * 32 + lane;
      logit[g] = (e < E) ? __bfloat162float(logits[n * E + e]) : 0.0f;
    }
    route_token<32, NG>(logit, n, lane, E, top_k, opts, bias, nullptr, topk_w, topk_idx, lse_out, mass, cnt, zsum);
  }
#pragma unroll
  for (int g = 0; g < NG; ++g) {
    const int e = g * 32 + lane;
    if (e < E) {
      s_mass[warp][e] = mass[g];
      s_cnt[warp][e] = cnt[g];
    }
  }
  if (lane == 0) s_z[warp] = zsum;
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += ROUTE_THREADS) {
    float m = 0.0f;
    int c = 0;
    for (int w = 0; w < ROUTE_WARPS; ++w) {
      m += s_mass[w][e];
      c += s_cnt[w][e];
    }
    block_mass[static_cast<long long>(blockIdx.x) * E + e] = m;
    block_hist[static_cast<long long>(blockIdx.x) * E + e] = c;
  }
  if (threadIdx.x == 0) {
    float z = 0.0f;
    for (int w = 0; w < ROUTE_WARPS; ++w) z += s_z[w];
    block_z[blockIdx.x] = z;
  }
}

// Histogram of given expert ids with the same block chunking (expert-parallel receive side).
__global__ void __launch_bounds__(ROUTE_THREADS)
route_hist_ids(const int32_t* __restrict__ ids, long long T, int E, int slots_per_block,
               int32_t* __restrict__ block_hist, int32_t* __restrict__ status) {
  __shared__ int s_cnt[MAX_E];
  for (int e = threadIdx.x; e < E; e += ROUTE_THREADS) s_cnt[e] = 0;
  __syncthreads();
  const long long begin = static_cast<long long>(blockIdx.x) * slots_per_block;
  long long end = begin + slots_per_block;
  if (end > T) end = T;
  for (long long i = begin + threadIdx.x; i < end; i += ROUTE_THREADS) {
    const int e = ids[i];
    if (e >= 0 && e < E) {
      atomicAdd(&s_cnt[e], 1);
    } else {
      atomicCAS(status, 0, FFM_STATUS_BAD_INDEX);
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += ROUTE_THREADS) block_hist[static_cast<long long>(blockIdx.x) * E + e] = s_cnt[e];
}

// One block. block_off[b][e] = sum_{b' < b} hist[b'][e]; counts; tile_start; stats.
// One warp per expert: the lanes sweep the block histograms 32 at a time (independent loads, a shuffle scan and a
// carry), so the kernel costs a few dozen dependent steps instead of one per block. All sums keep a fixed order.
__global__ void __launch_bounds__(ROUTE_THREADS)
route_scan(const int32_t* __restrict__ block_hist, const float* __restrict__ block_mass,
           const float* __restrict__ block_z, int blocks, int E, int32_t* __restrict__ block_off,
           int32_t* __restrict__ counts, int32_t* __restrict__ tile_start, float* __restrict__ stats) {
  __shared__ int s_counts[MAX_E];
  __shared__ float s_mass[MAX_E];
  __shared__ float s_zsum;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  for (int e = warp; e < E; e += ROUTE_WARPS) {
    int carry = 0;
    float m = 0.0f;
#pragma unroll 4
    for (int b0 = 0; b0 < blocks; b0 += 32) {
      const int b = b0 + lane;
      const long long o = static_cast<long long>(b) * E + e;
      const int v = (b < blocks) ? block_hist[o] : 0;
      if (block_mass != nullptr && b < blocks) m += block_mass[o];
      int x = v;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, x, d);
        if (lane >= d) x += t;
      }
      if (b < blocks) block_off[o] = carry + x - v;
      carry += __shfl_sync(0xffffffffu, x, 31);
    }
    m = warp_sum(m);
    if (lane == 0) {
      s_counts[e] = carry;
      s_mass[e] = m;
      counts[e] = carry;
      if (stats != nullptr) stats[e] = m;
    }
  }
  if (warp == ROUTE_WARPS - 1) {
    float z = 0.0f;
    if (block_z != nullptr) {
      for (int b = lane; b < blocks; b += 32) z += block_z[b];
    }
    z = warp_sum(z);
    if (lane == 0) s_zsum = z;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int tiles = 0;
    float dot = 0.0f;
    tile_start[0] = 0;
    for (int e = 0; e < E; ++e) {
      tiles += ((s_counts[e] + 255) >> 8) << 1;  // segments start on multiples of 256 rows
      tile_start[e + 1] = tiles;
      dot += static_cast<float>(s_counts[e]) * s_mass[e];
    }
    if (stats != nullptr) {
      stats[E] = s_zsum;
      stats[E + 1] = dot;
    }
  }
}

// Stable rank inside each expert segment. Each warp owns a contiguous run of the block's slots.
__global__ void __launch_bounds__(ROUTE_THREADS)
route_rank(const int32_t* __restrict__ ids, long long T, int E, int slots_per_block,
           const int32_t* __restrict__ block_off, const int32_t* __restrict__ tile_start, long long rows_cap,
           int32_t* __restrict__ pos, int32_t* __restrict__ src, int32_t* __restrict__ status) {
  __shared__ int s_run[ROUTE_WARPS][MAX_E];
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const long long begin = static_cast<long long>(blockIdx.x) * slots_per_block;
  long long end = begin + slots_per_block;
  if (end > T) end = T;
  const long long span = end > begin ? end - begin : 0;
  const long long per_warp = ((span + ROUTE_WARPS - 1) / ROUTE_WARPS + 31) / 32 * 32;
  const long long wb = begin + warp * per_warp;
  long long we = wb + per_warp;
  if (we > end) we = end;

  for (int e = lane; e < E; e += 32) s_run[warp][e] = 0;
  __syncwarp();
  // pass 1: per-warp counts
  for (long long i = wb + lane; i < we; i += 32) {
    const int e = ids[i];
    if (e >= 0 && e < E) atomicAdd(&s_run[warp][e], 1);
  }
  __syncthreads();
  // exclusive scan over warps, per expert, plus the block and segment bases
  for (int e = threadIdx.x; e < E; e += ROUTE_THREADS) {
    int run = tile_start[e] * 128 + block_off[static_cast<long long>(blockIdx.x) * E + e];
    for (int w = 0; w < ROUTE_WARPS; ++w) {
      const int c = s_run[w][e];
      s_run[w][e] = run;
      run += c;
    }
  }
  __syncthreads();
  // pass 2: walk the run in order, 32 slots at a time
  for (long long i0 = wb; i0 < we; i0 += 32) {
    const long long i = i0 + lane;
    const bool active = i < we;
    int e = active ? ids[i] : -1;
    if (active && (e < 0 || e >= E)) {
      atomicCAS(status, 0, FFM_STATUS_BAD_INDEX);
      e = -1;
    }
    const unsigned same = __match_any_sync(0xffffffffu, e);
    const int leader = __ffs(same) - 1;
    const int rank = __popc(same & ((1u << lane) - 1u));
    int base = 0;
    if (e >= 0 && lane == leader) {
      base = s_run[warp][e];
      s_run[warp][e] = base + __popc(same);
    }
    base = __shfl_sync(0xffffffffu, base, leader);
    __syncwarp();
    if (e >= 0) {
      const long long r = static_cast<long long>(base) + rank;
      if (r < rows_cap) {
        pos[i] = static_cast<int32_t>(r);
        src[r] = static_cast<int32_t>(i);
      } else {
        atomicCAS(status, 0, FFM_STATUS_BAD_INDEX);
      }
    }
  }
}

struct RouteWorkspace {
  int32_t* block_hist;
  int32_t* block_off;
  float* block_mass;
  float* block_z;
  size_t bytes;
};

RouteWorkspace carve_workspace(void* base, int blocks, int E) {
  RouteWorkspace w;
  size_t off = 0;
  auto take = [&](size_t n) {
    size_t o = off;
    off += (n + 255) / 256 * 256;
    return o;
  };
  const size_t per = static_cast<size_t>(blocks) * E * 4;
  size_t o_hist = take(per), o_off = take(per), o_mass = take(per), o_z = take(static_cast<size_t>(blocks) * 4);
  uint8_t* b = static_cast<uint8_t*>(base);
  w.block_hist = reinterpret_cast<int32_t*>(b + o_hist);
  w.block_off = reinterpret_cast<int32_t*>(b + o_off);
  w.block_mass = reinterpret_cast<float*>(b + o_mass);
  w.block_z = reinterpret_cast<float*>(b + o_z);
  w.bytes = off;
  return w;
}

template <int GW, int NG>
void launch_route(int blocks, cudaStream_t s, const bf16* hidden, const bf16* gate_w, const float* bias, long long N,
                  int D, int E, int top_k, const RouteOpts& opts, int tpb, bf16* logits, float* topk_w,
                  int32_t* topk_idx, float* lse, const RouteWorkspace& w) {
  auto kernel = route_gate_topk<GW, NG>;
  FFM_PREFER_MAX_SHARED(kernel);
  // gate matrix in shared memory when a warp owns all experts, E x D bf16 fits in 64 KiB and E > 8: with up to eight
  // experts staging gains nothing (the matrix stays hot in L1), and without it a block needs 2 KiB of shared memory
  // and can run on an SM that holds a GEMM CTA (the shared expert's GEMMs run beside the routing kernels)
  constexpr size_t kGateSmemMax = 64 * 1024;
  const size_t gate_bytes = static_cast<size_t>(E) * D * sizeof(bf16);
  static bool smem_ok = false, smem_tried = false;
  if (NG == 1 && !smem_tried) {
    smem_tried = true;
    smem_ok = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   static_cast<int>(kGateSmemMax)) == cudaSuccess;
    if (!smem_ok) cudaGetLastError();
  }
  const bool in_smem =
      NG == 1 && E > 8 && gate_bytes <= kGateSmemMax && (gate_bytes <= 48 * 1024 || smem_ok) && D % 8 == 0;
  route_gate_topk<GW, NG><<<blocks, ROUTE_THREADS, in_smem ? gate_bytes : 0, s>>>(
      hidden, gate_w, bias, N, D, E, top_k, opts, tpb, logits, topk_w, topk_idx, lse, w.block_hist, w.block_mass,
      w.block_z, in_smem ? 1 : 0);
}

// Expert capacity: a routed slot whose rank inside its expert segment is >= capacity is dropped. One thread
// per token: dropped slots get weight 0 and their grouped row becomes a padding row (src = -1, so every later
// kernel sees zeros there); the kept weights are renormalised by their sum, or left at zero when nothing is kept.
__global__ void __launch_bounds__(ROUTE_THREADS)
route_capacity_kernel(float* __restrict__ topk_w, const int32_t* __restrict__ topk_idx, const int32_t* __restrict__ pos,
                      int32_t* __restrict__ src, const int32_t* __restrict__ tile_start, long long N, int top_k, int E,
                      int capacity, int32_t* __restrict__ dropped) {
  const long long n = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (n >= N) return;
  float sum = 0.0f;
  int ndrop = 0;
  for (int j = 0; j < top_k; ++j) {
    const long long i = n * top_k + j;
    const int e = topk_idx[i];
    if (e < 0 || e >= E) continue;
    const int r = pos[i] - tile_start[e] * 128;
    float w = topk_w[i];
    if (r >= capacity) {
      w = 0.0f;
      src[pos[i]] = -1;
      ++ndrop;
    }
    topk_w[i] = w;
    sum += w;
  }
  const float denom = sum + (sum > 0.0f ? 0.0f : 1.0f);
  for (int j = 0; j < top_k; ++j) topk_w[n * top_k + j] /= denom;
  if (ndrop > 0) atomicAdd(dropped, ndrop);
}

// ---- scratch for the allocation-free entry point ---------------------------------------------
// Lives in the library image: every GPU that loads libffmoe holds these bytes until the process exits.
// Sized for the stated maximum of ffm_group_rows_static: 592 blocks x 256 experts x 4 bytes, twice.
static __device__ __align__(256) unsigned char g_static_scratch[FFM_STATIC_SCRATCH_BYTES];

// Device address of g_static_scratch on the current device. In host code the array's name is only a
// stand-in for the symbol, not a pointer a kernel could use, so the address is asked for once per device
// (with that device current) and remembered.
int static_scratch_address(void** out) {
  static std::atomic<void*> cached[64];  // (zero-initialised; host threads may race here: same value either way)
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
    cudaGetLastError();
    return FFM_ERR_LAUNCH;
  }
  void* p = cached[dev].load(std::memory_order_acquire);
  if (p == nullptr) {
    if (cudaGetSymbolAddress(&p, g_static_scratch) != cudaSuccess || p == nullptr) {
      cudaGetLastError();
      return FFM_ERR_LAUNCH;
    }
    cached[dev].store(p, std::memory_order_release);
  }
  *out = p;
  return FFM_OK;
}

}  // namespace

}  // namespace ffm

using namespace ffm;

extern "C" int64_t ffm_rows_capacity(int64_t T, int E) {
  if (T < 0 || E < 1) return 0;
  return ((T + 255LL * E) / 256) * 256;
}

extern "C" size_t ffm_route_workspace_bytes(int64_t N, int E, int top_k) {
  (void)top_k;
  if (N < 0 || E < 1) return 0;
  // The same workspace serves ffm_group_rows over N * top_k slots, whose grid is never larger.
  RouteGrid g = route_grid(N > 0 ? N : 1, route_granule(E));
  RouteGrid g2 = route_grid(N > 0 ? N * (top_k > 0 ? top_k : 1) : 1);
  int blocks = g.blocks > g2.blocks ? g.blocks : g2.blocks;
  return carve_workspace(nullptr, blocks, E).bytes;
}

extern "C" int ffm_route_forward(const void* hidden, const void* gate_w, const float* expert_bias, int64_t N, int D,
                                 int E, int top_k, int gating, float weight_scale, int pre_softmax, int n_group,
                                 int topk_group, void* logits, float* topk_w,
                                 int32_t* topk_idx, float* lse, int32_t* counts, int32_t* tile_start, int32_t* pos,
                                 int32_t* src, int64_t rows_cap, float* stats, void* workspace,
                                 size_t workspace_bytes, int32_t* status, ffm_stream_t stream) {
  if (!hidden || !gate_w || !topk_w || !topk_idx || !lse || !counts || !tile_start || !pos || !src || !stats ||
      !workspace || !status)
    return FFM_ERR_BAD_ARG;
  if (N < 0 || D <= 0 || E < 1 || top_k < 1) return FFM_ERR_BAD_ARG;
  if (gating != FFM_GATING_SOFTMAX && gating != FFM_GATING_SIGMOID) return FFM_ERR_BAD_ARG;
  if (D % 8 != 0 || E > MAX_E || top_k > E || top_k > 32) return FFM_ERR_UNSUPPORTED;
  if (n_group < 0 || (n_group > 0 && (topk_group < 1 || topk_group > n_group))) return FFM_ERR_BAD_ARG;
  if (n_group > 32 || (n_group > 0 && E % n_group != 0)) return FFM_ERR_UNSUPPORTED;
  if (rows_cap < ffm_rows_capacity(N * top_k, E)) return FFM_ERR_BAD_ARG;
  RouteOpts opts;
  opts.gating = gating;
  opts.weight_scale = weight_scale;
  opts.pre_softmax = (gating == FFM_GATING_SOFTMAX && pre_softmax) ? 1 : 0;
  opts.n_group = n_group;
  opts.topk_group = topk_group;
  if (workspace_bytes < ffm_route_workspace_bytes(N, E, top_k)) return FFM_ERR_WORKSPACE;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (cudaMemsetAsync(src, 0xFF, static_cast<size_t>(rows_cap) * 4, s) != cudaSuccess) return FFM_ERR_LAUNCH;
  const RouteGrid g = route_grid(N > 0 ? N : 1, route_granule(E));
  RouteWorkspace w = carve_workspace(workspace, g.blocks, E);
  const bf16* h = static_cast<const bf16*>(hidden);
  const bf16* gw = static_cast<const bf16*>(gate_w);
  bf16* lg = static_cast<bf16*>(logits);
  // Many experts: gate GEMM on the tensor cores (dense tcgen05 GEMM, fp32 accumulate, bf16 logits), then one
  // scoring kernel. Few experts: everything in one warp-level kernel.
  // (E = 32 included: one warp owning 32 experts keeps 64 accumulators per lane and ran at 0.12 TB/s)
  const bool tensor_gate = E >= 32 && D % 64 == 0 && E % 32 == 0 && logits != nullptr;
  if (tensor_gate) {
    const int rc = ffm_grouped_gemm(hidden, gate_w, FFM_B_KMAJOR, 1, nullptr, N, D, E, 1.0f, logits, nullptr, 0, status,
                                    stream);
    if (rc != FFM_OK) return rc;
#define FFM_LOGIT_CASE(NG)                                                                                      \
  route_from_logits<NG><<<g.blocks, ROUTE_THREADS, 0, s>>>(lg, expert_bias, N, E, top_k, opts, g.tokens_per_block, \
                                                           topk_w, topk_idx, lse, w.block_hist, w.block_mass, w.block_z)
    if (E <= 64) {
      FFM_LOGIT_CASE(2);
    } else if (E <= 128) {
      FFM_LOGIT_CASE(4);
    } else {
      FFM_LOGIT_CASE(8);
    }
#undef FFM_LOGIT_CASE
  } else {
#define FFM_ROUTE_CASE(GW, NG)                                                                                 \
  launch_route<GW, NG>(g.blocks, s, h, gw, expert_bias, N, D, E, top_k, opts, g.tokens_per_block, lg, topk_w, \
                       topk_idx, lse, w)
  if (E <= 8) {
    FFM_ROUTE_CASE(8, 1);
  } else if (E <= 16) {
    FFM_ROUTE_CASE(16, 1);
  } else if (E <= 32) {
    FFM_ROUTE_CASE(32, 1);
  } else if (E <= 64) {
    FFM_ROUTE_CASE(32, 2);
  } else if (E <= 128) {
    FFM_ROUTE_CASE(32, 4);
  } else {
    FFM_ROUTE_CASE(32, 8);
  }
#undef FFM_ROUTE_CASE
  }
  FFM_PREFER_MAX_SHARED(route_scan);
  route_scan<<<1, ROUTE_THREADS, 0, s>>>(w.block_hist, w.block_mass, w.block_z, g.blocks, E, w.block_off, counts,
                                         tile_start, stats);
  route_rank<<<g.blocks, ROUTE_THREADS, 0, s>>>(topk_idx, N * top_k, E, g.tokens_per_block * top_k, w.block_off,
                                                tile_start, rows_cap, pos, src, status);
  return cudaGetLastError() == cudaSuccess ? FFM_OK : FFM_ERR_LAUNCH;
}

extern "C" int ffm_group_rows(const int32_t* expert_ids, int64_t T, int E, int32_t* counts, int32_t* tile_start,
                              int32_t* pos, int32_t* src, int64_t rows_cap, void* workspace, size_t workspace_bytes,
                              int32_t* status, ffm_stream_t stream) {
  if (!expert_ids || !counts || !tile_start || !pos || !src || !workspace || !status) return FFM_ERR_BAD_ARG;
  if (T < 0 || E < 1) return FFM_ERR_BAD_ARG;
  if (E > MAX_E) return FFM_ERR_UNSUPPORTED;
  if (rows_cap < ffm_rows_capacity(T, E)) return FFM_ERR_BAD_ARG;
  const RouteGrid g = route_grid(T > 0 ? T : 1);
  if (workspace_bytes < carve_workspace(nullptr, g.blocks, E).bytes) return FFM_ERR_WORKSPACE;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (cudaMemsetAsync(src, 0xFF, static_cast<size_t>(rows_cap) * 4, s) != cudaSuccess) return FFM_ERR_LAUNCH;
  RouteWorkspace w = carve_workspace(workspace, g.blocks, E);
  route_hist_ids<<<g.blocks, ROUTE_THREADS, 0, s>>>(expert_ids, T, E, g.tokens_per_block, w.block_hist, status);
  route_scan<<<1, ROUTE_THREADS, 0, s>>>(w.block_hist, nullptr, nullptr, g.blocks, E, w.block_off, counts, tile_start,
                                         nullptr);
  route_rank<<<g.blocks, ROUTE_THREADS, 0, s>>>(expert_ids, T, E, g.tokens_per_block, w.block_off, tile_start,
                                                rows_cap, pos, src, status);
  return cudaGetLastError() == cudaSuccess ? FFM_OK : FFM_ERR_LAUNCH;
}

extern "C" int ffm_group_rows_static(const int32_t* expert_ids, int64_t T, int E, int32_t* counts,
                                     int32_t* tile_start, int32_t* pos, int32_t* src, int64_t rows_cap,
                                     int32_t* status, ffm_stream_t stream) {
  if (!expert_ids || !counts || !tile_start || !pos || !src || !status) return FFM_ERR_BAD_ARG;
  if (T < 0 || E < 1) return FFM_ERR_BAD_ARG;
  if (E > FFM_STATIC_MAX_EXPERTS || T > FFM_STATIC_MAX_ROWS) return FFM_ERR_STATIC_LIMIT;
  if (rows_cap < ffm_rows_capacity(T, E)) return FFM_ERR_BAD_ARG;
  const RouteGrid g = route_grid(T > 0 ? T : 1);
  const size_t per = (static_cast<size_t>(g.blocks) * E * 4 + 255) / 256 * 256;
  if (2 * per > FFM_STATIC_SCRATCH_BYTES) return FFM_ERR_STATIC_LIMIT;
  void* base = nullptr;
  const int rc = static_scratch_address(&base);
  if (rc != FFM_OK) return rc;
  // Every word of the scratch that the scan and rank kernels read is written by the histogram kernel of
  // this same call, so nothing left over from an earlier call is ever consumed and no clearing is needed.
  int32_t* block_hist = reinterpret_cast<int32_t*>(base);
  int32_t* block_off = reinterpret_cast<int32_t*>(static_cast<unsigned char*>(base) + per);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (cudaMemsetAsync(src, 0xFF, static_cast<size_t>(rows_cap) * 4, s) != cudaSuccess) return FFM_ERR_LAUNCH;
  route_hist_ids<<<g.blocks, ROUTE_THREADS, 0, s>>>(expert_ids, T, E, g.tokens_per_block, block_hist, status);
  route_scan<<<1, ROUTE_THREADS, 0, s>>>(block_hist, nullptr, nullptr, g.blocks, E, block_off, counts, tile_start,
                                         nullptr);
  route_rank<<<g.blocks, ROUTE_THREADS, 0, s>>>(expert_ids, T, E, g.tokens_per_block, block_off, tile_start, rows_cap,
                                                pos, src, status);
  return cudaGetLastError() == cudaSuccess ? FFM_OK : FFM_ERR_LAUNCH;
}

namespace ffm {
namespace {

// Positions of the routed rows in the grouped order with the 256-row padding squeezed out (the order in which an
// expert-parallel rank sends them), and the inverse map. Every block rebuilds the per-expert shift in shared memory.
__global__ void __launch_bounds__(ROUTE_THREADS)
compact_positions_kernel(const int32_t* __restrict__ pos, const int32_t* __restrict__ topk_idx,
                         const int32_t* __restrict__ counts, const int32_t* __restrict__ tile_start, long long T, int E,
                         int32_t* __restrict__ cpos, int32_t* __restrict__ src_c) {
  __shared__ int s_shift[MAX_E];  // padded position minus compact position for rows of expert e
  if (threadIdx.x == 0) {
    int before = 0;
    for (int e = 0; e < E; ++e) {
      s_shift[e] = tile_start[e] * 128 - before;
      before += counts[e];
    }
  }
  __syncthreads();
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < T) {
    const int c = pos[i] - s_shift[topk_idx[i]];
    cpos[i] = c;
    src_c[c] = static_cast<int32_t>(i);
  }
}

}  // namespace
}  // namespace ffm

extern "C" int ffm_compact_positions(const int32_t* pos, const int32_t* topk_idx, const int32_t* counts,
                                     const int32_t* tile_start, int64_t T, int E, int32_t* cpos, int32_t* src_c,
                                     ffm_stream_t stream) {
  if (!pos || !topk_idx || !counts || !tile_start || !cpos || !src_c) return FFM_ERR_BAD_ARG;
  if (T < 0 || E < 1) return FFM_ERR_BAD_ARG;
  if (E > ffm::MAX_E) return FFM_ERR_UNSUPPORTED;
  if (T == 0) return FFM_OK;
  const int blocks = static_cast<int>((T + ffm::ROUTE_THREADS - 1) / ffm::ROUTE_THREADS);
  ffm::compact_positions_kernel<<<blocks, ffm::ROUTE_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(
      pos, topk_idx, counts, tile_start, T, E, cpos, src_c);
  return cudaGetLastError() == cudaSuccess ? FFM_OK : FFM_ERR_LAUNCH;
}

extern "C" int ffm_route_apply_capacity(float* topk_w, const int32_t* topk_idx, const int32_t* pos, int32_t* src,
                                        const int32_t* tile_start, int64_t N, int top_k, int E, int capacity,
                                        int32_t* dropped_count, ffm_stream_t stream) {
  if (!topk_w || !topk_idx || !pos || !src || !tile_start || !dropped_count) return FFM_ERR_BAD_ARG;
  if (N < 0 || top_k < 1 || E < 1 || capacity < 0) return FFM_ERR_BAD_ARG;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (cudaMemsetAsync(dropped_count, 0, 4, s) != cudaSuccess) return FFM_ERR_LAUNCH;
  if (N == 0) return FFM_OK;
  const int blocks = static_cast<int>((N + ROUTE_THREADS - 1) / ROUTE_THREADS);
  route_capacity_kernel<<<blocks, ROUTE_THREADS, 0, s>>>(topk_w, topk_idx, pos, src, tile_start, N, top_k, E, capacity,
                                                         dropped_count);
  return cudaGetLastError() == cudaSuccess ? FFM_OK : FFM_ERR_LAUNCH;
}
