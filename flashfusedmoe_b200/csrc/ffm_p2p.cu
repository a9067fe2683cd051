// Peer-to-peer row exchange over NVLink for expert parallelism: plain vector loads from local memory, plain
// vector stores into the peers' receive buffers (memory mapped from the other GPUs of the box), and a flag
// barrier with bounded waits. No TMA and no multimem: only ordinary ld / st on peer pointers.
//
//   p2p_push_kernel     copies up to FFM_P2P_MAX_PEERS contiguous segments of the local send buffer to
//                       (peer base + offset); blockIdx.y selects the segment.
//   p2p_rows_kernel     the same copy at row granularity, driven by a table of segments in device memory
//                       {first source row, first destination row, rows, destination buffer}: a warp takes four
//                       consecutive rows, four of its lanes find their segments by binary search on the running row count. The source row may be looked up
//                       through an index (gather from the token matrix), or be absent (the rows are zeroed).
//   p2p_plan_kernel     builds those tables on the device from the [ep, E] matrix of row counts, so that a forward
//                       pass needs no host read of the counts (and can be captured in a CUDA graph).
//   p2p_signal_kernel   after the push (stream order), every rank stores the exchange's epoch into slot [my_rank]
//                       of every peer's flag array (release, system scope) and then waits until its own slots
//                       show that epoch from every peer (acquire, system scope). Epochs only grow, so flags are
//                       never reset. A wait that exceeds its cycle budget writes a status code and gives up.
#include <stdlib.h>

#include "ffm_common.cuh"

namespace ffm {

namespace {

struct PushArgs {
  const uint8_t* src[FFM_P2P_MAX_PEERS];
  uint8_t* dst[FFM_P2P_MAX_PEERS];
  long long bytes[FFM_P2P_MAX_PEERS];
};

__global__ void __launch_bounds__(256) p2p_push_kernel(PushArgs a) {
  const int seg = blockIdx.y;
  const long long n16 = a.bytes[seg] >> 4;
  const uint4* __restrict__ s = reinterpret_cast<const uint4*>(a.src[seg]);
  uint4* __restrict__ d = reinterpret_cast<uint4*>(a.dst[seg]);
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  // four independent 16-byte copies in flight per thread
  for (; i + 3 * stride < n16; i += 4 * stride) {
    const uint4 v0 = s[i], v1 = s[i + stride], v2 = s[i + 2 * stride], v3 = s[i + 3 * stride];
    d[i] = v0;
    d[i + stride] = v1;
    d[i + 2 * stride] = v2;
    d[i + 3 * stride] = v3;
  }
  for (; i < n16; i += stride) d[i] = s[i];
}

struct RowBases {
  uint8_t* base[FFM_P2P_MAX_PEERS];
};

// Four consecutive rows per warp and trip. Lanes 0..3 each find the segment of one row (binary search on the running
// row count), its source row (through the index, if any) and its destination address, and hand them to the warp by
// shuffle; then every lane moves one 16-byte chunk of each of the four rows per step, four loads in flight before the
// four stores. Consecutive rows mostly share a segment, so the four stores of a step land in one contiguous stretch
// of the destination.
constexpr int ROWS_PER_WARP = 4;

__global__ void __launch_bounds__(256) p2p_rows_kernel(const uint8_t* __restrict__ src, const int32_t* __restrict__ src_index,
                                                       int index_div, long long row_bytes,
                                                       const long long* __restrict__ segments,
                                                       const long long* __restrict__ seg_end, int n_segments,
                                                       long long total_rows,
                                                       const long long* __restrict__ total_rows_dev, RowBases bases,
                                                       int only_dst) {
  if (total_rows_dev != nullptr) total_rows = *total_rows_dev;
  const int warps = blockDim.x >> 5;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int chunks = static_cast<int>(row_bytes >> 4);
  for (long long row0 = (static_cast<long long>(blockIdx.x) * warps + warp) * ROWS_PER_WARP; row0 < total_rows;
       row0 += static_cast<long long>(gridDim.x) * warps * ROWS_PER_WARP) {
    // lanes 0..3: where row0 + lane comes from and where it goes
    unsigned long long my_src = 0ull, my_dst = 0ull;
    const long long row = row0 + lane;
    if (lane < ROWS_PER_WARP && row < total_rows) {
      int lo = 0, hi = n_segments - 1;  // smallest segment whose running end lies beyond this row
      while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        if (__ldg(seg_end + mid) > row) {
          hi = mid;
        } else {
          lo = mid + 1;
        }
      }
      const long long j = row - (lo > 0 ? __ldg(seg_end + lo - 1) : 0LL);
      const long long* seg = segments + 4LL * lo;
      long long src_row = __ldg(seg) + j;
      if (src_index != nullptr) src_row = __ldg(src_index + src_row) / index_div;
      const long long dst_rank = __ldg(seg + 3);
      // (measurement aid, see ffm_p2p_set_local_only: rows bound for another buffer are left where they are)
      if (only_dst < 0 || dst_rank == only_dst) {
        my_dst = reinterpret_cast<unsigned long long>(bases.base[dst_rank] + (__ldg(seg + 1) + j) * row_bytes);
        my_src = src != nullptr ? reinterpret_cast<unsigned long long>(src + src_row * row_bytes) : 0ull;
      }
    }
    const uint4* s[ROWS_PER_WARP];
    uint4* d[ROWS_PER_WARP];
#pragma unroll
    for (int q = 0; q < ROWS_PER_WARP; ++q) {
      s[q] = reinterpret_cast<const uint4*>(__shfl_sync(0xffffffffu, my_src, q));
      d[q] = reinterpret_cast<uint4*>(__shfl_sync(0xffffffffu, my_dst, q));  // null: no such row
    }
    if (src != nullptr) {
      for (int c = lane; c < chunks; c += 32) {
        uint4 v[ROWS_PER_WARP];
#pragma unroll
        for (int q = 0; q < ROWS_PER_WARP; ++q) {
          if (d[q] != nullptr) v[q] = s[q][c];
        }
#pragma unroll
        for (int q = 0; q < ROWS_PER_WARP; ++q) {
          if (d[q] != nullptr) d[q][c] = v[q];
        }
      }
    } else {
      const uint4 z = make_uint4(0u, 0u, 0u, 0u);
      for (int c = lane; c < chunks; c += 32) {
#pragma unroll
        for (int q = 0; q < ROWS_PER_WARP; ++q) {
          if (d[q] != nullptr) d[q][c] = z;
        }
      }
    }
  }
}

// Device-side twin of the host planner (p2p.SegmentPlan). One block. C[s * E + e] = rows rank s routes to expert e.
// Outputs (int64 unless noted): dispatch [E][4] + ends [E]; combine [El * ep][4] + ends; padding [El][4] + ends;
// tile_start int32 [El + 1]; totals [4] = {rows this rank sends, rows it receives, padding rows, grouped rows}.
// Runs with zero rows stay in the tables (their running end repeats), which the row kernel's search skips.
constexpr int PLAN_MAX_E = 256;

__global__ void __launch_bounds__(256) p2p_plan_kernel(const int32_t* __restrict__ C, int ep, int e_local, int rank,
                                                       long long* __restrict__ dispatch, long long* __restrict__ dispatch_end,
                                                       long long* __restrict__ combine, long long* __restrict__ combine_end,
                                                       long long* __restrict__ padding, long long* __restrict__ padding_end,
                                                       int32_t* __restrict__ tile_start, long long* __restrict__ totals,
                                                       long long max_grouped_rows, int32_t* __restrict__ status) {
  __shared__ long long s_R[PLAN_MAX_E];      // rows per expert over all sources
  __shared__ int s_overflow;
  __shared__ long long s_seg0[PLAN_MAX_E];   // first grouped row of expert e at its owner
  // first sender-order row of expert e at rank s, [ep][E]: sized by the launch, so that with few experts the block
  // needs little shared memory and can run on an SM that a GEMM CTA occupies
  extern __shared__ long long s_send0[];
  __shared__ long long s_rows_grouped;
  const int E = ep * e_local;
  const int t = threadIdx.x;
  if (t == 0) s_overflow = 0;
  for (int e = t; e < E; e += blockDim.x) {
    long long r = 0;
    for (int s = 0; s < ep; ++s) r += C[s * E + e];
    s_R[e] = r;
  }
  if (t < ep) {  // sender-order prefix of rank t
    long long acc = 0;
    for (int e = 0; e < E; ++e) {
      s_send0[t * E + e] = acc;
      acc += C[t * E + e];
    }
  }
  __syncthreads();
  if (t < ep) {  // grouped layout of owner t: segments aligned to 256 rows
    long long tiles = 0;
    for (int el = 0; el < e_local; ++el) {
      const int e = t * e_local + el;
      s_seg0[e] = tiles * 128;
      if (t == rank) tile_start[el] = static_cast<int32_t>(tiles);
      tiles += 2 * ((s_R[e] + 255) / 256);
    }
    if (t == rank) {
      tile_start[e_local] = static_cast<int32_t>(tiles);
      s_rows_grouped = tiles * 128;
    }
    // the grouped layout of owner t must fit its receive buffer; every rank evaluates every owner on the same counts
    if (max_grouped_rows > 0 && tiles * 128 > max_grouped_rows) s_overflow = 1;
  }
  __syncthreads();
  if (s_overflow) {
    // nothing may be stored past a buffer: tables that move nothing, and the status word says why
    for (int e = t; e < E; e += blockDim.x) {
      dispatch[4 * e + 0] = dispatch[4 * e + 1] = dispatch[4 * e + 2] = 0;
      dispatch[4 * e + 3] = e / e_local;
      dispatch_end[e] = 0;
    }
    for (int i = t; i < e_local * ep; i += blockDim.x) {
      combine[4 * i + 0] = combine[4 * i + 1] = combine[4 * i + 2] = 0;
      combine[4 * i + 3] = i % ep;
      combine_end[i] = 0;
    }
    for (int el = t; el <= e_local; el += blockDim.x) {
      tile_start[el] = 0;
      if (el < e_local) {
        padding[4 * el + 0] = padding[4 * el + 1] = padding[4 * el + 2] = 0;
        padding[4 * el + 3] = rank;
        padding_end[el] = 0;
      }
    }
    if (t == 0) {
      totals[0] = totals[1] = totals[2] = totals[3] = 0;
      if (status != nullptr) atomicCAS(status, 0, FFM_STATUS_EP_OVERFLOW);
    }
    return;
  }
  const int lo = rank * e_local;
  // dispatch: one run per expert, sender order -> owner's grouped layout
  for (int e = t; e < E; e += blockDim.x) {
    long long before = 0;
    for (int s = 0; s < rank; ++s) before += C[s * E + e];
    const long long rows = C[rank * E + e];
    dispatch[4 * e + 0] = s_send0[rank * E + e];
    dispatch[4 * e + 1] = s_seg0[e] + before;
    dispatch[4 * e + 2] = rows;
    dispatch[4 * e + 3] = e / e_local;
    dispatch_end[e] = s_send0[rank * E + e] + rows;
  }
  // combine: runs (expert, source) this rank holds, grouped layout -> the origin's sender order
  for (int i = t; i < e_local * ep; i += blockDim.x) {
    const int el = i / ep, s = i % ep, e = lo + el;
    long long before = 0;
    for (int s2 = 0; s2 < s; ++s2) before += C[s2 * E + e];
    long long prior = 0;  // valid rows of this rank's earlier experts
    for (int el2 = 0; el2 < el; ++el2) prior += s_R[lo + el2];
    const long long rows = C[s * E + e];
    combine[4 * i + 0] = s_seg0[e] + before;
    combine[4 * i + 1] = s_send0[s * E + e];
    combine[4 * i + 2] = rows;
    combine[4 * i + 3] = s;
    combine_end[i] = prior + before + rows;
  }
  // padding of this rank's own layout
  for (int el = t; el < e_local; el += blockDim.x) {
    const int e = lo + el;
    long long acc = 0;
    for (int el2 = 0; el2 <= el; ++el2) {
      const int e2 = lo + el2;
      acc += 256 * ((s_R[e2] + 255) / 256) - s_R[e2];
    }
    padding[4 * el + 0] = 0;
    padding[4 * el + 1] = s_seg0[e] + s_R[e];
    padding[4 * el + 2] = 256 * ((s_R[e] + 255) / 256) - s_R[e];
    padding[4 * el + 3] = rank;
    padding_end[el] = acc;
  }
  if (t == 0) {
    long long recv = 0, pad = 0;
    for (int el = 0; el < e_local; ++el) {
      recv += s_R[lo + el];
      pad += 256 * ((s_R[lo + el] + 255) / 256) - s_R[lo + el];
    }
    long long sent = 0;
    for (int e = 0; e < E; ++e) sent += C[rank * E + e];
    totals[0] = sent;
    totals[1] = recv;
    totals[2] = pad;
    totals[3] = s_rows_grouped;
  }
}

// Measurement aid: >= 0 makes the row kernels skip every row whose destination buffer index differs from it (with
// the caller's own rank: local rows still move, nothing crosses NVLink), so that a step can be timed without the
// payload of its exchanges while every kernel, barrier and local copy still runs. Results are then meaningless.
int g_only_dst = -1;

// Blocks of the row kernel per SM (FFM_P2P_BLOCKS_PER_SM, 1..8, default 2). The kernel runs on SMs that also hold a
// GEMM CTA, and NVLink, not the number of warps, bounds its rate: measured in the layer step (16,384 tokens per
// rank, replayed) 8 / 4 / 2 / 1 blocks per SM give 1.630 / 1.613 / 1.614 / - ms on 2 GPUs and 1.748 / - / 1.693 /
// 1.711 ms on 4, with the same 470-530 GB/s per direction inside the row kernels.
int rows_blocks_per_sm() {
  static int v = 0;
  if (v == 0) {
    const char* e = getenv("FFM_P2P_BLOCKS_PER_SM");
    const int x = e != nullptr ? atoi(e) : 2;
    v = x < 1 ? 1 : (x > 8 ? 8 : x);
  }
  return v;
}

struct SignalArgs {
  uint32_t* flags[FFM_P2P_MAX_PEERS];  // flag array of every rank (index = rank); [my_rank] is local memory
};

__global__ void p2p_signal_kernel(SignalArgs a, int my_rank, int world, uint32_t epoch, uint32_t* epoch_counter,
                                  int32_t* status, long long wait_cycles) {
  __shared__ uint32_t s_epoch;
  if (epoch_counter != nullptr) {
    // the epoch lives in device memory and grows by one per call, so that a captured graph can be replayed
    if (threadIdx.x == 0) s_epoch = atomicAdd(epoch_counter, 1u) + 1u;
    __syncthreads();
    epoch = s_epoch;
  }
  const int p = threadIdx.x;
  if (p >= world) return;
  __threadfence_system();  // the rows pushed by the preceding kernel are visible before the flag is
  uint32_t* remote = a.flags[p] + my_rank;
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(remote), "r"(epoch) : "memory");
  const uint32_t* mine = a.flags[my_rank] + p;
  const long long t0 = clock64();
  while (true) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
    if (static_cast<int32_t>(v - epoch) >= 0) break;
    if (clock64() - t0 > wait_cycles) {
      atomicCAS(status, 0, FFM_STATUS_WAIT_PEER);
      break;
    }
  }
}

}  // namespace

}  // namespace ffm

using namespace ffm;

extern "C" int ffm_p2p_set_local_only(int buffer_index) {
  const int old = g_only_dst;
  g_only_dst = buffer_index < 0 ? -1 : buffer_index;
  return old;
}

extern "C" int ffm_p2p_push(int n_segments, const void* const* src, void* const* dst, const int64_t* bytes,
                            ffm_stream_t stream) {
  if (n_segments < 0 || n_segments > FFM_P2P_MAX_PEERS) return FFM_ERR_UNSUPPORTED;
  if (n_segments == 0) return FFM_OK;
  if (!src || !dst || !bytes) return FFM_ERR_BAD_ARG;
  PushArgs a = {};
  long long max_bytes = 0;
  int n = 0;
  for (int i = 0; i < n_segments; ++i) {
    if (bytes[i] < 0 || (bytes[i] & 15) != 0) return FFM_ERR_UNSUPPORTED;
    if (bytes[i] == 0) continue;
    if (!src[i] || !dst[i]) return FFM_ERR_BAD_ARG;
    if ((reinterpret_cast<uintptr_t>(src[i]) & 15u) || (reinterpret_cast<uintptr_t>(dst[i]) & 15u)) return FFM_ERR_UNSUPPORTED;
    a.src[n] = static_cast<const uint8_t*>(src[i]);
    a.dst[n] = static_cast<uint8_t*>(dst[i]);
    a.bytes[n] = bytes[i];
    if (bytes[i] > max_bytes) max_bytes = bytes[i];
    ++n;
  }
  if (n == 0) return FFM_OK;
  long long blocks = (max_bytes / 16 + 256 * 4 - 1) / (256 * 4);
  const long long cap = (148LL * 8) / n > 0 ? (148LL * 8) / n : 1;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  dim3 grid(static_cast<unsigned>(blocks), static_cast<unsigned>(n), 1);
  p2p_push_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(a);
  return cudaGetLastError() == cudaSuccess ? FFM_OK : FFM_ERR_LAUNCH;
}

extern "C" int ffm_p2p_push_rows(const void* src, const int32_t* src_index, int index_div, int64_t row_bytes,
                                 const int64_t* segments, const int64_t* seg_end, int n_segments, int64_t total_rows,
                                 void* const* dst_bases, int n_bases, ffm_stream_t stream) {
  if (n_segments < 0 || total_rows < 0) return FFM_ERR_BAD_ARG;
  if (n_segments == 0 || total_rows == 0) return FFM_OK;
  if (!segments || !seg_end || !dst_bases) return FFM_ERR_BAD_ARG;
  if (n_bases < 1 || n_bases > FFM_P2P_MAX_PEERS) return FFM_ERR_UNSUPPORTED;
  if (row_bytes <= 0 || (row_bytes & 15) != 0) return FFM_ERR_UNSUPPORTED;
  if (src_index != nullptr && (src == nullptr || index_div < 1)) return FFM_ERR_BAD_ARG;
  if (src != nullptr && (reinterpret_cast<uintptr_t>(src) & 15u) != 0) return FFM_ERR_UNSUPPORTED;
  RowBases b = {};
  for (int i = 0; i < n_bases; ++i) {
    if (!dst_bases[i] || (reinterpret_cast<uintptr_t>(dst_bases[i]) & 15u) != 0) return FFM_ERR_BAD_ARG;
    b.base[i] = static_cast<uint8_t*>(dst_bases[i]);
  }
  long long blocks = (total_rows + 8 * ROWS_PER_WARP - 1) / (8 * ROWS_PER_WARP);
  if (blocks > 148LL * rows_blocks_per_sm()) blocks = 148LL * rows_blocks_per_sm();
  p2p_rows_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint8_t*>(src), src_index, index_div, row_bytes, reinterpret_cast<const long long*>(segments),
      reinterpret_cast<const long long*>(seg_end), n_segments, total_rows, nullptr, b, g_only_dst);
  return cudaGetLastError() == cudaSuccess ? FFM_OK : FFM_ERR_LAUNCH;
}

extern "C" int ffm_p2p_push_rows_dev(const void* src, const int32_t* src_index, int index_div, int64_t row_bytes,
                                     const int64_t* segments, const int64_t* seg_end, int n_segments,
                                     const int64_t* total_rows_dev, int64_t max_rows, void* const* dst_bases, int n_bases,
                                     ffm_stream_t stream) {
  if (n_segments < 0 || max_rows < 0) return FFM_ERR_BAD_ARG;
  if (n_segments == 0 || max_rows == 0) return FFM_OK;
  if (!segments || !seg_end || !dst_bases || !total_rows_dev) return FFM_ERR_BAD_ARG;
  if (n_bases < 1 || n_bases > FFM_P2P_MAX_PEERS) return FFM_ERR_UNSUPPORTED;
  if (row_bytes <= 0 || (row_bytes & 15) != 0) return FFM_ERR_UNSUPPORTED;
  if (src_index != nullptr && (src == nullptr || index_div < 1)) return FFM_ERR_BAD_ARG;
  if (src != nullptr && (reinterpret_cast<uintptr_t>(src) & 15u) != 0) return FFM_ERR_UNSUPPORTED;
  RowBases b = {};
  for (int i = 0; i < n_bases; ++i) {
    if (!dst_bases[i] || (reinterpret_cast<uintptr_t>(dst_bases[i]) & 15u) != 0) return FFM_ERR_BAD_ARG;
    b.base[i] = static_cast<uint8_t*>(dst_bases[i]);
  }
  long long blocks = (max_rows + 8 * ROWS_PER_WARP - 1) / (8 * ROWS_PER_WARP);
  if (blocks > 148LL * rows_blocks_per_sm()) blocks = 148LL * rows_blocks_per_sm();
  p2p_rows_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint8_t*>(src), src_index, index_div, row_bytes, reinterpret_cast<const long long*>(segments),
      reinterpret_cast<const long long*>(seg_end), n_segments, 0, reinterpret_cast<const long long*>(total_rows_dev), b,
      g_only_dst);
  return cudaGetLastError() == cudaSuccess ? FFM_OK : FFM_ERR_LAUNCH;
}

extern "C" int ffm_p2p_plan(const int32_t* counts, int ep, int e_local, int rank, int64_t* dispatch,
                            int64_t* dispatch_end, int64_t* combine, int64_t* combine_end, int64_t* padding,
                            int64_t* padding_end, int32_t* tile_start, int64_t* totals, int64_t max_grouped_rows,
                            int32_t* status, ffm_stream_t stream) {
  if (!counts || !dispatch || !dispatch_end || !combine || !combine_end || !padding || !padding_end || !tile_start ||
      !totals) {
    return FFM_ERR_BAD_ARG;
  }
  if (ep < 1 || ep > FFM_P2P_MAX_PEERS || e_local < 1 || rank < 0 || rank >= ep) return FFM_ERR_BAD_ARG;
  if (ep * e_local > PLAN_MAX_E) return FFM_ERR_UNSUPPORTED;
  if (max_grouped_rows < 0 || (max_grouped_rows > 0 && status == nullptr)) return FFM_ERR_BAD_ARG;
  const size_t table_bytes = static_cast<size_t>(ep) * ep * e_local * sizeof(long long);  // [ep][E], at most 32 KiB
  p2p_plan_kernel<<<1, 256, table_bytes, static_cast<cudaStream_t>(stream)>>>(
      counts, ep, e_local, rank, reinterpret_cast<long long*>(dispatch), reinterpret_cast<long long*>(dispatch_end),
      reinterpret_cast<long long*>(combine), reinterpret_cast<long long*>(combine_end),
      reinterpret_cast<long long*>(padding), reinterpret_cast<long long*>(padding_end), tile_start,
      reinterpret_cast<long long*>(totals), max_grouped_rows, status);
  return cudaGetLastError() == cudaSuccess ? FFM_OK : FFM_ERR_LAUNCH;
}

extern "C" int ffm_p2p_signal_wait(void* const* flag_arrays, int my_rank, int world, uint32_t epoch, int32_t* status,
                                   long long wait_cycles, ffm_stream_t stream) {
  if (!flag_arrays || !status) return FFM_ERR_BAD_ARG;
  if (world < 1 || world > FFM_P2P_MAX_PEERS || my_rank < 0 || my_rank >= world) return FFM_ERR_UNSUPPORTED;
  SignalArgs a = {};
  for (int i = 0; i < world; ++i) {
    if (!flag_arrays[i]) return FFM_ERR_BAD_ARG;
    a.flags[i] = static_cast<uint32_t*>(flag_arrays[i]);
  }
  if (wait_cycles <= 0) wait_cycles = 2000000000LL;
  p2p_signal_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(a, my_rank, world, epoch, nullptr, status,
                                                                     wait_cycles);
  return cudaGetLastError() == cudaSuccess ? FFM_OK : FFM_ERR_LAUNCH;
}

extern "C" int ffm_p2p_signal_wait_dev(void* const* flag_arrays, int my_rank, int world, uint32_t* epoch_counter,
                                       int32_t* status, long long wait_cycles, ffm_stream_t stream) {
  if (!flag_arrays || !status || !epoch_counter) return FFM_ERR_BAD_ARG;
  if (world < 1 || world > FFM_P2P_MAX_PEERS || my_rank < 0 || my_rank >= world) return FFM_ERR_UNSUPPORTED;
  SignalArgs a = {};
  for (int i = 0; i < world; ++i) {
    if (!flag_arrays[i]) return FFM_ERR_BAD_ARG;
    a.flags[i] = static_cast<uint32_t*>(flag_arrays[i]);
  }
  if (wait_cycles <= 0) wait_cycles = 2000000000LL;
  p2p_signal_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(a, my_rank, world, 0u, epoch_counter, status,
                                                                     wait_cycles);
  return cudaGetLastError() == cudaSuccess ? FFM_OK : FFM_ERR_LAUNCH;
}
