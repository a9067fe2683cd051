// Peer-to-peer row exchange over NVLink for expert parallelism: plain vector loads from local memory, plain
// vector stores into the peers' receive buffers (memory mapped from the other GPUs of the box), and a flag
// barrier with bounded waits. No TMA and no multimem: only ordinary ld / st on peer pointers.
//
//   p2p_push_kernel     copies up to FFM_P2P_MAX_PEERS contiguous segments of the local send buffer to
//                       (peer base + offset); blockIdx.y selects the segment.
//   p2p_signal_kernel   after the push (stream order), every rank stores the exchange's epoch into slot [my_rank]
//                       of every peer's flag array (release, system scope) and then waits until its own slots
//                       show that epoch from every peer (acquire, system scope). Epochs only grow, so flags are
//                       never reset. A wait that exceeds its cycle budget writes a status code and gives up.
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

struct SignalArgs {
  uint32_t* flags[FFM_P2P_MAX_PEERS];  // flag array of every rank (index = rank); [my_rank] is local memory
};

__global__ void p2p_signal_kernel(SignalArgs a, int my_rank, int world, uint32_t epoch, int32_t* status,
                                  long long wait_cycles) {
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
  p2p_signal_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(a, my_rank, world, epoch, status, wait_cycles);
  return cudaGetLastError() == cudaSuccess ? FFM_OK : FFM_ERR_LAUNCH;
}
