// Shared device helpers for the sm_100a fused-MoE kernels: status codes, bf16 packing,
// warp reductions and thin wrappers around the PTX this library issues by hand
// (mbarrier, TMA tiled loads, tcgen05 MMA / TMEM).
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/ffmoe.h"

namespace ffm {

typedef __nv_bfloat16 bf16;

// ----------------------------------------------------------------------------------------------
// Small numeric helpers
// ----------------------------------------------------------------------------------------------

__device__ __forceinline__ float bf16_round(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ float2 unpack_bf16x2(uint32_t u) {
  __nv_bfloat162 v = *reinterpret_cast<__nv_bfloat162*>(&u);
  return __bfloat1622float2(v);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float sigmoidf_(float x) { return 1.0f / (1.0f + __expf(-x)); }

// Sigmoid of a routing logit, for the scores that expert selection compares: 1 / (1 + exp(-x)) with every step
// rounded to fp32 as written (exp evaluated in double and rounded once, IEEE add and divide), the value a fp32
// evaluation of the reference's formula (kernels/fused_topk.py: tl.sigmoid) rounds to. The fast-math sigmoid above
// is off by a few units in the last place, enough to reorder experts whose scores nearly tie (saturated scores
// close to 1 above all), and top-k on sigmoid scores breaks ties by index.
__device__ __forceinline__ float sigmoid_rn(float x) {
  const float e = static_cast<float>(exp(-static_cast<double>(x)));
  return __fdiv_rn(1.0f, __fadd_rn(1.0f, e));
}

// GLU activation codes shared by every kernel and by the C ABI (FFM_ACT_*).
//   0 swiglu        : silu(g) * u
//   1 geglu (tanh)  : 0.5 g (1 + tanh(c (g + 0.044715 g^3))) * u, tanh(x) = 2 sigmoid(2x) - 1
//   2 relu_squared  : relu(g)^2 * u
//   3 geglu (erf)   : exact GELU, used only by the shared expert of the non-EP layer
__device__ __forceinline__ float glu_fwd(int act, float g, float u) {
  if (act == FFM_ACT_SWIGLU) {
    return g * sigmoidf_(g) * u;
  } else if (act == FFM_ACT_GEGLU_TANH) {
    const float c = 0.7978845608028654f;
    float inner = c * (g + 0.044715f * g * g * g);
    float th = 2.0f * sigmoidf_(2.0f * inner) - 1.0f;
    return 0.5f * g * (1.0f + th) * u;
  } else if (act == FFM_ACT_RELU2) {
    float r = fmaxf(g, 0.0f);
    return r * r * u;
  } else {
    return 0.5f * g * (1.0f + erff(g * 0.7071067811865476f)) * u;
  }
}

// d(act(g)*u): returns (d_gate, d_up) for upstream gradient ga.
__device__ __forceinline__ float2 glu_bwd(int act, float ga, float g, float u) {
  float dg, du;
  if (act == FFM_ACT_SWIGLU) {
    float s = sigmoidf_(g);
    du = ga * (g * s);
    dg = ga * u * (s * (1.0f + g * (1.0f - s)));
  } else if (act == FFM_ACT_GEGLU_TANH) {
    const float c = 0.7978845608028654f;
    float inner = c * (g + 0.044715f * g * g * g);
    float th = 2.0f * sigmoidf_(2.0f * inner) - 1.0f;
    float gelu = 0.5f * g * (1.0f + th);
    du = ga * gelu;
    float dth = 1.0f - th * th;
    float dinner = c * (1.0f + 3.0f * 0.044715f * g * g);
    dg = ga * u * (0.5f * (1.0f + th) + 0.5f * g * dth * dinner);
  } else if (act == FFM_ACT_RELU2) {
    float r = fmaxf(g, 0.0f);
    du = ga * r * r;
    dg = ga * u * 2.0f * r;
  } else {
    float cdf = 0.5f * (1.0f + erff(g * 0.7071067811865476f));
    float pdf = 0.3989422804014327f * __expf(-0.5f * g * g);
    du = ga * g * cdf;
    dg = ga * u * (cdf + g * pdf);
  }
  return make_float2(dg, du);
}

// ----------------------------------------------------------------------------------------------
// PTX wrappers (sm_100a)
// ----------------------------------------------------------------------------------------------

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok;
}

// Bounded wait. Returns false after `limit` clock cycles without completion, or as soon as another
// role of the CTA raised the abort flag; the first failing role records `code` in *status.
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                                  int* status, int code, long long limit) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  while (!mbar_try_wait(bar, parity)) {
    if (*abort_flag != 0) return false;
    if (clock64() - t0 > limit) {
      *abort_flag = 1;
      atomicCAS(status, 0, code);
      return false;
    }
  }
  return true;
}

}  // namespace ffm

// Ask for the largest shared-memory carve-out for a kernel that itself needs little or none. The persistent GEMM
// runs with the largest carve-out; a kernel launched on another stream can only share an SM with it (in the
// registers, thread slots and few KiB of shared memory the GEMM leaves free) if it does not ask for a different one.
#define FFM_PREFER_MAX_SHARED(kernel)                                                                              \
  do {                                                                                                             \
    static bool ffm_carveout_set = false;                                                                          \
    if (!ffm_carveout_set) {                                                                                       \
      ffm_carveout_set = true;                                                                                     \
      if (cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout,                             \
                               cudaSharedmemCarveoutMaxShared) != cudaSuccess) {                                   \
        cudaGetLastError();                                                                                        \
      }                                                                                                            \
    }                                                                                                              \
  } while (0)

namespace ffm {

__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void tma_prefetch_desc(const void* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

// Tiled 2-D TMA load into this CTA's shared memory (no cluster broadcast), completing on an mbarrier.
// c0 is the innermost coordinate: c0 * sizeof(element) must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const void* map, uint32_t bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1)
      : "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tmem_alloc(uint32_t slot_smem_addr, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot_smem_addr), "r"(cols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}

// D[tmem] (+)= A[smem desc] * B[smem desc], bf16 inputs, fp32 accumulate, issued by one thread.
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Arrive on an mbarrier once every MMA previously issued by this thread has completed.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// 32 lanes x 32 consecutive 32-bit columns: thread t receives lane (base_lane + t), columns [col, col+32).
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}

// 32 lanes x 16 consecutive 32-bit columns.
__device__ __forceinline__ void tmem_ld_32x16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}

// 32 lanes x 8 consecutive 32-bit columns.
__device__ __forceinline__ void tmem_ld_32x8(uint32_t taddr, uint32_t (&r)[8]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(taddr)
               : "memory");
}

__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor for tcgen05.mma, 128-byte swizzle, Blackwell descriptor version 1.
//   bits [0,14)  start address >> 4        bits [16,30) leading-dimension byte offset >> 4
//   bits [32,46) stride byte offset >> 4   bits [46,48) version = 1     bits [61,64) layout = 2 (SWIZZLE_128B)
__device__ __forceinline__ uint64_t make_smem_desc_sw128(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((saddr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}

// Instruction descriptor for kind::f16 with bf16 A/B and fp32 accumulation.
//   bits [4,6) D format (1 = f32)  [7,10) A format (1 = bf16)  [10,13) B format (1 = bf16)
//   bit 15 A major (1 = MN)  bit 16 B major (1 = MN)  [17,23) N >> 3  [24,29) M >> 4
__host__ __device__ constexpr uint32_t make_idesc_bf16(int m, int n, int a_mn, int b_mn) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(a_mn) << 15) |
         (static_cast<uint32_t>(b_mn) << 16) | (static_cast<uint32_t>(n >> 3) << 17) |
         (static_cast<uint32_t>(m >> 4) << 24);
}

}  // namespace ffm
