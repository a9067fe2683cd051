// Grouped GEMM for sm_100a: TMA-fed shared-memory ring, tcgen05.mma with fp32 accumulators in TMEM,
// persistent CTAs, warp-specialised roles, TMA-store epilogue.
//
//   warp 0      TMA producer   (one lane issues cp.async.bulk.tensor loads into the stage ring)
//   warp 1      MMA issuer     (one lane issues tcgen05.mma; the warp owns the TMEM allocation)
//   warps 2..5  epilogue       (tcgen05.ld of the fp32 accumulator one chunk ahead, math, bf16 rows staged in
//                               swizzled shared memory and written out with cp.async.bulk.tensor stores)
//   warps 6..13 passenger      (optional, PASS = 1: eight more warps run an independent HBM-bound job, the GLU
//                               backward, while the tensor pipe works. A resident GEMM CTA leaves no room on its SM
//                               for blocks of another kernel, so a memory-bound kernel launched beside a GEMM on
//                               another stream simply waits; riding inside the GEMM's own CTAs is how it overlaps.)
//
// Two tile shapes from one template:
//   CTA2 = 0   one CTA per 128 x 256 tile, tcgen05.mma.cta_group::1, 4 stages of (A 16 KiB + B 32 KiB)
//   CTA2 = 1   a cluster of two CTAs per 256 x 256 tile, tcgen05.mma.cta_group::2 issued by the even CTA.
//              Each CTA stages its own 128 rows of A and its own 128-column half of B (5-6 stages of 32 KiB), so
//              every byte of B is read from shared memory once for 256 rows of output instead of once for 128.
//              Both CTAs' loads complete on the even CTA's "full" barrier; MMA completion is committed to the
//              "empty" and "accumulator full" barriers of both CTAs; the odd CTA's epilogue hands its
//              accumulator back with a remote arrive. No load is broadcast to more than one CTA.
//
// The accumulator is double-buffered in TMEM (2 x 256 columns), so the epilogue of tile i overlaps the main
// loop of tile i + 1. Every mbarrier wait is bounded: when a wait runs out the role records a code in the
// caller's status word, raises a CTA-wide abort flag and all roles fall through to the common exit, where the
// cluster (if any) is joined and TMEM is released.
//
// Operand tiles in shared memory use the 128-byte swizzle that both TMA and the MMA descriptors understand:
//   K-major operand  (rows = M or N index, 64 contiguous K elements per row): box {64, 128 rows}
//       descriptor: SBO = 1024 B between 8-row groups; K step of 16 elements = +32 B on the start address
//   MN-major operand (rows = K index, 64 contiguous M/N elements per row):    box {64, 64 rows} per 64 columns
//       descriptor: LBO = 8192 B between 64-column blocks, SBO = 1024 B between 8-row K groups;
//       K step of 16 rows = +2048 B on the start address
// Output staging: every epilogue warp owns a few 32-row x 128-byte boxes (64 bf16 columns) with the 128-byte
// swizzle (16-byte chunk index ^= row & 7), stored with box {64 columns, 32 rows, 1}; stores clip at the tensor
// extents, so ragged row and column edges need no masking. A plain epilogue has one box per warp (two with one-CTA
// tiles); the GLU epilogue fills three (activation, gate, up) per 64-column step.
#include <stdlib.h>

#include "ffm_common.cuh"

namespace ffm {

namespace {

constexpr int BM = 128;  // rows per CTA
constexpr int BN = 256;  // columns per tile
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int NUM_ACC = 2;
constexpr int TMEM_COLS = 512;
constexpr int GEMM_THREADS = 192;
constexpr int PASSENGER_THREADS = 256;
constexpr int EPI_WARPS = 4;
constexpr int MAX_GROUPS = 256;
constexpr int A_STAGE_BYTES = BM * BK * 2;  // 16 KiB
constexpr int BOX_BYTES = 32 * 128;  // one staged box: 32 rows x 64 bf16
constexpr int SMEM_CTRL_BYTES = 2048;
constexpr int MAX_STAGES = 6;
constexpr int SMEM_LIMIT = 232448;  // 227 KiB of dynamic shared memory per CTA

enum { EPI_PLAIN = 0, EPI_GLU = 1, EPI_GLUBWD = 2 };
// The GLU epilogues get a second warp per TMEM lane quarter (helper warps 6..9, each taking the upper 32 columns of
// every 64-column step). The GLU backward does about 16 instructions and two MUFU operations per accumulator element,
// too much for one warp per scheduler inside a tile's main loop (0.174 -> 0.164 ms at 8 x 4096 rows, D 1024, H 2048);
// the e4m3 up-projection has half the main loop of the bf16 one under the same epilogue (1382 -> 1626 TFLOP/s); the
// bf16 up-projection gains 1 % (and needs 105 instead of 234 registers, since its loops are rolled).
constexpr int HELPER_THREADS = 128;
__host__ __device__ constexpr bool epilogue_helpers(int epi) { return epi == EPI_GLUBWD || epi == EPI_GLU; }
__host__ __device__ constexpr int gemm_threads(int epi, int pass) {
  return GEMM_THREADS + pass * PASSENGER_THREADS + (epilogue_helpers(epi) ? HELPER_THREADS : 0);
}

// Ring depth against staging depth for CTA pairs. Measured at 8 x 4096 rows, D 1024, H 2048: every split from 4 to
// 6 stages runs within 3 % of the others alone (the GEMMs sit at the board's power limit, not at a pipeline limit),
// and one, two or four staging steps per epilogue warp make no difference.
// What the split decides is who can run beside the resident GEMM CTA. Every block needs 1 KiB of shared memory of
// the SM even if it declares none, so a GEMM CTA that takes all 227 KiB shuts every other kernel out of its SM.
// With one staging step (plain) and two staging buffers (GLU backward) every shape leaves 16-32 KiB: blocks of
// kernels without shared memory of their own (the exchange's row and flag kernels, the row-wise HBM kernels) then
// run on SMs that hold a GEMM CTA. Measured in the layer step: no change on one GPU (1.712-1.716 ms either way),
// 1.650 -> 1.616 ms on two (expert parallel: the NVLink pushes no longer wait for a GEMM to drain).
// A 4-stage ring (~65 KiB free) also admits kernels with shared memory of their own; the GEMMs are then 0-4 % slower
// alone and the step does not gain (-DFFM_TUNE_PP_STAGES=4 -DFFM_TUNE_PG_STAGES=4 builds that one).
#ifndef FFM_TUNE_PP_STAGES
#define FFM_TUNE_PP_STAGES 6
#define FFM_TUNE_PP_STEPS 1
#endif
#ifndef FFM_TUNE_GB_STEPS
#define FFM_TUNE_GB_STEPS 2
#endif
#ifndef FFM_TUNE_PG_STAGES
#define FFM_TUNE_PG_STAGES 5
#define FFM_TUNE_PG_STEPS 1
#endif

// Shared-memory budget per tile shape and epilogue: ring stages against staging boxes per epilogue warp.
//   CTA pair, plain: 6 stages x 32 KiB + 1 box      CTA pair, GLU: 5 stages x 32 KiB + 3 boxes
//   one CTA,  plain: 4 stages x 48 KiB + 2 boxes    one CTA,  GLU: 3 stages x 48 KiB + 3 boxes
//   GLU backward epilogue (EPI_GLUBWD): 4 stages + 2 x 2 boxes (one CTA: 3 stages + 2 x 2 boxes)
// A GLU step stores three boxes (activation, gate, up) as one bulk group; a plain step stores one box; a GLU backward
// step stores two (gate gradient, up gradient).
template <int CTA2, int EPI>
struct Shape {
  static constexpr int STAGES = EPI == EPI_GLU      ? (CTA2 ? FFM_TUNE_PG_STAGES : 3)
                                : EPI == EPI_GLUBWD ? (CTA2 ? 4 : 3)
                                                    : (CTA2 ? FFM_TUNE_PP_STAGES : 4);
  static constexpr int B_STAGE_BYTES = (CTA2 ? 128 : 256) * BK * 2;
  static constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
  static constexpr int RING_BYTES = STAGES * STAGE_BYTES;
  static constexpr int BOXES_PER_STEP = EPI == EPI_GLU ? 3 : (EPI == EPI_GLUBWD ? 2 : 1);
  static constexpr int STEPS_BUFFERED = EPI == EPI_GLU      ? (CTA2 ? FFM_TUNE_PG_STEPS : 1)
                                        : EPI == EPI_GLUBWD ? (CTA2 ? FFM_TUNE_GB_STEPS : 2)
                                                            : (CTA2 ? FFM_TUNE_PP_STEPS : 2);
  static constexpr int STG_WARP_BYTES = BOXES_PER_STEP * STEPS_BUFFERED * BOX_BYTES;
  static constexpr int STG_BYTES = EPI_WARPS * STG_WARP_BYTES;
  static constexpr int SMEM_BYTES = RING_BYTES + STG_BYTES + SMEM_CTRL_BYTES + 1024;  // + 1 KiB alignment slack
  static_assert(SMEM_BYTES <= SMEM_LIMIT, "tile shape does not fit in shared memory");
  static_assert(STAGES <= MAX_STAGES, "ring deeper than the barrier arrays");
};

struct GemmParams {
  const int32_t* tile_start;  // [groups + 1] cumulative 128-row tiles, or null (dense)
  const int32_t* group_rows;  // [groups] valid rows per group, or null: when given (grouped-M only) the tiles of a
                              // group that hold no valid row are not computed
  int groups;
  int dense_m_tiles;
  int n_cols;              // output columns per group (GLU: H)
  int k_blocks;            // K / 64 (grouped-M / dense)
  long long b_group_rows;  // rows of the B tensor map per group
  int b1_row_offset;       // row offset of the second 128-row half of a K-major B tile
  int has_c2;              // GLU: also store the pre-activations
  int glu_h;
  float scale;
  int act;
  int m_tiles_per_group;  // grouped-K: 128-row tiles of M per group
  int n_tiles;            // number of BN (GLU: 128-column) blocks over n_cols
  int32_t* status;
  long long wait_cycles;
  // passenger job (PASS = 1): gU = GLU backward of (dAct, pre-activations), see ffm_glu_backward
  const bf16* pz_dact;
  const bf16* pz_pre;
  bf16* pz_gu;
  long long pz_rows;
  int pz_h;
  int pz_act;
};
// FP8 = 1 (e4m3 operands, never with a passenger): the epilogue multiplies the fp32 accumulator by
// a_scale[row] * b_scale[group]. The two pointers travel in the passenger's pointer fields: growing this
// struct changes ptxas's register allocation of the bf16 GLU-epilogue instantiation (234 -> 185 registers, a much
// slower kernel), so the struct keeps its size.
__device__ __forceinline__ const float* fp8_a_scale(const GemmParams& p) {
  return reinterpret_cast<const float*>(p.pz_dact);
}
__device__ __forceinline__ const float* fp8_b_scale(const GemmParams& p) {
  return reinterpret_cast<const float*>(p.pz_pre);
}

struct Ctrl {
  unsigned long long full_bar[MAX_STAGES];
  unsigned long long empty_bar[MAX_STAGES];
  unsigned long long acc_full_bar[NUM_ACC];
  unsigned long long acc_empty_bar[NUM_ACC];
  uint32_t tmem_base;
  int abort_flag;
  unsigned long long pre_bar[EPI_WARPS][3];  // GLU-backward epilogue: "pre-activation boxes have landed", per warp and buffer
  unsigned long long help_bar[EPI_WARPS][3];  // ... and "the helper warp has written its half of the step"
  unsigned long long free_bar[EPI_WARPS][3];  // GLU epilogue with helpers: "the step's staging boxes may be overwritten"
  int tile_start[MAX_GROUPS + 1];
};
static_assert(sizeof(Ctrl) <= SMEM_CTRL_BYTES, "control block too large");

struct TileCoord {
  int group;
  int m_tile;    // 128-row tile of this CTA: global (grouped-M / dense) or inside the group's M (grouped-K)
  int n_block;   // BN-column block (GLU: 128-column block of H)
  int k_row0;    // grouped-K: first K row; else 0
  int k_blocks;  // 64-deep K blocks to accumulate
};

// Walks the tiles of this CTA (or CTA pair) in launch order. The unit is one MMA tile: 128 rows, or with CTA2
// a pair of consecutive 128-row tiles (segments are aligned to 256 rows, so a pair never straddles experts).
// Grouped-M order is expert-major, then N block, then M (M fastest), so CTAs running side by side share one
// weight tile through L2.
template <int GROUPK, int CTA2>
struct TileWalker {
  const int* ts;             // cumulative tiles to walk (shared memory)
  const int32_t* layout_ts;  // cumulative tiles of the memory layout when it differs from `ts` (global), else null
  int groups, n_tiles, m_units_per_group, k_blocks, rank;
  long long total, cur, step;
  int g;

  __device__ static int units(int tiles) { return CTA2 ? (tiles + 1) / 2 : tiles; }

  __device__ TileWalker(const GemmParams& p, const int* ts_smem, int cta_rank) {
    ts = ts_smem;
    layout_ts = (!GROUPK && p.group_rows != nullptr) ? p.tile_start : nullptr;
    groups = p.groups;
    n_tiles = p.n_tiles;
    k_blocks = p.k_blocks;
    rank = cta_rank;
    m_units_per_group = units(p.m_tiles_per_group);
    if (GROUPK) {
      total = static_cast<long long>(groups) * m_units_per_group * n_tiles;
    } else {
      total = static_cast<long long>(units(ts[groups])) * n_tiles;
    }
    cur = CTA2 ? (blockIdx.x >> 1) : blockIdx.x;
    step = CTA2 ? (gridDim.x >> 1) : gridDim.x;
    g = 0;
  }

  __device__ bool next(TileCoord& t) {
    if (cur >= total) return false;
    int unit;
    if (GROUPK) {
      const int per_group = m_units_per_group * n_tiles;
      t.group = static_cast<int>(cur / per_group);
      const int r = static_cast<int>(cur % per_group);
      unit = r % m_units_per_group;
      t.n_block = r / m_units_per_group;
      t.k_row0 = ts[t.group] * BM;
      t.k_blocks = (ts[t.group + 1] - ts[t.group]) * (BM / BK);
    } else {
      while (g < groups - 1 && cur >= static_cast<long long>(units(ts[g + 1])) * n_tiles) ++g;
      const int u0 = units(ts[g]);
      const int cnt = units(ts[g + 1]) - u0;
      const int r = static_cast<int>(cur - static_cast<long long>(u0) * n_tiles);
      t.group = g;
      t.n_block = r / cnt;
      unit = (layout_ts != nullptr ? units(__ldg(layout_ts + g)) : u0) + r % cnt;
      t.k_row0 = 0;
      t.k_blocks = k_blocks;
    }
    t.m_tile = CTA2 ? (unit * 2 + rank) : unit;
    cur += step;
    return true;
  }
};

// ---- PTX used only by this kernel --------------------------------------------------------------

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}

// shared::cluster address of the same shared-memory offset in CTA `rank` of this cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}

__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}

// 2-D TMA load issued by either CTA of a pair into its own shared memory; the byte count completes on the
// mbarrier at `bar`, a shared::cluster address that may belong to the other CTA of the pair.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const void* map, uint32_t bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], "
      "[%2];" ::"r"(dst),
      "l"(map), "r"(bar), "r"(c0), "r"(c1)
      : "memory");
}

// 3-D TMA load into this CTA's shared memory (no cluster broadcast), completing on one of its own mbarriers.
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const void* map, uint32_t bar, int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}

__device__ __forceinline__ void ld_shared_v4(uint32_t addr, uint4& v) {
  asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr) : "memory");
}

__device__ __forceinline__ void tma_store_3d(const void* map, uint32_t src, int c0, int c1, int c2) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];" ::"l"(map), "r"(src),
               "r"(c0), "r"(c1), "r"(c2)
               : "memory");
}
// Ask the TMA unit to bring one box of a tensor into L2 (nothing lands in shared memory, nothing to wait for).
__device__ __forceinline__ void tma_prefetch_l2_2d(const void* map, int c0, int c1) {
  asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];" ::"l"(map), "r"(c0), "r"(c1)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// wait until at most N of this thread's bulk store groups have not finished reading shared memory
template <int N>
__device__ __forceinline__ void bulk_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void bulk_wait0() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

__device__ __forceinline__ void tmem_alloc2(uint32_t slot_smem_addr, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot_smem_addr), "r"(cols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish2() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc2(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}

__device__ __forceinline__ void umma_bf16_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                               uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// The same with 8-bit floating-point operands (e4m3 / e5m2 chosen by the instruction descriptor), 32 K elements per
// instruction, fp32 accumulation.
__device__ __forceinline__ void umma_f8(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_f8_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                             uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Instruction descriptor for kind::f8f6f4 with e4m3 A and B (format code 0) and fp32 accumulation, K-major operands.
__host__ __device__ constexpr uint32_t make_idesc_e4m3(int m, int n) {
  return (1u << 4) | (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(m >> 4) << 24);
}

// Arrive (once the pair's MMAs issued so far have completed) on one mbarrier given by shared::cluster address.
__device__ __forceinline__ void umma_commit_pair(uint32_t cluster_bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_bar)
               : "memory");
}

// 16-byte chunk q (0..7) of row r inside a 32-row x 128-byte box with the 128-byte TMA swizzle
__device__ __forceinline__ uint32_t box_offset(int r, int q) { return r * 128 + ((q ^ (r & 7)) << 4); }

__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

// GLU backward over rows [0, rows): (d gate | d up)[r, :] from dAct[r, :] and the saved pre-activations. `rows` is
// pz_rows cut at the end of the last group's tiles (buffers sized for a worst case hold far more rows than are used).
// `tid` / `nthreads` enumerate the passenger threads of the whole grid; four independent 16-byte column chunks per
// thread and trip keep enough loads in flight for 256 threads per SM to stream at HBM speed.
__device__ __forceinline__ void passenger_glu_backward(const GemmParams& p, long long rows, long long tid,
                                                       long long nthreads) {
  const int H = p.pz_h;
  const int chunks = H >> 3;
  const long long total = rows * chunks;
  for (long long base = tid; base < total; base += 4 * nthreads) {
    uint4 ga[4], gg[4], uu[4];
    long long r[4];
    int c[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const long long idx = base + u * nthreads;
      if (idx < total) {
        r[u] = idx / chunks;
        c[u] = static_cast<int>(idx % chunks);
        ga[u] = __ldg(reinterpret_cast<const uint4*>(p.pz_dact + r[u] * H) + c[u]);
        gg[u] = __ldg(reinterpret_cast<const uint4*>(p.pz_pre + r[u] * 2 * H) + c[u]);
        uu[u] = __ldg(reinterpret_cast<const uint4*>(p.pz_pre + r[u] * 2 * H + H) + c[u]);
      }
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const long long idx = base + u * nthreads;
      if (idx < total) {
        const uint32_t gav[4] = {ga[u].x, ga[u].y, ga[u].z, ga[u].w};
        const uint32_t ggv[4] = {gg[u].x, gg[u].y, gg[u].z, gg[u].w};
        const uint32_t uuv[4] = {uu[u].x, uu[u].y, uu[u].z, uu[u].w};
        uint32_t dg[4], du[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float2 a = unpack_bf16x2(gav[q]), g = unpack_bf16x2(ggv[q]), v = unpack_bf16x2(uuv[q]);
          const float2 r0 = glu_bwd(p.pz_act, a.x, g.x, v.x);
          const float2 r1 = glu_bwd(p.pz_act, a.y, g.y, v.y);
          dg[q] = pack_bf16x2(r0.x, r1.x);
          du[q] = pack_bf16x2(r0.y, r1.y);
        }
        reinterpret_cast<uint4*>(p.pz_gu + r[u] * 2 * H)[c[u]] = make_uint4(dg[0], dg[1], dg[2], dg[3]);
        reinterpret_cast<uint4*>(p.pz_gu + r[u] * 2 * H + H)[c[u]] = make_uint4(du[0], du[1], du[2], du[3]);
      }
    }
  }
}

// Eight columns of the GLU backward in the dAct epilogue: 16 bytes of this lane's row in the staged gate and up
// pre-activation boxes (128-byte swizzle) are read, combined with the bf16-rounded accumulator values v, and
// overwritten with the gate and up gradients.
template <int ACT>
__device__ __forceinline__ void glu_backward_8(const uint32_t (&v)[8], float scale, uint32_t buf, uint32_t o) {
  uint4 g4, u4;
  ld_shared_v4(buf + o, g4);
  ld_shared_v4(buf + BOX_BYTES + o, u4);
  const uint32_t gw4[4] = {g4.x, g4.y, g4.z, g4.w};
  const uint32_t uw4[4] = {u4.x, u4.y, u4.z, u4.w};
  uint32_t og[4], ou[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 da = unpack_bf16x2(
        pack_bf16x2(__uint_as_float(v[2 * j]) * scale, __uint_as_float(v[2 * j + 1]) * scale));
    const float2 gf = unpack_bf16x2(gw4[j]);
    const float2 uf = unpack_bf16x2(uw4[j]);
    const float2 r0 = glu_bwd(ACT, da.x, gf.x, uf.x);
    const float2 r1 = glu_bwd(ACT, da.y, gf.y, uf.y);
    og[j] = pack_bf16x2(r0.x, r1.x);
    ou[j] = pack_bf16x2(r0.y, r1.y);
  }
  st_shared_v4(buf + o, og[0], og[1], og[2], og[3]);
  st_shared_v4(buf + BOX_BYTES + o, ou[0], ou[1], ou[2], ou[3]);
}

// Half of a 64-column step (four 16-byte column groups from q_begin): the accumulator comes out of TMEM eight columns
// at a time, one load ahead of the math, in a loop that stays rolled (two loads per trip) so that its body stays
// resident in the instruction cache.
template <int ACT>
__device__ __forceinline__ void glu_backward_step(uint32_t tcol, float scale, uint32_t buf, int lane, int q_begin) {
  uint32_t a[8], b[8];
  tmem_ld_32x8(tcol + q_begin * 8, a);
#pragma unroll 1
  for (int q = q_begin; q < q_begin + 4; q += 2) {
    tmem_ld_wait();
    tmem_ld_32x8(tcol + (q + 1) * 8, b);
    glu_backward_8<ACT>(a, scale, buf, box_offset(lane, q));
    tmem_ld_wait();
    if (q + 2 < q_begin + 4) tmem_ld_32x8(tcol + (q + 2) * 8, a);
    glu_backward_8<ACT>(b, scale, buf, box_offset(lane, q + 1));
  }
}

// Eight GLU columns of the up-projection epilogue: gate and up accumulators g, u (scaled when they come from e4m3
// operands) are rounded to bf16 (the stored pre-activations), the activation is computed from the rounded values, and
// 16 bytes each go to this lane's row of the activation, gate and up boxes.
template <int ACT, int FP8>
__device__ __forceinline__ void glu_forward_8(const uint32_t (&g)[8], const uint32_t (&u)[8], float fp8_scale,
                                              bool store_pre, uint32_t buf, uint32_t o) {
  uint32_t pg[4], pu[4], pa[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    float g0 = __uint_as_float(g[2 * j]), g1 = __uint_as_float(g[2 * j + 1]);
    float u0 = __uint_as_float(u[2 * j]), u1 = __uint_as_float(u[2 * j + 1]);
    if (FP8) {
      g0 *= fp8_scale;
      g1 *= fp8_scale;
      u0 *= fp8_scale;
      u1 *= fp8_scale;
    }
    pg[j] = pack_bf16x2(g0, g1);
    pu[j] = pack_bf16x2(u0, u1);
    const float2 gf = unpack_bf16x2(pg[j]);
    const float2 uf = unpack_bf16x2(pu[j]);
    pa[j] = pack_bf16x2(glu_fwd(ACT, gf.x, uf.x), glu_fwd(ACT, gf.y, uf.y));
  }
  st_shared_v4(buf + o, pa[0], pa[1], pa[2], pa[3]);
  if (store_pre) {
    st_shared_v4(buf + BOX_BYTES + o, pg[0], pg[1], pg[2], pg[3]);
    st_shared_v4(buf + 2 * BOX_BYTES + o, pu[0], pu[1], pu[2], pu[3]);
  }
}

// 32 GLU columns (four 16-byte column groups from q_begin) of a 64-column step: gate at TMEM column tcol, up 128
// columns further, read eight columns at a time one load ahead of the math in a rolled loop.
template <int ACT, int FP8>
__device__ __forceinline__ void glu_forward_half_step_act(uint32_t tcol, float fp8_scale, bool store_pre, uint32_t buf,
                                                          int lane, int q_begin) {
  uint32_t ga[8], ua[8], gb[8], ub[8];
  tmem_ld_32x8(tcol, ga);
  tmem_ld_32x8(tcol + 128, ua);
#pragma unroll 1
  for (int i = 0; i < 4; i += 2) {
    tmem_ld_wait();
    tmem_ld_32x8(tcol + (i + 1) * 8, gb);
    tmem_ld_32x8(tcol + 128 + (i + 1) * 8, ub);
    glu_forward_8<ACT, FP8>(ga, ua, fp8_scale, store_pre, buf, box_offset(lane, q_begin + i));
    tmem_ld_wait();
    if (i + 2 < 4) {
      tmem_ld_32x8(tcol + (i + 2) * 8, ga);
      tmem_ld_32x8(tcol + 128 + (i + 2) * 8, ua);
    }
    glu_forward_8<ACT, FP8>(gb, ub, fp8_scale, store_pre, buf, box_offset(lane, q_begin + i + 1));
  }
}

template <int FP8>
__device__ __forceinline__ void glu_forward_half_step(uint32_t tcol, int act, float fp8_scale, bool store_pre,
                                                      uint32_t buf, int lane, int q_begin) {
  switch (act) {
    case FFM_ACT_SWIGLU: glu_forward_half_step_act<FFM_ACT_SWIGLU, FP8>(tcol, fp8_scale, store_pre, buf, lane, q_begin); break;
    case FFM_ACT_GEGLU_TANH: glu_forward_half_step_act<FFM_ACT_GEGLU_TANH, FP8>(tcol, fp8_scale, store_pre, buf, lane, q_begin); break;
    case FFM_ACT_RELU2: glu_forward_half_step_act<FFM_ACT_RELU2, FP8>(tcol, fp8_scale, store_pre, buf, lane, q_begin); break;
    default: glu_forward_half_step_act<FFM_ACT_GEGLU_ERF, FP8>(tcol, fp8_scale, store_pre, buf, lane, q_begin); break;
  }
}

// FP8 = 1: A and B hold e4m3 bytes, K-major only; a stage row is still 128 bytes, i.e. 128 K elements per block.
template <int A_MN, int B_MN, int EPI, int GROUPK, int CTA2, int PASS = 0, int FP8 = 0>
__global__ void __launch_bounds__(gemm_threads(EPI, PASS), 1)
ffm_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB0,
                const __grid_constant__ CUtensorMap tmB1, const __grid_constant__ CUtensorMap tmC,
                const __grid_constant__ CUtensorMap tmC2, const GemmParams p) {
  using S = Shape<CTA2, EPI>;
  constexpr int STAGES = S::STAGES;
  constexpr int STAGE_BYTES = S::STAGE_BYTES;
  constexpr bool HELPERS = epilogue_helpers(EPI);

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t pad = (1024u - (raw_addr & 1023u)) & 1023u;
  uint8_t* smem = smem_raw + pad;
  const uint32_t smem_base = raw_addr + pad;
  const uint32_t stg_base = smem_base + S::RING_BYTES;
  Ctrl* ctrl = reinterpret_cast<Ctrl*>(smem + S::RING_BYTES + S::STG_BYTES);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = CTA2 ? cluster_ctarank() : 0u;
  const bool leader = rank == 0;

  // ---- set-up ------------------------------------------------------------------------------
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(&ctrl->full_bar[s]), 1);
      mbar_init(smem_u32(&ctrl->empty_bar[s]), 1);
    }
    for (int a = 0; a < NUM_ACC; ++a) {
      mbar_init(smem_u32(&ctrl->acc_full_bar[a]), 1);
      // one arrival per epilogue warp (helpers included)
      mbar_init(smem_u32(&ctrl->acc_empty_bar[a]), (HELPERS ? 2 : 1) * EPI_WARPS * (CTA2 ? 2 : 1));
    }
    if (HELPERS) {
      for (int w = 0; w < EPI_WARPS; ++w) {
        for (int b = 0; b < 3; ++b) {
          mbar_init(smem_u32(&ctrl->pre_bar[w][b]), 1);
          mbar_init(smem_u32(&ctrl->help_bar[w][b]), 1);
          mbar_init(smem_u32(&ctrl->free_bar[w][b]), 1);
        }
      }
    }
    ctrl->abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB0);
    tma_prefetch_desc(&tmB1);
    tma_prefetch_desc(&tmC);
    tma_prefetch_desc(&tmC2);
  }
  if (!GROUPK && p.group_rows != nullptr) {
    // walk only the tiles that hold valid rows: per group ceil(rows / 128), rounded up to a pair with CTA2
    for (int i = threadIdx.x; i < p.groups; i += blockDim.x) {
      const int tiles = (p.group_rows[i] + BM - 1) / BM;
      ctrl->tile_start[i + 1] = CTA2 ? ((tiles + 1) & ~1) : tiles;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      int acc = 0;
      ctrl->tile_start[0] = 0;
      for (int i = 1; i <= p.groups; ++i) {
        acc += ctrl->tile_start[i];
        ctrl->tile_start[i] = acc;
      }
    }
  } else if (p.tile_start != nullptr) {
    for (int i = threadIdx.x; i <= p.groups; i += blockDim.x) ctrl->tile_start[i] = p.tile_start[i];
  } else if (threadIdx.x == 0) {
    ctrl->tile_start[0] = 0;
    ctrl->tile_start[1] = p.dense_m_tiles;
  }
  if (warp == 1) {
    if (CTA2) {
      tmem_alloc2(smem_u32(&ctrl->tmem_base), TMEM_COLS);
      tmem_relinquish2();
    } else {
      tmem_alloc(smem_u32(&ctrl->tmem_base), TMEM_COLS);
      tmem_relinquish();
    }
  }
  tc_fence_before();
  __syncthreads();
  if (CTA2) cluster_sync_all();  // the peer's barriers exist before anything arrives on them
  tc_fence_after();

  const uint32_t tmem_base = ctrl->tmem_base;
  volatile int* abort_flag = &ctrl->abort_flag;

  // ---- roles -------------------------------------------------------------------------------
  if (warp == 0) {
    // ================= TMA producer =================
    if (lane == 0) {
      TileWalker<GROUPK, CTA2> walker(p, ctrl->tile_start, rank);
      TileCoord t;
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      while (ok && walker.next(t)) {
        const int m0 = t.m_tile * BM;
#ifdef FFM_TUNE_GLUBWD_L2_PREFETCH
        if (EPI == EPI_GLUBWD) {
          // pull the tile's pre-activations into L2 a whole main loop ahead (tmC2 maps them with a 256 x 128 box)
          tma_prefetch_l2_2d(&tmC2, t.n_block * BN, m0);
          tma_prefetch_l2_2d(&tmC2, p.pz_h + t.n_block * BN, m0);
        }
#endif
        for (int kb = 0; kb < t.k_blocks && ok; ++kb) {
          ok = mbar_wait_bounded(smem_u32(&ctrl->empty_bar[stage]), phase ^ 1u, abort_flag, p.status,
                                 FFM_STATUS_WAIT_PRODUCER, p.wait_cycles);
          if (!ok) break;
          const uint32_t full_local = smem_u32(&ctrl->full_bar[stage]);
          const uint32_t full = CTA2 ? map_to_cta(full_local, 0) : full_local;  // the even CTA's barrier
          const uint32_t a_dst = smem_base + stage * STAGE_BYTES;
          const uint32_t b_dst = a_dst + A_STAGE_BYTES;
          if (leader) mbar_expect_tx(full_local, STAGE_BYTES * (CTA2 ? 2 : 1));
          const int k0 = kb * (FP8 ? 2 * BK : BK);
          // A tile: this CTA's 128 rows
          if (A_MN) {
            const int krow = t.k_row0 + k0;
            if (CTA2) {
              tma_load_2d_pair(a_dst, &tmA, full, m0, krow);
              tma_load_2d_pair(a_dst + 8192, &tmA, full, m0 + 64, krow);
            } else {
              tma_load_2d(a_dst, &tmA, full, m0, krow);
              tma_load_2d(a_dst + 8192, &tmA, full, m0 + 64, krow);
            }
          } else {
            if (CTA2) {
              tma_load_2d_pair(a_dst, &tmA, full, k0, m0);
            } else {
              tma_load_2d(a_dst, &tmA, full, k0, m0);
            }
          }
          // B tile: all 256 columns, or with CTA2 this CTA's 128-column half
          if (B_MN) {
            const int krow = GROUPK ? (t.k_row0 + k0) : static_cast<int>(t.group * p.b_group_rows + k0);
            const int n0 = t.n_block * BN + (CTA2 ? static_cast<int>(rank) * 128 : 0);
            if (CTA2) {
              tma_load_2d_pair(b_dst, &tmB0, full, n0, krow);
              tma_load_2d_pair(b_dst + 8192, &tmB0, full, n0 + 64, krow);
            } else {
#pragma unroll
              for (int j = 0; j < 4; ++j) tma_load_2d(b_dst + j * 8192, &tmB0, full, n0 + 64 * j, krow);
            }
          } else {
            const int nrow = static_cast<int>(t.group * p.b_group_rows) + t.n_block * (EPI == EPI_GLU ? 128 : BN);
            if (CTA2) {
              if (rank == 0) {
                tma_load_2d_pair(b_dst, &tmB0, full, k0, nrow);
              } else {
                tma_load_2d_pair(b_dst, &tmB1, full, k0, nrow + p.b1_row_offset);
              }
            } else {
              tma_load_2d(b_dst, &tmB0, full, k0, nrow);
              tma_load_2d(b_dst + 16384, &tmB1, full, k0, nrow + p.b1_row_offset);
            }
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ================= MMA issuer (with CTA2: only in the even CTA of the pair) =================
    if (lane == 0 && leader) {
      constexpr uint32_t idesc = FP8 ? make_idesc_e4m3(CTA2 ? 256 : 128, BN)
                                     : make_idesc_bf16(CTA2 ? 256 : 128, BN, A_MN, B_MN);
      TileWalker<GROUPK, CTA2> walker(p, ctrl->tile_start, rank);
      TileCoord t;
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      while (ok && walker.next(t)) {
        if (t.k_blocks == 0) continue;  // empty group: the epilogue stores zeros without an accumulator
        ok = mbar_wait_bounded(smem_u32(&ctrl->acc_empty_bar[acc]), acc_phase ^ 1u, abort_flag, p.status,
                               FFM_STATUS_WAIT_MMA, p.wait_cycles);
        if (!ok) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < t.k_blocks; ++kb) {
          ok = mbar_wait_bounded(smem_u32(&ctrl->full_bar[stage]), phase, abort_flag, p.status, FFM_STATUS_WAIT_MMA,
                                 p.wait_cycles);
          if (!ok) break;
          tc_fence_after();
          const uint32_t a_src = smem_base + stage * STAGE_BYTES;
          const uint32_t b_src = a_src + A_STAGE_BYTES;
#pragma unroll
          for (int kk = 0; kk < BK / UMMA_K; ++kk) {
            const uint64_t adesc = A_MN ? make_smem_desc_sw128(a_src + kk * 2048, 8192, 1024)
                                        : make_smem_desc_sw128(a_src + kk * 32, 16, 1024);
            const uint64_t bdesc = B_MN ? make_smem_desc_sw128(b_src + kk * 2048, 8192, 1024)
                                        : make_smem_desc_sw128(b_src + kk * 32, 16, 1024);
            const uint32_t accumulate = (kb > 0 || kk > 0) ? 1u : 0u;
            if (FP8) {
              if (CTA2) {
                umma_f8_pair(d_tmem, adesc, bdesc, idesc, accumulate);
              } else {
                umma_f8(d_tmem, adesc, bdesc, idesc, accumulate);
              }
            } else if (CTA2) {
              umma_bf16_pair(d_tmem, adesc, bdesc, idesc, accumulate);
            } else {
              umma_bf16(d_tmem, adesc, bdesc, idesc, accumulate);
            }
          }
          // free the stage (in both CTAs) once these MMAs retire
          const uint32_t empty_local = smem_u32(&ctrl->empty_bar[stage]);
          if (CTA2) {
            umma_commit_pair(empty_local);
            umma_commit_pair(map_to_cta(empty_local, 1));
          } else {
            umma_commit(empty_local);
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        const uint32_t accf_local = smem_u32(&ctrl->acc_full_bar[acc]);
        if (CTA2) {
          umma_commit_pair(accf_local);
          umma_commit_pair(map_to_cta(accf_local, 1));
        } else {
          umma_commit(accf_local);
        }
        if (++acc == NUM_ACC) {
          acc = 0;
          acc_phase ^= 1u;
        }
      }
    }
  } else if (PASS && warp >= 2 + EPI_WARPS) {
    // ================= passenger (warps 6..13) =================
    long long pz_rows = p.pz_rows;
    const long long used = static_cast<long long>(ctrl->tile_start[p.groups]) * BM;
    if (used < pz_rows) pz_rows = used;
    passenger_glu_backward(p, pz_rows,
                           static_cast<long long>(blockIdx.x) * PASSENGER_THREADS + (threadIdx.x - GEMM_THREADS),
                           static_cast<long long>(gridDim.x) * PASSENGER_THREADS);
  } else {
    // ================= epilogue (warps 2..5; with the GLU backward also helper warps 6..9) =================
    const int quarter = warp & 3;  // TMEM lanes [32 * quarter, 32 * quarter + 32) belong to this warp
    const int wi = (warp - 2) & 3;  // staging area and barriers; a helper shares those of the warp of its quarter
    const bool helper = HELPERS && warp >= 2 + EPI_WARPS;
    const uint32_t stg = stg_base + wi * S::STG_WARP_BYTES;
    constexpr int STEP_BYTES = S::BOXES_PER_STEP * BOX_BYTES;
    int step_slot = 0;  // staging slot of the next store step; advances per step actually stored
    uint32_t pre_phase = 0u;  // GLU-backward epilogue: bit b = parity to wait for on buffer b's load barrier
    uint32_t help_phase = 0u;  // the same for the helper's "half written" barriers (waited for by warps 2..5)
    uint32_t free_phase = 0u;  // ... and for the "boxes may be overwritten" barriers (waited for by the helpers)
    TileWalker<GROUPK, CTA2> walker(p, ctrl->tile_start, rank);
    TileCoord t;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    while (ok && walker.next(t)) {
      const int row0 = t.m_tile * BM + quarter * 32;  // first row of this warp's 32-row slab
      const int zdim = GROUPK ? t.group : 0;
      const bool have_acc = t.k_blocks > 0;
      if (EPI == EPI_GLUBWD) {
        // pre-activation boxes of this tile's first step, requested before the accumulator is waited for (the MMAs of
        // this tile may still be running): wait until the store that last read this buffer has drained, then load
        if (!helper && lane == 0) {
          bulk_wait_read<S::STEPS_BUFFERED - 1>();  // the store that last read this buffer is STEPS_BUFFERED groups back
          const uint32_t bar = smem_u32(&ctrl->pre_bar[wi][step_slot]);
          const uint32_t buf = stg + step_slot * STEP_BYTES;
          mbar_expect_tx(bar, STEP_BYTES);
          tma_load_3d(buf, &tmB1, bar, t.n_block * BN, row0, 0);
          tma_load_3d(buf + BOX_BYTES, &tmB1, bar, p.pz_h + t.n_block * BN, row0, 0);
        }
        __syncwarp();
      }
      if (have_acc) {
        ok = mbar_wait_bounded(smem_u32(&ctrl->acc_full_bar[acc]), acc_phase, abort_flag, p.status,
                               FFM_STATUS_WAIT_EPILOGUE, p.wait_cycles);
        ok = __all_sync(0xffffffffu, ok ? 1 : 0) != 0;
        if (!ok) break;
        tc_fence_after();
      }
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * BN;
      // FP8: de-quantisation factor of this lane's row in this tile = scale of the row of A x scale of the group's B
      float fp8_scale = 1.0f;
      if (FP8) fp8_scale = __ldg(fp8_a_scale(p) + row0 + lane) * __ldg(fp8_b_scale(p) + t.group);

      if (EPI == EPI_GLU) {
        // two steps of 64 GLU columns; warp wi takes the lower 32 columns of a step, its helper the upper 32, eight
        // columns of gate and up per trip of a rolled loop. A step fills three boxes (activation, gate, up), stored as
        // one group by warp wi once the helper has written its half.
        const int h0 = t.n_block * 128;
        const int qb = helper ? 4 : 0;
#pragma unroll 1
        for (int st = 0; st < 2 && h0 + st * 64 < p.n_cols; ++st) {
          const uint32_t buf = stg + step_slot * STEP_BYTES;
          const uint32_t slot_bit = 1u << step_slot;
          if (!helper) {
            // the slot is free once the step stored STEPS_BUFFERED steps ago has been read out
            if (lane == 0) {
              bulk_wait_read<S::STEPS_BUFFERED - 1>();
              mbar_arrive(smem_u32(&ctrl->free_bar[wi][step_slot]));
            }
            __syncwarp();
          } else {
            ok = mbar_wait_bounded(smem_u32(&ctrl->free_bar[wi][step_slot]), (free_phase & slot_bit) ? 1u : 0u,
                                   abort_flag, p.status, FFM_STATUS_WAIT_EPILOGUE, p.wait_cycles);
            ok = __all_sync(0xffffffffu, ok ? 1 : 0) != 0;
            if (!ok) break;
            free_phase ^= slot_bit;
          }
          if (h0 + st * 64 + qb * 8 < p.n_cols) {
            glu_forward_half_step<FP8>(taddr + st * 64 + qb * 8, p.act, fp8_scale, p.has_c2 != 0, buf, lane, qb);
          }
          fence_proxy_async();
          __syncwarp();
          if (helper) {
            if (lane == 0) mbar_arrive(smem_u32(&ctrl->help_bar[wi][step_slot]));
          } else {
            ok = mbar_wait_bounded(smem_u32(&ctrl->help_bar[wi][step_slot]), (help_phase & slot_bit) ? 1u : 0u,
                                   abort_flag, p.status, FFM_STATUS_WAIT_EPILOGUE, p.wait_cycles);
            ok = __all_sync(0xffffffffu, ok ? 1 : 0) != 0;
            if (!ok) break;
            help_phase ^= slot_bit;
            if (lane == 0) {
              const int col = h0 + st * 64;
              tma_store_3d(&tmC, buf, col, row0, 0);
              if (p.has_c2) {
                tma_store_3d(&tmC2, buf + BOX_BYTES, col, row0, 0);
                tma_store_3d(&tmC2, buf + 2 * BOX_BYTES, p.glu_h + col, row0, 0);
              }
              bulk_commit();
            }
          }
          if (++step_slot == S::STEPS_BUFFERED) step_slot = 0;
        }
        if (!ok) break;
      } else if (EPI == EPI_GLUBWD) {
        // The accumulator is dAct (gradient of the GLU output). Rounded to bf16 as the stand-alone dAct GEMM would
        // store it, it goes through the GLU backward with the saved pre-activations of the same rows and columns, and
        // the gate and up gradients leave as two boxes per 64-column step: dAct itself never touches memory.
        // The pre-activations come in by TMA, one step (a gate box and an up box of 32 rows x 64 columns) ahead, into
        // the boxes that the step's results are then written over and stored from (tmB1 maps them).
        // The step loop is deliberately not unrolled and the activation is a template argument of the step's math:
        // unrolled with the activation switch inlined at every element, the epilogue did not fit the instruction
        // cache and its warps spent most of their time waiting for instructions (ncu: stall_no_instruction 4.9 per
        // issue, 3.4 x the run time of the plain dAct GEMM).
        const int n0 = t.n_block * BN;
        const int Hh = p.pz_h;
        const int steps = (p.n_cols - n0 >= BN) ? BN / 64 : (p.n_cols - n0 + 63) / 64;  // 64-column steps of this tile
#pragma unroll 1
        for (int st = 0; st < steps; ++st) {
          const uint32_t buf = stg + step_slot * STEP_BYTES;
          // next step's boxes into the next buffer of the rotation (the store that last read it lies
          // STEPS_BUFFERED - 1 groups back, so the wait leaves the latest STEPS_BUFFERED - 2 stores alone)
          if (st + 1 < steps && !helper && lane == 0) {
            bulk_wait_read<(S::STEPS_BUFFERED >= 2 ? S::STEPS_BUFFERED - 2 : 0)>();
            const int nslot = (step_slot + 1 == S::STEPS_BUFFERED) ? 0 : step_slot + 1;
            const uint32_t nbar = smem_u32(&ctrl->pre_bar[wi][nslot]);
            const uint32_t nbuf = stg + nslot * STEP_BYTES;
            mbar_expect_tx(nbar, STEP_BYTES);
            tma_load_3d(nbuf, &tmB1, nbar, n0 + (st + 1) * 64, row0, 0);
            tma_load_3d(nbuf + BOX_BYTES, &tmB1, nbar, Hh + n0 + (st + 1) * 64, row0, 0);
          }
          const uint32_t parity = (pre_phase >> step_slot) & 1u;
          ok = mbar_wait_bounded(smem_u32(&ctrl->pre_bar[wi][step_slot]), parity, abort_flag, p.status,
                                 FFM_STATUS_WAIT_EPILOGUE, p.wait_cycles);
          ok = __all_sync(0xffffffffu, ok ? 1 : 0) != 0;
          if (!ok) break;
          pre_phase ^= 1u << step_slot;
          const int qb = helper ? 4 : 0;  // first 16-byte column group of this warp's half of the step
          switch (p.pz_act) {
            case FFM_ACT_SWIGLU: glu_backward_step<FFM_ACT_SWIGLU>(taddr + st * 64, p.scale, buf, lane, qb); break;
            case FFM_ACT_GEGLU_TANH: glu_backward_step<FFM_ACT_GEGLU_TANH>(taddr + st * 64, p.scale, buf, lane, qb); break;
            case FFM_ACT_RELU2: glu_backward_step<FFM_ACT_RELU2>(taddr + st * 64, p.scale, buf, lane, qb); break;
            default: glu_backward_step<FFM_ACT_GEGLU_ERF>(taddr + st * 64, p.scale, buf, lane, qb); break;
          }
          fence_proxy_async();
          __syncwarp();
          if (helper) {
            // the step's buffer is reused only after warp wi has stored it and loaded the next boxes into it, and this
            // warp sees those through pre_bar: no wait in this direction
            if (lane == 0) mbar_arrive(smem_u32(&ctrl->help_bar[wi][step_slot]));
          } else {
            ok = mbar_wait_bounded(smem_u32(&ctrl->help_bar[wi][step_slot]), (help_phase >> step_slot) & 1u, abort_flag,
                                   p.status, FFM_STATUS_WAIT_EPILOGUE, p.wait_cycles);
            ok = __all_sync(0xffffffffu, ok ? 1 : 0) != 0;
            if (!ok) break;
            help_phase ^= 1u << step_slot;
            if (lane == 0) {
              tma_store_3d(&tmC, buf, n0 + st * 64, row0, 0);
              tma_store_3d(&tmC, buf + BOX_BYTES, Hh + n0 + st * 64, row0, 0);
              bulk_commit();
            }
          }
          if (++step_slot == S::STEPS_BUFFERED) step_slot = 0;
        }
        if (!ok) break;
      } else {
        // four steps of 64 columns (one box each), two 32-column chunks per step, TMEM loads one chunk ahead
        const int n0 = t.n_block * BN;
        const float scale = FP8 ? p.scale * fp8_scale : p.scale;
        uint32_t v[2][32];
        if (have_acc) tmem_ld_32x32(taddr, v[0]);
#pragma unroll
        for (int c = 0; c < BN / 32; ++c) {
          if (have_acc) {
            tmem_ld_wait();
            if (c + 1 < BN / 32) tmem_ld_32x32(taddr + (c + 1) * 32, v[(c + 1) & 1]);
          }
          const int col = n0 + (c >> 1) * 64;  // first column of this step's box
          if (col < p.n_cols) {
            const uint32_t buf = stg + step_slot * STEP_BYTES;
            if ((c & 1) == 0) {
              if (lane == 0) bulk_wait_read<S::STEPS_BUFFERED - 1>();
              __syncwarp();
            }
            if (n0 + c * 32 < p.n_cols) {
              uint32_t o[16];
#pragma unroll
              for (int i = 0; i < 16; ++i) {
                o[i] = have_acc ? pack_bf16x2(__uint_as_float(v[c & 1][2 * i]) * scale,
                                              __uint_as_float(v[c & 1][2 * i + 1]) * scale)
                                : 0u;
              }
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                st_shared_v4(buf + box_offset(lane, (c & 1) * 4 + q), o[4 * q], o[4 * q + 1], o[4 * q + 2], o[4 * q + 3]);
              }
            }
            if (c & 1) {
              fence_proxy_async();
              __syncwarp();
              if (lane == 0) {
                tma_store_3d(&tmC, buf, col, row0, zdim);
                bulk_commit();
              }
              if (++step_slot == S::STEPS_BUFFERED) step_slot = 0;
            }
          }
        }
      }
      if (have_acc) {
        // hand the accumulator back to the MMA issuer (from the odd CTA of a pair: a remote arrive)
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          const uint32_t bar = smem_u32(&ctrl->acc_empty_bar[acc]);
          if (CTA2) {
            mbar_arrive_cluster(map_to_cta(bar, 0));
          } else {
            mbar_arrive(bar);
          }
        }
        if (++acc == NUM_ACC) {
          acc = 0;
          acc_phase ^= 1u;
        }
      }
    }
    if (lane == 0) bulk_wait0();  // this lane's bulk stores have landed before the CTA's shared memory goes away
  }

  // ---- common exit: every role reaches this point, also after an abort ----------------------
  tc_fence_before();
  __syncthreads();
  if (CTA2) cluster_sync_all();  // neither CTA leaves while its peer may still touch its barriers or operands
  if (warp == 1) {
    tc_fence_after();
    if (CTA2) {
      tmem_dealloc2(tmem_base, TMEM_COLS);
    } else {
      tmem_dealloc(tmem_base, TMEM_COLS);
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------------

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
    }
  }
  return fn;
}

// 2-D tensor map over a row-major [rows, cols] matrix of bf16 (elt_bytes 2) or bytes (elt_bytes 1: e4m3 operands),
// 128-byte swizzle, zero fill out of bounds.
int make_map_2d(CUtensorMap* map, const void* base, long long rows, long long cols, int box_cols, int box_rows,
                int elt_bytes = 2) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) return FFM_ERR_NO_DRIVER;
  if (rows <= 0 || cols <= 0) return FFM_ERR_BAD_ARG;
  if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0 || (cols * elt_bytes) % 16 != 0) return FFM_ERR_UNSUPPORTED;
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(cols) * elt_bytes};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(box_cols), static_cast<cuuint32_t>(box_rows)};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, elt_bytes == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                  const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? FFM_OK : FFM_ERR_LAUNCH;
}

// 2-D bf16 map used only for L2 prefetches (cp.async.bulk.prefetch.tensor): box {256 columns, 128 rows}, no swizzle.
int make_prefetch_map(CUtensorMap* map, const void* base, long long rows, long long cols) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) return FFM_ERR_NO_DRIVER;
  if (rows <= 0 || cols <= 0) return FFM_ERR_BAD_ARG;
  if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0 || (cols * 2) % 16 != 0) return FFM_ERR_UNSUPPORTED;
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(cols) * 2};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(cols < 256 ? cols : 256), static_cast<cuuint32_t>(rows < 128 ? rows : 128)};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? FFM_OK : FFM_ERR_LAUNCH;
}

// 3-D bf16 output map over [groups, rows, cols] (row-major, contiguous), 128-byte swizzle, box {64, 32, 1}.
int make_out_map(CUtensorMap* map, void* base, long long groups, long long rows, long long cols) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) return FFM_ERR_NO_DRIVER;
  if (groups <= 0 || rows <= 0 || cols <= 0) return FFM_ERR_BAD_ARG;
  if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0 || (cols * 2) % 16 != 0) return FFM_ERR_UNSUPPORTED;
  cuuint64_t dims[3] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows), static_cast<cuuint64_t>(groups)};
  cuuint64_t strides[2] = {static_cast<cuuint64_t>(cols) * 2, static_cast<cuuint64_t>(cols) * rows * 2};
  cuuint32_t box[3] = {64, 32, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, base, dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? FFM_OK : FFM_ERR_LAUNCH;
}

int num_sms() {
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (sms <= 0) sms = 148;
  }
  return sms;
}

long long g_wait_cycles = 2000000000LL;
int g_cta_pair = -1;  // -1: read FFM_GEMM_CTA_PAIR from the environment on first use (default on)

bool use_cta_pair() {
  if (g_cta_pair < 0) {
    const char* e = getenv("FFM_GEMM_CTA_PAIR");
    g_cta_pair = (e != nullptr && e[0] == '0') ? 0 : 1;
  }
  return g_cta_pair != 0;
}

template <int A_MN, int B_MN, int EPI, int GROUPK, int CTA2, int PASS = 0, int FP8 = 0>
int launch_gemm_shape(const CUtensorMap& tmA, const CUtensorMap& tmB0, const CUtensorMap& tmB1, const CUtensorMap& tmC,
                      const CUtensorMap& tmC2, const GemmParams& p, long long max_units, cudaStream_t stream) {
  static int max_ctas = 0;  // persistent grid size, found once per instantiation
  auto kernel = ffm_gemm_kernel<A_MN, B_MN, EPI, GROUPK, CTA2, PASS, FP8>;
  constexpr int threads = gemm_threads(EPI, PASS);
  constexpr int smem_bytes = Shape<CTA2, EPI>::SMEM_BYTES;
  if (max_ctas == 0) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes) != cudaSuccess) {
      cudaGetLastError();
      return FFM_ERR_LAUNCH;
    }
    max_ctas = num_sms();
    if (CTA2) {
      // co-resident CTA pairs: a GPC with an odd number of usable SMs leaves one SM without a partner
      cudaLaunchConfig_t q = {};
      q.gridDim = dim3(num_sms() & ~1, 1, 1);
      q.blockDim = dim3(threads, 1, 1);
      q.dynamicSmemBytes = smem_bytes;
      cudaLaunchAttribute qa[1];
      qa[0].id = cudaLaunchAttributeClusterDimension;
      qa[0].val.clusterDim.x = 2;
      qa[0].val.clusterDim.y = 1;
      qa[0].val.clusterDim.z = 1;
      q.attrs = qa;
      q.numAttrs = 1;
      int clusters = 0;
      if (cudaOccupancyMaxActiveClusters(&clusters, kernel, &q) != cudaSuccess || clusters <= 0) {
        cudaGetLastError();
        clusters = num_sms() / 2 - 4;
      }
      max_ctas = 2 * clusters;
    }
  }
  if (max_units <= 0 && !(PASS && p.pz_rows > 0)) return FFM_OK;
  long long ctas = CTA2 ? 2 * max_units : max_units;
  if (PASS && p.pz_rows > 0) ctas = max_ctas;  // the passenger job wants every SM, whatever the GEMM's tile count
  if (ctas > max_ctas) ctas = max_ctas;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(ctas), 1, 1);
  cfg.blockDim = dim3(threads, 1, 1);
  cfg.dynamicSmemBytes = smem_bytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = CTA2 ? 2 : 1;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = CTA2 ? 1 : 0;  // the one-CTA shape is an ordinary launch
  if (cudaLaunchKernelEx(&cfg, kernel, tmA, tmB0, tmB1, tmC, tmC2, p) != cudaSuccess) {
    cudaGetLastError();
    return FFM_ERR_LAUNCH;
  }
  return FFM_OK;
}

// max_m_tiles: upper bound on the 128-row tiles of M the walker can see (per group for grouped-K);
// multiplier: tiles per M tile (N blocks, times groups for grouped-K).
template <int A_MN, int B_MN, int EPI, int GROUPK, int PASS = 0, int FP8 = 0>
int launch_gemm(const CUtensorMap& tmA, const CUtensorMap& tmB0, const CUtensorMap& tmB1, const CUtensorMap& tmC,
                const CUtensorMap& tmC2, const GemmParams& p, long long max_m_tiles, long long multiplier,
                cudaStream_t stream, int tile_rows = 0) {
  const bool pair = tile_rows == 256 ? true : (tile_rows == 128 ? false : use_cta_pair());
  if (pair) {
    return launch_gemm_shape<A_MN, B_MN, EPI, GROUPK, 1, PASS, FP8>(tmA, tmB0, tmB1, tmC, tmC2, p,
                                                                    ((max_m_tiles + 1) / 2) * multiplier, stream);
  }
  return launch_gemm_shape<A_MN, B_MN, EPI, GROUPK, 0, PASS, FP8>(tmA, tmB0, tmB1, tmC, tmC2, p,
                                                                   max_m_tiles * multiplier, stream);
}

}  // namespace

}  // namespace ffm

using namespace ffm;

extern "C" long long ffm_set_wait_cycles(long long cycles) {
  long long old = g_wait_cycles;
  if (cycles > 0) g_wait_cycles = cycles;
  return old;
}

extern "C" int ffm_set_gemm_cta_pair(int enable) {
  const int old = use_cta_pair() ? 1 : 0;
  if (enable == 0 || enable == 1) g_cta_pair = enable;
  return old;
}

extern "C" int ffm_grouped_gemm_glu(const void* A, const void* w_gate, const void* w_up, int64_t group_rows,
                                    int groups, const int32_t* tile_start, int64_t rows, int K, int H,
                                    int activation, void* act, void* preact, const int32_t* valid_rows, int tile_rows,
                                    int32_t* status, ffm_stream_t stream) {
  if (!A || !w_gate || !w_up || !act || !status) return FFM_ERR_BAD_ARG;
  if (groups < 1 || groups > MAX_GROUPS || rows < 0 || K <= 0 || H <= 0 || group_rows < H) return FFM_ERR_BAD_ARG;
  if (activation < 0 || activation > 3) return FFM_ERR_BAD_ARG;
  if (tile_start == nullptr && groups != 1) return FFM_ERR_BAD_ARG;
  if (tile_rows != 0 && tile_rows != 128 && tile_rows != 256) return FFM_ERR_BAD_ARG;
  if (valid_rows != nullptr && tile_start == nullptr) return FFM_ERR_BAD_ARG;
  if (K % 64 != 0 || H % 64 != 0) return FFM_ERR_UNSUPPORTED;  // a 64-column box of gate must not reach into up
  if (rows == 0) return FFM_OK;
  CUtensorMap tmA, tmB0, tmB1, tmC, tmC2;
  int rc;
  if ((rc = make_map_2d(&tmA, A, rows, K, 64, 128)) != FFM_OK) return rc;
  const long long wrows = static_cast<long long>(groups - 1) * group_rows + H;
  if ((rc = make_map_2d(&tmB0, w_gate, wrows, K, 64, 128)) != FFM_OK) return rc;
  if ((rc = make_map_2d(&tmB1, w_up, wrows, K, 64, 128)) != FFM_OK) return rc;
  if ((rc = make_out_map(&tmC, act, 1, rows, H)) != FFM_OK) return rc;
  if (preact != nullptr) {
    if ((rc = make_out_map(&tmC2, preact, 1, rows, 2LL * H)) != FFM_OK) return rc;
  } else {
    tmC2 = tmC;
  }
  GemmParams p = {};
  p.tile_start = tile_start;
  p.groups = groups;
  p.dense_m_tiles = static_cast<int>((rows + BM - 1) / BM);
  p.n_cols = H;
  p.k_blocks = K / BK;
  p.b_group_rows = group_rows;
  p.b1_row_offset = 0;
  p.has_c2 = preact != nullptr ? 1 : 0;
  p.glu_h = H;
  p.scale = 1.0f;
  p.act = activation;
  p.n_tiles = (H + 127) / 128;
  p.status = status;
  p.wait_cycles = g_wait_cycles;
  p.group_rows = valid_rows;
  return launch_gemm<0, 0, EPI_GLU, 0>(tmA, tmB0, tmB1, tmC, tmC2, p, (rows + BM - 1) / BM, p.n_tiles,
                                       static_cast<cudaStream_t>(stream), tile_rows);
}

extern "C" int ffm_grouped_gemm(const void* A, const void* B, int b_major, int groups, const int32_t* tile_start,
                                int64_t rows, int K, int Nout, float scale, void* out, const int32_t* valid_rows,
                                int tile_rows, int32_t* status, ffm_stream_t stream) {
  if (!A || !B || !out || !status) return FFM_ERR_BAD_ARG;
  if (groups < 1 || groups > MAX_GROUPS || rows < 0 || K <= 0 || Nout <= 0) return FFM_ERR_BAD_ARG;
  if (b_major != FFM_B_KMAJOR && b_major != FFM_B_NMAJOR) return FFM_ERR_BAD_ARG;
  if (tile_start == nullptr && groups != 1) return FFM_ERR_BAD_ARG;
  if (tile_rows != 0 && tile_rows != 128 && tile_rows != 256) return FFM_ERR_BAD_ARG;
  if (valid_rows != nullptr && tile_start == nullptr) return FFM_ERR_BAD_ARG;
  if (K % 64 != 0 || Nout % 32 != 0) return FFM_ERR_UNSUPPORTED;
  if (b_major == FFM_B_NMAJOR && Nout % 64 != 0) return FFM_ERR_UNSUPPORTED;
  if (rows == 0) return FFM_OK;
  CUtensorMap tmA, tmB, tmC;
  int rc;
  if ((rc = make_map_2d(&tmA, A, rows, K, 64, 128)) != FFM_OK) return rc;
  if ((rc = make_out_map(&tmC, out, 1, rows, Nout)) != FFM_OK) return rc;
  GemmParams p = {};
  p.tile_start = tile_start;
  p.groups = groups;
  p.dense_m_tiles = static_cast<int>((rows + BM - 1) / BM);
  p.n_cols = Nout;
  p.k_blocks = K / BK;
  p.scale = scale;
  p.n_tiles = (Nout + BN - 1) / BN;
  p.status = status;
  p.wait_cycles = g_wait_cycles;
  p.group_rows = valid_rows;
  const long long m_tiles = (rows + BM - 1) / BM;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (b_major == FFM_B_KMAJOR) {
    if ((rc = make_map_2d(&tmB, B, static_cast<long long>(groups) * Nout, K, 64, 128)) != FFM_OK) return rc;
    p.b_group_rows = Nout;
    p.b1_row_offset = 128;
    return launch_gemm<0, 0, EPI_PLAIN, 0>(tmA, tmB, tmB, tmC, tmC, p, m_tiles, p.n_tiles, s, tile_rows);
  }
  if ((rc = make_map_2d(&tmB, B, static_cast<long long>(groups) * K, Nout, 64, 64)) != FFM_OK) return rc;
  p.b_group_rows = K;
  return launch_gemm<0, 1, EPI_PLAIN, 0>(tmA, tmB, tmB, tmC, tmC, p, m_tiles, p.n_tiles, s, tile_rows);
}

extern "C" int ffm_grouped_gemm_wgrad(const void* A, const void* B, int groups, const int32_t* tile_start,
                                      int64_t rows_cap, int M, int Nout, float scale, void* dW, int32_t* status,
                                      ffm_stream_t stream) {
  if (!A || !B || !dW || !status || !tile_start) return FFM_ERR_BAD_ARG;
  if (groups < 1 || groups > MAX_GROUPS || rows_cap <= 0 || M <= 0 || Nout <= 0) return FFM_ERR_BAD_ARG;
  if (M % 64 != 0 || Nout % 64 != 0) return FFM_ERR_UNSUPPORTED;
  CUtensorMap tmA, tmB, tmC;
  int rc;
  if ((rc = make_map_2d(&tmA, A, rows_cap, M, 64, 64)) != FFM_OK) return rc;
  if ((rc = make_map_2d(&tmB, B, rows_cap, Nout, 64, 64)) != FFM_OK) return rc;
  if ((rc = make_out_map(&tmC, dW, groups, M, Nout)) != FFM_OK) return rc;
  GemmParams p = {};
  p.tile_start = tile_start;
  p.groups = groups;
  p.n_cols = Nout;
  p.scale = scale;
  p.m_tiles_per_group = (M + BM - 1) / BM;
  p.n_tiles = (Nout + BN - 1) / BN;
  p.status = status;
  p.wait_cycles = g_wait_cycles;
  return launch_gemm<1, 1, EPI_PLAIN, 1>(tmA, tmB, tmB, tmC, tmC, p, p.m_tiles_per_group,
                                         static_cast<long long>(groups) * p.n_tiles,
                                         static_cast<cudaStream_t>(stream));
}

extern "C" int ffm_grouped_gemm_wgrad_glu_backward(const void* A, const void* B, int groups, const int32_t* tile_start,
                                                   int64_t rows_cap, int M, int Nout, float scale, void* dW,
                                                   const void* dAct, const void* preact, int64_t glu_rows, int H,
                                                   int activation, void* gU, int32_t* status, ffm_stream_t stream) {
  if (!dAct || !preact || !gU || glu_rows < 0 || H <= 0 || H % 8 != 0) return FFM_ERR_BAD_ARG;
  if (activation < 0 || activation > 3) return FFM_ERR_BAD_ARG;
  if (!A || !B || !dW || !status || !tile_start) return FFM_ERR_BAD_ARG;
  if (groups < 1 || groups > MAX_GROUPS || rows_cap <= 0 || M <= 0 || Nout <= 0) return FFM_ERR_BAD_ARG;
  if (M % 64 != 0 || Nout % 64 != 0) return FFM_ERR_UNSUPPORTED;
  CUtensorMap tmA, tmB, tmC;
  int rc;
  if ((rc = make_map_2d(&tmA, A, rows_cap, M, 64, 64)) != FFM_OK) return rc;
  if ((rc = make_map_2d(&tmB, B, rows_cap, Nout, 64, 64)) != FFM_OK) return rc;
  if ((rc = make_out_map(&tmC, dW, groups, M, Nout)) != FFM_OK) return rc;
  GemmParams p = {};
  p.tile_start = tile_start;
  p.groups = groups;
  p.n_cols = Nout;
  p.scale = scale;
  p.m_tiles_per_group = (M + BM - 1) / BM;
  p.n_tiles = (Nout + BN - 1) / BN;
  p.status = status;
  p.wait_cycles = g_wait_cycles;
  p.pz_dact = static_cast<const bf16*>(dAct);
  p.pz_pre = static_cast<const bf16*>(preact);
  p.pz_gu = static_cast<bf16*>(gU);
  p.pz_rows = glu_rows;
  p.pz_h = H;
  p.pz_act = activation;
  return launch_gemm<1, 1, EPI_PLAIN, 1, 1>(tmA, tmB, tmB, tmC, tmC, p, p.m_tiles_per_group,
                                         static_cast<long long>(groups) * p.n_tiles,
                                         static_cast<cudaStream_t>(stream));
}

// ---- FP8 (e4m3) forward projections: quantised operands, fp32 accumulation, scales applied in the epilogue ----

extern "C" int ffm_grouped_gemm_glu_fp8(const void* Aq, const float* a_scale, const void* Wq, const float* w_scale,
                                        int groups, const int32_t* tile_start, int64_t rows, int K, int H,
                                        int activation, void* act, void* preact, int tile_rows, int32_t* status,
                                        ffm_stream_t stream) {
  if (!Aq || !a_scale || !Wq || !w_scale || !act || !status) return FFM_ERR_BAD_ARG;
  if (groups < 1 || groups > MAX_GROUPS || rows < 0 || K <= 0 || H <= 0) return FFM_ERR_BAD_ARG;
  if (activation < 0 || activation > 3) return FFM_ERR_BAD_ARG;
  if (tile_start == nullptr && groups != 1) return FFM_ERR_BAD_ARG;
  if (tile_rows != 0 && tile_rows != 128 && tile_rows != 256) return FFM_ERR_BAD_ARG;
  if (K % 128 != 0 || H % 64 != 0) return FFM_ERR_UNSUPPORTED;
  if (rows == 0) return FFM_OK;
  CUtensorMap tmA, tmB0, tmB1, tmC, tmC2;
  int rc;
  if ((rc = make_map_2d(&tmA, Aq, rows, K, 128, 128, 1)) != FFM_OK) return rc;
  const long long wrows = static_cast<long long>(groups) * 2 * H;
  const uint8_t* w = static_cast<const uint8_t*>(Wq);
  // gate rows of every group through one map, up rows (H rows further down) through a second one
  if ((rc = make_map_2d(&tmB0, w, wrows - H, K, 128, 128, 1)) != FFM_OK) return rc;
  if ((rc = make_map_2d(&tmB1, w + static_cast<long long>(H) * K, wrows - H, K, 128, 128, 1)) != FFM_OK) return rc;
  if ((rc = make_out_map(&tmC, act, 1, rows, H)) != FFM_OK) return rc;
  if (preact != nullptr) {
    if ((rc = make_out_map(&tmC2, preact, 1, rows, 2LL * H)) != FFM_OK) return rc;
  } else {
    tmC2 = tmC;
  }
  GemmParams p = {};
  p.tile_start = tile_start;
  p.groups = groups;
  p.dense_m_tiles = static_cast<int>((rows + BM - 1) / BM);
  p.n_cols = H;
  p.k_blocks = K / 128;
  p.b_group_rows = 2LL * H;
  p.b1_row_offset = 0;
  p.has_c2 = preact != nullptr ? 1 : 0;
  p.glu_h = H;
  p.scale = 1.0f;
  p.act = activation;
  p.n_tiles = (H + 127) / 128;
  p.status = status;
  p.wait_cycles = g_wait_cycles;
  p.pz_dact = reinterpret_cast<const bf16*>(a_scale);   // see fp8_a_scale / fp8_b_scale
  p.pz_pre = reinterpret_cast<const bf16*>(w_scale);
  return launch_gemm<0, 0, EPI_GLU, 0, 0, 1>(tmA, tmB0, tmB1, tmC, tmC2, p, (rows + BM - 1) / BM, p.n_tiles,
                                             static_cast<cudaStream_t>(stream), tile_rows);
}

extern "C" int ffm_grouped_gemm_fp8(const void* Aq, const float* a_scale, const void* Bq, const float* b_scale,
                                    int groups, const int32_t* tile_start, int64_t rows, int K, int Nout, void* out,
                                    int tile_rows, int32_t* status, ffm_stream_t stream) {
  if (!Aq || !a_scale || !Bq || !b_scale || !out || !status) return FFM_ERR_BAD_ARG;
  if (groups < 1 || groups > MAX_GROUPS || rows < 0 || K <= 0 || Nout <= 0) return FFM_ERR_BAD_ARG;
  if (tile_start == nullptr && groups != 1) return FFM_ERR_BAD_ARG;
  if (tile_rows != 0 && tile_rows != 128 && tile_rows != 256) return FFM_ERR_BAD_ARG;
  if (K % 128 != 0 || Nout % 32 != 0) return FFM_ERR_UNSUPPORTED;
  if (rows == 0) return FFM_OK;
  CUtensorMap tmA, tmB, tmC;
  int rc;
  if ((rc = make_map_2d(&tmA, Aq, rows, K, 128, 128, 1)) != FFM_OK) return rc;
  if ((rc = make_map_2d(&tmB, Bq, static_cast<long long>(groups) * Nout, K, 128, 128, 1)) != FFM_OK) return rc;
  if ((rc = make_out_map(&tmC, out, 1, rows, Nout)) != FFM_OK) return rc;
  GemmParams p = {};
  p.tile_start = tile_start;
  p.groups = groups;
  p.dense_m_tiles = static_cast<int>((rows + BM - 1) / BM);
  p.n_cols = Nout;
  p.k_blocks = K / 128;
  p.scale = 1.0f;
  p.n_tiles = (Nout + BN - 1) / BN;
  p.status = status;
  p.wait_cycles = g_wait_cycles;
  p.b_group_rows = Nout;
  p.b1_row_offset = 128;
  p.pz_dact = reinterpret_cast<const bf16*>(a_scale);   // see fp8_a_scale / fp8_b_scale
  p.pz_pre = reinterpret_cast<const bf16*>(b_scale);
  return launch_gemm<0, 0, EPI_PLAIN, 0, 0, 1>(tmA, tmB, tmB, tmC, tmC, p, (rows + BM - 1) / BM, p.n_tiles,
                                               static_cast<cudaStream_t>(stream), tile_rows);
}

// ---- dAct GEMM with the GLU backward in its epilogue ----

extern "C" int ffm_grouped_gemm_dact_glu_backward(const void* gY, const void* Wd, int groups, const int32_t* tile_start,
                                                  int64_t rows, int K, int H, int activation, const void* preact,
                                                  void* gU, int tile_rows, int32_t* status, ffm_stream_t stream) {
  if (!gY || !Wd || !preact || !gU || !status) return FFM_ERR_BAD_ARG;
  if (groups < 1 || groups > MAX_GROUPS || rows < 0 || K <= 0 || H <= 0) return FFM_ERR_BAD_ARG;
  if (activation < 0 || activation > 3) return FFM_ERR_BAD_ARG;
  if (tile_start == nullptr && groups != 1) return FFM_ERR_BAD_ARG;
  if (tile_rows != 0 && tile_rows != 128 && tile_rows != 256) return FFM_ERR_BAD_ARG;
  if (K % 64 != 0 || H % 64 != 0) return FFM_ERR_UNSUPPORTED;
  if (rows == 0) return FFM_OK;
  CUtensorMap tmA, tmB, tmC, tmP;
  int rc;
  if ((rc = make_map_2d(&tmA, gY, rows, K, 64, 128)) != FFM_OK) return rc;
  if ((rc = make_map_2d(&tmB, Wd, static_cast<long long>(groups) * K, H, 64, 64)) != FFM_OK) return rc;
  if ((rc = make_out_map(&tmC, gU, 1, rows, 2LL * H)) != FFM_OK) return rc;
  if ((rc = make_prefetch_map(&tmP, preact, rows, 2LL * H)) != FFM_OK) return rc;
  CUtensorMap tmL;  // the epilogue's loads of the pre-activations: 64 x 32 boxes, same swizzle as the stores
  if ((rc = make_out_map(&tmL, const_cast<void*>(preact), 1, rows, 2LL * H)) != FFM_OK) return rc;
  GemmParams p = {};
  p.tile_start = tile_start;
  p.groups = groups;
  p.dense_m_tiles = static_cast<int>((rows + BM - 1) / BM);
  p.n_cols = H;
  p.k_blocks = K / BK;
  p.scale = 1.0f;
  p.n_tiles = (H + BN - 1) / BN;
  p.status = status;
  p.wait_cycles = g_wait_cycles;
  p.b_group_rows = K;
  p.pz_pre = static_cast<const bf16*>(preact);
  p.pz_rows = rows;
  p.pz_h = H;
  p.pz_act = activation;
  return launch_gemm<0, 1, EPI_GLUBWD, 0>(tmA, tmB, tmL, tmC, tmP, p, (rows + BM - 1) / BM, p.n_tiles,
                                          static_cast<cudaStream_t>(stream), tile_rows);
}
