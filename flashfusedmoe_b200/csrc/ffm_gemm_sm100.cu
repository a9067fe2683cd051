// Grouped GEMM for sm_100a: TMA-fed shared-memory ring, tcgen05.mma with fp32 accumulators in TMEM,
// persistent CTAs, warp-specialised roles.
//
//   warp 0      TMA producer   (one lane issues cp.async.bulk.tensor loads into a 4-stage ring)
//   warp 1      MMA issuer     (one lane issues tcgen05.mma; owns the TMEM allocation)
//   warps 2..5  epilogue       (tcgen05.ld of the 128 x 256 fp32 accumulator, math, bf16 stores)
//
// The accumulator is double-buffered in TMEM (2 x 256 columns), so the epilogue of tile i overlaps the
// main loop of tile i + 1. Every mbarrier wait is bounded: when a wait runs out the role records a code in
// the caller's status word, raises a CTA-wide abort flag and all roles fall through to the common exit,
// where TMEM is released.
//
// Operand tiles in shared memory use the 128-byte swizzle that both TMA and the MMA descriptors understand:
//   K-major operand  (rows = M or N index, 64 contiguous K elements per row): box {64, 128 rows}
//       descriptor: SBO = 1024 B between 8-row groups; K step of 16 elements = +32 B on the start address
//   MN-major operand (rows = K index, 64 contiguous M/N elements per row):    box {64, 64 rows} per 64 columns
//       descriptor: LBO = 8192 B between 64-column blocks, SBO = 1024 B between 8-row K groups;
//       K step of 16 rows = +2048 B on the start address
#include "ffm_common.cuh"

namespace ffm {

namespace {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int STAGES = 4;
constexpr int A_STAGE_BYTES = BM * BK * 2;  // 16 KiB
constexpr int B_STAGE_BYTES = BN * BK * 2;  // 32 KiB
constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
constexpr int NUM_ACC = 2;
constexpr int TMEM_COLS = 512;
constexpr int GEMM_THREADS = 192;
constexpr int MAX_GROUPS = 256;
constexpr int SMEM_CTRL_BYTES = 2048;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + SMEM_CTRL_BYTES + 1024;  // + slack for 1 KiB alignment

enum { EPI_PLAIN = 0, EPI_GLU = 1 };

struct GemmParams {
  const int32_t* tile_start;  // [groups + 1] cumulative 128-row tiles, or null (dense)
  int groups;
  int dense_m_tiles;
  long long m_rows;        // store bound on output rows (grouped-M / dense)
  int n_cols;              // output columns per group (GLU: H)
  int k_blocks;            // K / 64 (grouped-M / dense)
  long long b_group_rows;  // rows of the B tensor map per group
  int b1_row_offset;       // row offset of the second 128-row half of a K-major B tile
  bf16* C;
  long long ldc;
  long long c_group_stride;  // grouped-K: elements between consecutive groups of C
  bf16* C2;                  // GLU: pre-activations [rows, 2H] or null
  long long ldc2;
  int glu_h;
  float scale;
  int act;
  int m_tiles_per_group;  // grouped-K
  int n_tiles;            // number of BN (GLU: 128-column) blocks over n_cols
  int32_t* status;
  long long wait_cycles;
};

struct Ctrl {
  unsigned long long full_bar[STAGES];
  unsigned long long empty_bar[STAGES];
  unsigned long long acc_full_bar[NUM_ACC];
  unsigned long long acc_empty_bar[NUM_ACC];
  uint32_t tmem_base;
  int abort_flag;
  int tile_start[MAX_GROUPS + 1];
};
static_assert(sizeof(Ctrl) <= SMEM_CTRL_BYTES, "control block too large");

struct TileCoord {
  int group;
  int m_tile;    // grouped-M: global 128-row tile; grouped-K: 128-row tile of M within the group
  int n_block;   // BN-column block (GLU: 128-column block of H)
  int k_row0;    // grouped-K: first K row; else 0
  int k_blocks;  // 64-deep K blocks to accumulate
};

// Walks this CTA's tiles in launch order. Grouped-M order is expert-major, then N block, then M tile
// (M fastest), so CTAs running side by side share one weight tile through L2.
template <int GROUPK>
struct TileWalker {
  const int* ts;
  int groups, n_tiles, m_tiles_per_group, k_blocks;
  long long total;
  long long cur;
  int g;  // cursor for grouped-M

  __device__ TileWalker(const GemmParams& p, const int* ts_smem) {
    ts = ts_smem;
    groups = p.groups;
    n_tiles = p.n_tiles;
    m_tiles_per_group = p.m_tiles_per_group;
    k_blocks = p.k_blocks;
    if (GROUPK) {
      total = static_cast<long long>(groups) * m_tiles_per_group * n_tiles;
    } else {
      total = static_cast<long long>(ts[groups]) * n_tiles;
    }
    cur = blockIdx.x;
    g = 0;
  }

  __device__ bool next(TileCoord& t) {
    if (cur >= total) return false;
    if (GROUPK) {
      const int per_group = m_tiles_per_group * n_tiles;
      t.group = static_cast<int>(cur / per_group);
      const int r = static_cast<int>(cur % per_group);
      t.m_tile = r % m_tiles_per_group;
      t.n_block = r / m_tiles_per_group;
      t.k_row0 = ts[t.group] * BM;
      t.k_blocks = (ts[t.group + 1] - ts[t.group]) * (BM / BK);
    } else {
      while (g < groups - 1 && cur >= static_cast<long long>(ts[g + 1]) * n_tiles) ++g;
      const int cnt = ts[g + 1] - ts[g];
      const int r = static_cast<int>(cur - static_cast<long long>(ts[g]) * n_tiles);
      t.group = g;
      t.n_block = r / cnt;
      t.m_tile = ts[g] + r % cnt;
      t.k_row0 = 0;
      t.k_blocks = k_blocks;
    }
    cur += gridDim.x;
    return true;
  }
};

template <int A_MN, int B_MN, int EPI, int GROUPK>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
ffm_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB0,
                const __grid_constant__ CUtensorMap tmB1, const GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t pad = (1024u - (raw_addr & 1023u)) & 1023u;
  uint8_t* smem = smem_raw + pad;
  const uint32_t smem_base = raw_addr + pad;
  Ctrl* ctrl = reinterpret_cast<Ctrl*>(smem + STAGES * STAGE_BYTES);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  // ---- set-up ------------------------------------------------------------------------------
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(&ctrl->full_bar[s]), 1);
      mbar_init(smem_u32(&ctrl->empty_bar[s]), 1);
    }
    for (int a = 0; a < NUM_ACC; ++a) {
      mbar_init(smem_u32(&ctrl->acc_full_bar[a]), 1);
      mbar_init(smem_u32(&ctrl->acc_empty_bar[a]), 4);  // one arrival per epilogue warp
    }
    ctrl->abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB0);
    tma_prefetch_desc(&tmB1);
  }
  if (p.tile_start != nullptr) {
    for (int i = threadIdx.x; i <= p.groups; i += GEMM_THREADS) ctrl->tile_start[i] = p.tile_start[i];
  } else if (threadIdx.x == 0) {
    ctrl->tile_start[0] = 0;
    ctrl->tile_start[1] = p.dense_m_tiles;
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&ctrl->tmem_base), TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();

  const uint32_t tmem_base = ctrl->tmem_base;
  volatile int* abort_flag = &ctrl->abort_flag;

  // ---- roles -------------------------------------------------------------------------------
  if (warp == 0) {
    // ================= TMA producer =================
    if (lane == 0) {
      TileWalker<GROUPK> walker(p, ctrl->tile_start);
      TileCoord t;
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      while (ok && walker.next(t)) {
        const int m0 = t.m_tile * BM;
        for (int kb = 0; kb < t.k_blocks && ok; ++kb) {
          ok = mbar_wait_bounded(smem_u32(&ctrl->empty_bar[stage]), phase ^ 1u, abort_flag, p.status,
                                 FFM_STATUS_WAIT_PRODUCER, p.wait_cycles);
          if (!ok) break;
          const uint32_t full = smem_u32(&ctrl->full_bar[stage]);
          const uint32_t a_dst = smem_base + stage * STAGE_BYTES;
          const uint32_t b_dst = a_dst + A_STAGE_BYTES;
          mbar_expect_tx(full, STAGE_BYTES);
          const int k0 = kb * BK;
          // A tile
          if (A_MN) {
            const int krow = t.k_row0 + k0;
            tma_load_2d(a_dst, &tmA, full, m0, krow);
            tma_load_2d(a_dst + 8192, &tmA, full, m0 + 64, krow);
          } else {
            tma_load_2d(a_dst, &tmA, full, k0, m0);
          }
          // B tile
          if (B_MN) {
            const int krow = GROUPK ? (t.k_row0 + k0) : static_cast<int>(t.group * p.b_group_rows + k0);
            const int n0 = t.n_block * BN;
#pragma unroll
            for (int j = 0; j < 4; ++j) tma_load_2d(b_dst + j * 8192, &tmB0, full, n0 + 64 * j, krow);
          } else {
            const int nrow = static_cast<int>(t.group * p.b_group_rows) + t.n_block * (EPI == EPI_GLU ? 128 : BN);
            tma_load_2d(b_dst, &tmB0, full, k0, nrow);
            tma_load_2d(b_dst + 16384, &tmB1, full, k0, nrow + p.b1_row_offset);
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ================= MMA issuer =================
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(BM, BN, A_MN, B_MN);
      TileWalker<GROUPK> walker(p, ctrl->tile_start);
      TileCoord t;
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      while (ok && walker.next(t)) {
        if (t.k_blocks == 0) continue;  // empty group: the epilogue writes zeros without an accumulator
        ok = mbar_wait_bounded(smem_u32(&ctrl->acc_empty_bar[acc]), acc_phase ^ 1u, abort_flag, p.status,
                               FFM_STATUS_WAIT_MMA, p.wait_cycles);
        if (!ok) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < t.k_blocks; ++kb) {
          ok = mbar_wait_bounded(smem_u32(&ctrl->full_bar[stage]), phase, abort_flag, p.status,
                                 FFM_STATUS_WAIT_MMA, p.wait_cycles);
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
            umma_bf16(d_tmem, adesc, bdesc, idesc, (kb > 0 || kk > 0) ? 1u : 0u);
          }
          umma_commit(smem_u32(&ctrl->empty_bar[stage]));  // frees the stage once these MMAs retire
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        umma_commit(smem_u32(&ctrl->acc_full_bar[acc]));
        if (++acc == NUM_ACC) {
          acc = 0;
          acc_phase ^= 1u;
        }
      }
    }
  } else {
    // ================= epilogue (warps 2..5) =================
    const int quarter = warp & 3;  // TMEM lanes [32 * quarter, 32 * quarter + 32) belong to this warp
    const int row_in_tile = quarter * 32 + lane;
    TileWalker<GROUPK> walker(p, ctrl->tile_start);
    TileCoord t;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    while (ok && walker.next(t)) {
      const long long row = static_cast<long long>(t.m_tile) * BM + row_in_tile;
      if (t.k_blocks == 0) {
        // grouped-K with an empty group: the gradient tile is zero
        if (GROUPK && row < p.m_rows) {
          bf16* crow = p.C + t.group * p.c_group_stride + row * p.ldc;
          const int n0 = t.n_block * BN;
          for (int c = 0; c < BN / 8; ++c) {
            const int col = n0 + c * 8;
            if (col < p.n_cols) *reinterpret_cast<uint4*>(crow + col) = make_uint4(0, 0, 0, 0);
          }
        }
        continue;
      }
      ok = mbar_wait_bounded(smem_u32(&ctrl->acc_full_bar[acc]), acc_phase, abort_flag, p.status,
                             FFM_STATUS_WAIT_EPILOGUE, p.wait_cycles);
      ok = __all_sync(0xffffffffu, ok ? 1 : 0) != 0;
      if (!ok) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * BN;

      if (EPI == EPI_GLU) {
        const int h0 = t.n_block * 128;
        const bool row_ok = row < p.m_rows;
        bf16* act_row = p.C + row * p.ldc + h0;
        bf16* pre_row = p.C2 ? (p.C2 + row * p.ldc2 + h0) : nullptr;
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          if (h0 + c * 32 >= p.n_cols) break;
          uint32_t g[32], u[32];
          tmem_ld_32x32(taddr + c * 32, g);
          tmem_ld_32x32(taddr + 128 + c * 32, u);
          tmem_ld_wait();
          uint32_t pg[16], pu[16], pa[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            pg[i] = pack_bf16x2(__uint_as_float(g[2 * i]), __uint_as_float(g[2 * i + 1]));
            pu[i] = pack_bf16x2(__uint_as_float(u[2 * i]), __uint_as_float(u[2 * i + 1]));
            const float2 gf = unpack_bf16x2(pg[i]);
            const float2 uf = unpack_bf16x2(pu[i]);
            pa[i] = pack_bf16x2(glu_fwd(p.act, gf.x, uf.x), glu_fwd(p.act, gf.y, uf.y));
          }
          if (row_ok) {
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              *reinterpret_cast<uint4*>(act_row + c * 32 + v * 8) =
                  make_uint4(pa[4 * v], pa[4 * v + 1], pa[4 * v + 2], pa[4 * v + 3]);
            }
            if (pre_row != nullptr) {
#pragma unroll
              for (int v = 0; v < 4; ++v) {
                *reinterpret_cast<uint4*>(pre_row + c * 32 + v * 8) =
                    make_uint4(pg[4 * v], pg[4 * v + 1], pg[4 * v + 2], pg[4 * v + 3]);
                *reinterpret_cast<uint4*>(pre_row + p.glu_h + c * 32 + v * 8) =
                    make_uint4(pu[4 * v], pu[4 * v + 1], pu[4 * v + 2], pu[4 * v + 3]);
              }
            }
          }
        }
      } else {
        const int n0 = t.n_block * BN;
        bf16* crow = p.C + (GROUPK ? t.group * p.c_group_stride : 0LL) + row * p.ldc + n0;
        const bool row_ok = row < p.m_rows;
        const float scale = p.scale;
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          if (n0 + c * 32 >= p.n_cols) break;
          uint32_t v[32];
          tmem_ld_32x32(taddr + c * 32, v);
          tmem_ld_wait();
          if (row_ok) {
            uint32_t o[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              o[i] = pack_bf16x2(__uint_as_float(v[2 * i]) * scale, __uint_as_float(v[2 * i + 1]) * scale);
            }
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              *reinterpret_cast<uint4*>(crow + c * 32 + q * 8) = make_uint4(o[4 * q], o[4 * q + 1], o[4 * q + 2], o[4 * q + 3]);
            }
          }
        }
      }
      // hand the accumulator back to the MMA issuer
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&ctrl->acc_empty_bar[acc]));
      if (++acc == NUM_ACC) {
        acc = 0;
        acc_phase ^= 1u;
      }
    }
  }

  // ---- common exit: every role reaches this point, also after an abort ----------------------
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
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

// 2-D bf16 tensor map over a row-major [rows, cols] matrix, 128-byte swizzle, zero fill out of bounds.
int make_map_2d(CUtensorMap* map, const void* base, long long rows, long long cols, int box_cols, int box_rows) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) return FFM_ERR_NO_DRIVER;
  if (rows <= 0 || cols <= 0) return FFM_ERR_BAD_ARG;
  if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0 || (cols * 2) % 16 != 0) return FFM_ERR_UNSUPPORTED;
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(cols) * 2};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(box_cols), static_cast<cuuint32_t>(box_rows)};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
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

template <int A_MN, int B_MN, int EPI, int GROUPK>
int launch_gemm(const CUtensorMap& tmA, const CUtensorMap& tmB0, const CUtensorMap& tmB1, const GemmParams& p,
                long long max_tiles, cudaStream_t stream) {
  static bool configured = false;
  auto kernel = ffm_gemm_kernel<A_MN, B_MN, EPI, GROUPK>;
  if (!configured) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess) {
      cudaGetLastError();
      return FFM_ERR_LAUNCH;
    }
    configured = true;
  }
  if (max_tiles <= 0) return FFM_OK;
  const int grid = static_cast<int>(max_tiles < num_sms() ? max_tiles : num_sms());
  kernel<<<grid, GEMM_THREADS, SMEM_BYTES, stream>>>(tmA, tmB0, tmB1, p);
  return cudaGetLastError() == cudaSuccess ? FFM_OK : FFM_ERR_LAUNCH;
}

}  // namespace

}  // namespace ffm

using namespace ffm;

extern "C" long long ffm_set_wait_cycles(long long cycles) {
  long long old = g_wait_cycles;
  if (cycles > 0) g_wait_cycles = cycles;
  return old;
}

extern "C" int ffm_grouped_gemm_glu(const void* A, const void* w_gate, const void* w_up, int64_t group_rows,
                                    int groups, const int32_t* tile_start, int64_t rows, int K, int H,
                                    int activation, void* act, void* preact, int32_t* status,
                                    ffm_stream_t stream) {
  if (!A || !w_gate || !w_up || !act || !status) return FFM_ERR_BAD_ARG;
  if (groups < 1 || groups > MAX_GROUPS || rows < 0 || K <= 0 || H <= 0 || group_rows < H) return FFM_ERR_BAD_ARG;
  if (activation < 0 || activation > 3) return FFM_ERR_BAD_ARG;
  if (tile_start == nullptr && groups != 1) return FFM_ERR_BAD_ARG;
  if (K % 64 != 0 || H % 32 != 0) return FFM_ERR_UNSUPPORTED;
  if (rows == 0) return FFM_OK;
  CUtensorMap tmA, tmB0, tmB1;
  int rc;
  if ((rc = make_map_2d(&tmA, A, rows, K, 64, 128)) != FFM_OK) return rc;
  const long long wrows = static_cast<long long>(groups - 1) * group_rows + H;
  if ((rc = make_map_2d(&tmB0, w_gate, wrows, K, 64, 128)) != FFM_OK) return rc;
  if ((rc = make_map_2d(&tmB1, w_up, wrows, K, 64, 128)) != FFM_OK) return rc;
  GemmParams p = {};
  p.tile_start = tile_start;
  p.groups = groups;
  p.dense_m_tiles = static_cast<int>((rows + BM - 1) / BM);
  p.m_rows = rows;
  p.n_cols = H;
  p.k_blocks = K / BK;
  p.b_group_rows = group_rows;
  p.b1_row_offset = 0;
  p.C = static_cast<bf16*>(act);
  p.ldc = H;
  p.C2 = static_cast<bf16*>(preact);
  p.ldc2 = 2LL * H;
  p.glu_h = H;
  p.scale = 1.0f;
  p.act = activation;
  p.n_tiles = (H + 127) / 128;
  p.status = status;
  p.wait_cycles = g_wait_cycles;
  const long long max_tiles = ((rows + BM - 1) / BM) * p.n_tiles;
  return launch_gemm<0, 0, EPI_GLU, 0>(tmA, tmB0, tmB1, p, max_tiles, static_cast<cudaStream_t>(stream));
}

extern "C" int ffm_grouped_gemm(const void* A, const void* B, int b_major, int groups, const int32_t* tile_start,
                                int64_t rows, int K, int Nout, float scale, void* out, int32_t* status,
                                ffm_stream_t stream) {
  if (!A || !B || !out || !status) return FFM_ERR_BAD_ARG;
  if (groups < 1 || groups > MAX_GROUPS || rows < 0 || K <= 0 || Nout <= 0) return FFM_ERR_BAD_ARG;
  if (b_major != FFM_B_KMAJOR && b_major != FFM_B_NMAJOR) return FFM_ERR_BAD_ARG;
  if (tile_start == nullptr && groups != 1) return FFM_ERR_BAD_ARG;
  if (K % 64 != 0 || Nout % 32 != 0) return FFM_ERR_UNSUPPORTED;
  if (b_major == FFM_B_NMAJOR && Nout % 64 != 0) return FFM_ERR_UNSUPPORTED;
  if (rows == 0) return FFM_OK;
  CUtensorMap tmA, tmB;
  int rc;
  if ((rc = make_map_2d(&tmA, A, rows, K, 64, 128)) != FFM_OK) return rc;
  GemmParams p = {};
  p.tile_start = tile_start;
  p.groups = groups;
  p.dense_m_tiles = static_cast<int>((rows + BM - 1) / BM);
  p.m_rows = rows;
  p.n_cols = Nout;
  p.k_blocks = K / BK;
  p.C = static_cast<bf16*>(out);
  p.ldc = Nout;
  p.scale = scale;
  p.n_tiles = (Nout + BN - 1) / BN;
  p.status = status;
  p.wait_cycles = g_wait_cycles;
  const long long max_tiles = ((rows + BM - 1) / BM) * p.n_tiles;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (b_major == FFM_B_KMAJOR) {
    if ((rc = make_map_2d(&tmB, B, static_cast<long long>(groups) * Nout, K, 64, 128)) != FFM_OK) return rc;
    p.b_group_rows = Nout;
    p.b1_row_offset = 128;
    return launch_gemm<0, 0, EPI_PLAIN, 0>(tmA, tmB, tmB, p, max_tiles, s);
  }
  if ((rc = make_map_2d(&tmB, B, static_cast<long long>(groups) * K, Nout, 64, 64)) != FFM_OK) return rc;
  p.b_group_rows = K;
  return launch_gemm<0, 1, EPI_PLAIN, 0>(tmA, tmB, tmB, p, max_tiles, s);
}

extern "C" int ffm_grouped_gemm_wgrad(const void* A, const void* B, int groups, const int32_t* tile_start,
                                      int64_t rows_cap, int M, int Nout, float scale, void* dW, int32_t* status,
                                      ffm_stream_t stream) {
  if (!A || !B || !dW || !status || !tile_start) return FFM_ERR_BAD_ARG;
  if (groups < 1 || groups > MAX_GROUPS || rows_cap <= 0 || M <= 0 || Nout <= 0) return FFM_ERR_BAD_ARG;
  if (M % 64 != 0 || Nout % 64 != 0) return FFM_ERR_UNSUPPORTED;
  CUtensorMap tmA, tmB;
  int rc;
  if ((rc = make_map_2d(&tmA, A, rows_cap, M, 64, 64)) != FFM_OK) return rc;
  if ((rc = make_map_2d(&tmB, B, rows_cap, Nout, 64, 64)) != FFM_OK) return rc;
  GemmParams p = {};
  p.tile_start = tile_start;
  p.groups = groups;
  p.m_rows = M;
  p.n_cols = Nout;
  p.C = static_cast<bf16*>(dW);
  p.ldc = Nout;
  p.c_group_stride = static_cast<long long>(M) * Nout;
  p.scale = scale;
  p.m_tiles_per_group = (M + BM - 1) / BM;
  p.n_tiles = (Nout + BN - 1) / BN;
  p.status = status;
  p.wait_cycles = g_wait_cycles;
  const long long max_tiles = static_cast<long long>(groups) * p.m_tiles_per_group * p.n_tiles;
  return launch_gemm<1, 1, EPI_PLAIN, 1>(tmA, tmB, tmB, p, max_tiles, static_cast<cudaStream_t>(stream));
}
