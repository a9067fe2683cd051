/*
 * libffmoe — C ABI of the sm_100a fused Mixture-of-Experts layer.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream; none of them allocates,
 * synchronises or throws. They enqueue work on `stream` and return FFM_OK or a negative FFM_ERR_* code
 * (argument validation and launch errors). Failures that can only be seen on the device (a bounded wait
 * that ran out) are written to the caller's `status` word, which must be zero-initialised device memory;
 * the first failure wins and later kernels keep running on whatever data is there.
 *
 * The reference project (FlashFusedMoE, Python + Triton + torch.bmm) has no C boundary of its own; each
 * declaration below cites the reference Python/Triton routine whose work it takes over.
 *
 * Data layout shared by all entry points
 * --------------------------------------
 *   N tokens, D model width, H = ffn_dim / 2, E experts (E_local with expert parallelism), k = top_k,
 *   T = N * k routed rows. All activations and weights are bf16, row-major, contiguous.
 *   "Grouped rows": routed rows sorted by expert, stable in (token, slot) order, each expert's segment
 *   starting on a multiple of 256 rows (the height of the two-CTA MMA tile). Rows between the end of an
 *   expert's tokens and the next multiple of 256 are zero. Buffers hold ffm_rows_capacity(T, E) rows.
 *     tile_start[E + 1]  int32  cumulative count of 128-row tiles per expert, always even
 *                               (tile_start[E] = tiles in use)
 *     pos[T]             int32  grouped row of flat slot i = n * k + j          (reference: expand_to_batch)
 *     src[rows_cap]      int32  flat slot held by a grouped row, -1 for padding (reference: sorted_order)
 */
#ifndef FFMOE_H_
#define FFMOE_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FFM_VERSION 100

/* Return codes */
#define FFM_OK 0
#define FFM_ERR_BAD_ARG (-1)      /* null pointer, negative size, unknown enum */
#define FFM_ERR_UNSUPPORTED (-2)  /* shape outside what the kernels handle (see each function) */
#define FFM_ERR_LAUNCH (-3)       /* cudaGetLastError() after a launch, or a driver call failed */
#define FFM_ERR_WORKSPACE (-4)    /* workspace too small */
#define FFM_ERR_NO_DRIVER (-5)    /* cuTensorMapEncodeTiled could not be resolved */
#define FFM_ERR_STATIC_LIMIT (-6) /* problem larger than the built-in scratch of ffm_group_rows_static */

/* Device-side status codes written into *status (0 = fine) */
#define FFM_STATUS_WAIT_PRODUCER 101 /* TMA producer gave up waiting for a free stage */
#define FFM_STATUS_WAIT_MMA 102      /* MMA issuer gave up waiting for operands or a free accumulator */
#define FFM_STATUS_WAIT_EPILOGUE 103 /* epilogue gave up waiting for an accumulator */
#define FFM_STATUS_BAD_INDEX 104     /* an expert index or row position was out of range */
#define FFM_STATUS_WAIT_PEER 105     /* a peer GPU's flag did not arrive within the wait budget */
#define FFM_STATUS_EP_OVERFLOW 106   /* a rank would receive more rows than its declared bound: the call moved nothing */

/* Gating */
#define FFM_GATING_SOFTMAX 0
#define FFM_GATING_SIGMOID 1

/* GLU activations (gate = first H rows of w_up, up = last H rows) */
#define FFM_ACT_SWIGLU 0
#define FFM_ACT_GEGLU_TANH 1
#define FFM_ACT_RELU2 2
#define FFM_ACT_GEGLU_ERF 3

/* Operand majorness for ffm_grouped_gemm */
#define FFM_B_KMAJOR 0  /* B stored [groups * n, k]: out = A * B^T   (forward projections) */
#define FFM_B_NMAJOR 1  /* B stored [groups * k, n]: out = A * B     (input-gradient GEMMs) */

typedef void* ffm_stream_t; /* cudaStream_t */

int ffm_version(void);
const char* ffm_error_string(int code);

/* Rows a grouped buffer must hold for T routed rows over E experts: 256 * floor((T + 255 E) / 256). */
int64_t ffm_rows_capacity(int64_t T, int E);

/* Set the cycle budget of every bounded device-side wait (default 2e9, about one second). Returns the old value. */
long long ffm_set_wait_cycles(long long cycles);

/* Choose the GEMM tile shape: 1 (default) = 256 x 256 tiles on pairs of CTAs (tcgen05.mma.cta_group::2),
 * 0 = 128 x 256 tiles on single CTAs. Results are identical; the environment variable FFM_GEMM_CTA_PAIR=0
 * selects 0 at first use. Any other argument only queries. Returns the previous setting. */
int ffm_set_gemm_cta_pair(int enable);

/* -------------------------------------------------------------------------------------------------
 * Routing forward: gate GEMM + scoring + top-k + renormalisation + loss statistics + grouped-row map.
 * Replaces fused_moe.py:327-348 (gate matmul, _apply_routing, argsort/bincount/cumsum),
 * kernels/fused_topk.py:31-136 (iterative-argmax top-k, lowest index wins ties, descending order) and the
 * loss block fused_moe.py:1160-1194.
 *
 * Logits are accumulated in fp32, rounded to bf16 and re-widened before selection, as the reference's
 * bf16 GEMM output is. Selection uses logit (+ expert_bias) for softmax gating and sigmoid(logit)
 * (+ expert_bias) for sigmoid gating; weights always come from the unbiased values and are multiplied by
 * weight_scale (scoring_factor / top_k, or 1).
 * pre_softmax != 0 (softmax gating): scores are the softmax probabilities over all experts, selection on
 * probability (+ bias), weights = p / (sum p + 1e-6)                          (fused_moe.py:146-162).
 * n_group > 0: group-limited selection (fused_moe.py:203-251): experts form n_group contiguous groups, a group's
 * score is the sum of its top (top_k / topk_group) selection values (its maximum if that count is 1 or exceeds
 * the group size), the topk_group best groups stay eligible. Limits: n_group <= 32, E % n_group == 0.
 *
 *   hidden [N, D] bf16, gate_w [E, D] bf16, expert_bias [E] f32 or NULL
 *   logits [N, E] bf16 out (may be NULL), topk_w [N, k] f32 out, topk_idx [N, k] int32 out, lse [N] f32 out
 *   counts [E] int32 out, tile_start [E + 1] int32 out, pos [T] int32 out, src [rows_cap] int32 out
 *   stats [E + 2] f32 out: stats[e] = sum of routing probability mass of expert e (softmax: selected
 *     weights; sigmoid: all scores), stats[E] = sum_n lse[n]^2, stats[E + 1] = sum_e counts[e] * stats[e]
 *   workspace: ffm_route_workspace_bytes(N, E, k) bytes
 * Limits: D % 8 == 0, 1 <= k <= min(E, 32), E <= 256.
 * ------------------------------------------------------------------------------------------------- */
size_t ffm_route_workspace_bytes(int64_t N, int E, int top_k);
int ffm_route_forward(const void* hidden, const void* gate_w, const float* expert_bias, int64_t N, int D, int E,
                      int top_k, int gating, float weight_scale, int pre_softmax, int n_group, int topk_group,
                      void* logits, float* topk_w, int32_t* topk_idx,
                      float* lse, int32_t* counts, int32_t* tile_start, int32_t* pos, int32_t* src,
                      int64_t rows_cap, float* stats, void* workspace, size_t workspace_bytes, int32_t* status,
                      ffm_stream_t stream);

/* Expert capacity with token dropping (fused_moe.py:351-390): a slot whose rank inside its expert is >= capacity
 * is dropped: its weight becomes 0, its grouped row a padding row (src = -1), and each token's kept weights are
 * renormalised by their sum (left at zero when nothing is kept). Call after ffm_route_forward, before
 * ffm_permute_rows. dropped_count [1] int32 out: number of dropped slots. */
int ffm_route_apply_capacity(float* topk_w, const int32_t* topk_idx, const int32_t* pos, int32_t* src,
                             const int32_t* tile_start, int64_t N, int top_k, int E, int capacity,
                             int32_t* dropped_count, ffm_stream_t stream);

/* Grouped-row map from given expert ids (no gate GEMM): used on the receiving side of expert parallelism,
 * where rows arrive already tagged with a local expert id. Replaces fused_moe.py:704-707.
 *   expert_ids [T] int32 in; outputs as in ffm_route_forward. */
int ffm_group_rows(const int32_t* expert_ids, int64_t T, int E, int32_t* counts, int32_t* tile_start, int32_t* pos,
                   int32_t* src, int64_t rows_cap, void* workspace, size_t workspace_bytes, int32_t* status,
                   ffm_stream_t stream);

/* Allocation-free variant of ffm_group_rows. It has no counterpart in the reference; it exists for callers
 * that cannot hand over a workspace because they are not allowed to allocate device memory at the point of the
 * call: code running inside a memory-pool-managed region that forbids cudaMalloc (for example a serving loop
 * whose allocator is frozen after start-up), or a host language binding that owns no device allocator at all
 * and only passes through pointers it was given. The histogram / offset scratch that ffm_group_rows takes
 * from the caller lives here in a fixed array inside the library image (FFM_STATIC_SCRATCH_BYTES per GPU,
 * held from library load until process exit). Inputs and outputs are still the caller's buffers.
 *
 * Limits: E <= FFM_STATIC_MAX_EXPERTS and T <= FFM_STATIC_MAX_ROWS, otherwise FFM_ERR_STATIC_LIMIT is
 * returned and nothing is launched. The call performs no cudaMalloc / cudaFree and calls no allocating
 * library routine. The first call on each device looks up the device address of the built-in array (a
 * one-time, per-device query made with that device current); make that first call outside any CUDA stream
 * capture. All calls on a device share the one array: two calls whose kernels can overlap on the GPU (different
 * streams without an ordering between them, or different host threads) race on it and corrupt each other's
 * result; calls ordered on one stream are safe. The array keeps whatever the last call left in it; each
 * call overwrites every word it later reads, so stale contents never leak into a result. */
#define FFM_STATIC_SCRATCH_BYTES 1310720 /* 1.25 MiB */
#define FFM_STATIC_MAX_EXPERTS 256
#define FFM_STATIC_MAX_ROWS 1048576
int ffm_group_rows_static(const int32_t* expert_ids, int64_t T, int E, int32_t* counts, int32_t* tile_start,
                          int32_t* pos, int32_t* src, int64_t rows_cap, int32_t* status, ffm_stream_t stream);

/* -------------------------------------------------------------------------------------------------
 * Permute: grouped[r, :] = x[src[r] / k, :] for src[r] >= 0; other rows are zeroed, or with zero_padding == 0 left
 * as they are (forward without gradients: nothing sums over padding rows).
 * Replaces fused_routing_scatter (kernels/moe_ops.py:53-149) without the padded [E, max_tokens, D] buffer.
 * Limits: D % 8 == 0.
 * ------------------------------------------------------------------------------------------------- */
int ffm_permute_rows(const void* x, const int32_t* src, int64_t rows_cap, int top_k, int D, int zero_padding,
                     void* grouped, ffm_stream_t stream);

/* -------------------------------------------------------------------------------------------------
 * Grouped GEMMs on tcgen05 / TMEM tiles fed by TMA (256 x 256 x 64 tiles on CTA pairs, fp32 accumulation,
 * outputs written with TMA stores).
 * tile_start == NULL selects the dense case: one group, `rows` rows of A (any value, masked at the edge).
 *
 * ffm_grouped_gemm_glu:  act[r, :] = glu(A[r, :] * Wg[e]^T, A[r, :] * Wu[e]^T), optional preact[r, 0:2H].
 *   Replaces torch.bmm up-projection + activation_forward (fused_moe.py:435-438,
 *   kernels/activations.py:28-74). Gate and up pre-activations are rounded to bf16 before the activation,
 *   as the reference's bf16 bmm output is. w_gate / w_up are [groups * group_rows, K] row-major with the
 *   group's gate rows starting at row e * group_rows of w_gate and its up rows at e * group_rows of w_up;
 *   for stacked expert weights pass w_gate = w_up_tensor, w_up = w_up_tensor + H * K, group_rows = 2H.
 *   Limits: K % 64 == 0, H % 64 == 0.
 *
 * ffm_grouped_gemm: out[r, 0:Nout] = scale * A[r, :] * op(B[e]).
 *   Replaces the down-projection bmm (fused_moe.py:441) and the input-gradient bmms (:547, :553).
 *   Limits: K % 64 == 0, Nout % 32 == 0 (b_major = FFM_B_NMAJOR also needs Nout % 64 == 0).
 *
 * ffm_grouped_gemm_wgrad: dW[e][m, n] = scale * sum over the rows r of expert e of A[r, m] * B[r, n].
 *   Replaces the weight-gradient bmms (fused_moe.py:564-565, :961-966). A is [rows_cap, M], B is
 *   [rows_cap, Nout], dW is [groups, M, Nout]. Padding rows must be finite in A and zero in A or B.
 *   Limits: M % 64 == 0, Nout % 64 == 0.
 * valid_rows / tile_rows (the two grouped-M entry points): valid_rows, when not NULL, is an int32 [groups] device array
 *   of the valid rows of every group; 128-row tiles beyond them are then not computed (their output rows stay
 *   unwritten). tile_rows picks the tile shape for this call: 256 = CTA pair, 128 = one CTA per tile, 0 = the
 *   library default (ffm_set_gemm_cta_pair). With few rows per group (decode) 128 with valid_rows halves the
 *   tensor-core work, which is then hidden behind the weight stream.
 * ------------------------------------------------------------------------------------------------- */
int ffm_grouped_gemm_glu(const void* A, const void* w_gate, const void* w_up, int64_t group_rows, int groups,
                         const int32_t* tile_start, int64_t rows, int K, int H, int activation, void* act,
                         void* preact, const int32_t* valid_rows, int tile_rows, int32_t* status,
                         ffm_stream_t stream);
int ffm_grouped_gemm(const void* A, const void* B, int b_major, int groups, const int32_t* tile_start,
                     int64_t rows, int K, int Nout, float scale, void* out, const int32_t* valid_rows,
                     int tile_rows, int32_t* status, ffm_stream_t stream);
int ffm_grouped_gemm_wgrad(const void* A, const void* B, int groups, const int32_t* tile_start, int64_t rows_cap,
                           int M, int Nout, float scale, void* dW, int32_t* status, ffm_stream_t stream);
/* dAct GEMM with the GLU backward fused into its epilogue: gU [rows, 2H] = GLU backward of (gY Wd (N-major B, as
 * ffm_grouped_gemm with FFM_B_NMAJOR) rounded to bf16, preact [rows, 2H]), bit-identical to ffm_grouped_gemm followed by
 * ffm_glu_backward (reference: the bmm + activation_backward pair, fused_moe.py:520-531); dAct is never written. The
 * epilogue warps pull the tile's pre-activations in by TMA, one 64-column step ahead, into the staging boxes that the
 * gradients are then written over and stored from.
 * gY [rows, K], Wd [groups, K, H], K % 64 == 0, H % 64 == 0. */
int ffm_grouped_gemm_dact_glu_backward(const void* gY, const void* Wd, int groups, const int32_t* tile_start,
                                       int64_t rows, int K, int H, int activation, const void* preact, void* gU,
                                       int tile_rows, int32_t* status, ffm_stream_t stream);
/* ffm_grouped_gemm_wgrad with a passenger: the same launch also computes gU = GLU backward of (dAct [glu_rows, H],
 * preact [glu_rows, 2H]) exactly as ffm_glu_backward does, on eight extra warps per CTA that stream through HBM while
 * the tensor pipe works on the weight gradient. The two jobs are independent (in the layer: dW_down needs the output
 * gradient and the activations, the GLU backward needs dAct); a GEMM CTA leaves no room on its SM for another
 * kernel's blocks, so this is how the HBM-bound job overlaps a GEMM. Results are bit-identical to the two calls.
 * Only rows below tile_start[groups] * 128 are converted (as ffm_glu_backward does when given tile_start): the row
 * buffers may be sized for a worst case far above the rows in use. */
int ffm_grouped_gemm_wgrad_glu_backward(const void* A, const void* B, int groups, const int32_t* tile_start,
                                        int64_t rows_cap, int M, int Nout, float scale, void* dW, const void* dAct,
                                        const void* preact, int64_t glu_rows, int H, int activation, void* gU,
                                        int32_t* status, ffm_stream_t stream);
/* -------------------------------------------------------------------------------------------------
 * Combine forward: out[n, :] = sum_j w[n, j] * Y[pos[n k + j], :] (+ addend[n, :]), fp32 accumulation.
 * w (f32) is rounded to bf16 before the multiply, as the reference does (fused_moe.py:412); w == NULL
 * means 1. Replaces fused_gather_reduce (kernels/moe_ops.py:166-241). Limits: D % 8 == 0, k <= 32.
 * ------------------------------------------------------------------------------------------------- */
int ffm_combine_forward(const void* Y, const int32_t* pos, const float* w, const void* addend, int64_t N,
                        int top_k, int D, void* out, ffm_stream_t stream);

/* -------------------------------------------------------------------------------------------------
 * Combine backward, one pass over the grouped rows:
 *   gw[i]     = <Y[r, :], go[n, :]>         (f32; routing-weight gradient, fused_moe.py:527-535)
 *   gYw[r, :] = go[n, :] * bf16(w[i])       (fused_weighted_scatter, kernels/moe_ops.py:258-332)
 * with i = src[r], n = i / k; padding rows of gYw are written as zero. Y may be NULL (gw not produced).
 * ------------------------------------------------------------------------------------------------- */
int ffm_combine_backward(const void* go, const void* Y, const float* w, const int32_t* src, int64_t rows_cap,
                         int top_k, int D, void* gYw, float* gw, ffm_stream_t stream);

/* -------------------------------------------------------------------------------------------------
 * GLU backward: gU[r, 0:H] = d gate, gU[r, H:2H] = d up from dAct[r, 0:H] and preact[r, 0:2H].
 * Replaces activation_backward (kernels/activations.py:78-231). tile_start/groups bound the rows in use
 * (NULL: all `rows`). Limits: H % 8 == 0.
 * ------------------------------------------------------------------------------------------------- */
int ffm_glu_backward(const void* dAct, const void* preact, const int32_t* tile_start, int groups, int64_t rows,
                     int H, int activation, void* gU, ffm_stream_t stream);

/* -------------------------------------------------------------------------------------------------
 * Routing backward (fused_moe.py:573-591, :915-932) plus the analytic gradients of the two losses.
 *   gl[n, :]  = bf16( scatter(softmax/sigmoid Jacobian applied to gw + aux term)
 *                     + gz * 2 lse[n] / N * softmax(logits[n, :])                 (z-loss, fused_moe.py:1193)
 *                     + sigmoid gating only: gaux_e * s (1 - s) / N )              (aux loss, :1186-1189)
 *   dH[n, :] += gl[n, :] * gate_w           (accumulate = 0 overwrites)
 *   dGate     = gl^T * hidden
 * gaux [E] f32 or NULL: d loss / d P_e (softmax gating: added to gw of every slot routed to e).
 * gz: device pointer to one f32 = d loss / d (sum_n lse^2 / N), i.e. z_loss_coeff * upstream gradient;
 *     NULL (or a stored 0) disables the term. A device scalar keeps the backward pass free of host syncs.
 * workspace: ffm_route_backward_workspace_bytes(N, D, E). status: the library's status word (with E % 64 == 0,
 * D % 64 == 0 and N >= 1024 the dGate product runs as a tensor-core GEMM over the tokens, whose waits report there).
 * ------------------------------------------------------------------------------------------------- */
size_t ffm_route_backward_workspace_bytes(int64_t N, int D, int E);
int ffm_route_backward(const float* gw, const float* topk_w, const int32_t* topk_idx, const void* logits,
                       const float* lse, const float* gaux, const float* gz, const void* hidden, const void* gate_w,
                       int64_t N, int D, int E, int top_k, int gating, int accumulate, void* dH, void* dGate,
                       void* workspace, size_t workspace_bytes, int32_t* status, ffm_stream_t stream);

/* -------------------------------------------------------------------------------------------------
 * ffm_compact_positions: cpos[i] = position of flat slot i in the grouped order without the 256-row padding (the
 *   order in which an expert-parallel rank sends its rows, expert-major), src_c = the inverse map (int32 [T]).
 *   Inputs are ffm_route_forward's pos, topk_idx, counts and tile_start. Replaces the stable sort by destination
 *   rank of the reference's dispatcher (expert_parallel.py:225-236). E <= 256.
 * ------------------------------------------------------------------------------------------------- */
int ffm_compact_positions(const int32_t* pos, const int32_t* topk_idx, const int32_t* counts,
                          const int32_t* tile_start, int64_t T, int E, int32_t* cpos, int32_t* src_c,
                          ffm_stream_t stream);

/* -------------------------------------------------------------------------------------------------
 * FP8 (e4m3) forward projections, opt-in. The reference has FP8 only for the dense nn.Linear layers of its training
 * benchmark (benchmarks/train_multigpu.py:283-336, torch._scaled_mm); this is the same idea for the routed experts'
 * up- and down-projection.
 * ffm_quantize_rows_e4m3: q[r, :] = e4m3(x[r, :] / scale[r]), scale[r] = max |x[r, :]| / 448 (1 for an all-zero row);
 *   x bf16 [rows, K], K % 16 == 0; q uint8 [rows, K]; scale f32 [rows]. Used for activations (a scale per row).
 * ffm_quantize_rows_given_scale_e4m3: the same conversion with the caller's scales, row r uses
 *   scale_in[r / rows_per_scale]: weights viewed as [groups * N, K] with one scale per group (per expert).
 * ffm_grouped_gemm_glu_fp8 / ffm_grouped_gemm_fp8: ffm_grouped_gemm_glu / ffm_grouped_gemm (K-major B) on quantised
 *   operands with tcgen05.mma.kind::f8f6f4, fp32 accumulation, out[r, n] = acc * a_scale[r] * b_scale[group];
 *   K % 128 == 0. Wq is [groups, 2H, K] (gate rows, then up rows), Bq is [groups, Nout, K], w_scale / b_scale f32
 *   [groups]. a_scale must hold an entry for every row up to the next multiple of 128.
 *   Outputs are bf16 as in the bf16 entry points.
 * ------------------------------------------------------------------------------------------------- */
int ffm_quantize_rows_e4m3(const void* x, int64_t rows, int K, void* q, float* scale, ffm_stream_t stream);
int ffm_quantize_rows_given_scale_e4m3(const void* x, int64_t rows, int K, int64_t rows_per_scale,
                                       const float* scale_in, void* q, ffm_stream_t stream);
int ffm_grouped_gemm_glu_fp8(const void* Aq, const float* a_scale, const void* Wq, const float* w_scale, int groups,
                             const int32_t* tile_start, int64_t rows, int K, int H, int activation, void* act,
                             void* preact, int tile_rows, int32_t* status, ffm_stream_t stream);
int ffm_grouped_gemm_fp8(const void* Aq, const float* a_scale, const void* Bq, const float* b_scale, int groups,
                         const int32_t* tile_start, int64_t rows, int K, int Nout, void* out, int tile_rows,
                         int32_t* status, ffm_stream_t stream);

/* -------------------------------------------------------------------------------------------------
 * Expert-parallel exchange over NVLink with plain peer stores. Replaces the c10d all_to_all_single calls of the
 * reference's dispatcher (expert_parallel.py:253-258, :290-292; fused_moe.py:901-910).
 * The caller owns the receive buffers and the flag arrays, which must be mapped on every GPU of the group
 * (CUDA IPC / virtual-memory handles; the Python package uses torch's symmetric memory for this).
 *
 * ffm_p2p_push: copy n_segments (<= FFM_P2P_MAX_PEERS) contiguous byte ranges src[i] -> dst[i], dst[i] usually in a
 *   peer's memory. Ranges and sizes must be multiples of 16 bytes; empty segments are skipped.
 * ffm_p2p_push_rows: the same at row granularity, for layouts that are not one contiguous range per peer. A table in
 *   device memory lists n_segments runs of rows: segments[i] = {first source row, first destination row, rows,
 *   index into dst_bases} (int64 x 4), seg_end[i] = rows of segments 0..i (int64, growing); total_rows = seg_end[last].
 *   Row r of run i goes from src + (first source row + r) * row_bytes to dst_bases[..] + (first destination row + r)
 *   * row_bytes. With src_index the source row is src_index[first source row + r] / index_div instead (a gather
 *   from the token matrix by flat slot); with src == NULL the destination rows are zeroed. row_bytes % 16 == 0.
 *   This is how rows travel straight between the sender's expert-sorted order and the receiver's 256-row-aligned
 *   grouped layout (and back), without a staging permute on either side.
 * ffm_p2p_push_rows_dev: ffm_p2p_push_rows with the row total read from device memory at run time (max_rows only
 *   sizes the grid) and tables that may contain empty runs, as ffm_p2p_plan writes them.
 * ffm_p2p_plan: builds on the device, from counts[s * E + e] = rows rank s routes to expert e (int32 [ep][E],
 *   E = ep * e_local <= 256, the same on every rank), the tables of one expert-parallel call for `rank`:
 *   dispatch int64 [E][4] + dispatch_end [E] (sender order -> the owners' grouped layouts), combine
 *   int64 [e_local * ep][4] + combine_end (this rank's grouped layout -> the origins' sender order), padding
 *   int64 [e_local][4] + padding_end (rows of its own layout to zero), tile_start int32 [e_local + 1] for the grouped
 *   GEMM, totals int64 [4] = {rows sent, rows received, padding rows, grouped rows}. With it a forward pass needs no
 *   host read of the counts and can be captured in a CUDA graph. max_grouped_rows (0 = no bound) is the size of every
 *   rank's receive buffer in rows: if ANY rank's grouped layout would exceed it, every rank (they all see the same
 *   counts) writes tables that move nothing (all run lengths, totals and tile_start zero) and sets
 *   FFM_STATUS_EP_OVERFLOW in *status, so no row is ever stored past a buffer.
 * ffm_p2p_signal_wait: all ranks call it with the same, growing epoch after their pushes: stores epoch into
 *   slot [my_rank] of every rank's flag array (release), then waits (bounded by wait_cycles, 0 = default) until its
 *   own array holds epoch in every slot (acquire). Kernels enqueued after it may read what the peers pushed.
 *   flag_arrays[r] points at rank r's array of `world` uint32 flags, zero-initialised once.
 * ffm_p2p_signal_wait_dev: the same with the epoch kept in device memory (*epoch_counter grows by one per call, and
 *   by the same amount on every rank), so that the call can sit in a CUDA graph that is replayed. Give it flag
 *   arrays of its own: the two kinds of barrier must not share flags.
 * ------------------------------------------------------------------------------------------------- */
#define FFM_P2P_MAX_PEERS 16
int ffm_p2p_push(int n_segments, const void* const* src, void* const* dst, const int64_t* bytes,
                 ffm_stream_t stream);
/* Measurement aid: buffer_index >= 0 makes ffm_p2p_push_rows(_dev) skip rows bound for any other destination buffer
 * (pass the caller's rank: local rows move, nothing crosses NVLink); -1 restores normal operation. Returns the old
 * value. The difference between a step timed this way and a normal one is the exposed exchange time. */
int ffm_p2p_set_local_only(int buffer_index);
int ffm_p2p_push_rows(const void* src, const int32_t* src_index, int index_div, int64_t row_bytes,
                      const int64_t* segments, const int64_t* seg_end, int n_segments, int64_t total_rows,
                      void* const* dst_bases, int n_bases, ffm_stream_t stream);
int ffm_p2p_push_rows_dev(const void* src, const int32_t* src_index, int index_div, int64_t row_bytes,
                          const int64_t* segments, const int64_t* seg_end, int n_segments,
                          const int64_t* total_rows_dev, int64_t max_rows, void* const* dst_bases, int n_bases,
                          ffm_stream_t stream);
int ffm_p2p_plan(const int32_t* counts, int ep, int e_local, int rank, int64_t* dispatch, int64_t* dispatch_end,
                 int64_t* combine, int64_t* combine_end, int64_t* padding, int64_t* padding_end, int32_t* tile_start,
                 int64_t* totals, int64_t max_grouped_rows, int32_t* status, ffm_stream_t stream);
int ffm_p2p_signal_wait_dev(void* const* flag_arrays, int my_rank, int world, uint32_t* epoch_counter,
                            int32_t* status, long long wait_cycles, ffm_stream_t stream);
int ffm_p2p_signal_wait(void* const* flag_arrays, int my_rank, int world, uint32_t epoch, int32_t* status,
                        long long wait_cycles, ffm_stream_t stream);

#ifdef __cplusplus
}
#endif

#endif /* FFMOE_H_ */
