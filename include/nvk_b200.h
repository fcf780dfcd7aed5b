/*
 * libnvk_b200 -- C ABI of the B200 (sm_100a) NVFP4 linear path.
 *
 * Drop-in boundary: every `nv_kernels_*` symbol below has the name, argument order, argument
 * meaning and return convention of the declaration it replaces in the reference project's
 * hand-written kernel header (rust/crates/nv-kernels/include/nv_kernels.h, cited per symbol),
 * which the reference binds with bindgen and re-exports 1:1 as `nv_kernels::cuda::<name>`.
 * `nvk_b200_*` symbols are additions with no counterpart there.
 *
 * Conventions (as in the reference):
 *   - `stream` is a cudaStream_t / CUstream passed as void*; every call only enqueues work on it,
 *     never synchronises and never allocates device memory.
 *   - bf16 tensors are uint16_t*, packed e2m1 (two values per byte, even k in the low nibble)
 *     and ue4m3 block scales are uint8_t*; all pointers are device pointers owned by the caller.
 *   - Weight matrices are row-major [N, K/2] bytes; their block scales use the 128x4 swizzled
 *     layout, ceil(N/128)*128 * ceil(K/64)*4 bytes: scale of (row n, block kb) sits at
 *       ((n/128 * ceil(K/64) + kb/4) * 32 + n%32) * 16 + ((n/32)%4) * 4 + kb%4.
 *   - Return value: 0 = enqueued (or an empty problem); -1 = shape/route refused, nothing
 *     launched; -2 = bad argument or alignment; -3 = resource limit; -9 = grid axis too large;
 *     a positive value is a cudaError_t.  Checks run in that order; a NULL operand that a launch
 *     would dereference is refused with -2 after the shape checks (the reference does not check
 *     for NULL; a call it would accept with valid pointers is accepted here unchanged).
 */
#pragma once
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* replaces rust/crates/nv-kernels/include/nv_kernels.h:11 */
int nv_kernels_capability(int* sm_major, int* sm_minor);

/* ---- W4A16 linear: y = bf16(alpha * x W^T), fp32 accumulate ---------------------------------- */

/* M = 1.  Refuses K % 16 != 0 with -1; N <= 0 or K <= 0 is a no-op returning 0.
 * replaces rust/crates/nv-kernels/include/nv_kernels.h:534-543
 * (kernel: rust/crates/nv-kernels/cuda/gemv_nvfp4.cu:224-312) */
int nv_kernels_nvfp4_gemv_bf16act(void* stream, const uint8_t* W_packed, const uint8_t* W_scales,
                                  const uint16_t* x_bf16, uint16_t* y, float alpha, int N, int K);

/* M = 1 with the activation row in NVFP4 as well (packed e2m1 + a FLAT [K/16] ue4m3 scale array, as
 * nv_kernels_nvfp4_quantize_row_bf16 writes it): y = bf16(alpha * sum_kb ws*xs * dot16(w, x)).  The
 * reference keeps this pair for tests and as the mirror of its WGSL kernel; its serving path does
 * not call it.  Refuses K % 16 != 0 with -1, packed pointers not 8-byte aligned with -2.
 * replaces rust/crates/nv-kernels/include/nv_kernels.h:545-555
 * (rust/crates/nv-kernels/cuda/gemv_nvfp4.cu:117-177,314-340) */
int nv_kernels_nvfp4_gemv_bf16(void* stream, const uint8_t* W_packed, const uint8_t* W_scales, const uint8_t* x_packed,
                               const uint8_t* x_scales, uint16_t* y, float alpha, int N, int K);

/* M = 1, two weight matrices sharing one x (gate + up); wq_b == sc_b == y_b == NULL runs one arm.
 * Refuses K % 32 != 0, N <= 0, K <= 0 or a half-null second arm with -1.
 * replaces rust/crates/nv-kernels/include/nv_kernels.h:584-597
 * (rust/crates/nv-kernels/cuda/gemv_nvfp4_w4a16_decode.cu:111-150,186-220) */
int nv_kernels_gemv_nvfp4_w4a16_dual_m1(void* stream, const uint8_t* wq_a, const uint8_t* sc_a,
                                        const uint8_t* wq_b, const uint8_t* sc_b, const uint16_t* x,
                                        uint16_t* y_a, uint16_t* y_b, float alpha_a, float alpha_b, int N,
                                        int K);

/* M = 1 down projection whose activation is bf16(SiLU(gate) * up), computed in fp32 and rounded
 * to bf16 before the contraction.
 * replaces rust/crates/nv-kernels/include/nv_kernels.h:615-625
 * (rust/crates/nv-kernels/cuda/gemv_nvfp4_w4a16_decode.cu:152-182,222-251) */
int nv_kernels_gemv_nvfp4_w4a16_silu_gate_up_in_m1(void* stream, const uint8_t* wq, const uint8_t* sc,
                                                   const uint16_t* gate, const uint16_t* up, uint16_t* y,
                                                   float alpha, int N, int K);

/* 1 <= M <= 16, x is [M, K], y is [M, N]; optional second arm.  Refuses M > 16, K % 32 != 0 and
 * N % 32 != 0 with -1, as the reference does.
 * replaces rust/crates/nv-kernels/include/nv_kernels.h:599-613
 * (rust/crates/nv-kernels/cuda/gemm_nvfp4_w4a16_mk_mma.cu:57-231,290-326) */
int nv_kernels_gemm_nvfp4_w4a16_mk_dual(void* stream, const uint8_t* wq_a, const uint8_t* sc_a,
                                        const uint8_t* wq_b, const uint8_t* sc_b, const uint16_t* x,
                                        uint16_t* y_a, uint16_t* y_b, float alpha_a, float alpha_b, int M, int N,
                                        int K);

/* No counterpart in the reference: the same contraction for 1 <= M <= 64, any N, K % 16 == 0,
 * optional second arm, optional SiLU prologue (x = gate, x2 = up; x2 == NULL for a plain x). */
int nvk_b200_linear_nvfp4_w4a16(void* stream, const uint8_t* wq_a, const uint8_t* sc_a, const uint8_t* wq_b,
                                const uint8_t* sc_b, const uint16_t* x, const uint16_t* x2, uint16_t* y_a,
                                uint16_t* y_b, float alpha_a, float alpha_b, int M, int N, int K);

/* No counterpart in the reference: the same linear with a caller-supplied workspace.  For M >= 3
 * the activations are converted once into the workspace (one small extra launch) and every CTA
 * streams them from there instead of converting its whole K range itself; results are bit-identical
 * to nvk_b200_linear_nvfp4_w4a16.  `workspace` is device memory, 16-byte aligned, at least
 * nvk_b200_linear_workspace_bytes(M, K) bytes, and must not be used by another call until this one
 * has completed on the GPU (calls on one stream may share it).  workspace == NULL falls back to
 * nvk_b200_linear_nvfp4_w4a16; a workspace that is too small or misaligned returns -2. */
size_t nvk_b200_linear_workspace_bytes(int M, int K);
int nvk_b200_linear_nvfp4_w4a16_ws(void* stream, const uint8_t* wq_a, const uint8_t* sc_a, const uint8_t* wq_b,
                                   const uint8_t* sc_b, const uint16_t* x, const uint16_t* x2, uint16_t* y_a,
                                   uint16_t* y_b, float alpha_a, float alpha_b, int M, int N, int K,
                                   void* workspace, size_t workspace_bytes);

/* No counterpart in the reference (its residual epilogues take int8 activations only): the W4A16 linear
 * as a residual update, y[m, n] = bf16(fma(sum_k W[n, k] a[m, k], alpha, residual[m, n])), one rounding,
 * with a = x or, when x2 is given, a = bf16(SiLU(x) * x2) -- a decoder MLP's tail or an attention output
 * projection in one launch.  y may alias residual.  1 <= M <= 64.  0 for an empty problem (N or K <= 0);
 * -1 for M outside [1, 64] or K % 32 != 0; -2 for a null operand (x2 excepted) or one not 16-byte
 * aligned; -9 when N needs more than 65535 row tiles. */
int nvk_b200_linear_nvfp4_w4a16_residual(void* stream, const uint8_t* wq, const uint8_t* sc, const uint16_t* x,
                                         const uint16_t* x2, const uint16_t* residual, uint16_t* y, float alpha, int M,
                                         int N, int K);

/* The same for one row (M = 1), also leaving 1/rms of the new row for the RMSNorm that follows:
 * rstd_pack[0] = rsqrt(mean(y^2) + eps) over the N rounded outputs.  rstd_pack: three floats in device
 * memory {rstd, running sum of squares, arrival count}; the last two zero before the first launch, and
 * returned to zero by every launch.  Partial sums meet through float atomics in arrival order: the last
 * bits of rstd may differ from run to run, as in the reference's int8 form
 * (rust/crates/nv-kernels/include/nv_kernels.h:652-678).  -2 for a null rstd_pack. */
int nvk_b200_linear_nvfp4_w4a16_residual_rstd_emit(void* stream, const uint8_t* wq, const uint8_t* sc,
                                                   const uint16_t* x, const uint16_t* x2, const uint16_t* residual,
                                                   uint16_t* y, float alpha, float* rstd_pack, float eps, int N, int K);

/* No counterpart in the reference with this signature (its fused norms feed the quantizing routes): the
 * W4A16 linear with an RMSNorm in front, y = bf16(alpha * sum_k W[n, k] a[m, k]) with
 * a[m, k] = bf16(x[m, k] * rstd[m] * norm_weight[k]), rstd[m] = rsqrt(mean_k x[m, k]^2 + eps), for one or
 * two matrices sharing x (wq_b, sc_b, y_b all null: one).  Bit-identical to nv_kernels_rmsnorm_bf16
 * followed by the plain linear.  rstd null: every CTA sums its rows' squares itself, M <= 8; rstd given
 * (one f32 per row, e.g. the first float of a rstd_pack): M <= 64.  0 for an empty problem; -1 for M
 * outside that range, K % 32 != 0 or a half-given second matrix; -2 for a null or not 16-byte aligned
 * operand. */
int nvk_b200_linear_nvfp4_w4a16_normed(void* stream, const uint8_t* wq_a, const uint8_t* sc_a, const uint8_t* wq_b,
                                       const uint8_t* sc_b, const uint16_t* x, const uint16_t* norm_weight,
                                       const float* rstd, float eps, uint16_t* y_a, uint16_t* y_b, float alpha_a,
                                       float alpha_b, int M, int N, int K);

/* No counterpart in the reference (it has no multi-GPU path): a row-parallel (K-sharded) W4A16 linear and
 * its all-reduce in one launch per GPU.  y [M, N] = bf16(sum over ranks of bf16(alpha * x_r W_r^T) (+ residual)),
 * the same bits on every rank and the same bits as the linear followed by nvk_b200_tp_allreduce_bf16.
 * Each CTA stores its partials into its own region of every GPU's inbox (plain peer stores), raises one
 * flag per GPU, waits -- bounded, nvk_b200_set_wait_limit -- for the CTA of the same index on every other
 * GPU and writes the sum in rank order.  wq / sc / x / x2: this rank's K slice (K = its length);
 * peer_bufs: `world` device pointers to the ranks' exchange buffers as mapped here, each
 * nvk_b200_tp_fused_buffer_bytes(world, max_ctas, max_rows) bytes of plain device memory, zero before the
 * first call; epoch: max_ctas uint32 of local device memory, zero before the first call; err: one int
 * that becomes 1 + r if rank r never arrived.  All ranks make the same sequence of calls with the same
 * M, N and K (the K slices have equal length): CTAs are paired across the ranks by their index.
 * 1 <= M <= max_rows <= 64.  0 for an empty problem; -1 for M outside that range or K % 32 != 0; -2 for
 * null / misaligned operands, a rank outside the world or a row capacity outside [1, 64]; -3 when the
 * launch needs more than max_ctas CTAs. */
int nvk_b200_tp_linear_nvfp4_w4a16_allreduce(void* stream, const void* const* peer_bufs, int rank, int world,
                                             const uint8_t* wq, const uint8_t* sc, const uint16_t* x, const uint16_t* x2,
                                             const uint16_t* residual, uint16_t* y, float alpha, int M, int N, int K,
                                             int max_ctas, int max_rows, uint32_t* epoch, int* err);
size_t nvk_b200_tp_fused_buffer_bytes(int world, int max_ctas, int max_rows);

/* No counterpart in the reference (it has no multi-GPU path): the expert-parallel MoE combine and the sum
 * over GPUs in one launch.  Every rank passes the rows of ITS experts' slots (inv_perm < 0, or zero rows,
 * for the others); y_acc [n_tokens, hidden] f32 receives the sum over ranks of the ranks' weighted
 * combines, added in rank order -- the same bits on every rank.  Each CTA stores its partials into its
 * own region of every GPU's inbox (plain peer stores), raises one flag per GPU and waits, bounded, for
 * the CTA of the same index on the other GPUs.  hidden % 8 == 0, rows 16-byte aligned.  peer_bufs:
 * `world` pointers to the ranks' exchange buffers (nvk_b200_moe_combine_buffer_bytes(world, max_ctas)
 * bytes of plain device memory each, zero before the first call); epoch: max_ctas uint32, zero before
 * the first call; err: becomes 1 + r if rank r never arrived.  -2 for bad arguments; -3 when
 * ceil(hidden / 1024) * n_tokens exceeds max_ctas. */
int nvk_b200_moe_combine_allreduce(void* stream, const void* const* peer_bufs, int rank, int world,
                                   const uint16_t* y_sorted_bf16, const float* topk_weights, const int32_t* inv_perm,
                                   float* y_acc_f32, int n_tokens, int k, int hidden, int y_sorted_row_stride,
                                   int sorted_rows, int* status, int max_ctas, uint32_t* epoch, int* err);
size_t nvk_b200_moe_combine_buffer_bytes(int world, int max_ctas);

/* No counterpart in the reference: tuning/test hook.  force_ksplit in {0 (auto), 1, 2, 4, 8} fixes
 * how many CTAs of a cluster share one row tile's K range; force_rows_per_cta in {0 (auto), 16, 32,
 * 64, 128} fixes the rows one CTA owns (M <= 16 only). */
int nvk_b200_set_tuning(int force_ksplit, int force_rows_per_cta);

/* No counterpart in the reference: tuning/test hook for the calling thread.  When the 128-row tiles of
 * a W4A16 launch (M <= 64, no K split) fit the GPU at once but not evenly -- more CTAs than SMs, fewer
 * than a whole number of CTAs per SM -- the launch instead starts the same number of CTAs on every SM
 * and deals the 16-row units round-robin over all of them, so that no SM carries a whole CTA more than
 * another.  A row's result does not depend on which warp computes it.  mode 0 = decide per launch
 * (default), 1 = deal whenever the route allows it, 2 = never.  -2 for another value. */
int nvk_b200_set_row_balance(int mode);

/* The rule behind mode 0, as a host-only query (no GPU needed): for a launch of tile_ctas 128-row-tile
 * CTAs that each need smem_bytes of shared memory and of which registers allow max_ctas_per_sm per SM,
 * the number of CTAs the dealt launch starts instead (a multiple of 148), or 0 when the per-tile launch
 * is kept: tile_ctas <= 148, more CTAs than are resident at once, or no SM would carry fewer warps. */
int nvk_b200_row_balance_grid(int tile_ctas, size_t smem_bytes, int max_ctas_per_sm);

/* No counterpart in the reference.  The decode-path launches use programmatic dependent launch: a
 * kernel may be scheduled while the previous kernel of the stream is still running and waits for that
 * kernel (griddepcontrol.wait) before it reads anything that kernel may have written or writes
 * anything -- the W4A16 kernels fill their weight ring first, every other kernel waits first of all.
 * enabled = 0 turns this off for the calling thread's launches (plain stream order); default on. */
int nvk_b200_set_pdl(int enabled);
/* Polls a kernel of this library spends in ONE wait on another CTA or another GPU (the peer
 * all-reduce's flags, a persistent step's dependency counters) before it gives up, sets its error
 * word and returns -- no wait is unbounded.  0 restores the default (2,000,000 polls, about a second).
 * Applies to later calls made by the calling thread.  No counterpart in the reference. */
int nvk_b200_set_wait_limit(unsigned polls);

/* bf16 weights, M = 1 (lm_head): y[n] = bf16(sum_k W[n,k] x[k]).
 * replaces rust/crates/nv-kernels/include/nv_kernels.h:116-123
 * (rust/crates/nv-kernels/cuda/gemv_bf16.cu:22-76,467-533) */
int nv_kernels_gemv_bf16(void* stream, const uint16_t* W, const uint16_t* x, uint16_t* y, int N, int K);

/* No counterpart with this signature in the reference, which sends a bf16 linear with several rows to
 * a library GEMM (rust/crates/nv-layers/src/linear.rs:717-804): y [M, N] = bf16(x [M, K] W^T), bf16 W
 * [N, K], fp32 accumulate, 1 <= M <= 64 (-1 otherwise), in ONE pass over W for all M rows (the lm_head
 * of a batched decode step).  Needs K % 8 == 0 and 16-byte aligned W and x for that; other shapes and
 * M == 1 run nv_kernels_gemv_bf16 once per row. */
int nvk_b200_linear_bf16(void* stream, const uint16_t* W, const uint16_t* x, uint16_t* y, int M, int N, int K);

/* ---- bf16 -> NVFP4 quantizers (byte-exact with nv_quant::nvfp4::quantize_block_with_global,
 *      rust/crates/nv-quant/src/nvfp4.rs:91-129) -------------------------------------------------- */

/* Rows [m_logical, m_padded) quantize zeros.  -2 if m_logical is outside [0, m_padded].
 * replaces rust/crates/nv-kernels/include/nv_kernels.h:1370-1379
 * (rust/crates/nv-kernels/cuda/quantize_nvfp4_bf16.cu:73-120,352-377) */
int nv_kernels_quantize_nvfp4_bf16(void* stream, const uint16_t* x_bf16, uint8_t* packed_out,
                                   uint8_t* scales_out_swizzled, float stored_global, int m_padded,
                                   int m_logical, int K);

/* replaces rust/crates/nv-kernels/include/nv_kernels.h:1381-1389 (quantize_nvfp4_bf16.cu:327-350) */
int nv_kernels_quantize_nvfp4_bf16_rows(void* stream, const uint16_t* x_bf16, uint8_t* packed_out,
                                        uint8_t* scales_out_swizzled, float stored_global, int m_rows, int K);

/* One row, scales written linearly ([K/16]).
 * replaces rust/crates/nv-kernels/include/nv_kernels.h:525-532
 * (rust/crates/nv-kernels/cuda/gemv_nvfp4.cu:79-120,181-199) */
int nv_kernels_nvfp4_quantize_row_bf16(void* stream, const uint16_t* x, uint8_t* packed_out, uint8_t* scales_out,
                                       float stored_global, int K);

/* Stored global of row r is stored_globals[r / m_per_expert] (device array).  The `_strided`
 * forms touch only row 0 of every m_per_expert-row tile and return -3 unless
 * m_total % m_per_expert == 0.
 * replace rust/crates/nv-kernels/include/nv_kernels.h:1348-1368
 * (rust/crates/nv-kernels/cuda/quantize_nvfp4_bf16.cu:122-170,277-325) */
int nv_kernels_quantize_nvfp4_bf16_per_expert(void* stream, const uint16_t* x_bf16, uint8_t* packed_out,
                                              uint8_t* scales_out_swizzled, const float* stored_globals,
                                              int m_per_expert, int m_total, int K);
int nv_kernels_quantize_nvfp4_bf16_per_expert_strided(void* stream, const uint16_t* x_bf16, uint8_t* packed_out,
                                                      uint8_t* scales_out_swizzled, const float* stored_globals,
                                                      int m_per_expert, int m_total, int K);

/* Quantizes SiLU(gate) * up evaluated in fp32 (no bf16 rounding in between).
 * replace rust/crates/nv-kernels/include/nv_kernels.h:1324-1346
 * (rust/crates/nv-kernels/cuda/quantize_nvfp4_bf16.cu:172-275) */
int nv_kernels_silu_mul_quantize_nvfp4_bf16_per_expert(void* stream, const uint16_t* y_gate_bf16,
                                                       const uint16_t* y_up_bf16, uint8_t* packed_out,
                                                       uint8_t* scales_out_swizzled, const float* stored_globals,
                                                       int m_per_expert, int m_total, int K);
int nv_kernels_silu_mul_quantize_nvfp4_bf16_per_expert_strided(void* stream, const uint16_t* y_gate_bf16,
                                                               const uint16_t* y_up_bf16, uint8_t* packed_out,
                                                               uint8_t* scales_out_swizzled,
                                                               const float* stored_globals, int m_per_expert,
                                                               int m_total, int K);

/* RMSNorm fused in front of the quantizer; the row is staged in shared memory (K * 2 bytes), and
 * K * 2 > 48 KiB is refused with -3.
 * replaces rust/crates/nv-kernels/include/nv_kernels.h:1391-1402
 * (rust/crates/nv-kernels/cuda/rmsnorm_quantize_nvfp4_bf16.cu:92-197) */
int nv_kernels_rmsnorm_quantize_nvfp4_bf16(void* stream, const uint16_t* x_bf16, const uint16_t* weight_bf16,
                                           uint8_t* packed_out, uint8_t* scales_out_swizzled, float stored_global,
                                           float eps, int m_padded, int m_logical, int K);

/* ---- W4A8 decode MLP: NVFP4 weights x int8 activation rows (one dequant scale per row) -----------
 *   y[m, n] = bf16( fma( sum_k W[n, k] * q[m, k],  alpha * scale[m],  residual[m, n] ) )
 * W = e2m1 x ue4m3 block scale, q int8 in [-127, 127], fp32 accumulate, one rounding.  N, K > 0 and
 * K % 32 == 0 (-1 otherwise, nothing launched); weights and scales 16-byte aligned, x_q8 8-byte
 * aligned, no NULL operand except residual (-2).  The reference refuses K > 98304 (its shared-memory
 * staging); this library has no such limit.
 * replace rust/crates/nv-kernels/include/nv_kernels.h:627-715, 746-776
 * (rust/crates/nv-kernels/cuda/gemv_nvfp4_w4a8_decode.cu) */
int nv_kernels_gemv_nvfp4_w4a8_dual_m1(void* stream, const uint8_t* wq_a, const uint8_t* sc_a, const uint8_t* wq_b,
                                       const uint8_t* sc_b, const int8_t* x_q8, const float* x_dequant_scale,
                                       uint16_t* y_a, uint16_t* y_b, float alpha_a, float alpha_b, int N, int K);
int nv_kernels_gemv_nvfp4_w4a8_dual_mk(void* stream, const uint8_t* wq_a, const uint8_t* sc_a, const uint8_t* wq_b,
                                       const uint8_t* sc_b, const int8_t* x_q8, const float* x_dequant_scales,
                                       uint16_t* y_a, uint16_t* y_b, float alpha_a, float alpha_b, int M, int N, int K);
int nv_kernels_gemv_nvfp4_w4a8_down_residual_m1(void* stream, const uint8_t* wq, const uint8_t* sc, const int8_t* x_q8,
                                                const float* x_dequant_scale, const uint16_t* residual, uint16_t* y,
                                                float alpha, int N, int K);
int nv_kernels_gemv_nvfp4_w4a8_down_residual_mk(void* stream, const uint8_t* wq, const uint8_t* sc, const int8_t* x_q8,
                                                const float* x_dequant_scales, const uint16_t* residual, uint16_t* y,
                                                float alpha, int M, int N, int K);
/* ... and leaves 1/rms of the new row for the next RMSNorm: rstd_ssq_count_pack = {rstd, running sum
 * of squares, arrival count} (three 32-bit words the caller zeroes once); after the launch word 0 is
 * rsqrt(sum(y^2) / N + rstd_eps) and words 1, 2 are zero again.  The CTAs' partial sums are added in
 * arrival order (as in the reference), so word 0 may differ in its last bits between runs. */
int nv_kernels_gemv_nvfp4_w4a8_down_residual_m1_rstd_emit(void* stream, const uint8_t* wq, const uint8_t* sc,
                                                          const int8_t* x_q8, const float* x_dequant_scale,
                                                          const uint16_t* residual, uint16_t* y, float alpha,
                                                          float* rstd_ssq_count_pack, float rstd_eps, int N, int K);
/* The down projection reading the staged bf16 activation of nv_kernels_silu_mul_stage_partial_absmax_m1
 * and quantizing it to int8 while it stages it: bit-identical to nv_kernels_silu_mul_rowquant_i8_m1
 * followed by nv_kernels_gemv_nvfp4_w4a8_down_residual_m1.  num_partials > 0 (-1 otherwise). */
int nv_kernels_gemv_nvfp4_w4a8_down_residual_quant_prologue_m1(void* stream, const uint8_t* wq, const uint8_t* sc,
                                                               const uint16_t* act_staged_bf16,
                                                               const float* partial_absmax, int num_partials,
                                                               const uint16_t* residual, uint16_t* y, float alpha, int N,
                                                               int K);
/* act = bf16(SiLU(gate) * up); scale = max|act| / 127; q = clamp(rn(act / scale), +-127) (ties to even).
 * _m1: one row, K % 4 == 0 and K * 2 bytes <= 96 KiB (-1 otherwise).  _mk: M rows in two passes --
 * act_staged_bf16 [M, K] and partial_absmax [nv_kernels_silu_mul_rowquant_i8_mk_partials_len(M, K)]
 * are caller buffers; K % 16 == 0.  _stage_partial_absmax_m1 is the first pass alone for one row. */
int nv_kernels_silu_mul_rowquant_i8_m1(void* stream, const uint16_t* gate, const uint16_t* up, int8_t* act_q8,
                                       float* act_dequant_scale, int K);
int nv_kernels_silu_mul_rowquant_i8_mk_partials_len(int M, int K);
int nv_kernels_silu_mul_rowquant_i8_mk(void* stream, const uint16_t* gate, const uint16_t* up, uint16_t* act_staged_bf16,
                                       float* partial_absmax, int8_t* act_q8, float* act_dequant_scales, int M, int K);
int nv_kernels_silu_mul_stage_partial_absmax_m1(void* stream, const uint16_t* gate, const uint16_t* up,
                                                uint16_t* act_staged_bf16, float* partial_absmax, int K);
/* res_out = bf16(x + res_in); v = bf16(res_out * rsqrt(mean((x + res_in)^2) + eps) * weight).
 * _rowquant_i8_m1 (one row, hidden <= 24576 else -1) quantizes v to int8 like the kernels above;
 * _bf16 writes v for `batch` rows.
 * replace rust/crates/nv-kernels/include/nv_kernels.h:717-727 (cuda/gemv_nvfp4_w4a8_decode.cu:323-386)
 * and :1195-1205 (cuda/rmsnorm_residual_writeout.cu) */
int nv_kernels_rmsnorm_residual_writeout_rowquant_i8_m1(void* stream, const uint16_t* x, const uint16_t* res_in,
                                                        const uint16_t* weight, uint16_t* res_out, int8_t* out_q8,
                                                        float* out_dequant_scale, int hidden, float eps);
int nv_kernels_rmsnorm_residual_writeout_bf16(void* stream, const uint16_t* x, const uint16_t* res_in,
                                              const uint16_t* weight, uint16_t* res_out, uint16_t* out, size_t batch,
                                              size_t hidden, float eps);

/* ---- MoE decode ------------------------------------------------------------------------------ */

/* mode 0: top-K of the (optionally tanh soft-capped) logits, softmax over the K winners;
 * mode 1: sigmoid scores, selection on score + bias, optional renormalisation.  Larger score first,
 * ties to the lower expert id; weights are multiplied by routed_scaling.  A NaN score never wins and
 * an expert wins at most once: a row with fewer than K usable scores is padded with id -1 /
 * weight 0 (the reference re-selects an expert it already chose there).  -2 if E > 4096, K > 32 or
 * K > E.
 * replace rust/crates/nv-kernels/include/nv_kernels.h:1538-1567
 * (rust/crates/nv-kernels/cuda/moe_route.cu:75-329) */
int nv_kernels_moe_route_topk(void* stream, const float* logits, const float* bias, int32_t* topk_ids,
                              float* topk_weights, int n_tokens, int E, int K, int mode, float softcap,
                              int norm_topk, float routed_scaling);
int nv_kernels_moe_route_topk_shared_tail(void* stream, const float* logits, const float* bias, int32_t* topk_ids,
                                          float* topk_weights, int n_tokens, int E, int K, int mode, float softcap,
                                          int norm_topk, float routed_scaling, int shared_tail_id);

/* out[r, :] = x[src_idx[r], :], a zero row when src_idx[r] is outside [0, n_tokens).  The strided
 * form touches rows 0, row_stride, 2*row_stride, ...
 * replace rust/crates/nv-kernels/include/nv_kernels.h:1433-1452 (cuda/gather_rows_bf16.cu) */
int nv_kernels_gather_rows_bf16(void* stream, const uint16_t* x_bf16, const int32_t* src_idx, uint16_t* out_bf16,
                                int m_total_padded, int hidden, int n_tokens);
int nv_kernels_gather_rows_bf16_strided(void* stream, const uint16_t* x_bf16, const int32_t* src_idx,
                                        uint16_t* out_bf16, int m_total_padded, int hidden, int n_tokens,
                                        int row_stride);

/* dst[i] = ids[i] >= 0 ? src[ids[i]] : 0.
 * replaces rust/crates/nv-kernels/include/nv_kernels.h:1593-1599 (cuda/moe_route.cu:536-561) */
int nv_kernels_gather_f32_by_ids(void* stream, const float* src, const int32_t* ids, float* dst, int n);

/* y_acc[n,h] = sum_s w[n,s] * y_sorted[inv_perm[n,s], h] in fp32, s ascending; a slot with a
 * negative inv_perm (one the sort left out) contributes nothing.
 * replaces rust/crates/nv-kernels/include/nv_kernels.h:1526-1536 (cuda/moe_unpermute_scatter.cu:6-32) */
int nv_kernels_moe_unpermute_scatter(void* stream, const uint16_t* y_sorted_bf16, const float* topk_weights,
                                     const int32_t* inv_perm, float* y_acc_f32, int n_tokens, int k, int hidden,
                                     int y_sorted_row_stride);

/* out = bf16(resid + bf16(combine + shared)).
 * replaces rust/crates/nv-kernels/include/nv_kernels.h:1454-1466 (cuda/moe_unpermute_scatter.cu:34-64) */
int nv_kernels_moe_unpermute_scatter_tail(void* stream, const uint16_t* y_sorted_bf16, const float* topk_weights,
                                          const int32_t* inv_perm, const float* shared_f32,
                                          const uint16_t* resid_bf16, uint16_t* out_bf16, int n_tokens, int k,
                                          int hidden, int y_sorted_row_stride);

/* No counterpart in the reference (whose entry point trusts inv_perm): the same combine with the
 * sorted buffer's row count known.  A row index not below sorted_rows is skipped and reported in
 * bit 2 of *status (one device int the caller zeroes; may be NULL). */
int nvk_b200_moe_combine(void* stream, const uint16_t* y_sorted_bf16, const float* topk_weights, const int32_t* inv_perm,
                         float* y_acc_f32, int n_tokens, int k, int hidden, int y_sorted_row_stride, int sorted_rows,
                         int* status);

/* Sort the n_tokens*k routed slots by expert: expert_offsets[E+1], permuted_token_idx[pos] = token,
 * inv_perm[slot] = pos.  Slots of one expert keep their original order (the reference leaves that
 * order to atomics).  An expert id outside [0, E) -- a router's -1 included -- is never used as an
 * index: that slot gets inv_perm = -1 and is left out.  scratch_counts is E int32 of caller scratch
 * (any contents).  One launch.
 * replaces rust/crates/nv-kernels/include/nv_kernels.h:1601-1611 (cuda/moe_permute.cu) */
int nv_kernels_moe_permute(void* stream, const int32_t* topk_ids, int32_t* permuted_token_idx,
                           int32_t* expert_offsets, int32_t* inv_perm, int32_t* scratch_counts, int n_tokens, int k,
                           int num_experts);

/* No counterpart in the reference (its decode step launches the router and the permutation
 * separately): both in one launch for decode-sized batches, with exactly the outputs of
 * nv_kernels_moe_route_topk followed by nv_kernels_moe_permute and no scratch buffer.  When
 * active_experts / n_active are given (both or neither), the ascending list of experts that
 * received at least one slot ([min(E, n_tokens*K)] int32) and its length are written as well, for
 * nvk_b200_moe_grouped_w4a16.
 * Limits: E <= 256 and n_tokens * K <= 4096, otherwise -3 and nothing is launched; K > E or K > 32
 * returns -2. */
int nvk_b200_moe_route_permute(void* stream, const float* logits, const float* bias, int32_t* topk_ids,
                               float* topk_weights, int32_t* permuted_token_idx, int32_t* expert_offsets,
                               int32_t* inv_perm, int32_t* active_experts, int32_t* n_active, int n_tokens, int E,
                               int K, int mode, float softcap, int norm_topk, float routed_scaling);

/* One decode token: route it, copy each winner's (and the shared tail's, when shared_tail_id >= 0)
 * stored activation globals into gu_mini / dn_mini, and quantize the token's row once per tile with
 * that tile's gate/up global into row t * min_tile of x_fp4 (swizzled scale in x_sf).
 * -1 non-positive sizes, -2 E > 256 / K + 1 > 32 / K > E / misaligned or NULL pointers,
 * -3 hidden % 16 != 0 or min_tile % 128 != 0.
 * replaces rust/crates/nv-kernels/include/nv_kernels.h:1569-1591 (cuda/moe_route.cu:331-470) */
int nv_kernels_moe_route_gather_quant_m1(void* stream, const float* logits, const float* bias, const uint16_t* x_bf16,
                                         const float* globals_gu, const float* globals_dn, int32_t* topk_ids,
                                         float* topk_weights, float* gu_mini, float* dn_mini, uint8_t* x_fp4,
                                         uint8_t* x_sf, int E, int K, int mode, float softcap, int norm_topk,
                                         float routed_scaling, int shared_tail_id, int hidden, int min_tile);

/* Writes the GPU's global nanosecond timer into *out when the stream reaches this point (also
 * inside a captured graph): two stamps time the kernels between them.
 * replaces rust/crates/nv-kernels/include/nv_kernels.h:1701-1704 (cuda/laguna_step.cu:565-576) */
int nv_kernels_prof_timestamp(void* stream, unsigned long long* out);

/* No counterpart in the reference.  The same permutation as nv_kernels_moe_permute for callers that
 * cannot supply (or allocate) the scratch_counts buffer: the per-expert counters live in a 16 KiB
 * array inside the library (held by every GPU that loads it, until the process exits), so the call
 * allocates nothing and takes no scratch argument.  Limits and rules:
 *   - num_experts <= 4096, otherwise -3 and nothing is launched;
 *   - the first call on each device looks up the array's device address (a one-time set-up step
 *     with that device current); make that first call before any stream capture;
 *   - all calls on a device share the one array, whose counters the kernel clears before it counts:
 *     two calls that may run on the GPU at the same time (different streams) race -- keep them on
 *     one stream or otherwise ordered. */
int nvk_b200_moe_permute_static(void* stream, const int32_t* topk_ids, int32_t* permuted_token_idx,
                                int32_t* expert_offsets, int32_t* inv_perm, int n_tokens, int k,
                                int num_experts);

/* Grouped M=1 expert GEMV with NVFP4 weights AND NVFP4 activations: group g multiplies row 0 of its
 * a_tile_stride_rows-row activation tile by expert group_expert_ids[g]; an id outside
 * [0, num_experts_total) writes zeros.  -1 on bad shapes, -2 unless a_packed/b_packed are 8-byte
 * aligned, -9 if num_groups > 65535.
 * replaces rust/crates/nv-kernels/include/nv_kernels.h:1020-1035
 * (rust/crates/nv-kernels/cuda/moe_grouped_fp4_gemv.cu:77-180) */
int nv_kernels_moe_grouped_fp4_gemv_m1_bf16(void* stream, const uint8_t* a_packed, const uint8_t* a_scales,
                                            const uint8_t* b_packed, const uint8_t* b_scales, const float* alphas,
                                            uint16_t* d_bf16, const int32_t* group_expert_ids, int num_groups,
                                            int num_experts_total, int n, int k, int a_tile_stride_rows,
                                            long long d_group_stride_elems);

/* ---- prefill-sized block-scaled GEMM (both operands NVFP4) --------------------------------------
 * D[m,n] = bf16(*global_sf * sum_k A[m,k] * B[n,k]); a_fp4 [m, k/2], b_fp4 [n, k/2] packed e2m1, a_sf / b_sf
 * their 128x4-swizzled ue4m3 scales (padded to 128 rows), global_sf one fp32 in device memory.
 * Runs tcgen05 kind::mxf4nvf4 block-scaled MMA on sm_100a.  Workspace protocol as in the reference:
 * *required_workspace is always written; all five data pointers NULL is a pure size query (returns 0,
 * launches nothing); a workspace that is too small returns -10.  k % 32 != 0 or n % 8 != 0 returns -1.
 *   ..._bf16          data-parallel scheduler, the tile nvk_b200_set_prefill_config selected;
 *   ..._bf16_streamk  the 1-SM tile under the stream-K scheduler (its own, larger workspace: query it
 *                     through this symbol);
 *   ..._bf16_tiled    `tile` 0..2 names one of the reference's sm_120 tile shapes -- all three map to the
 *                     1-SM 128x128x256 tile here, any other value is -3 as in the reference -- and
 *                     `stream_k` keeps its meaning: 0 data-parallel, 1 stream-K, >= 2 that many forced
 *                     splits of every output tile along K.
 * replace rust/crates/nv-kernels/include/nv_kernels.h:1037-1049,1924-1955
 * (rust/crates/nv-kernels/cuda_sm120/cutlass_fp4_gemm.cu:14-221) */
int nv_kernels_cutlass_fp4_gemm_sm120_bf16(void* stream, const void* a_fp4, const void* a_sf, const void* b_fp4,
                                           const void* b_sf, const float* global_sf, void* d_bf16, int m, int n, int k,
                                           void* workspace, size_t workspace_bytes, size_t* required_workspace);
int nv_kernels_cutlass_fp4_gemm_sm120_bf16_streamk(void* stream, const void* a_fp4, const void* a_sf,
                                                   const void* b_fp4, const void* b_sf, const float* global_sf,
                                                   void* d_bf16, int m, int n, int k, void* workspace,
                                                   size_t workspace_bytes, size_t* required_workspace);
int nv_kernels_cutlass_fp4_gemm_sm120_bf16_tiled(void* stream, const void* a_fp4, const void* a_sf, const void* b_fp4,
                                                 const void* b_sf, const float* global_sf, void* d_bf16, int m, int n,
                                                 int k, int tile, int stream_k, void* workspace,
                                                 size_t workspace_bytes, size_t* required_workspace);

/* Grouped block-scaled FP4 x FP4 GEMM for prefill-sized MoE steps: for every group g,
 * D_g[m_g, N] = bf16(alphas[e_g] * A_g B[e_g]^T) with every size and offset in device memory.
 *   group g: rows [expert_offsets[g], +m_g) of the stacked packed activations and of D; activation
 *   scales from row sf_offsets[g] (a multiple of 128) of the stacked swizzled scale buffer; weights of
 *   expert e_g = active_expert_indices ? active_expert_indices[g] : g; (m_g, n_g, k_g) =
 *   problem_sizes[3g .. 3g+2].  meta_scratch (>= 64 KiB, device) receives the per-group argument
 *   arrays; all of a_packed, b_packed, d_bf16 NULL is a workspace query.  -10 meta scratch too small,
 *   -11 meta scratch overflow, -12 workspace too small, -13..-15 set-up stages of the GEMM.
 * Both symbols run the same sm_100a kernel (1-SM 128x128x256 tile, tcgen05 kind::mxf4nvf4).
 * replaces rust/crates/nv-kernels/include/nv_kernels.h:970-1018
 * (rust/crates/nv-kernels/cuda_sm120/moe_grouped_fp4_gemm.cu:116-470) */
int nv_kernels_cutlass_moe_grouped_fp4_gemm_sm120_bf16(
    void* stream, const void* a_packed, const void* a_scales, const void* b_packed, const void* b_scales,
    const float* alphas, void* d_bf16, const int32_t* expert_offsets, const int32_t* sf_offsets,
    const int32_t* problem_sizes, const int32_t* active_expert_indices, int N, int K, int num_experts,
    int64_t a_row_stride_elems, int64_t b_row_stride_elems, int64_t c_row_stride_elems, void* meta_scratch,
    size_t meta_scratch_bytes, void* gemm_workspace, size_t gemm_workspace_bytes, size_t* required_workspace);
int nv_kernels_cutlass_moe_grouped_fp4_gemm_sm120_bf16_decode(
    void* stream, const void* a_packed, const void* a_scales, const void* b_packed, const void* b_scales,
    const float* alphas, void* d_bf16, const int32_t* expert_offsets, const int32_t* sf_offsets,
    const int32_t* problem_sizes, const int32_t* active_expert_indices, int N, int K, int num_experts,
    int64_t a_row_stride_elems, int64_t b_row_stride_elems, int64_t c_row_stride_elems, void* meta_scratch,
    size_t meta_scratch_bytes, void* gemm_workspace, size_t gemm_workspace_bytes, size_t* required_workspace);

/* No counterpart in the reference: tuning hook for the prefill GEMM, per calling thread.  1 = 1-SM
 * 128x128x256 tile (default), 2 = 2-SM (cta_group::2) 256x128x256 tile with a 2x1x1 cluster, whose
 * operand loads use cluster multicast: single-GPU processes and this GPU's own memory only. */
int nvk_b200_set_prefill_config(int cfg);

/* The library route of the same contraction: d [m, n] = bf16(alpha * a [m, k] * b [n, k]^T) through
 * cuBLASLt (CUDA_R_4F_E2M1 operands, VEC16_UE4M3 block scaling, TN, weights as the library's A), what
 * the reference's runner does with SPEACHES_NVFP4_BACKEND=cublaslt
 * (rust/crates/nv-quant/src/nvfp4.rs:866-1067; the reference binds cuBLASLt from Rust, so there is no
 * nv_kernels symbol to keep).  alpha is a host value.  cuBLASLt is opened at run time.  0 for an empty
 * problem; -1 unless k % 16 == 0 and m, n, k >= 128 (the reference's rule for this route,
 * nvfp4.rs:564-590); -2 null or not 16-byte aligned operands; -3 cuBLASLt cannot be opened or gives no
 * handle; -100 - s for a cuBLASLt status s (-115: no algorithm for the shape).  The first call for a
 * shape makes its plan and must not be inside a graph capture; later calls are capturable.
 * nvk_b200_cublaslt_fp4_workspace_bytes() = the 64 MiB the reference gives this route per stream. */
int nvk_b200_cublaslt_fp4_gemm_bf16(void* stream, const uint8_t* a_packed, const uint8_t* a_scales,
                                    const uint8_t* b_packed, const uint8_t* b_scales, uint16_t* d, int m, int n,
                                    int k, float alpha, void* workspace, size_t workspace_bytes);
size_t nvk_b200_cublaslt_fp4_workspace_bytes(void);

/* RMSNorm over bf16 rows, y = bf16(x * rsqrt(mean(x^2) + eps) * weight): the launch the reference's
 * M = 1 GEMV route puts in front of nv_kernels_nvfp4_gemv_bf16act when a norm precedes the linear
 * (rust/crates/nv-layers/src/linear.rs:1475-1510).  y may alias x.
 * replaces rust/crates/nv-kernels/include/nv_kernels.h:23-31 (rust/crates/nv-kernels/cuda/rmsnorm.cu:46-120) */
int nv_kernels_rmsnorm_bf16(void* stream, const uint16_t* x, const uint16_t* weight, uint16_t* y, size_t batch,
                            size_t hidden, float eps);

/* y[r, h] = x[r, h] * sigmoid(gate_logits[r]), fp32: the gate of the MoE block's shared expert
 * (rust/crates/nv-layers/src/moe.rs:386-398).  y may alias x.
 * replaces rust/crates/nv-kernels/include/nv_kernels.h:1424-1431
 * (rust/crates/nv-kernels/cuda/capture_copy.cu:52-85) */
int nv_kernels_mul_sigmoid_rowgate_f32(void* stream, const float* x, const float* gate_logits, float* y, int rows,
                                       int hidden);

/* No counterpart in the reference: a decode step's W4A16 linears (M <= 8 tokens) as ONE persistent
 * cooperative launch.  The step is a list of operations; operation i may name one EARLIER operation
 * `dep` whose outputs are its activations (x, and x2 for the SiLU(x) * x2 prologue), and is then held
 * back until that operation has completed -- inside the kernel, with the weight prefetch of the
 * waiting tiles already in flight.  An operation may overwrite a buffer only if every reader of the
 * old contents is, directly or through the chain of `dep`s, one of its dependencies.  Every item
 * computes exactly what nvk_b200_linear_nvfp4_w4a16 computes for the same rows with no split of K:
 * with nvk_b200_set_tuning(1, rows_per_item) the stand-alone launches give the same bits.
 *   nvk_b200_stack_plan_bytes(n_ops)   device bytes the plan needs (0 if n_ops is out of range)
 *   nvk_b200_stack_build(...)          SET-UP call: validates, writes the plan to plan_dev (host->device
 *                                      copy, synchronises) and returns launch_out[0] = CTAs,
 *                                      launch_out[1] = dynamic shared memory bytes.  -1 shape (K % 32,
 *                                      M > 8, half-null second arm), -2 argument / alignment / dep not
 *                                      earlier, -3 too many operations (> 1024) or no resident CTA
 *   nvk_b200_stack_run(...)            enqueue one step: clears the plan's counters on the stream and
 *                                      launches; allocates nothing, never synchronises.  `err` is a
 *                                      device int owned and zeroed by the caller, set to 1 if a wait
 *                                      inside the kernel ran out (nvk_b200_set_wait_limit).  n_ops, M and
 *                                      smem_bytes must be the values the plan was built with and grid at
 *                                      most the CTAs nvk_b200_stack_build returned, else -2 (a plan that
 *                                      this process did not build is refused the same way). */
typedef struct NvkStackOp {
    const uint8_t* wq_a;   /* packed weights [N, K/2] and swizzled scales of the (first) matrix */
    const uint8_t* sc_a;
    const uint8_t* wq_b;   /* optional second matrix sharing x (gate + up); all three NULL for one arm */
    const uint8_t* sc_b;
    const uint16_t* x;     /* [M, K] bf16 */
    const uint16_t* x2;    /* optional: the activation is bf16(SiLU(x) * x2) */
    uint16_t* y_a;         /* [M, N] bf16 */
    uint16_t* y_b;
    float alpha_a, alpha_b;
    int N, K;
    int dep;               /* index of the earlier operation that writes x (and x2), or -1 */
    int rows_per_item;     /* 0 = chosen from the shape; 128 or 16 */
} NvkStackOp;
size_t nvk_b200_stack_plan_bytes(int n_ops);
int nvk_b200_stack_build(const NvkStackOp* ops, int n_ops, int M, void* plan_dev, size_t plan_dev_bytes,
                         int* launch_out);
int nvk_b200_stack_run(void* stream, void* plan_dev, int n_ops, int M, int grid, int smem_bytes, int* err);

/* No counterpart in the reference (its grouped decode path quantizes activations to NVFP4 and gives
 * every (token, expert) pair its own 128-row tile): grouped-expert W4A16 linear with the tokens of
 * one expert sharing one pass over that expert's weights.
 *   banks:   expert e's packed weights at wq_bank + e * N*K/2, its swizzled scales at
 *            sc_bank + e * ceil(N/128)*128 * ceil(K/64)*4 (the layout of MoeGroupedWeights,
 *            rust/crates/nv-layers/src/moe_grouped.rs:98-281), its alpha at alphas[e] (device).
 *   tokens:  the routed slots sorted by expert, as nv_kernels_moe_permute produces them: expert e
 *            owns sorted slots [expert_offsets[e], expert_offsets[e+1]).  Slot i reads activation row
 *            row_index[i] of x (row i when row_index is NULL) and writes output row i of y.
 *   arms:    wq_bank_b/sc_bank_b/alphas_b/y_b give a second matrix sharing the activations
 *            (gate + up); all four NULL for one arm.
 *   x2:      when not NULL the activation is bf16(SiLU(x) * x2), rows taken the same way.
 *   active:  active_experts / n_active (device; both or neither) as nvk_b200_moe_route_permute
 *            writes them: the launch then covers min(num_experts, num_slots) experts instead of
 *            all of them, and experts without tokens cost nothing.  Without the list an expert
 *            without tokens costs one empty CTA per row tile.
 *   bounds:  num_slots = rows of y (and entries of row_index), x_rows = rows of x.  Offsets and row
 *            indices outside them are never followed: such slots are skipped (offset) or read as
 *            zeros (row) and bit 0 / bit 1 of *status (one device int the caller zeroes; may be
 *            NULL) is set.
 *   order:   a slot's result does not depend on the other slots or on how many experts are active:
 *            whether K is split over a cluster is decided from one expert's N and K alone.
 * K % 32 == 0 (-1 otherwise), 16-byte aligned pointers (-2 otherwise). */
int nvk_b200_moe_grouped_w4a16(void* stream, const uint8_t* wq_bank_a, const uint8_t* sc_bank_a,
                               const uint8_t* wq_bank_b, const uint8_t* sc_bank_b, const float* alphas_a,
                               const float* alphas_b, const uint16_t* x, const uint16_t* x2,
                               const int32_t* row_index, const int32_t* expert_offsets,
                               const int32_t* active_experts, const int32_t* n_active, uint16_t* y_a,
                               uint16_t* y_b, int num_experts, int N, int K, int num_slots, int x_rows,
                               int* status);

/* ---- tensor-parallel exchange (no counterpart in the reference, which has no multi-GPU code) ---
 * One-shot all-reduce of a small bf16 vector over peer memory for the row-parallel linears of a
 * decode step: every rank stores its partial into an inbox on every peer (plain peer stores, no
 * multicast), flags it, waits (bounded) for all peers and sums the slots in rank order in fp32, so
 * every rank gets the same bits.  The call number lives in device memory, so captured graphs replay.
 *   peer_bufs  `world` device pointers: the symmetric buffer of each rank as mapped here, each of
 *              nvk_b200_tp_allreduce_buffer_bytes(world, max_elems) bytes, zero-filled before first use
 *   epoch      32 uint32 of local device memory, zero-filled before first use
 *   err        one int of local device memory; non-zero (1 + missing peer) if a wait gave up
 * n % 8 == 0, n <= max_elems <= 262144, 16-byte aligned x and y, world <= 8; every rank must issue
 * the same sequence of calls.  -2 bad argument, -3 vector too long. */
size_t nvk_b200_tp_allreduce_buffer_bytes(int world, int max_elems);
/* Set-up helpers for that buffer (host side, they allocate and synchronise; never on the launch path):
 * plain cudaMalloc'd, zero-filled device memory shared between the ranks of one node with CUDA IPC
 * handles (64 bytes each, exchanged by the caller over its own host-side channel).  No memory is bound
 * to a multicast object.  Each returns 0 or a cudaError_t (-2 on a null argument). */
int nvk_b200_tp_buffer_alloc(size_t bytes, void** dev_ptr);
int nvk_b200_tp_buffer_free(void* dev_ptr);
int nvk_b200_tp_ipc_export(void* dev_ptr, void* handle_out_64_bytes);
int nvk_b200_tp_ipc_open(const void* handle_64_bytes, void** dev_ptr);
int nvk_b200_tp_ipc_close(void* dev_ptr);
int nvk_b200_tp_allreduce_bf16(void* stream, const void* const* peer_bufs, int rank, int world, const uint16_t* x,
                               uint16_t* y, int n, int max_elems, uint32_t* epoch, int* err);

#ifdef __cplusplus
}
#endif
