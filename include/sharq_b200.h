/*
 * sharq_b200 - C ABI of the B200 (sm_100a) SharQ quantized-linear kernels.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream handle
 * (cudaStream_t passed as void*; NULL = the legacy default stream), enqueues its work
 * on that stream and returns without synchronising.  Return value: 0 on success,
 * non-zero on an argument or launch error; sharq_last_error() then returns a message
 * (thread-local).  Unless stated otherwise an entry point allocates nothing and keeps
 * no state: every buffer, including scratch, is provided by the caller.
 *
 * The entry points are what a binding of the reference's `sharq_ops` module would call:
 * each comment names the reference op it stands behind (file:line in the reference
 * project, kernels/src/bindings.cpp unless another file is named).
 *
 * Buffer formats (identical to the reference's):
 *   payload     e2m1, two elements per byte (element 2i in the low nibble), row-major [rows, K/2]
 *   A_comp      per 8 logical K the two kept pair-bytes, row-major [M, K/4]
 *   E           per 8 logical K one nibble idx0 | idx1 << 2; layout [ceil(K/256)][ceil128(M)][16 B]
 *   scales      UE4M3, blocked: 512-byte tiles of 128 rows x 4 scales
 *               offset = (r/128)*(G/4)*512 + (g/4)*512 + (r%32)*16 + ((r/32)%4)*4 + g%4,
 *               G = K/16 (dense) or K/32 (sparse main path); allocation (rows/128+1)*128*K/16
 *   outputs     bf16 row-major [M, N]
 */
#ifndef SHARQ_B200_H_
#define SHARQ_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Library version (major*10000 + minor*100 + patch). */
int sharq_version(void);

/* Message of the last failing call on this thread ("" if none). */
const char *sharq_last_error(void);

/* get_sparse_nvfp4_buffer_sizes(M,N,K) -> (A_comp, E, SFA, SFB) bytes.  bindings.cpp:232-241 */
int sharq_get_sparse_nvfp4_buffer_sizes(int m, int n, int k, int64_t out_bytes[4]);

/* get_fused_sparse_residual_buffer_sizes(M,N,K) -> (A_comp, E, SFA_sparse, Q_res, SF_res) bytes.
 * bindings.cpp:243-253 */
int sharq_get_fused_sparse_residual_buffer_sizes(int m, int n, int k, int64_t out_bytes[5]);

/* fused_sparse_residual_quantize_x(X, N): X is a pre-scaled bf16 [M,K], K % 128 == 0.
 * Writes every byte of the five output buffers (sizes from the call above), padding
 * included, so they need not be zero-initialised.  bindings.cpp:255-289 */
int sharq_fused_sparse_residual_quantize_x(const void *x_bf16, int m, int n, int k, void *a_comp, void *e,
                                           void *sfa_sparse, void *q_res, void *sf_res, void *stream);

/* fused_sparse_residual_quantize_x_debug(X, N): dense sparse payload [M,K/2] instead of
 * A_comp/E.  bindings.cpp:357-390 */
int sharq_fused_sparse_residual_quantize_x_debug(const void *x_bf16, int m, int n, int k, void *q_sparse,
                                                 void *sfa_sparse, void *q_res, void *sf_res, void *stream);

/* Scratch bytes needed by the scaled prepare calls below for M rows.  Layout:
 * bytes [0,4) tensor absmax (float bits), bytes [4,8) arrival counter of the grid-wide barrier,
 * bytes [256, 256+4*M) per-row inv_rms (float).  The calls initialise what they use. */
size_t sharq_prepare_workspace_bytes(int m);

/* The scaled prepare calls run statistics and quantisation in ONE cooperative launch whose CTAs
 * meet at a grid-wide barrier with a bounded wait (about one second).  Returns how many such
 * waits ran out on the current device since the library was loaded: 0 in a healthy process (the
 * outputs of a call that timed out are undefined), -1 if the counter cannot be read.  Synchronises
 * nothing itself: call it after synchronising the stream.  No counterpart in the reference. */
int sharq_prepare_timeouts(void);

/* fused_rmsnorm_sparse_residual_quantize_x(X, rmsnorm_weight, eps, N): RMSNorm, tensor
 * scale = clamp(amax/2688, 1e-9) and prepare: an 8-byte memset and one cooperative launch (row
 * statistics, grid barrier, quantisation; the rows of a CTA stay in shared memory in between).
 * The normalised values are divided by the float32 scale, as the reference's kernel does
 * (kernels/src/fused_rmsnorm_sparse_prepare.cu:195-204).
 * K % 128 == 0 and K/32 <= 1024.  scale_out: one device float.  bindings.cpp:291-355 */
int sharq_fused_rmsnorm_sparse_residual_quantize_x(const void *x_bf16, const void *rmsnorm_weight_bf16,
                                                   float rmsnorm_eps, int m, int n, int k, void *workspace,
                                                   size_t workspace_bytes, void *a_comp, void *e, void *sfa_sparse,
                                                   void *q_res, void *sf_res, float *scale_out, void *stream);

/* The same with the decoder's residual add folded in (no counterpart in the reference, whose
 * layer wrapper adds with ATen before the call, model/qLlamaLayer.py:216-221): the input is
 * S = bf16(X + residual), rounded like the ATen add; the statistics kernel forms S, writes it
 * to sum_out [M,K] (may alias neither input) and the prepare reads it.  Outputs equal
 * sharq_fused_rmsnorm_sparse_residual_quantize_x(S, ...). */
int sharq_fused_add_rmsnorm_sparse_residual_quantize_x(const void *x_bf16, const void *residual_bf16, void *sum_out_bf16,
                                                       const void *rmsnorm_weight_bf16, float rmsnorm_eps, int m, int n,
                                                       int k, void *workspace, size_t workspace_bytes, void *a_comp,
                                                       void *e, void *sfa_sparse, void *q_res, void *sf_res,
                                                       float *scale_out, void *stream);

/* The non-RMSNorm activation path with its host-side passes folded in: computes
 * scale = clamp(max|X|/2688, 1e-9), X' = (X / scale).to(bf16) and the prepare of X'.  Equals
 * global_nvfp4_scale + divide + fused_sparse_residual_quantize_x of the reference
 * (model/quantize.py:43-44,179-183) as torch evaluates them on a CUDA device: dividing a bf16
 * tensor by a 0-dim float32 tensor there casts the divisor to bf16 first, so X' =
 * bf16(float(X) / float(bf16(scale))), while scale_out receives the unrounded float32 scale
 * (which the reference multiplies into the GEMM output). */
int sharq_scaled_sparse_residual_quantize_x(const void *x_bf16, int m, int n, int k, void *workspace,
                                            size_t workspace_bytes, void *a_comp, void *e, void *sfa_sparse,
                                            void *q_res, void *sf_res, float *scale_out, void *stream);

/* Decoder-layer steps between the SharQ linears, which the reference leaves to
 * HuggingFace's PyTorch code; each intermediate is rounded to bf16 where the PyTorch
 * composition rounds, so the results are those of the ATen ops.
 *
 * sharq_rope_inplace: rotary embedding x*cos + rotate_half(x)*sin, in place, on the first
 * `heads` heads of every row of a bf16 matrix (the query and key heads of a merged qkv
 * activation); row_stride in elements; position of a row = row % seq_len; cos/sin are bf16
 * [seq_len, head_dim].  Stands behind apply_rotary_pos_emb at model/qLlamaLayer.py:137-141.
 *
 * sharq_swiglu: H[rows, ffn] = silu(gate) * up of a contiguous merged activation
 * gate_up[rows, 2*ffn] (gate columns first).  model/qLlamaLayer.py:183-185.
 *
 * sharq_swiglu_sparse_residual_quantize_x: the same H (written to h_bf16, [M, K]) and the
 * scaled prepare of H for down_proj in two launches instead of the reference's five passes
 * (silu, mul, amax, divide, prepare): the SwiGLU kernel leaves max|H| in the workspace, so
 * the statistics pass of sharq_scaled_sparse_residual_quantize_x is not needed.  Outputs
 * equal sharq_scaled_sparse_residual_quantize_x(H). */
int sharq_rope_inplace(void *x_bf16, int rows, int row_stride, int seq_len, int heads, int head_dim,
                       const void *cos_bf16, const void *sin_bf16, void *stream);
/* sharq_scatter_add_scaled: out[rows[i], :] += y[i, :] * w[i] in bf16 with the roundings of
 * `final.index_add_(0, rows, y * w[:, None])` (the expert loop of model/qMixtralLayer.py:228-231);
 * out [out_rows, width] and y [n_rows, width] contiguous bf16, rows int64 and pairwise distinct, w bf16;
 * an index outside [0, out_rows) is skipped. */
int sharq_scatter_add_scaled(void *out_bf16, int out_rows, const void *y_bf16, const int64_t *rows, const void *w_bf16,
                             int n_rows, int width, void *stream);
int sharq_swiglu(const void *gate_up_bf16, int rows, int ffn, void *h_bf16, void *stream);
/* sharq_add_rmsnorm: out[rows, K] = bf16(s * rsqrt(mean(s^2) + eps) * gamma) with s = bf16(x + residual) written to
 * sum_out (both NULL: s = x); mean and products in float, one rounding per element.  The normalised bf16
 * activation that the router and the experts of a mixture-of-experts layer both read
 * (model/qMixtralLayer.py:205-213; the reference calls HuggingFace's RMSNorm module there).  K % 8 == 0, K <= 8192. */
int sharq_add_rmsnorm(const void *x_bf16, const void *residual_bf16, void *sum_out_bf16, const void *gamma_bf16, float eps,
                      int rows, int k, void *out_bf16, void *stream);
int sharq_swiglu_sparse_residual_quantize_x(const void *gate_up_bf16, int m, int n, int k, void *h_bf16,
                                            void *workspace, size_t workspace_bytes, void *a_comp, void *e,
                                            void *sfa_sparse, void *q_res, void *sf_res, float *scale_out,
                                            void *stream);

/* quantize_w32_shared(W): bf16 [N,K] (already divided by the weight tensor scale),
 * K % 32 == 0 -> QW [N,K/2], SFW_sparse (32-groups), SFW_dense (each scale duplicated
 * into two 16-group slots).  bindings.cpp:392-417 */
int sharq_quantize_w32_shared(const void *w_bf16, int n, int k, void *qw, void *sfw_sparse, void *sfw_dense,
                              void *stream);

/* duplicate_sfa32_to_sfa16(SFA_sparse, M, N, K).  bindings.cpp:419-437 */
int sharq_duplicate_sfa32_to_sfa16(const void *sfa_sparse, int m, int n, int k, void *sfa_dense, void *stream);

/* quantize_x_nvfp4(X) / quantize_w_nvfp4(W) (and reorder_quantize_x/w with the identity
 * index and KE == 0): dense NVFP4, one scale per 16.  K % 16 == 0.  Only the used bytes
 * of the scale buffer are written, as in the reference.  bindings.cpp:74-160 */
int sharq_quantize_nvfp4(const void *x_bf16, int rows, int k, void *q, void *sf, void *stream);

/* compress_sparse_a(A_q_dense, N): dense payload with at most two non-zero bytes per
 * 4-byte chunk -> A_comp, E.  bindings.cpp:164-230 */
int sharq_compress_sparse_a(const void *a_q_dense, int m, int n, int k, void *a_comp, void *e, void *stream);

/* matmul / matmul_tensor_scale / matmul_accum / matmul_accum_tensor_scale:
 * D = bf16(alpha * (A . B^T) + beta * C_in).  With alpha_dev (one device float) non-NULL
 * the factor is alpha * (*alpha_dev) (the reference passes alpha = 1 then); c_in may be
 * NULL when beta == 0.  K % 64 == 0.
 * error_flag: one device int the kernel sets non-zero if an internal bounded wait ran
 * out (never expected; the output is then undefined).  bindings.cpp:441-569 */
int sharq_matmul(const void *a, const void *b, const void *sfa, const void *sfb, int m, int n, int k, float alpha,
                 const float *alpha_dev, const void *c_in, float beta, void *d, int *error_flag, void *stream);

/* sparse_matmul / sparse_matmul_tensor_scale: beta must be 0.  K % 128 == 0.
 * bindings.cpp:571-701 */
int sharq_sparse_matmul(const void *a_comp, const void *b, const void *e, const void *sfa, const void *sfb, int m,
                        int n, int k, float alpha, const float *alpha_dev, float beta, void *d, int *error_flag,
                        void *stream);

/* The SharQ linear GEMM in one launch: D = bf16(alpha * (A_sparse + A_res) . W^T) (+ bias
 * in bf16), the sparse main pass and the dense residual pass reading the same weight tile
 * and accumulating into one tensor-memory tile.  Stands behind the two-launch composition
 * of model/qLinearLayer.py:130-154 (+ bias add at :177-179) and is what the optional
 * `sharq_linear_forward` op probed by benchmarks/vllm/sharq.py:206-213 runs. */
int sharq_linear_gemm(const void *a_comp, const void *e, const void *sfa_sparse, const void *q_res,
                      const void *sf_res, const void *qw, const void *sfw_sparse, const void *sfw_dense, int m, int n,
                      int k, float alpha, const float *alpha_dev, const void *bias_bf16, void *d, int *error_flag,
                      void *stream);

/* The three GEMMs with caller-provided scratch (no counterpart in the reference).  With
 * sharq_gemm_workspace_bytes(M, N) bytes (non-zero for M <= 128: M * N floats; contents
 * need not be initialised) a small-M GEMM, which is bound by streaming the weights, splits K
 * over the SMs: units add their fp32 partial sums into the scratch with vector reductions
 * and a second kernel applies alpha / beta / bias and writes bf16.  The order of those fp32
 * additions is not fixed, so the last bits of the sums may vary from call to call.  With
 * workspace == NULL, or M > 128, these are the plain entry points. */
size_t sharq_gemm_workspace_bytes(int m, int n);
int sharq_matmul_ws(const void *a, const void *b, const void *sfa, const void *sfb, int m, int n, int k, float alpha,
                    const float *alpha_dev, const void *c_in, float beta, void *d, void *workspace,
                    size_t workspace_bytes, int *error_flag, void *stream);
int sharq_sparse_matmul_ws(const void *a_comp, const void *b, const void *e, const void *sfa, const void *sfb, int m,
                           int n, int k, float alpha, const float *alpha_dev, float beta, void *d, void *workspace,
                           size_t workspace_bytes, int *error_flag, void *stream);
int sharq_linear_gemm_ws(const void *a_comp, const void *e, const void *sfa_sparse, const void *q_res,
                         const void *sf_res, const void *qw, const void *sfw_sparse, const void *sfw_dense, int m, int n,
                         int k, float alpha, const float *alpha_dev, const void *bias_bf16, void *d, void *workspace,
                         size_t workspace_bytes, int *error_flag, void *stream);

/* No counterpart in the reference.  Same work and outputs as
 * sharq_fused_rmsnorm_sparse_residual_quantize_x, for callers that cannot allocate device
 * memory and have no spare buffer to pass as workspace (a server that has given all free
 * HBM to its own pool; a thread on which cudaMalloc's device-wide synchronisation is not
 * allowed): the scratch lives in a fixed array inside the library (256 KiB + 256 B per GPU
 * that loads it).  M <= sharq_noalloc_max_rows() (65536), larger M is an error.  The first
 * call on a device looks up the array's address and should come before any stream capture;
 * no call allocates.  All calls on a device share the array: calls that overlap on the GPU
 * race, so order them on one stream (or with events).  Errors: non-zero return,
 * message from sharq_noalloc_last_error(). */
int sharq_fused_rmsnorm_sparse_residual_quantize_x_noalloc(const void *x_bf16, const void *rmsnorm_weight_bf16,
                                                           float rmsnorm_eps, int m, int n, int k, void *a_comp,
                                                           void *e, void *sfa_sparse, void *q_res, void *sf_res,
                                                           float *scale_out, void *stream);
int sharq_noalloc_max_rows(void);
const char *sharq_noalloc_last_error(void);

/* No counterpart in the reference (it has no tensor parallelism).  In-place sum, over the
 * `world` GPUs of one NVSwitch domain, of a bf16 buffer that every rank holds at the same
 * offset of a symmetric-memory allocation bound to an NVLink multicast object: the partial
 * outputs of a row-parallel SharQ linear (o_proj, down_proj).  One kernel per rank: rank r
 * reduces bytes [r, r+1) * n_bytes / world inside the switch (multimem.ld_reduce, fp32
 * accumulation) and stores the rounded bf16 sums to every rank's copy (multimem.st).
 *   multicast_data   multicast address of the buffer
 *   rank_flag_ptrs   HOST array of `world` device pointers: rank p's flag area as mapped in
 *                    this process (peer mapping; entry `rank` is the local one).  Each area
 *                    holds sharq_allreduce_flag_bytes() bytes, zeroed once (on every rank,
 *                    followed by a barrier) before the first call; afterwards it holds the
 *                    kernels' barrier counters and must not be touched.
 *   n_bytes          multiple of 16 * world; max_ctas: 0 = default.
 * All ranks must make the same calls in the same order with the same sizes.  The kernels of
 * the ranks wait for one another with bounded spins (about two seconds); a wait that runs
 * out sets *error_flag non-zero.  world <= 16. */
int sharq_allreduce_bf16_multimem(void *multicast_data, void *const *rank_flag_ptrs, int rank, int world,
                                  size_t n_bytes, int max_ctas, int *error_flag, void *stream);
size_t sharq_allreduce_flag_bytes(void);
/* The same sum with plain peer loads and stores instead of the multicast object, for
 * world <= 4 (it moves fewer bytes per link than the in-switch form at world == 2):
 * rank_data_ptrs[p] = rank p's copy of the buffer as mapped in this process.  Rank r sums
 * slice r of all copies in rank order (fp32) and writes the bf16 result into every copy. */
int sharq_allreduce_bf16_peer(void *const *rank_data_ptrs, void *const *rank_flag_ptrs, int rank, int world,
                              size_t n_bytes, int max_ctas, int *error_flag, void *stream);

/* Mixture-of-experts FFN in grouped launches.  The reference runs its experts in a Python loop
 * (model/qMixtralLayer.py:223-231): per expert a gather of its tokens, prepare, two GEMMs, SwiGLU, a
 * routing-weight multiply and index_add_.  These entry points do each step once for ALL experts on a
 * GROUPED activation: the token slots are sorted by expert, every expert's segment is padded to a
 * multiple of 256 rows, M is the padded total, and unit_group[u] (device, M/256 ints) is the expert
 * of rows [256u, 256u+256) or < 0 for a unit without rows.  Arithmetic per row is that of the
 * per-expert calls: every expert's rows are divided by that expert's own tensor scale.
 *   sharq_grouped_sparse_residual_quantize_x: per-expert max|X| (into amax_workspace, `groups`
 *     uint32 words) + scaled prepare; scale_vec_out[g] = clamp(amax_g / 2688, 1e-9).  src_row (optional,
 *     device, M ints) gathers: grouped row r is row src_row[r] of the token-major X (< 0: padding row).
 *   sharq_grouped_swiglu_sparse_residual_quantize_x: H = silu(gate) * up of gate_up [M, 2K] (written
 *     to h_bf16 [M, K]), per-expert max|H| and the scaled prepare of H.
 *   sharq_linear_gemm_grouped: D[r] = alpha * alpha_vec[g] * (A_sparse[r] + A_res[r]) . W_g^T for every
 *     row r of a unit of expert g (one launch; qw / sfw_sparse / sfw_dense: host arrays of `groups`
 *     device pointers; alpha_vec: device, e.g. activation scale x weight scale per expert).
 *   sharq_moe_combine: out[t] = sum over the top_k slots of token t, in ascending expert order, of
 *     y[dest[t,j]] * w[t,j] with bf16 rounding after every product and addition, which is what the
 *     reference's sequence of index_add_ calls on a zero buffer computes. */
int sharq_grouped_sparse_residual_quantize_x(const void *x_bf16, const int *src_row, int m, int n, int k,
                                            const int *unit_group, int groups, void *amax_workspace, void *a_comp, void *e,
                                            void *sfa_sparse, void *q_res, void *sf_res, float *scale_vec_out, void *stream);
int sharq_grouped_swiglu_sparse_residual_quantize_x(const void *gate_up_bf16, int m, int n, int k, void *h_bf16,
                                                   const int *unit_group, int groups, void *amax_workspace, void *a_comp,
                                                   void *e, void *sfa_sparse, void *q_res, void *sf_res,
                                                   float *scale_vec_out, void *stream);
int sharq_linear_gemm_grouped(const void *a_comp, const void *e, const void *sfa_sparse, const void *q_res, const void *sf_res,
                              int groups, const void *const *qw, const void *const *sfw_sparse, const void *const *sfw_dense,
                              const int *unit_group, const float *alpha_vec, float alpha, int m, int n, int k, void *d,
                              int *error_flag, void *stream);
int sharq_moe_combine(void *out_bf16, const void *y_bf16, const int *dest, const int64_t *selected, const void *w_bf16,
                      int tokens, int top_k, int width, void *stream);

/* No counterpart in the reference (it has no tensor parallelism).  Row-parallel SharQ linear and the
 * transition to the next column-parallel one over the GPUs of one NVLink domain, with the residual
 * stream sharded by rows (GPU r owns rows [r*M/world, (r+1)*M/world)), in two launches per GPU:
 *
 * sharq_linear_gemm_scatter: sharq_linear_gemm whose epilogue deals the output rows to their owners:
 *   row q of this GPU's partial product goes, through the peer mapping d_rank_ptrs[o] of owner
 *   o = q / (M/world), into block `rank` of GPU o's collection buffer [world][M/world, N] bf16 (plain
 *   peer stores, so the transfer runs while the GEMM computes).  M % (128*world) == 0, N % 8 == 0.
 *
 * sharq_tp_reduce_rmsnorm_prepare_allgather (one cooperative kernel): waits until every GPU has delivered,
 *   S   = sum over the `world` blocks of partial_blocks (this GPU's collection buffer) in fp32 in rank
 *         order, rounded to bf16 (partial_blocks == NULL: no sum),
 *   X'  = bf16(residual_in + S) for this GPU's rows, written to residual_out [M/world, K]
 *         (partial_blocks == NULL: X' = residual_in; residual_in == NULL: X' = S),
 *   then RMSNorm statistics of X', the tensor scale from the absmax over ALL GPUs' rows, the
 *   4:8 sparse + residual prepare of this GPU's rows, and the packed rows stored into EVERY
 *   GPU's copy of the prepared activation (plain peer stores; multimem.st with SHARQ_TP_ALLGATHER=multicast).
 * On return of the kernel every GPU's (a_comp, e, sfa_sparse, q_res, sf_res, *scale_out) hold
 * exactly what sharq_fused_rmsnorm_sparse_residual_quantize_x produces for the whole [M,K]
 * matrix X' on one GPU.  The five output buffers are this GPU's copy inside ONE symmetric
 * allocation whose multicast mapping is at local address + multicast_delta; rank_state_ptrs[r]
 * is GPU r's state block (sharq_tp_transition_state_bytes() bytes inside the SAME symmetric
 * allocation, zero-filled once, then owned by these calls) as mapped on this GPU: the kernel
 * reaches GPU r's copy of an output byte at its local address + (rank_state_ptrs[r] -
 * rank_state_ptrs[rank]).  workspace:
 * sharq_tp_transition_workspace_bytes(M/world) bytes of local scratch.
 * Requirements: M % (128*world) == 0, K % 128 == 0, K/32 <= 1024, 16-byte aligned buffers, the
 * same sequence of calls on every GPU.  Every cross-GPU wait is bounded (about ten seconds); one
 * that runs out stores a code 0x301..0x306 in *error_flag and the outputs are undefined.  Uses
 * plain peer stores and multimem.st only. */
int sharq_linear_gemm_scatter(const void *a_comp, const void *e, const void *sfa_sparse, const void *q_res, const void *sf_res,
                              const void *qw, const void *sfw_sparse, const void *sfw_dense, int m, int n, int k, float alpha,
                              const float *alpha_dev, void *const *d_rank_ptrs, int rank, int world, int *error_flag,
                              void *stream);
size_t sharq_tp_transition_state_bytes(void);
size_t sharq_tp_transition_workspace_bytes(int rows);
int sharq_tp_reduce_rmsnorm_prepare_allgather(const void *partial_blocks, const void *residual_in_bf16,
                                              void *residual_out_bf16, const void *rmsnorm_weight_bf16, float rmsnorm_eps,
                                              int m, int n, int k, void *workspace, size_t workspace_bytes, void *a_comp,
                                              void *e, void *sfa_sparse, void *q_res, void *sf_res,
                                              long long multicast_delta, float *scale_out, void *const *rank_state_ptrs,
                                              int rank, int world, int *error_flag, void *stream);

/* Test/tuning hook: how many SM clock cycles a cross-GPU wait of the all-reduce and transition
 * kernels may take before the kernel gives up, stores its error code and returns (0 restores the
 * defaults of two to ten seconds).  Applies to launches made after the call. */
int sharq_set_wait_limit_cycles(long long cycles);

/* Test/tuning hook: force the GEMM kernel variant (0 = automatic; 128 or 256 = single-CTA kernel
 * with that tile width; 512 = CTA-pair kernel, 256 x 256 tile per pair).  Process-wide. */
int sharq_set_gemm_tile_n(int tile_n);

#ifdef __cplusplus
}
#endif

#endif /* SHARQ_B200_H_ */
