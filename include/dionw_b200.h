/*
 * dionw_b200 — C ABI of the B200 (sm_100a) optimizer-step kernels.
 *
 * Every entry point takes raw device pointers, sizes and the CUDA stream to
 * launch on (passed as void* so that this header needs no CUDA include), runs
 * asynchronously on that stream, allocates nothing, never synchronises (the two
 * status reads, dionw_device_status and dionw_check_device, and the CPU EMA
 * job's waits excepted), and returns DIONW_OK or a negative code;
 * dionw_last_error() then gives the text.
 * The reference has no FFI of its own: each entry replaces the Python/Triton
 * function cited beside it (paths are relative to the reference project).
 *
 * Conventions
 *   - "blocks x rows x cols": the bucket layout of src/dionw/_buckets.py:154-178
 *     (momentum [blocks, rows, cols] fp32, variance [blocks, rows] fp32).
 *   - a "run" is a range of consecutive blocks of one bucket whose parameters
 *     are separate tensors: pointer tables are HOST arrays of DEVICE pointers,
 *     with rows_per_tensor[i] = rows that tensor i contributes (its blocks x rows).
 *   - dtype codes: DIONW_F32 / DIONW_F16 / DIONW_BF16.
 */
#ifndef DIONW_B200_H_
#define DIONW_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define DIONW_OK 0
#define DIONW_ERR_ARGUMENT (-1)
#define DIONW_ERR_CUDA (-2)
#define DIONW_ERR_WORKSPACE (-3)
#define DIONW_ERR_UNSUPPORTED (-4)
#define DIONW_ERR_DEVICE_WAIT (-5)
#define DIONW_ERR_WORKER (-6)

#define DIONW_F32 0
#define DIONW_F16 1
#define DIONW_BF16 2

/* Newton-Schulz kinds (src/dionw/newton_schulz.py:33-40). */
#define DIONW_NS_GRAM 0
#define DIONW_NS_POLAR_EXPRESS 1
#define DIONW_NS_KELLER 2
/* GRAM with the products among symmetric matrices computed in full, as the
 * reference's cuBLAS calls do, instead of on one triangle of tiles. */
#define DIONW_NS_GRAM_FULL 3

/* Text of the last error on the calling thread (copied, NUL-terminated). */
void dionw_last_error(char* buffer, size_t size);
/* Library version string. */
const char* dionw_version(void);
/* Kernels this library has launched in this process so far (all threads). */
int64_t dionw_launch_count(void);
/* Reads and clears the device status word (non-zero: a bounded wait inside a
 * kernel ran out).  Synchronises the device; meant for tests and diagnostics. */
int dionw_device_status(int* status);
/* Synchronises the device, reads and clears the status word, and returns
 * DIONW_ERR_DEVICE_WAIT (with the code in the error text) when a bounded wait
 * ran out since the last check, DIONW_OK otherwise.  The reference fails fast and
 * never swallows an error (src/dionw/ema/_cpu_job.py:108-137); this is the call
 * the host makes wherever it synchronises anyway (checkpoints, weight swaps). */
int dionw_check_device(void);
/* Self-test of the bounded wait: one small kernel waits `limit_us` microseconds
 * (1 .. 100000) on a barrier nothing arrives on, gives up, stores the wait code
 * in the status word and returns normally; *gave_up (device int, may be NULL) is
 * set to 1.  dionw_check_device() afterwards returns DIONW_ERR_DEVICE_WAIT once.
 * No counterpart in the reference. */
int dionw_selftest_wait_timeout(int64_t limit_us, int* gave_up, void* stream);

/* How the two-CTA tensor-core products hand tiles to SM pairs: 0 (default) a
 * fixed stride, 1 from a counter in device memory (one atomic per tile), so that a
 * product running beside other kernels (NCCL's collectives in the sharded step)
 * loses only the SMs those hold instead of waiting for the pairs that start late.
 * Same arithmetic, same results.  Process-wide; on < 0 only queries.  Returns the
 * previous setting.  DIONW_GEMM_DYNAMIC_TILES=1 sets the initial value.  No
 * counterpart in the reference (its products are cuBLAS's and Triton's). */
int dionw_gemm_dynamic_tiles(int on);

/* ---- momentum passes ---------------------------------------------------- */

/* M += G for every row of a run, plus per-row sum|M| (scores) and sum M^2.
 * Replaces accumulate_row_l1 / _accumulate_row_l1_kernel
 * (src/dionw/_momentum_kernels.py:40-55, :89-103) as called once per parameter
 * by _accumulate_with_scores (src/dionw/_matrix_step.py:188-199); here one
 * launch covers the whole run.  Score order: 1024 strided lanes, folded by
 * halving (lane[i] += lane[i+w], w = 512..1). */
int dionw_accumulate_row_l1_run(const void* const* grads, int grad_dtype,
                                const int64_t* rows_per_tensor, int n_tensors,
                                float* momentum, float* scores, float* sumsq,
                                int64_t cols, void* stream);

/* m = M + G; M = decay*m; u = m (heavy ball) or G + decay*m (Nesterov); also
 * per-row sum u^2.  Replaces accumulate_copy_decay
 * (src/dionw/_momentum_kernels.py:58-77, :106-133; caller
 * src/dionw/_matrix_step.py:217-237). */
int dionw_accumulate_copy_decay_run(const void* const* grads, int grad_dtype,
                                    const int64_t* rows_per_tensor, int n_tensors,
                                    float* momentum, float* u, float* sumsq,
                                    int64_t cols, float decay, int nesterov, void* stream);

/* Top-k rows of each block by score.  Writes the selected rows in ascending
 * order (ties go to the lower row), the inverse map rowmap[b, r] = position of
 * row r in index[b, :] or -1, and frob[b] = sqrt(sum of sumsq over the selected
 * rows).  Replaces torch.topk + the Frobenius norm of the gathered rows
 * (src/dionw/_matrix_step.py:172-176, src/dionw/_gram.py:85-86). */
int dionw_select_rows(const float* scores, const float* sumsq, int64_t blocks,
                      int64_t rows, int64_t k, int32_t* index, int32_t* rowmap,
                      float* frob, void* stream);

/* frob[b] = sqrt(sum_r sumsq[b, r]) for blocks that update every row. */
int dionw_block_norms(const float* sumsq, int64_t blocks, int64_t rows, float* frob,
                      void* stream);

/* For each listed row: x = half(src_row / (frob[b] + eps)) and, when
 * decay_rows != 0, src_row *= decay in place (error feedback).  index may be
 * NULL (every row, k == rows).  x is [blocks, k, ldx] in x_dtype (F16 or BF16;
 * BF16 also rounds the input first and scales the norm by norm_scale, the
 * form of src/dionw/_polar_express.py:88-92).  Replaces gather + mul +
 * scatter_ + normalise + cast (src/dionw/_matrix_step.py:176-179,
 * src/dionw/_gram.py:85-87). */
int dionw_pack_rows(float* src, const int32_t* index, const float* frob,
                    int64_t blocks, int64_t rows, int64_t k, int64_t cols,
                    float decay, int decay_rows, float eps, float norm_scale,
                    void* x, int x_dtype, int64_t ldx, void* stream);

/* out[b, c, r] = in[b, r, c] for 2-byte elements (tall blocks are iterated in
 * their wide orientation, src/dionw/_gram.py:83-84, :89). */
int dionw_transpose_2byte(const void* in, void* out, int64_t blocks, int64_t rows,
                          int64_t cols, int64_t ld_in, int64_t ld_out, void* stream);

/* ---- Newton-Schulz ------------------------------------------------------ */

/* Bytes of scratch dionw_newton_schulz needs for this problem. */
size_t dionw_newton_schulz_workspace_bytes(int64_t blocks, int64_t m, int64_t n, int kind);

/* Five quintic steps on wide or square [blocks, m, ldx] operands (m <= n),
 * already normalised and rounded to fp16 (GRAM) or bf16 (the other kinds);
 * x is overwritten; out receives bf16 [blocks, m, ldx].  out may alias x.
 * GRAM and GRAM_FULL follow gram_polar_express / _gram / _standard
 * (src/dionw/_gram.py:41-89) product by product (GRAM mirrors the m x m products
 * that are symmetric, GRAM_FULL computes them in full), with the symmetric products (ns_line_1, ns_line_2,
 * src/dionw/_symmetric_kernels.py:252-312) computed on one triangle of tiles
 * by tcgen05 tensor-core kernels fed by TMA.  POLAR_EXPRESS / KELLER follow
 * quintic_triton (src/dionw/_polar_express.py:74-104, src/dionw/_keller.py). */
/* rowsq (nullable, fp32 [blocks * m, dionw_newton_schulz_rowsq_parts(n)]): the
 * epilogue of the last product also writes, per output row, the sum of the
 * squares of its bf16 results over each 128 columns -- what normalize_rows
 * (src/dionw/_row_normalization.py:41-60) reduces the output to -- so NorMuon
 * needs no second pass over the output (dionw_normuon_rows adds the parts). */
int dionw_newton_schulz(void* x, void* out, int64_t blocks, int64_t m, int64_t n,
                        int64_t ldx, int kind, void* workspace, size_t workspace_bytes,
                        float* rowsq, void* stream);
/* Partial sums per output row that dionw_newton_schulz writes into rowsq. */
int64_t dionw_newton_schulz_rowsq_parts(int64_t n);

/* The same iteration for callers that have no scratch to give: a host bound to
 * this ABI without torch's allocator, a serving loop whose memory was budgeted at
 * start-up, a process whose device memory already belongs to a framework's pool,
 * a loop that may not stall on cudaMalloc/cudaFree.  The scratch is a fixed
 * DIONW_STATIC_SCRATCH_BYTES (64 MiB) array inside the library's device image: a
 * GPU holds it from the moment the CUDA runtime loads the image there (with lazy
 * module loading, as late as this entry's first call on that GPU) until the
 * process exits.  A problem whose dionw_newton_schulz_workspace_bytes() exceeds
 * it is refused with DIONW_ERR_WORKSPACE; the ceiling holds for operands with
 * ldx == n rounded up to 8, any other ldx is refused with DIONW_ERR_ARGUMENT.
 * The call allocates nothing.  Its first call on a device looks the array's
 * device address up (cudaGetSymbolAddress, with the current device) and may be
 * the call that loads the image, which fails with DIONW_ERR_CUDA if the GPU's
 * memory is already full: make that call once per device during set-up, before
 * memory pools are filled and before any stream capture is begun.  All calls on
 * a device share the one array, which keeps whatever the last call left in it
 * (nothing needs clearing: each product writes its output whole before it is
 * read); two calls that overlap on the GPU, e.g. on different streams, race on
 * it.  Arguments as dionw_newton_schulz (without the workspace and the row sums).
 * This entry has no counterpart in the reference. */
#define DIONW_STATIC_SCRATCH_BYTES (64u << 20)
int dionw_newton_schulz_static(void* x, void* out, int64_t blocks, int64_t m, int64_t n,
                               int64_t ldx, int kind, void* stream);

/* C = alpha * A B^T + beta * Cin for a product that is symmetric: computed on
 * the lower triangle of tiles and mirrored, so C is exactly symmetric; out2
 * (optional) = C + diag * I.  A and B are [blocks, m, ld] with kdim columns;
 * b == NULL means B = A.  dtype F16 or BF16 for every operand.  ns_line_1 is
 * b=NULL, alpha=1, beta=0, cin=NULL; ns_line_2 is A = Cin = the symmetric input
 * (src/dionw/_symmetric_kernels.py:252-312).  With B != A the caller asserts
 * that A B^T is symmetric (both symmetric and commuting, as the polynomials of
 * one Gram matrix at src/dionw/_gram.py:64-68 are). */
int dionw_symmetric_product(const void* a, const void* b, int64_t blocks, int64_t m,
                            int64_t kdim, int64_t lda, int64_t ldb, const void* cin,
                            int64_t ldc, float alpha, float beta, void* out, int64_t ldo,
                            void* out2, float diag, int dtype, void* stream);

/* C = A B + beta * Cin, A [blocks, m, lda] (m x kdim).  b_is_nk = 0: B is
 * [blocks, kdim, ldb] row-major (kdim x n); b_is_nk = 1: B is given as
 * [blocks, n, ldb] (n x kdim) and used transposed.  cin may be NULL (beta
 * ignored).  in_dtype F16/BF16; out_dtype F16/BF16 (torch.bmm / torch.baddbmm
 * at src/dionw/_gram.py:46,58,64,67-69). */
int dionw_batched_gemm(const void* a, int64_t lda, const void* b, int64_t ldb, int b_is_nk,
                       const void* cin, int64_t ldc, float beta, void* out, int64_t ldo,
                       int64_t blocks, int64_t m, int64_t n, int64_t kdim, int in_dtype,
                       int out_dtype, void* stream);

/* ---- NorMuon and the weight update -------------------------------------- */

/* s[b*k + r] = sum_c o[b, r, c]^2 for a bf16 batch [blocks, k, ldo] (used where
 * dionw_newton_schulz cannot hand the row sums over: tall blocks, which are
 * iterated transposed, and foreign orthogonalizers). */
int dionw_row_sumsq_bf16(const void* o, int64_t blocks, int64_t k, int64_t cols,
                         int64_t ldo, float* s, void* stream);

/* Per-row and per-block scales of NorMuon (normalize_rows,
 * src/dionw/_row_normalization.py:41-60): v <- lerp(v, s/cols, weight) written
 * back to variance[b, index[b, r]] (index NULL: row r); denom = sqrt(v) + eps;
 * scale[b] = ||O|| / max(||O/denom||, eps) * step.  normalize = 0 gives
 * denom = 1, scale = step and leaves variance alone
 * (RowNormalization.NONE, src/dionw/_row_normalization.py:35-36).
 * s is [blocks * k, parts]: a row's sum of squares is the sum of its parts,
 * taken left to right (parts = 1: dionw_row_sumsq_bf16's output).
 * step_device (nullable) overrides step with a value read from device memory,
 * as the reference keeps -step_size in a 0-d device tensor so that a scheduled
 * learning rate costs nothing (src/dionw/_buckets.py:57-58,
 * src/dionw/_row_normalization.py:48-49). */
int dionw_normuon_rows(const float* s, int64_t parts, float* variance, const int32_t* index,
                       int64_t blocks, int64_t rows, int64_t k, int64_t cols,
                       float weight, float eps, float step, const float* step_device,
                       int normalize, float* denom, float* scale, void* stream);

/* W <- W * decay_factor on every row (when has_decay), then
 * W[row] += (float(o[b, p, :]) / denom[b, p]) * scale[b] for each selected row
 * (p = rowmap[b, row] >= 0; rowmap NULL: every row, p = row).  Replaces _apply
 * / _add_blocks_ (src/dionw/_matrix_step.py:274-304). */
int dionw_apply_run(void* const* weights, const int64_t* rows_per_tensor, int n_tensors,
                    const void* o, int64_t ldo, const int32_t* rowmap, const float* denom,
                    const float* scale, int64_t rows, int64_t k, int64_t cols,
                    float decay_factor, int has_decay, void* stream);

/* The same update for tensors whose update rows do not lie in one buffer (a
 * round of the sharded step applies the contributions of every rank with one
 * launch): o[i], rowmap[i] (array or entries nullable), denom[i], scale[i] point
 * at the first block of tensor i.  decay_device (nullable) overrides
 * decay_factor with a value read from device memory (the reference's decay is
 * `1 - lr * wd` of the current lr, src/dionw/_matrix_step.py:280).  cta_warps
 * (0 = the default 8, else 1..8) sets the CTA size, one row per warp: CTAs of
 * four warps are small enough in registers to run beside a resident tensor-core
 * CTA, for a launch that overlaps the Newton-Schulz of the next round. */
int dionw_apply_round(void* const* weights, const int64_t* rows_per_tensor,
                      const void* const* o, const int32_t* const* rowmap,
                      const float* const* denom, const float* const* scale, int n_tensors,
                      int64_t ldo, int64_t rows, int64_t k, int64_t cols, float decay_factor,
                      const float* decay_device, int has_decay, int cta_warps,
                      const void* decay_job, void* stream);

/* A decay job: the decoupled decay of the UNSELECTED rows of a round's weights,
 * done by the tensor-core kernels' epilogue warps while they wait for their
 * accumulators, so that it runs beside the Newton-Schulz of the round instead
 * of after it (no counterpart in the reference, which decays with one
 * elementwise multiply, src/dionw/_matrix_step.py:280).  `job` is
 * dionw_decay_job_bytes() of 16-byte aligned device memory that must stay
 * untouched until the dionw_apply_round that is given the same pointer has run;
 * weights / rowmap / rows_per_tensor describe the round's tensors in the order
 * dionw_apply_round will get them (at most 64; every tensor needs a row map).
 * dionw_decay_job_begin writes the job (stream-ordered).  dionw_gemm_side_job(job)
 * makes the products launched by the calling thread from then on carry it
 * (NULL: none): a waiting epilogue warp draws up to rows_per_wait rows per tile
 * from the job's cursor and multiplies the unselected ones by the decay factor.
 * dionw_apply_round(..., decay_job = job, ...) then skips the unselected rows
 * below the cursor.  Each element is multiplied once, by the same factor: the
 * weights come out bit-identical to the update doing all of it. */
size_t dionw_decay_job_bytes(void);
int dionw_decay_job_begin(void* job, void* const* weights, const int32_t* const* rowmap,
                          const int64_t* rows_per_tensor, int n_tensors, int64_t rows,
                          int64_t cols, float decay_factor, const float* decay_device,
                          int rows_per_wait, void* stream);
void dionw_gemm_side_job(void* job);

/* dst[0..n) <- values[0..n) (host array), stream-ordered: the values are copied
 * into the launch, so the host array may be reused at once.  The step's scalars
 * (-step_size per bucket, 1 - lr*wd per group, lr and wd per AdamW group) live
 * in device memory so that a recorded step can be replayed under a learning-rate
 * schedule (src/dionw/_buckets.py:57-58 keeps them in 0-d device tensors). */
int dionw_write_scalars(float* dst, const float* values, int64_t n, void* stream);

/* ---- AdamW and EMA ------------------------------------------------------ */

/* Adds one to every fp32 step counter, then one fused decoupled-decay AdamW
 * update per tensor (bias-corrected, amsgrad off).  Replaces adamw_step
 * (src/dionw/_adamw.py:25-61: torch._foreach_add_ + torch._fused_adamw_). */
int dionw_adamw_multi(void* const* params, const void* const* grads, void* const* exp_avg,
                      void* const* exp_avg_sq, void* const* steps, const int64_t* numels,
                      int n_tensors, float lr, float beta1, float beta2, float weight_decay,
                      float eps, const float* hyper_device, void* stream);
/* hyper_device (nullable): {lr, weight_decay} read from device memory instead. */

/* shadow <- source (first = 1) or shadow += weight * (source - shadow) for
 * every tensor (weight = 1 - decay < 0.5 form of torch.lerp; else
 * source - (source - shadow) * (1 - weight)).  source_dtype F32/F16/BF16.
 * Replaces _finalize_gpu_updates / foreach_ema_update_
 * (src/dionw/ema/tracker.py:139-152, src/dionw/ema/_update.py:32-70). */
int dionw_ema_multi(void* const* shadows, const void* const* sources, const int64_t* numels,
                    int n_tensors, int source_dtype, float weight, int first, void* stream);

/* Gathers n tensors into one contiguous fp32 staging buffer on the device
 * (element offsets[i]); the caller then issues ONE device-to-host copy.
 * Replaces the per-parameter copies of _stage_cpu_snapshot
 * (src/dionw/ema/tracker.py:229-248). */
int dionw_ema_stage_pack(const void* const* sources, const int64_t* numels,
                         const int64_t* offsets, int n_tensors, int source_dtype,
                         float* staging, void* stream);

/* Host worker of the CPU EMA (AsyncCpuEmaJob, src/dionw/ema/_cpu_job.py:46-137):
 * start() spawns a thread that waits for `cuda_event` (a cudaEvent_t, may be
 * NULL), then for each of n segments copies (first[i] != 0) or lerps
 * shadow_i <- shadow_i + weight * (staged_i - shadow_i) on `threads` host threads.
 * wait_copy() returns once the event has completed, wait_update() once the
 * shadows are written; done() polls; destroy() joins and frees.  At most the
 * caller's one job at a time is expected, as in the reference. */
typedef struct dionw_cpu_ema_job dionw_cpu_ema_job;
dionw_cpu_ema_job* dionw_cpu_ema_job_start(float* const* shadows, const float* const* staged,
                                           const int64_t* numels, const uint8_t* first,
                                           int n, float weight, void* cuda_event, int threads);
int dionw_cpu_ema_job_wait_copy(dionw_cpu_ema_job* job);
int dionw_cpu_ema_job_wait_update(dionw_cpu_ema_job* job);
int dionw_cpu_ema_job_done(dionw_cpu_ema_job* job);
void dionw_cpu_ema_job_destroy(dionw_cpu_ema_job* job);

#ifdef __cplusplus
}
#endif
#endif /* DIONW_B200_H_ */
