/*
 * loopback_b200 -- C ABI of the B200 (sm_100a) kernels for Loopback's depth-attention residual read.
 *
 * Every entry point takes plain device pointers and sizes, launches on the CUDA stream it is given
 * (a cudaStream_t passed as void*; NULL = the default stream), never synchronises, never allocates device memory,
 * and returns LB_OK or a negative LB_ERR_* code; lb_last_error_string() describes the last failure of the calling
 * thread. There is no CPU fallback: on a machine without an sm_100 GPU every compute call fails with LB_ERR_CUDA.
 *
 * Shapes: n_tok = batch * sequence tokens; d = model width; N = K * R block applications ("steps") of one forward
 * pass; NQ = N - 1 read queries; a read at step s sees n = s + 1 stored updates and uses query row s - 1.
 * dtype selects the storage type of activations (LB_DTYPE_BF16 or LB_DTYPE_F32); all arithmetic is fp32.
 * Constraints: d * sizeof(element) is a multiple of 16 and at most 16384 bytes; activation pointers are 16-byte
 * aligned; n <= LB_MAX_SOURCES.
 *
 * Layouts (row-major, contiguous):
 *   V, dV   [N][n_tok][d]   storage dtype      the stack of updates / their gradients
 *   R, dR   [N][n_tok]      fp32               key scales rsqrt(mean(v^2) + eps) / their gradients
 *   DOTS    [NQ][N][n_tok]  fp32               cached scores q_j . V[s, t, :]; private to this library
 *   cbar, TC, LG, dcbar, gt  [n_tok][n] fp32;  LSE, LSE0 [n_tok] fp32;  c0 [n] fp32;  Q [NQ][d] fp32
 *
 * The reference interface each entry point replaces is cited by file:line of the reference project
 * (fused_dattn.py is the Triton implementation, looped_transformer.py the model with the reference read).
 */
#ifndef LOOPBACK_B200_H
#define LOOPBACK_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define LB_VERSION 1

#define LB_DTYPE_F32 0
#define LB_DTYPE_BF16 1

#define LB_MAX_SOURCES 128

#define LB_OK 0
#define LB_ERR_ARG (-1)          /* null pointer, negative size, n out of range ... */
#define LB_ERR_ALIGN (-2)        /* pointer or row size not 16-byte aligned */
#define LB_ERR_UNSUPPORTED (-3)  /* shape outside what the kernels cover (d too large, n > LB_MAX_SOURCES) */
#define LB_ERR_CUDA (-4)         /* a CUDA runtime/driver call failed (includes: no sm_100 device) */
#define LB_ERR_DEVICE (-5)       /* a kernel reported a bounded wait that ran out (lb_device_error) */

/* Library version (LB_VERSION of the build). */
int lb_version(void);

/* Message of the last error returned to the calling thread ("" if none). The pointer stays valid until the
 * thread's next failing call. */
const char *lb_last_error_string(void);

/* Reads (and, if clear != 0, resets) the current device's error word. 0 = no kernel gave up a wait; otherwise the
 * code of the first wait that ran out. SYNCHRONISES the device; meant for tests and for the end of a step. */
int lb_device_error(int clear);

/* Tuning knobs for sweeps: "fwd_stages", "bwd_stages" (TMA ring depth), "fwd_fr" (chunks per consumer warp),
 * "fwd_warps", "bwd_warps" (consumer warps per CTA: 8, 12 or 16), "bwd_wpt" (warps per token), "grid_cap" (CTAs),
 * "tma_per_chunk" (one 3-D box per chunk instead of one 4-D box per stage), "write_tt" (1 or 2: tokens per lane of the
 * tiled write kernel, whatever the batch size; 3: the tensor-core write kernel whatever the batch size),
 * "write_mt" (16-token tiles per consumer warp of the tensor-core write kernel: 1 or 2),
 * "write_tile" (tokens per tile of the tensor-core write kernel: a multiple of 32 up to 256), "write_stages" (its TMA
 * ring depth, 2..8), "fwd_sps" (sources per TMA stage of the forward read: 1, 2 or 4), "wait_cycles" (the limit of
 * every bounded wait inside the kernels, in GPU clock cycles; default 4e9), "test_skip_item" (test hook: the first
 * CTA of the next forward reads leaves out its k-th tile copy, so that a bounded wait runs out, the CTA unwinds and
 * lb_device_error reports it; nothing traps or hangs). Value 0 restores the default
 * (chosen by size); the name "reset_all" restores every knob. Returns LB_ERR_ARG for an unknown name.
 * The knobs are one process-wide table without a lock: set them from one thread, while no other thread is inside
 * a call of this library. */
int lb_set_option(const char *name, int value);

/* Update write: V[s] = round(h - x); R[s] = key scale of the rounded update; if Q != NULL also the cached scores
 * DOTS[j][s][:] = Q[j] . V[s] for the queries j >= max(s - 1, 0) (the reads that will see update s).
 * R may be NULL (then only V[s] is written and Q is ignored).
 * The scores are fp32 sums of exact products: on the fp32 pipes, or -- bf16 rows, at least 32 tokens per SM, at most
 * 32 queries -- as bf16 tensor-core products of the update with a three-term bf16 split of each fp32 query, summed in fp32.
 * Replaces DattnStack.write / _WriteDelta.forward and the kernel _write_stk_kernel (fused_dattn.py:561-585,
 * :663-691) and, when R is requested without Q, the scale kernel used by DattnStack.rstd (fused_dattn.py:698-708). */
int lb_write(const void *h, const void *x, void *V, float *R, const float *Q, float *DOTS, int64_t n_tok, int d, int N,
             int NQ, int s, float eps, int dtype, void *stream);

/* Gradient of the write for the block input: dx = -g (dh is g itself).
 * Replaces _WriteDelta.backward (fused_dattn.py:693-695). */
int lb_write_bwd_dx(const void *g, void *dx, int64_t n_elem, int dtype, void *stream);

/* Key scale of a free-standing update: r[t] = rsqrt(mean(x[t,:]^2) + eps).
 * Replaces rstd / _Rstd.forward and _rstd_fwd_kernel (fused_dattn.py:206-215, :232-243, :257-261). */
int lb_rstd_fwd(const void *x, float *r, int64_t n_tok, int d, float eps, int dtype, void *stream);

/* Gradient of the key scale, written: gx = gr * (-r^3 / d) * x.
 * Replaces _Rstd.backward and _rstd_bwd_kernel (fused_dattn.py:218-229, :245-254). */
int lb_rstd_bwd(const void *x, const float *r, const float *gr, void *gx, int64_t n_tok, int d, int dtype,
                void *stream);

/* Gradient of the key scale, accumulated: dv = round(dv + round(gr * (-r^3 / d) * x)) in the storage dtype.
 * Replaces _RstdStk.backward and _rstd_bwd_acc_kernel (fused_dattn.py:539-552, :711-722). */
int lb_rstd_bwd_acc(const void *x, const float *r, const float *gr, void *dv, int64_t n_tok, int d, int dtype,
                    void *stream);

/* Scores of one query against the first n updates of a stack whose writes did not cache them:
 * dots[i][t] = q . V[i, t, :], dots laid out [N][n_tok] (one query block of DOTS, or caller scratch).
 * Replaces the score half of the online read kernel _dattn_fwd_stk_kernel (fused_dattn.py:426-433). */
int lb_scores(const void *V, const float *q, float *dots, int64_t n_tok, int d, int N, int n, int dtype, void *stream);

/* Forward read at step s = n - 1 from cached scores (query row qi of DOTS):
 *   l_i = DOTS[qi][i] * R[i] / sqrt(d) + log(max(c0_i, 1e-8));  p = softmax(l);  p0 = softmax(log-prior)
 *   TC_i = c0_i + sum(c0) * (p_i - p0_i);   out = base + sum_i (TC_i - cbar_i) * V[i]
 * Saves LG (= l), LSE, LSE0 for the backward when they are non-NULL (all three or none).
 * Replaces FusedDattnReadStk.forward with its host preparation and the kernels _dattn_fwd_dots_kernel /
 * _dattn_fwd_stk_kernel (fused_dattn.py:729-759, :588-625, :410-456); the reference read it reproduces is
 * LoopDeltaAttnRes.combine (looped_transformer.py:410-424). */
int lb_read_fwd(const void *V, const float *R, const float *DOTS, int qi, const void *base, const float *cbar,
                const float *c0, void *out, float *TC, float *LG, float *LSE, float *LSE0, int64_t n_tok, int d, int N,
                int n, int dtype, void *stream);

/* One whole forward step in one launch, for decode-sized batches (tens to hundreds of tokens, where a step is bound by
 * launches, not bytes): the write of update s = what lb_write(h, x, ..., s) stores in V[s] and R[s], and the read that
 * follows it = lb_combine_fwd with n = s + 1 and the query row s - 1 of Q [N-1][d], the new update never leaving the
 * chip in between. No cached scores are needed or written (DOTS is not an argument): the stored updates, which at
 * these sizes live in L2, are swept twice, once for the scores and once for the weighted sum. Results agree
 * with lb_write + lb_combine_fwd to fp32 round-off (another summation order); V[s] is bit-identical; a zero query
 * with cbar == c0 gives out == base and TC == c0 bit for bit. One CTA per token: use it for batches that cannot fill
 * the GPU with token tiles. h0 == NULL: base = h; else base = h + beta (h0 - h) as in lb_combine_fwd.
 * Replaces the reference's per-step pair DattnStack.write + FusedDattnReadStk.forward with their kernels
 * _write_stk_kernel and _dattn_fwd_stk_kernel (fused_dattn.py:561-585, :410-456, :663-691, :729-759), called back to
 * back by the model (modeling_looped_transformer.py:472-481). */
int lb_step_fwd(const void *h, const void *x, const void *h0, float beta, void *V, float *R, const float *Q,
                const float *tc_prev, float lam, const float *c0, void *out, float *TC, float *LG, float *LSE, float *LSE0,
                int64_t n_tok, int d, int N, int s, float eps, int dtype, void *stream);

/* Bytes of scratch lb_read_bwd needs for the per-CTA partial rows of the query gradient (depends on d only). */
size_t lb_read_bwd_scratch_bytes(int d);

/* Backward read: from g = dL/dout [n_tok][d] and gt = dL/dTC [n_tok][n] (NULL = zeros) and the forward's saves,
 *   dq [d] (written), dcbar [n_tok][n] (written), dV[i], dR[i] for i < n (written if accum == 0, else added into,
 *   with the storage-dtype rounding of an in-place autograd add). dL/dbase is g itself.
 * `scratch` must hold lb_read_bwd_scratch_bytes(d) bytes; it is fully overwritten.
 * Replaces FusedDattnReadStk.backward, the kernels _dattn_bwd1_stk_kernel / _dattn_bwd2_stk_kernel and the torch
 * reduction of the query-gradient partials (fused_dattn.py:761-793, :459-536). */
int lb_read_bwd(const void *V, const float *R, void *dV, float *dR, const float *q, const void *g, const float *gt,
                const float *cbar, const float *c0, const float *LG, const float *LSE, const float *LSE0, float *dcbar,
                float *dq, void *scratch, int64_t n_tok, int d, int N, int n, int accum, int dtype, void *stream);

/* lb_read_bwd that also finishes the gradient of the newest source (index n - 1), for the read that is the last, in
 * backward order, to touch it: after adding its own contribution it adds the term that reaches the update through
 * its key scale, dV[n-1] = round(dV[n-1] + round(dR[n-1] * (-R[n-1]^3 / d) * V[n-1])) with the complete dR[n-1], and,
 * if neg_out != NULL, writes -dV[n-1] ([n_tok][d], storage dtype) there: the gradient of the block input.
 * Fuses _RstdStk.backward / _rstd_bwd_acc_kernel and _WriteDelta.backward into the read's backward
 * (fused_dattn.py:539-552, :711-722, :693-695): same values, two passes over the update less. */
int lb_read_bwd_final(const void *V, const float *R, void *dV, float *dR, const float *q, const void *g,
                      const float *gt, const float *cbar, const float *c0, const float *LG, const float *LSE,
                      const float *LSE0, float *dcbar, float *dq, void *scratch, void *neg_out, int64_t n_tok, int d,
                      int N, int n, int accum, int dtype, void *stream);

/* lb_read_fwd with the caller's prologue folded in (LoopDeltaAttnRes.combine, looped_transformer.py:380-391):
 *   base = proposal                                   when h0 == NULL (a read inside an iteration)
 *        = proposal + beta * (h0 - proposal)          at the end of an iteration, each operation rounded to the storage
 *                                                     dtype as the caller's tensor arithmetic would round it
 *   cbar = lam * (tc_prev, 1)                         tc_prev [n_tok][n-1] = the previous read's TC; lam = 1 or 1 - beta
 * Needs n >= 2. Everything else as lb_read_fwd. */
int lb_combine_fwd(const void *V, const float *R, const float *DOTS, int qi, const void *proposal, const void *h0,
                   float beta, const float *tc_prev, float lam, const float *c0, void *out, float *TC, float *LG,
                   float *LSE, float *LSE0, int64_t n_tok, int d, int N, int n, int dtype, void *stream);

/* Backward of lb_combine_fwd: as lb_read_bwd / lb_read_bwd_final (finalize != 0, neg_out may be NULL), with the
 * installed coefficients given as (tc_prev, lam) and dtc_prev [n_tok][n-1] = dL/d tc_prev written instead of dcbar.
 * dL/d base is g; the caller applies the blend's factors (1 - beta to the proposal, beta to h0). */
int lb_combine_bwd(const void *V, const float *R, void *dV, float *dR, const float *q, const void *g, const float *gt,
                   const float *tc_prev, float lam, const float *c0, const float *LG, const float *LSE,
                   const float *LSE0, float *dtc_prev, float *dq, void *scratch, void *neg_out, int finalize,
                   int64_t n_tok, int d, int N, int n, int accum, int dtype, void *stream);

/* The backward of one whole step -- the write of update n-1 and the read that follows it -- for callers that make
 * the two one autograd node: lb_combine_bwd with finalize, handing out the step's own gradients instead of dV[n-1]:
 *   dx  [n_tok][d] = -dV[n-1]                      the gradient of the block input (the write's x)
 *   dh  [n_tok][d] = round(dV[n-1] + dbase/dh)     the gradient of the block output: the finished gradient of the
 *                    update plus what reaches it as the read's base: g inside an iteration (blend == 0); at an
 *                    iteration's end (blend != 0, base = h + beta (h0 - h)) g - round(beta g), as autograd forms it
 *   dh0 [n_tok][d] or NULL: the blend's gradient of h0, round(beta g): written when dh0_accum == 0, else added to what
 *                    dh0 holds with the storage-dtype rounding of an in-place add (a pass's reads, last to first,
 *                    build the loop input's gradient in one buffer)
 * dV[n-1] itself is not stored (no later backward reads it); dV[i], dR[i] for i < n-1, dtc_prev and dq as
 * lb_combine_bwd. Replaces, on top of what lb_combine_bwd replaces, _WriteDelta.backward and the autograd
 * accumulation of the block output's two gradients (fused_dattn.py:693-695) and the blend's backward
 * (modeling_looped_transformer.py:148-149). */
int lb_step_bwd(const void *V, const float *R, void *dV, float *dR, const float *q, const void *g, const float *gt,
                const float *tc_prev, float lam, const float *c0, const float *LG, const float *LSE, const float *LSE0,
                float *dtc_prev, float *dq, void *scratch, void *dh, void *dx, void *dh0, int dh0_accum, int blend,
                float beta, int64_t n_tok, int d, int N, int n, int accum, int dtype, void *stream);

/* lb_step_bwd without a gradient stack. The plain forms add every read's contribution into dV[i] as the reads'
 * backwards run (each source row read and written once per later read: N^2 row transfers per pass). This form defers:
 * the backward of step s = n - 1 keeps its upstream gradient (G[s] = g, a stack like V) and, per older source i and
 * token, the two scalars of its contribution (Wt[s][i], KQt[s][i]: the coefficients of g and of the step's query), and
 * forms the finished gradient of ITS OWN update in one go from what the backward steps before it left:
 *   dV_s = sum over s' >= s of (Wt[s'][s] G[s'] + KQt[s'][s] Q[s'-1]) + the key-scale term,   fp32, rounded once
 * (N^2 / 2 row reads, no gradient row written except the outputs). Outputs, blend and dh0 exactly as lb_step_bwd; dR is
 * still accumulated in place (first != 0: written). The step-1 backward (n == 2) also finishes update 0, which has no
 * step of its own: dv0 receives its gradient (key-scale term included), dx0 the negation; NULL otherwise.
 * G [N][n_tok][d] storage dtype; Wt, KQt [N][N][n_tok] fp32; Q [N-1][d] fp32 (every query; this step's is row n - 2);
 * Qp = the same queries in the order the kernel's lanes read them from shared memory, made once per pass by
 * lb_permute_queries ([N-1][lb_permuted_query_row_floats(d, dtype)] fp32).
 * Every backward step of a pass must use this form, last step first, for the sums to be complete.
 * More accurate than the in-place accumulation it replaces (autograd's, fused_dattn.py:528-531, rounds after every
 * add); same reference code replaced as lb_step_bwd. */
size_t lb_permuted_query_row_floats(int d, int dtype);
int lb_permute_queries(const float *Q, float *Qp, int NQ, int d, int dtype, void *stream);
int lb_step_bwd_deferred(const void *V, const float *R, void *G, float *dR, float *Wt, float *KQt, const float *Q,
                         const float *Qp, const void *g, const float *gt, const float *tc_prev, float lam, const float *c0, const float *LG,
                         const float *LSE, const float *LSE0, float *dtc_prev, float *dq, void *scratch, void *dh, void *dx,
                         void *dh0, int dh0_accum, int blend, float beta, void *dv0, void *dx0, int64_t n_tok, int d, int N,
                         int n, int first, int dtype, void *stream);

/* The widest row lb_read_bwd_noalloc accepts. */
#define LB_NOALLOC_MAX_D 3072

/* lb_read_bwd without the `scratch` argument, for callers that are not able to allocate device memory (a runtime
 * that plans all its memory up front and forbids allocation afterwards, a plugin host that only passes the tensors
 * of the current call). The partial rows of the query gradient go to a fixed array inside the library instead
 * (about 3.6 MiB, resident on every GPU that uses the library, until the process exits). Arguments, results and
 * rounding are exactly those of lb_read_bwd. It allocates nothing and calls no allocating routine.
 * Limits: d <= LB_NOALLOC_MAX_D, otherwise LB_ERR_UNSUPPORTED; all calls on a device share the array, so calls that
 * overlap in time on that GPU race (serialise them on one stream; nothing needs clearing between calls); the first
 * call on a device resolves the array's device address and should be made outside any stream capture.
 * This entry point has no counterpart in the reference. */
int lb_read_bwd_noalloc(const void *V, const float *R, void *dV, float *dR, const float *q, const void *g,
                        const float *gt, const float *cbar, const float *c0, const float *LG, const float *LSE,
                        const float *LSE0, float *dcbar, float *dq, int64_t n_tok, int d, int N, int n, int accum,
                        int dtype, void *stream);

/* The most ranks lb_peer_allreduce serves (the GPUs of one NVLink node). */
#define LB_MAX_PEERS 16

/* 32-bit words of the flag block every rank provides to lb_peer_allreduce (zeroed once, before the first call of any
 * rank; never touched by the host afterwards). */
int lb_peer_flag_words(void);

/* One-shot all-reduce (fp32 sum) of the query gradient over the GPUs of one node through peer memory: the pass's
 * last backward leaves each rank's (N - 1, d) gradient in bufs[rank]; this one small launch per rank then sums all
 * ranks' buffers in rank order (every rank gets the same bits) into `out`.
 *   bufs, flags  HOST arrays of `world` DEVICE pointers, rank-ordered: every rank's gradient buffer (n floats) and
 *                flag block (lb_peer_flag_words() words), addressable from this GPU (peer-mapped: CUDA IPC or
 *                symmetric memory); bufs[rank] / flags[rank] are this rank's own
 *   out          [n] local result; n a multiple of 4; all ranks pass the same n
 * The ranks' kernels wait on one another (plain flag words, ld.acquire.sys / st.release.sys; no multicast), so each
 * rank needs a GPU of its own. Every wait is bounded by the "wait_cycles" option: a rank whose peer does not arrive
 * records error 6 in the device error word (lb_device_error), skips its sum and returns. When the launch has
 * completed, no peer reads bufs[rank] any more: the next pass may overwrite it. The call counter lives in the flag
 * block, so the launch can be captured in a CUDA graph and replayed.
 * Replaces the reduce-scatter FSDP issues for query.grad (trainer/flame/models/parallelize_fla.py:549-554) and the
 * NCCL all-reduce of loopback_b200.dist.allreduce_query_grad. */
int lb_peer_allreduce(const float *const *bufs, unsigned int *const *flags, int rank, int world, float *out, int64_t n,
                      void *stream);

#ifdef __cplusplus
}
#endif
#endif /* LOOPBACK_B200_H */
