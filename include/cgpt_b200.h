/*
 * cgpt_b200 -- C ABI of the B200 (sm_100a) training hot path for CGPT.
 *
 * Every function is `extern "C"`, takes raw DEVICE pointers, plain integer sizes, option scalars and
 * a CUDA stream (passed as `void*` so the header needs no CUDA include), is asynchronous on that
 * stream unless stated otherwise, and returns an int status:
 *      0  CGPT_OK
 *    > 0  an argument error class (CGPT_ERR_*); nothing was launched
 *    < 0  the negated cudaError_t of the CUDA runtime/driver call that failed
 * Nothing throws, nothing calls exit(). The C++ shim that re-creates CGPT's own `Tensor&` functions
 * on top of this ABI turns CGPT_ERR_* into std::invalid_argument, as CGPT's validators do.
 *
 * All tensors are contiguous row-major. `dtype` is one of CGPT_DTYPE_* and applies to every
 * floating-point tensor of the call unless a parameter says otherwise (CGPT uses one storage dtype
 * per op, see `include/core/dtype.h:12-21` of the reference; the numeric codes are the same).
 *
 * Scratch memory: ops that need global scratch take it from a per-device arena inside the library,
 * grown with cudaMalloc on first use of a given size. Run each op once eagerly before capturing it
 * in a CUDA graph (CGPT's trainer does exactly that, `train/train.cpp:545-548`).
 */
#ifndef CGPT_B200_H_
#define CGPT_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define CGPT_DTYPE_F16 0
#define CGPT_DTYPE_BF16 1
#define CGPT_DTYPE_F32 2

#define CGPT_OK 0
#define CGPT_ERR_NULL 1      /* a required pointer is NULL */
#define CGPT_ERR_DTYPE 2     /* unsupported dtype for this op */
#define CGPT_ERR_SHAPE 3     /* zero / inconsistent / overflowing dimensions */
#define CGPT_ERR_OPTION 4    /* invalid option scalar (epsilon <= 0, beta outside [0,1), ...) */
#define CGPT_ERR_ALIGN 5     /* pointer not aligned to the element size */
#define CGPT_ERR_UNSUPPORTED 6 /* valid for CGPT but outside what this build implements */
#define CGPT_ERR_STATE 7     /* object used in a state it does not allow (changed entry list, ...) */
#define CGPT_ERR_DEVICE 8    /* device-side bounded wait ran out (status word set by a kernel) */

typedef void* cgpt_stream_t; /* a cudaStream_t */

/* Library / build information. Returns a static string such as "cgpt_b200 sm_100a". */
const char* cgpt_b200_version(void);
/* Number of kernel launches issued by this library in the calling process since load (a host-side
 * counter incremented next to every `<<<>>>`); bench.py reports the difference over the timed
 * region. */
uint64_t cgpt_b200_launch_count(void);

/* Reads (and with clear != 0 resets) the device status word of the tensor-core kernels. Every wait in
 * those kernels (on an mbarrier fed by TMA or by tcgen05.commit) is bounded; a kernel whose wait ran out
 * sets the word to non-zero and returns. Synchronises the device. */
int cgpt_b200_device_status(unsigned int* status_out, int clear);
/* The transformer block's attention branch and MLP branch are independent until the block's last operation (parallel
 * residual; reference src/core/transformer_block.cu:466-595, :644-748 issues them one after the other on one stream).
 * When enabled, cgpt_block_forward / cgpt_block_backward (and the model functions built on them) issue the MLP branch on
 * a side stream owned by the library, forked from and joined back into the caller's stream with events, so that the memory-bound
 * kernels of one branch run underneath the tensor-core kernels of the other. Under stream capture the fork and join
 * become graph edges. The side stream is created by the first call on a device, which must therefore be made outside
 * of a capture (a first call inside a capture runs both branches on the caller's stream). enable = 0 (the initial
 * state unless the environment variable CGPT_B200_BRANCH_STREAMS=1 is set) keeps both branches on the caller's stream:
 * the 104m training step is power-capped on B200 and gained only 0.3-0.6 % from the overlap. */
int cgpt_b200_set_branch_streams(int enable);

/* Measurement aid for benchmarks: with enable != 0 the library records a CUDA event pair around every
 * tensor-core GEMM launch (eager mode only; do not enable while capturing a graph) together with the
 * launch's algorithmic FLOPs (2*m*n*k); cgpt_b200_gemm_timing_read synchronises the device and returns the
 * summed kernel milliseconds, FLOPs and launch count since enabling. */
int cgpt_b200_gemm_timing(int enable);
int cgpt_b200_gemm_timing_read(double* total_ms, double* total_flops, uint64_t* launches);
/* Pre-sizes the per-device scratch arena so that later ops (and CUDA graphs that captured them) never
 * see it move. Call outside stream capture. */
int cgpt_b200_reserve_scratch(size_t bytes);

/* ------------------------------------------------------------------------------------------------
 * Linear layer Y = X W^T and its backward, fp32 accumulation.
 * Replaces linear_forward (reference include/ops/linear.h:30-56, src/ops/linear.cu: cuBLASLt) and
 * linear_backward (reference include/ops/backward/linear_backward.h:10-46,
 * src/ops/backward/linear_backward.cu:135-148,181-200,268-285: two cuBLASLt GEMMs + a bias reduction):
 *      dX[rows,in] = dY[rows,out] W[out,in];  dW[out,in] = dY^T X;  db[out] = sum_rows dY.
 * dx, dw or db may be NULL to skip that product (the reference always computes all three; CGPT's model
 * has no biases). accumulate_* != 0 adds to the existing output (read in storage dtype, added in fp32,
 * rounded once), as the reference's beta = 1.
 * 16-bit dtypes run on the tensor cores (tcgen05 + TMA) when bases are 16-byte aligned and in/out
 * features are multiples of 8; everything else (fp32 tensors, odd shapes) runs a plain fp32 SIMT kernel.
 *
 * cgpt_gemm is the underlying contraction C[m,n] (+)= A B: a_layout 0 = A stored [m,k], 1 = [k,m];
 * b_layout 0 = B stored [n,k], 1 = [k,n]; force_simt != 0 selects the SIMT kernel (for tests).
 * ---------------------------------------------------------------------------------------------- */
int cgpt_gemm(void* c, const void* a, const void* b, size_t m, size_t n, size_t k, int a_layout,
              int b_layout, int accumulate, int dtype, int force_simt, cgpt_stream_t stream);
int cgpt_linear_forward(void* y, const void* x, const void* w, size_t rows, size_t in_features,
                        size_t out_features, int dtype, cgpt_stream_t stream);
int cgpt_linear_backward(void* dx, void* dw, void* db, const void* dy, const void* x, const void* w,
                         size_t rows, size_t in_features, size_t out_features, int accumulate_input,
                         int accumulate_weight, int accumulate_bias, int dtype, cgpt_stream_t stream);

/* `count` (1..3) projections of the same input as one launch: y_i[rows,out_i] = x[rows,in] W_i[out_i,in]^T.
 * Replaces consecutive linear_forward calls on one input (reference src/core/transformer_block.cu:496-510: query, key
 * and value projections): one work list over all output tiles fills the SMs better than three launches whose tile
 * counts are not multiples of the SM count. Results are bit-identical to the separate calls. y, w: host arrays of
 * `count` device pointers. Runs as separate calls when the tensor-core path does not apply (fp32, unaligned, tiny). */
int cgpt_linear_forward_fused(void* const* y, const void* x, const void* const* w, const size_t* out_features,
                              size_t count, size_t rows, size_t in_features, int dtype, cgpt_stream_t stream);

/* Weight gradients of `count` (1..3) projections of the same input as one launch:
 *      dW_i[out_i,in] (+)= dY_i[rows,out_i]^T X[rows,in].
 * Replaces consecutive linear_backward calls that share `input` (reference src/core/transformer_block.cu:669-675 gate/up,
 * :726-744 q/k/v): the output tiles of all products form one work list, so small products (key/value projections of a
 * grouped-query model) no longer run as launches of their own, each with its own K split and reduction.
 * dw, dy: host arrays of `count` device pointers. Runs as separate products when the tensor-core path does not apply. */
int cgpt_linear_backward_weight_fused(void* const* dw, const void* const* dy, const void* x, const size_t* out_features,
                                      size_t count, size_t rows, size_t in_features, int accumulate_weight, int dtype,
                                      cgpt_stream_t stream);

/* Gate and up projections with the SwiGLU activation in the GEMM epilogue:
 *      gate = X Wg^T, up = X Wu^T, activated = gate / (1 + exp(-gate)) * up      (all [rows, intermediate]).
 * Replaces the sequence linear_forward, linear_forward, swiglu_forward of the block forward (reference
 * src/core/transformer_block.cu:566-579, src/ops/swiglu.cu:69-71) with one launch: both projections are rounded to the
 * storage dtype and written (the backward pass reads them), and the activation is computed from the rounded values, so
 * results equal the three-call sequence. Runs as that sequence when the tensor-core path does not apply (fp32, unaligned). */
int cgpt_linear_swiglu_forward(void* gate, void* up, void* activated, const void* x, const void* w_gate, const void* w_up,
                               size_t rows, size_t in_features, size_t intermediate, int dtype, cgpt_stream_t stream);

/* Input gradient of `count` (1..3) projections that read the same input, in one pass:
 *      dX[rows,in] (+)= sum_i dY_i[rows,out_i] W_i[out_i,in].
 * No single counterpart in the reference: it is what the block backward obtains from consecutive
 * linear_backward calls whose later ones accumulate into grad_input (reference src/core/transformer_block.cu:
 * 669-675 for gate/up, 726-744 for q/k/v). The sum over i stays in the fp32 accumulator, so dX is rounded to the
 * storage dtype once instead of after every projection. dy, w: arrays of `count` device pointers (host arrays);
 * out_features: `count` sizes. Falls back to one SIMT launch per projection for fp32 or unaligned operands. */
int cgpt_linear_backward_input_fused(void* dx, const void* const* dy, const void* const* w,
                                     const size_t* out_features, size_t count, size_t rows, size_t in_features,
                                     int accumulate_input, int dtype, cgpt_stream_t stream);
/* Sum of `count` (1..3) projections into the same output, plus an optional residual, in one pass:
 *      Y[rows,out] = R[rows,out] + sum_i X_i[rows,in_i] W_i[out,in_i]^T.
 * No single counterpart in the reference: it is the end of the parallel-residual block, where the reference runs the
 * output projection, the down projection and two in-place adds (src/core/transformer_block.cu:541-546, 580-595). The
 * products share the fp32 accumulator and the residual is added to it before the one rounding to the storage dtype.
 * x, w: arrays of `count` device pointers (host arrays); in_features: `count` sizes; residual may be NULL. Y may alias
 * R only where the tensor-core epilogue adds it (16-bit, out % 64 == 0, rows >= 256): otherwise the product is written
 * first and R added by an elementwise pass, and aliasing returns CGPT_ERR_OPTION. */
int cgpt_linear_forward_sum(void* y, const void* const* x, const void* const* w, const size_t* in_features,
                            size_t count, size_t rows, size_t out_features, const void* residual, int dtype,
                            cgpt_stream_t stream);

/* ------------------------------------------------------------------------------------------------
 * Grouped-query softmax attention, forward with saved log-sum-exp and backward.
 * Replaces flash_gqa_attention_forward_with_lse (reference include/ops/attention.h:60-81,
 * src/ops/attention.cu), flash_gqa_attention_backward_with_lse and flash_gqa_attention_backward
 * (reference include/ops/backward/attention_backward.h:24-35,57-70,
 * src/ops/backward/attention_backward.cu:1914-2069).
 * q, out, dout, dq: [batch, sq, hq, head_dim]; k, v, dk, dv: [batch, sk, hkv, head_dim];
 * lse: fp32 [batch, sq, hq] = log sum exp of the scaled scores (natural log). hq % hkv == 0.
 * Key k is visible to query q iff !causal or k <= offset + q (causal requires offset + sq <= sk).
 * scale <= 0 selects 1/sqrt(head_dim).
 *   P = exp(scale QK^T - lse); delta = rowsum(dout*out); dS = P (dout V^T - delta);
 *   dq = scale dS K; dk = scale dS^T Q; dv = P^T dout.   accumulate != 0 adds into dq, dk, dv.
 * Backward with out == NULL or lse == NULL recomputes the forward statistics first (the reference's
 * flash_gqa_attention_backward). 16-bit tensors with head_dim 64 or 128 run on the tensor cores;
 * everything else (and force_generic != 0) runs a warp-per-row kernel. No atomics: bit-reproducible.
 * ---------------------------------------------------------------------------------------------- */
int cgpt_attention_forward(void* out, float* lse, const void* q, const void* k, const void* v,
                           size_t batch, size_t sq, size_t sk, size_t hq, size_t hkv, size_t head_dim,
                           float scale, int causal, size_t offset, int dtype, int force_generic,
                           cgpt_stream_t stream);
int cgpt_attention_backward(void* dq, void* dk, void* dv, const void* dout, const void* out,
                            const float* lse, const void* q, const void* k, const void* v, size_t batch,
                            size_t sq, size_t sk, size_t hq, size_t hkv, size_t head_dim, float scale,
                            int causal, size_t offset, int accumulate, int dtype, int force_generic,
                            cgpt_stream_t stream);

/* ------------------------------------------------------------------------------------------------
 * RMSNorm  y = x * rsqrt(mean(x^2) + eps) * w
 * Replaces rmsnorm_forward  (reference include/ops/rmsnorm.h:36-52, src/ops/rmsnorm.cu:812-906)
 *      and rmsnorm_backward (reference include/ops/backward/rmsnorm_backward.h:21-29,
 *                            src/ops/backward/rmsnorm_backward.cu:529-547).
 * x, y, dy, dx: [rows, hidden]; w, dw: [hidden]. fp32 math, one rounding on store.
 * Backward overwrites dx and dw:  inv = rsqrt(mean(x^2)+eps); c = sum(dy*w*x) * inv^3 / hidden;
 *      dx = dy*w*inv - x*c (+ residual_a + residual_b when given);  dw = sum_rows dy*x*inv.
 * residual_a / residual_b (may be NULL) are [rows, hidden] tensors added to dx in fp32 before the
 * single rounding: they fold the reference's `add_inplace` passes
 * (src/core/transformer_block.cu:678-681,747) into this kernel. dx may be the same buffer as residual_a or
 * residual_b (each element is read before it is written, by the same thread); it may not alias dy or x.
 * ---------------------------------------------------------------------------------------------- */
int cgpt_rmsnorm_forward(void* y, const void* x, const void* w, size_t rows, size_t hidden,
                         float epsilon, int dtype, cgpt_stream_t stream);
int cgpt_rmsnorm_backward(void* dx, void* dw, const void* dy, const void* x, const void* w,
                          const void* residual_a, const void* residual_b, size_t rows,
                          size_t hidden, float epsilon, int dtype, cgpt_stream_t stream);

/* RMSNorm backward that never allocates. No counterpart in the reference: it exists for hosts that
 * cannot call the device allocator at call time (a process whose pool allocator owns all device memory,
 * a latency-critical loop that may not take the allocator's lock, a sandbox that filters allocator
 * calls). Arguments, results and error codes are those of cgpt_rmsnorm_backward; the [grid, hidden] fp32
 * partial sums live in a fixed 4 MiB array inside the library image (present on every GPU that loads
 * the library, for the life of the process). Limits: hidden <= 8192, otherwise CGPT_ERR_SHAPE. The first
 * call on a device resolves the array's device address and should be made outside stream capture.
 * Calls share the array: order them on one stream; calls that overlap on the GPU race on it. */
int cgpt_rmsnorm_backward_noalloc(void* dx, void* dw, const void* dy, const void* x, const void* w,
                                  const void* residual_a, const void* residual_b, size_t rows,
                                  size_t hidden, float epsilon, int dtype, cgpt_stream_t stream);
/* Both RMSNorms of a parallel-residual block's input in one pass (the attention branch's and the MLP branch's norm read
 * the same x and share rsqrt(mean(x^2) + eps); reference src/core/transformer_block.cu:483-487, :556-560 forward and
 * :678-681, :745-747 backward, where they are separate calls plus a copy and two in-place adds):
 *   forward   y_a = rmsnorm(x; w_a), y_b = rmsnorm(x; w_b)
 *   backward  dx = residual + rmsnorm_backward(dy_a; x, w_a) + rmsnorm_backward(dy_b; x, w_b), dw_a, dw_b
 * with the three terms of dx summed in fp32 and rounded once. residual may be NULL; dx may alias it. 16-bit rows of
 * 256..1024 elements take the one-pass kernels, every other shape runs the single-norm operators one after the other. */
int cgpt_rmsnorm_forward_dual(void* y_a, void* y_b, const void* x, const void* w_a, const void* w_b, size_t rows,
                              size_t hidden, float epsilon, int dtype, cgpt_stream_t stream);
int cgpt_rmsnorm_backward_dual(void* dx, void* dw_a, void* dw_b, const void* dy_a, const void* dy_b, const void* x,
                               const void* w_a, const void* w_b, const void* residual, size_t rows, size_t hidden,
                               float epsilon, int dtype, cgpt_stream_t stream);

/* ------------------------------------------------------------------------------------------------
 * RoPE on adjacent pairs (x[2p], x[2p+1]) of the first rotary_dim dims of each head, angle index
 * (position_offset + s, p), tables [max_seq, rotary_dim/2] in the tensors' dtype.
 * Replaces rope_forward (reference include/ops/rope.h:13-39, in place on q and k) and rope_backward
 * (reference include/ops/backward/rope_backward.h:22-31, src/ops/backward/rope_backward.cu:318-389).
 * q-like tensors [batch, seq, q_heads, head_dim], k-like [batch, seq, kv_heads, head_dim].
 * Backward: dx0 = dy0*c + dy1*s, dx1 = -dy0*s + dy1*c; dims >= rotary_dim are copied. In-place
 * (dq == dq_rot) is allowed. rotary_dim == 0 means head_dim.
 * ---------------------------------------------------------------------------------------------- */
int cgpt_rope_forward(void* q, void* k, const void* cos_table, const void* sin_table, size_t batch,
                      size_t seq, size_t q_heads, size_t kv_heads, size_t head_dim,
                      size_t rotary_dim, size_t position_offset, size_t max_seq, int dtype,
                      cgpt_stream_t stream);
int cgpt_rope_backward(void* dq, void* dk, const void* dq_rot, const void* dk_rot,
                       const void* cos_table, const void* sin_table, size_t batch, size_t seq,
                       size_t q_heads, size_t kv_heads, size_t head_dim, size_t rotary_dim,
                       size_t position_offset, size_t max_seq, int dtype, cgpt_stream_t stream);

/* Fused per-head QK-RMSNorm + RoPE: one pass instead of the reference's rmsnorm_forward(q), rmsnorm_forward(k),
 * rope_forward sequence (src/core/transformer_block.cu:496-521) and, backward, rope_backward, rmsnorm_backward(q),
 * rmsnorm_backward(k) (:705-720). q_pre/k_pre are the projections before the norm ([batch, seq, heads, head_dim]),
 * q_norm/k_norm the [head_dim] weights; rounding points are the reference's (the normalised value / the un-rotated
 * gradient are rounded to the storage dtype between the two stages). 16-bit dtypes, head_dim a power of two in
 * [8, 256], rotary_dim a multiple of 8; otherwise CGPT_ERR_UNSUPPORTED (callers then use the separate ops). */
int cgpt_qknorm_rope_forward(void* q, void* k, const void* q_pre, const void* k_pre, const void* q_norm,
                             const void* k_norm, const void* cos_table, const void* sin_table, size_t batch, size_t seq,
                             size_t q_heads, size_t kv_heads, size_t head_dim, size_t rotary_dim,
                             size_t position_offset, size_t max_seq, float epsilon, int dtype, cgpt_stream_t stream);
int cgpt_qknorm_rope_backward(void* dq_pre, void* dk_pre, void* dq_norm, void* dk_norm, const void* dq_rot,
                              const void* dk_rot, const void* q_pre, const void* k_pre, const void* q_norm,
                              const void* k_norm, const void* cos_table, const void* sin_table, size_t batch,
                              size_t seq, size_t q_heads, size_t kv_heads, size_t head_dim, size_t rotary_dim,
                              size_t position_offset, size_t max_seq, float epsilon, int dtype, cgpt_stream_t stream);

/* ------------------------------------------------------------------------------------------------
 * SwiGLU  y = silu(gate) * up.
 * Replaces swiglu_forward (reference include/ops/swiglu.h) and swiglu_backward
 * (reference include/ops/backward/swiglu_backward.h:6-38, src/ops/backward/swiglu_backward.cu:760-883):
 *      s = 1/(1+exp(-g));  dgate = dy*up*s*(1+g*(1-s));  dup = dy*g*s.
 * accumulate_* != 0 adds to the existing output instead of overwriting it. count = number of
 * elements of each tensor.
 * ---------------------------------------------------------------------------------------------- */
int cgpt_swiglu_forward(void* y, const void* gate, const void* up, size_t count, int dtype,
                        cgpt_stream_t stream);
int cgpt_swiglu_backward(void* dgate, void* dup, const void* dy, const void* gate, const void* up,
                         size_t count, int accumulate_gate, int accumulate_up, int dtype,
                         cgpt_stream_t stream);

/* ------------------------------------------------------------------------------------------------
 * Embedding gather and its backward.
 * Replaces embedding_forward (reference include/ops/embedding.h) and embedding_backward
 * (reference include/ops/backward/embedding_backward.h:6-42, src/ops/backward/embedding_backward.cu:207-254):
 *      grad_weight[ids[t], :] += grad_output[t, :]   for ids[t] < vocab (others skipped when
 *      bounds_check != 0), after zeroing grad_weight unless accumulate != 0.
 * Deterministic: tokens are grouped by id and each table row is summed in fp32 in token order, then
 * rounded once (the reference uses storage-dtype atomics in arrival order).
 * ids: uint32 device buffer of `tokens` entries.
 * ---------------------------------------------------------------------------------------------- */
int cgpt_embedding_forward(void* out, const uint32_t* ids, const void* weight, size_t tokens,
                           size_t vocab, size_t hidden, int dtype, cgpt_stream_t stream);
int cgpt_embedding_backward(void* grad_weight, const void* grad_output, const uint32_t* ids,
                            size_t tokens, size_t vocab, size_t hidden, int bounds_check,
                            int accumulate, int dtype, cgpt_stream_t stream);

/* ------------------------------------------------------------------------------------------------
 * Residual adds. Replaces add_tensors / add_inplace (reference src/core/transformer_block.cu:161-215,
 * 261-288). out = a + b (+ c when c != NULL), fp32 add, one rounding. out may alias a.
 * ---------------------------------------------------------------------------------------------- */
int cgpt_add(void* out, const void* a, const void* b, const void* c, size_t count, int dtype,
             cgpt_stream_t stream);

/* ------------------------------------------------------------------------------------------------
 * Softmax cross-entropy on materialised logits.
 * Replaces cross_entropy_forward_backward / cross_entropy_forward (reference
 * include/ops/cross_entropy.h:25-42, src/ops/cross_entropy.cu:352-410).
 * logits, grad: [rows, vocab] in `dtype`; loss: fp32 [1], overwritten with the mean over `rows` of
 * (log sum exp - logit[target]); rows whose target >= vocab add nothing to the loss and get no -1.
 * grad = (softmax - onehot) / rows * gradient_scale. grad == NULL computes the loss only.
 * ---------------------------------------------------------------------------------------------- */
int cgpt_cross_entropy(float* loss, void* grad, const void* logits, const uint32_t* targets,
                       size_t rows, size_t vocab, float gradient_scale, int dtype,
                       cgpt_stream_t stream);

/* ------------------------------------------------------------------------------------------------
 * AdamW over a list of tensors, fp32 master weights / moments, loss-scale unscale, non-finite skip,
 * optional global-norm clip, device-side step counter.
 * Replaces AdamWWorkspace, adamw_step_many_async, adamw_check (reference include/optim/adamw.h:12-136,
 * src/optim/adamw.cu:269-359). Math per element (expression tree kept for 1e-6 parity):
 *      g = float(grad) / loss_scale * clip
 *      m = b1*m + (1-b1)*g;  v = b2*v + (1-b2)*g*g
 *      n = m / bc1 / (sqrtf(v / bc2) + eps),  bc_i = 1 - powf(b_i, float(step))   (on device)
 *      master = master*(1 - lr*wd) - lr*n;  param = (T)master
 * clip = max_grad_norm / norm when norm = sqrt(sum (grad/loss_scale)^2 over ALL entries) exceeds a
 * finite max_grad_norm, else 1. A non-finite unscaled gradient or norm skips the whole step: no
 * tensor changes, the step counter does not advance, and a sticky flag is raised.
 *
 * cgpt_adamw_create binds the workspace to `count` tensors (the reference binds on first use and
 * rejects a changed list, adamw.cu:283-305). Pointers are device pointers; dtype applies to param
 * and grad. `initial_step` seeds the device counter. The handle owns small device buffers; it is
 * created and destroyed outside stream capture. cgpt_adamw_step is capturable and launches a fixed
 * number of kernels regardless of `count`. cgpt_adamw_check copies {sticky flag, step} to the host,
 * synchronises the stream, clears the sticky flag, writes the step to *step_out and the flag to
 * *non_finite_out.
 * ---------------------------------------------------------------------------------------------- */
typedef struct cgpt_adamw_tensor {
    void* param;        /* [count] in `dtype`, updated in place */
    const void* grad;   /* [count] in `dtype` */
    float* master;      /* [count] fp32 */
    float* m;           /* [count] fp32 */
    float* v;           /* [count] fp32 */
    uint64_t count;     /* elements */
    int32_t dtype;      /* CGPT_DTYPE_* of param and grad */
    int32_t reserved;
} cgpt_adamw_tensor;

typedef struct cgpt_adamw_options {
    float learning_rate, beta1, beta2, epsilon, weight_decay, loss_scale, max_grad_norm;
} cgpt_adamw_options;

typedef struct cgpt_adamw_workspace cgpt_adamw_workspace;

int cgpt_adamw_create(cgpt_adamw_workspace** out, const cgpt_adamw_tensor* tensors, size_t count,
                      uint64_t initial_step, cgpt_stream_t stream);
int cgpt_adamw_destroy(cgpt_adamw_workspace* ws);
int cgpt_adamw_step(cgpt_adamw_workspace* ws, const cgpt_adamw_options* options,
                    cgpt_stream_t stream);
/* The same step with the learning rate read from a device scalar (fp32 [1]) when the update kernel runs, instead of
 * options->learning_rate: the three launches can then sit inside a captured CUDA graph while the schedule changes the
 * rate every step by writing the scalar (a 4-byte copy enqueued before the replay). The reference launches its optimizer
 * outside its graph for exactly this reason (train/train.cpp:554-556: the rate is a by-value kernel argument). */
int cgpt_adamw_step_device_lr(cgpt_adamw_workspace* ws, const cgpt_adamw_options* options,
                              const float* learning_rate_device, cgpt_stream_t stream);
int cgpt_adamw_check(cgpt_adamw_workspace* ws, uint64_t* step_out, int* non_finite_out,
                     cgpt_stream_t stream);
/* Reads back the statistics of the last step (sum of squared unscaled gradients, clip factor).
 * Synchronises the stream. For tests and logging. */
int cgpt_adamw_last_stats(cgpt_adamw_workspace* ws, float* squared_norm, float* clip,
                          cgpt_stream_t stream);

/* ------------------------------------------------------------------------------------------------
 * Cut cross-entropy: mean CE of X C^T against targets, with dX and dC, without a [rows, vocab] logits
 * tensor. Replaces cut_cross_entropy_forward_backward (reference include/ops/cut_cross_entropy.h:25-33,
 * src/ops/cut_cross_entropy.cu:97-221, F32 only there) and, in the training step, the composition
 * linear_forward -> cross_entropy_forward_backward -> linear_backward that CGPT's trainer runs on
 * materialised fp16 logits (train/train.cpp:536-544).
 * x, dx: [rows, hidden]; c (classifier), dc: [vocab, hidden]; targets: uint32 [rows]; loss: fp32 [1].
 *   loss = mean_rows(log sum exp(x C^T) - (x C^T)[target]);  G = (softmax - onehot) / rows * gradient_scale
 *   dx = G C;  dc (+)= G^T x.   Rows whose target >= vocab add no loss and no -1 (as cross_entropy).
 * Rows are processed in chunks of at most chunk_rows (0 = library default, 18944 = 74 x 256 rows): logits of one chunk
 * live in scratch ([chunk_rows, vocab]), are turned into G in place and feed the two gradient GEMMs.
 * accumulate_dc != 0 adds into dc instead of overwriting it.
 * ---------------------------------------------------------------------------------------------- */
int cgpt_cut_cross_entropy(float* loss, void* dx, void* dc, const void* x, const void* c,
                           const uint32_t* targets, size_t rows, size_t vocab, size_t hidden,
                           float gradient_scale, int accumulate_dc, size_t chunk_rows, int dtype,
                           cgpt_stream_t stream);
/* The same operator with the form of a chunk chosen by the caller (cgpt_cut_cross_entropy uses the fastest measured):
 *   CGPT_CCE_ROWS       logits product into the scratch, one row kernel turns them into G in place;
 *   CGPT_CCE_TILES      the logits product's epilogue also leaves (max, sum exp) of every 256-column tile of every row,
 *                       so G is one streaming pass over the scratch without row reductions;
 *   CGPT_CCE_RECOMPUTE  the logits are never stored: a first product leaves only the tile statistics, a second one
 *                       recomputes the logits and its epilogue writes G from tensor memory (four products, not three).
 * The last two need 16-bit tensors, chunks of at least 256 rows, vocab >= 256 and % 8 == 0, hidden % 8 == 0 and return
 * CGPT_ERR_UNSUPPORTED otherwise. All forms give the same loss and gradients up to the rounding of the row sums. */
enum { CGPT_CCE_DEFAULT = 0, CGPT_CCE_ROWS = 1, CGPT_CCE_TILES = 2, CGPT_CCE_RECOMPUTE = 3 };
int cgpt_cut_cross_entropy_form(int form, float* loss, void* dx, void* dc, const void* x, const void* c,
                                const uint32_t* targets, size_t rows, size_t vocab, size_t hidden,
                                float gradient_scale, int accumulate_dc, size_t chunk_rows, int dtype,
                                cgpt_stream_t stream);

/* ------------------------------------------------------------------------------------------------
 * Transformer block / model forward and backward (host orchestration in C++ inside the library).
 * Replaces transformer_block_forward / transformer_block_backward (reference
 * include/core/transformer_block.h:10-242, src/core/transformer_block.cu:405-748) and
 * transformer_model_forward / transformer_model_backward (reference include/core/transformer_model.h,
 * src/core/transformer_model.cu:170-381). Block graph (parallel residual, per-head QK-RMSNorm before
 * RoPE):   out = x + W_o Attn(RoPE(qnorm(W_q n_a)), RoPE(knorm(W_k n_a)), W_v n_a) + W_down SwiGLU(W_gate n_f, W_up n_f)
 * with n_a = RMSNorm(x; attention_norm), n_f = RMSNorm(x; ffn_norm).
 * Every struct member is a device pointer to a contiguous tensor in `dtype`
 * (attention_logsumexp: fp32). The same struct type describes weights and their gradients.
 * ---------------------------------------------------------------------------------------------- */
typedef struct cgpt_block_params {
    void* attention_norm; /* [hidden] */
    void* q_projection;   /* [q_heads*head_dim, hidden] */
    void* k_projection;   /* [kv_heads*head_dim, hidden] */
    void* q_norm;         /* [head_dim] */
    void* k_norm;         /* [head_dim] */
    void* v_projection;   /* [kv_heads*head_dim, hidden] */
    void* o_projection;   /* [hidden, q_heads*head_dim] */
    void* ffn_norm;       /* [hidden] */
    void* gate_proj;      /* [intermediate, hidden] */
    void* up_proj;        /* [intermediate, hidden] */
    void* down_proj;      /* [hidden, intermediate] */
} cgpt_block_params;

/* Activations saved by the forward for the backward (TransformerBlockWorkspace in the reference,
 * include/core/transformer_block.h:65-93), rows = batch*seq. */
typedef struct cgpt_block_saved {
    void* norm;                  /* [rows, hidden] output of the FFN RMSNorm */
    void* query;                 /* [batch, seq, q_heads, head_dim] after QK-norm and RoPE */
    void* key;                   /* [batch, seq, kv_heads, head_dim] after QK-norm and RoPE */
    void* value;                 /* [batch, seq, kv_heads, head_dim] */
    void* query_pre_norm;        /* [batch, seq, q_heads, head_dim] */
    void* key_pre_norm;          /* [batch, seq, kv_heads, head_dim] */
    void* attention_output;      /* [batch, seq, q_heads, head_dim] */
    float* attention_logsumexp;  /* [batch, seq, q_heads] fp32 */
    void* gate;                  /* [rows, intermediate] */
    void* up;                    /* [rows, intermediate] */
    void* activated;             /* [rows, intermediate] */
    void* attention_norm_output; /* optional [rows, hidden]: output of the attention RMSNorm. The reference's
                                    workspace has no such buffer and recomputes the norm in the backward
                                    (src/core/transformer_block.cu:725); NULL keeps that behaviour, a buffer
                                    trades rows*hidden elements per layer for one RMSNorm pass per layer */
} cgpt_block_saved;

typedef struct cgpt_model_config {
    uint64_t vocab, layers, hidden, intermediate, q_heads, kv_heads, head_dim, rotary_dim;
    uint64_t max_seq;        /* rows of the cos/sin tables */
    float rms_epsilon;
    int32_t dtype;           /* CGPT_DTYPE_* of every weight / activation */
    int32_t tied_embeddings; /* != 0: lm_head and token_embedding share weight and gradient */
    int32_t reserved;
} cgpt_model_config;

/* Bytes of scratch the block / model calls need for (batch, seq); pass a buffer of at least this size. */
size_t cgpt_block_workspace_bytes(const cgpt_model_config* cfg, size_t batch, size_t seq);

int cgpt_block_forward(void* out, const void* in, const cgpt_block_params* weights, const cgpt_block_saved* saved,
                       void* workspace, const void* cos_table, const void* sin_table, const cgpt_model_config* cfg,
                       size_t batch, size_t seq, size_t position_offset, cgpt_stream_t stream);
int cgpt_block_backward(void* grad_in, const void* grad_out, const void* in, const cgpt_block_params* weights,
                        const cgpt_block_params* grads, const cgpt_block_saved* saved, void* workspace,
                        const void* cos_table, const void* sin_table, const cgpt_model_config* cfg, size_t batch,
                        size_t seq, size_t position_offset, cgpt_stream_t stream);

typedef struct cgpt_model_tensors {
    void* token_embedding;          /* [vocab, hidden] */
    const cgpt_block_params* layers; /* host array of `layers` entries */
    void* final_norm;               /* [hidden] */
    void* lm_head;                  /* [vocab, hidden] (== token_embedding when tied) */
} cgpt_model_tensors;

typedef struct cgpt_model_saved {
    const cgpt_block_saved* layers; /* host array of `layers` entries */
    void* const* layer_inputs;      /* host array of `layers` device pointers, each [rows, hidden] */
    void* hidden;                   /* [rows, hidden] output of the last block */
    void* normalized;               /* [rows, hidden] output of the final RMSNorm */
} cgpt_model_saved;

/* Forward: embedding -> blocks -> final RMSNorm (saved->normalized); with logits != NULL also the LM head
 * into logits [rows, vocab] (the reference's transformer_model_forward). */
int cgpt_model_forward(void* logits, const uint32_t* token_ids, const cgpt_model_tensors* weights,
                       const cgpt_model_saved* saved, void* workspace, const void* cos_table, const void* sin_table,
                       const cgpt_model_config* cfg, size_t batch, size_t seq, cgpt_stream_t stream);
/* Backward. Either grad_logits [rows, vocab] is given (the reference's transformer_model_backward: LM-head
 * backward first, grads->lm_head overwritten), or grad_logits == NULL and grad_normalized [rows, hidden]
 * already holds the gradient of the final-norm output with grads->lm_head already written (the cut
 * cross-entropy path). grad_normalized is scratch of [rows, hidden] in the first case. With tied embeddings
 * the lookup gradient is added into grads->lm_head, else grads->token_embedding is overwritten. */
int cgpt_model_backward(const void* grad_logits, void* grad_normalized, const uint32_t* token_ids,
                        const cgpt_model_tensors* weights, const cgpt_model_tensors* grads,
                        const cgpt_model_saved* saved, void* workspace, const void* cos_table, const void* sin_table,
                        const cgpt_model_config* cfg, size_t batch, size_t seq, cgpt_stream_t stream);
/* The same backward in pieces, for callers that interleave it with other work (a data-parallel driver starts the
 * all-reduce of the gradients that are already final). Steps: 0 = LM head (if grad_logits) + final norm,
 * 1 .. layers = the blocks from the last to the first (step s is layer `layers - s`), layers + 1 = embedding.
 * Runs steps [step_begin, step_end); consecutive calls on one stream covering 0 .. layers + 2 in order equal one
 * cgpt_model_backward call (which is implemented as exactly that). The reference has only the whole-model call
 * (include/core/transformer_model.h:176-190). */
int cgpt_model_backward_steps(const void* grad_logits, void* grad_normalized, const uint32_t* token_ids,
                              const cgpt_model_tensors* weights, const cgpt_model_tensors* grads,
                              const cgpt_model_saved* saved, void* workspace, const void* cos_table,
                              const void* sin_table, const cgpt_model_config* cfg, size_t batch, size_t seq,
                              size_t step_begin, size_t step_end, cgpt_stream_t stream);

#ifdef __cplusplus
} /* extern "C" */
#endif

#endif /* CGPT_B200_H_ */
