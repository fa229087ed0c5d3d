/*
 * tb200.h — C ABI of libtb200.so: hand-written sm_100a CUDA kernels that stand in
 * for the Triton kernel layer of kakaobrain/trident (trident/kernel/*.py and
 * trident/language/*.py) for attention, linear, GEGLU, LayerNorm, RMSNorm, Softmax
 * and MaskedSoftmax, forward and backward.
 *
 * Conventions
 *   - every pointer is a DEVICE pointer owned by the caller; the library never
 *     allocates, frees, synchronises or reads memory back, and launches only on
 *     the stream it is given;
 *   - `dtype`: 0 = float32, 1 = float16, 2 = bfloat16 (the floating-point subset of
 *     trident/util/util.py:48-58);
 *   - strides are in ELEMENTS;
 *   - nullable pointers play the role of the reference's `None` arguments;
 *   - return value: 0 = launched; < 0 = rejected before any launch (text in
 *     tb200_last_error()); > 0 = a cudaError_t raised by the launch;
 *   - statistics saved for backward (mean, rstd, rms, log-sum-exp) are float32
 *     whatever the input dtype is.
 */
#ifndef TB200_H_
#define TB200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TB200_F32 0
#define TB200_F16 1
#define TB200_BF16 2

#define TB200_ERR_INVALID (-1)     /* bad argument (null, size, dtype) */
#define TB200_ERR_UNSUPPORTED (-2) /* shape/stride outside every kernel's domain */
#define TB200_ERR_WORKSPACE (-3)   /* workspace missing or too small */

/* ---- library / device --------------------------------------------------- */
const char* tb200_last_error(void); /* thread-local text of the last failure */
int tb200_version(void);
/* 0 iff `device` has compute capability 10.x (the only target of this library). */
int tb200_device_check(int device);

/* ---- LayerNorm ----------------------------------------------------------
 * Replaces kernel.LayerNorm.forward (trident/kernel/layer_norm.py:19-126),
 * launched at trident/operation/layer_norm.py:64. */
int tb200_layer_norm_fwd(void* y, float* mean, float* rstd, const void* x,
                         const void* weight /*nullable*/, const void* bias /*nullable*/,
                         int64_t rows, int64_t cols, float eps, int dtype, void* stream);
/* Replaces kernel.LayerNorm.backward (trident/kernel/layer_norm.py:128-246) launched at
 * trident/operation/layer_norm.py:97 together with the two torch.sum reductions at
 * :114 and :121. dweight/dbias may be null. The workspace holds per-CTA column
 * partials; its size comes from the query below. */
size_t tb200_layer_norm_bwd_workspace(int64_t rows, int64_t cols);
int tb200_layer_norm_bwd(void* dx, void* dweight /*nullable*/, void* dbias /*nullable*/,
                         const void* dy, const void* x, const void* weight /*nullable*/,
                         const float* mean, const float* rstd, void* workspace,
                         size_t workspace_bytes, int64_t rows, int64_t cols, int dtype,
                         void* stream);

/* Same result as tb200_layer_norm_bwd, but the caller passes no workspace and nothing is
 * allocated: the column partials of dweight/dbias go to a 2 MiB array that is part of the
 * library image on every GPU that loads it. It exists for callers that cannot allocate
 * device memory at the point of the call: a process that gave its whole GPU to a private
 * arena at start-up, or code under a no-cudaMalloc rule on its request path. (It has no
 * counterpart in the reference, whose operation layer always allocates its staging
 * buffers with torch.)
 *   - cols may be at most 8192; wider rows are rejected with TB200_ERR_UNSUPPORTED and
 *     should use tb200_layer_norm_bwd with a workspace;
 *   - the first call on each device resolves the array's device address (the device must
 *     be current); make that first call before any stream capture begins;
 *   - all calls on one device share the array: two calls that may run on the GPU at the
 *     same time (different streams) race on it and must be serialised by the caller.
 *     Nothing in the array has to be cleared between calls; each call overwrites every
 *     element it later reads;
 *   - the resolved address is remembered per device ordinal for the life of the process: a
 *     process that calls cudaDeviceReset and then uses this entry point again on the same
 *     device would be handed the address of the destroyed context. */
int tb200_layer_norm_bwd_static(void* dx, void* dweight /*nullable*/, void* dbias /*nullable*/,
                                const void* dy, const void* x, const void* weight /*nullable*/,
                                const float* mean, const float* rstd, int64_t rows, int64_t cols,
                                int dtype, void* stream);

/* ---- RMSNorm ------------------------------------------------------------
 * Replaces kernel.RMSNorm.forward (trident/kernel/rms_norm.py:19-117), launched at
 * trident/operation/rms_norm.py:60. rms = sqrt(mean(x[:partial_cols]^2));
 * y = x / (rms + eps) * weight (+ bias). x is addressed with (row_stride,
 * col_stride); y is contiguous. y may be null: then only rms is written (the row
 * statistic for tb200_geglu_fwd_row_scaled). */
int tb200_rms_norm_fwd(void* y, float* rms, const void* x, const void* weight,
                       const void* bias /*nullable*/, int64_t rows, int64_t cols,
                       int64_t row_stride, int64_t col_stride, int64_t partial_cols,
                       float eps, int dtype, void* stream);
/* Replaces kernel.RMSNorm.backward (trident/kernel/rms_norm.py:119-232) launched at
 * trident/operation/rms_norm.py:98, the torch.sum at :117 and the Sum launch at :122.
 * dy and dx are contiguous; x uses (row_stride, col_stride). */
size_t tb200_rms_norm_bwd_workspace(int64_t rows, int64_t cols);
int tb200_rms_norm_bwd(void* dx, void* dweight, void* dbias /*nullable*/, const void* dy,
                       const void* x, const void* weight, const float* rms, void* workspace,
                       size_t workspace_bytes, int64_t rows, int64_t cols, int64_t row_stride,
                       int64_t col_stride, int64_t partial_cols, float eps, int dtype,
                       void* stream);

/* ---- Softmax / MaskedSoftmax -------------------------------------------
 * Replaces kernel.Softmax.forward (trident/kernel/softmax.py:29-106, launched at
 * trident/operation/softmax.py:57) and kernel.MaskedSoftmax.forward
 * (trident/kernel/masked_softmax.py:21-81, launched at
 * trident/operation/masked_softmax.py:57). `mask` is nullable; it holds one byte per
 * element (non-zero = masked out) and is addressed with its own strides. x, y share
 * (row_stride, col_stride): the softmax runs along the `cols` axis. */
int tb200_softmax_fwd(void* y, const void* x, const uint8_t* mask /*nullable*/,
                      int64_t rows, int64_t cols, int64_t row_stride, int64_t col_stride,
                      int64_t mask_row_stride, int64_t mask_col_stride, int dtype,
                      void* stream);
/* Replaces Softmax.backward_delta + Softmax.backward (trident/kernel/softmax.py:108-238,
 * launched at trident/operation/softmax.py:81,:97) and their MaskedSoftmax twins
 * (trident/kernel/masked_softmax.py:83-199; trident/operation/masked_softmax.py:83,:100).
 * dx, dy and y share the strides. */
int tb200_softmax_bwd(void* dx, const void* dy, const void* y, int64_t rows, int64_t cols,
                      int64_t row_stride, int64_t col_stride, int dtype, void* stream);

/* ---- Linear --------------------------------------------------------------
 * y[b,m,n] = sum_k x[b,m,k] * w[n,k] (+ bias[n]).
 * Replaces kernel.Linear.forward (trident/kernel/linear.py:113-190; launched at
 * trident/operation/linear.py:61). y is contiguous [B,M,N]. */
int tb200_linear_fwd(void* y, const void* x, const void* w, const void* bias /*nullable*/,
                     int64_t B, int64_t M, int64_t N, int64_t K, int64_t x_sb, int64_t x_sm,
                     int64_t x_sk, int64_t w_sn, int64_t w_sk, int allow_tf32, int dtype,
                     void* stream);
/* dx[b,m,k] = sum_n dy[b,m,n] * w[n,k]; dy contiguous [B,M,N]; dx strided.
 * Replaces kernel.Linear.backward (trident/kernel/linear.py:192-265; launched at
 * trident/operation/linear.py:95 and trident/operation/geglu.py:119). */
int tb200_linear_bwd_input(void* dx, const void* dy, const void* w, int64_t B, int64_t M,
                           int64_t N, int64_t K, int64_t dx_sb, int64_t dx_sm, int64_t dx_sk,
                           int64_t w_sn, int64_t w_sk, int allow_tf32, int dtype, void* stream);
/* dw[n,k] = sum_{b,m} dy[b,m,n] * x[b,m,k]; dw contiguous [N,K], already reduced over
 * the batch. Replaces kernel.Linear.backward_weight (trident/kernel/linear.py:267-342;
 * launched at trident/operation/linear.py:117, trident/operation/geglu.py:141) and the
 * torch.sum over the batch staging buffer (trident/operation/linear.py:133). */
int tb200_linear_bwd_weight(void* dw, const void* dy, const void* x, int64_t B, int64_t M,
                            int64_t N, int64_t K, int64_t x_sb, int64_t x_sm, int64_t x_sk,
                            int allow_tf32, int dtype, void* stream);
/* dbias[n] = sum_{rows} dy[row,n]; dy contiguous [rows,N].
 * Replaces kernel.Linear.backward_bias (trident/kernel/linear.py:344-378; launched at
 * trident/operation/linear.py:143, trident/operation/geglu.py:167) and the torch.sum at
 * trident/operation/linear.py:153. */
size_t tb200_linear_bwd_bias_workspace(int64_t rows, int64_t N);
int tb200_linear_bwd_bias(void* dbias, const void* dy, void* workspace, size_t workspace_bytes,
                          int64_t rows, int64_t N, int dtype, void* stream);

/* ---- GEGLU ---------------------------------------------------------------
 * state_gate = x w^T + bias  ([B,M,N], N even); out = state * gelu(gate) with
 * state = state_gate[..., :N/2], gate = state_gate[..., N/2:]  ([B,M,N/2]).
 * Replaces kernel.GEGLU.forward (trident/kernel/geglu.py:54-177; launched at
 * trident/operation/geglu.py:65). gelu_tanh != 0 selects the tanh approximation of
 * trident/language/math/gelu.py:19-31, 0 the exact erf form of the test oracle
 * (tests/test_geglu.py:22-24). */
int tb200_geglu_fwd(void* out, void* state_gate, const void* x, const void* w,
                    const void* bias /*nullable*/, int64_t B, int64_t M, int64_t N, int64_t K,
                    int64_t x_sb, int64_t x_sm, int64_t x_sk, int64_t w_sn, int64_t w_sk,
                    int gelu_tanh, int allow_tf32, int dtype, void* stream);
/* The same with every accumulator row m multiplied by row_scale[m] (fp32, [B*M]) before the bias:
 * state_gate = row_scale * (x w^T) + bias. Given row_scale = 1 / (rms + eps) (tb200_rms_norm_fwd
 * with y = null returns rms alone) and w = W * diag(norm weight), this is GEGLU applied to
 * RMSNorm(x), the two reference launches trident/function/function.py:202-208 and :70-80 that run
 * back to back, without the normalised copy of x going through memory. 16-bit operands with unit
 * inner strides only; anything else returns TB200_ERR_UNSUPPORTED and the caller runs the two
 * operations one after the other. */
int tb200_geglu_fwd_row_scaled(void* out, void* state_gate, const void* x, const void* w,
                               const void* bias /*nullable*/, const float* row_scale, int64_t B, int64_t M,
                               int64_t N, int64_t K, int64_t x_sb, int64_t x_sm, int64_t x_sk,
                               int64_t w_sn, int64_t w_sk, int gelu_tanh, int dtype, void* stream);
/* d_state_gate[:, :N/2] = dout * gelu(gate); d_state_gate[:, N/2:] = dout * state *
 * gelu'(gate). Replaces kernel.GEGLU.backward (trident/kernel/geglu.py:179-242;
 * launched at trident/operation/geglu.py:101). */
int tb200_geglu_bwd_elementwise(void* d_state_gate, const void* dout, const void* state_gate,
                                int64_t rows, int64_t N, int gelu_tanh, int dtype, void* stream);
/* The same step fused with the bias gradient of the Linear backward that follows it
 * (dbias[N] = column sums of d_state_gate, summed in fp32 before rounding): replaces
 * kernel.GEGLU.backward plus kernel.Linear.backward_bias (trident/kernel/linear.py, launched at
 * trident/operation/geglu.py:150-178) in one pass over d_state_gate. `workspace` as for
 * tb200_linear_bwd_bias (tb200_linear_bwd_bias_workspace(rows, N) bytes). */
int tb200_geglu_bwd_elementwise_bias(void* d_state_gate, void* dbias, const void* dout,
                                     const void* state_gate, void* workspace, size_t workspace_bytes,
                                     int64_t rows, int64_t N, int gelu_tanh, int dtype, void* stream);

/* ---- Row reductions: Sum, Mean, Var, VarMean --------------------------------
 * The problem as util.size_and_stride describes it (trident/util/util.py:65-76): y_size
 * outputs, output y reduces the x_size elements x[y*y_stride + i*x_stride]. kind: 0 sum,
 * 1 mean, 2 var, 3 var_mean. out_a[y_size] = sum | mean | var | var, out_b[y_size] = mean
 * (var_mean only, else ignored); var divides by (x_size - correction).
 * Replaces kernel.Sum/Mean/Var/VarMean.forward (trident/kernel/sum.py:35, mean.py:35, var.py:35,
 * var_mean.py:35; launched at trident/operation/sum.py:57, mean.py:58, var.py:59, var_mean.py:60). */
int tb200_reduce_fwd(void* out_a, void* out_b /*nullable*/, const void* x, int64_t y_size, int64_t x_size,
                     int64_t y_stride, int64_t x_stride, int kind, float correction, int dtype,
                     void* stream);
/* dx (same strides as x) from dout_a[y_size] (and dout_b, the gradient of the mean output of
 * var_mean, nullable); x is needed for var and var_mean only. Replaces kernel.*.backward of the
 * same files (trident/kernel/sum.py:65, mean.py:66, var.py:76, var_mean.py:86; launched at
 * trident/operation/sum.py:79, mean.py:80, var.py:82, var_mean.py:86); no zero fill of dx is needed. */
int tb200_reduce_bwd(void* dx, const void* dout_a, const void* dout_b /*nullable*/, const void* x /*nullable for sum, mean*/,
                     int64_t y_size, int64_t x_size, int64_t y_stride, int64_t x_stride, int kind,
                     float correction, int dtype, void* stream);

/* ---- Attention -----------------------------------------------------------
 * out = softmax(scale * q k^T + M) v per (batch, head); M is the additive `mask`
 * (nullable; same dtype as q; stride 0 broadcasts a dimension) or the causal mask.
 * q, k, v, out: [B,H,S,D] with per-tensor element strides (4 each). lse[b,h,s] is the
 * natural-log sum of exponentials of a score row (float32).
 * Replaces kernel.Attention.forward (trident/kernel/attention.py:30-165; launched at
 * trident/operation/attention.py:109). */
int tb200_attention_fwd(void* out, float* lse, const void* q, const void* k, const void* v,
                        const void* mask /*nullable*/, int64_t B, int64_t H, int64_t S,
                        int64_t D, const int64_t* q_strides, const int64_t* k_strides,
                        const int64_t* v_strides, const int64_t* out_strides,
                        const int64_t* mask_strides /*nullable iff mask is*/, int is_causal,
                        float softmax_scale, int dtype, void* stream);
/* dq, dk, dv (and dmask when non-null: dense [B,H,S,S], same dtype; the gradient of the additive
 * mask is dS, which the tensor-core kernel writes from the registers it computes it in) from dout.
 * Replaces Softmax.backward_delta as launched at trident/operation/attention.py:161 and
 * kernel.Attention.backward (trident/kernel/attention.py:167-339; launched at
 * trident/operation/attention.py:170). dq/dk/dv/dout are contiguous [B,H,S,D]; q, k, v,
 * out keep their strides. The workspace (fp32 delta and fp32 dq accumulator) is sized
 * by the query below. */
size_t tb200_attention_bwd_workspace(int64_t B, int64_t H, int64_t S, int64_t D, int dtype);
int tb200_attention_bwd(void* dq, void* dk, void* dv, void* dmask /*nullable*/,
                        const void* dout, const void* q, const void* k, const void* v,
                        const void* out, const float* lse, const void* mask /*nullable*/,
                        void* workspace, size_t workspace_bytes, int64_t B, int64_t H,
                        int64_t S, int64_t D, const int64_t* q_strides,
                        const int64_t* k_strides, const int64_t* v_strides,
                        const int64_t* out_strides, const int64_t* mask_strides,
                        int is_causal, float softmax_scale, int dtype, void* stream);

/* ---- introspection used by the tests and the bench ----------------------
 * Name of the kernel family the last successful call on this thread dispatched to
 * ("row_vec", "row_generic", "gemm_tcgen05", "gemm_simt", "attn_tcgen05", "attn_simt", ...)
 * and how many kernels that call launched. */
const char* tb200_last_kernel(void);
int tb200_last_launch_count(void);
/* Kernels launched by this process through the library so far. */
int64_t tb200_total_launches(void);
/* Every wait inside the tensor-core kernels is bounded; a wait that gives up records a
 * non-zero code in a device status word and the kernel still runs to its end. This call
 * synchronises the device and returns that word (0 = healthy); `reset` != 0 clears it. */
int tb200_device_status(int reset);
/* The norm backward kernels fold their per-CTA weight/bias gradient rows inside the same
 * (cooperative) launch when on != 0 (the default), or in a second finalize kernel when
 * on == 0. Both orders of summation are fixed. Used by tests to cover both paths (the
 * second is otherwise only taken when the grid cannot be co-resident). The setting belongs to
 * the calling thread and applies to the norm backward calls that thread makes; other threads
 * keep their own. Returns the old value. */
int tb200_set_norm_fused_finalize(int on);
/* Test hook of the calling thread for the bounded waits of the tensor-core kernels. mode 1: the
 * attention forward launches this thread makes next run with a wait limit of about a
 * millisecond and the producer of CTA (0, 0) leaves out the copy of its second key tile, so one
 * wait runs out: the launch must still complete, free its tensor memory and leave a non-zero
 * code in the device status word (tb200_device_status); its output is invalid. mode 0: normal
 * operation. Returns the old mode. No memory is touched that a normal launch would not touch. */
int tb200_test_wait_fault(int mode);

#ifdef __cplusplus
}
#endif
#endif /* TB200_H_ */
