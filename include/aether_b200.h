/* aether_b200.h -- C ABI of libaether_b200.so.
 *
 * A B200 (sm_100a) implementation of the convolution hot path of Aether-ML
 * (https://github.com/AlexanderSoftCode/Aether-ML) and of the bandwidth-bound layers around it.
 * Each entry point replaces the arithmetic of one method of the reference's layer classes in
 * CNN/models/CNN_classes_cupy.py (cited per function as file:line); the Python classes of the same
 * names in aether_ml_b200/layers.py call these through ctypes.
 *
 * Conventions
 *   - Every pointer is a raw DEVICE address (e.g. arr.__cuda_array_interface__['data'][0], torch
 *     tensor.data_ptr()) of a C-contiguous fp32 array unless stated otherwise.  Activations are NHWC,
 *     filters are (fH, fW, Cin, Cout) -- the reference's own layouts.  Arrays must be 16-byte aligned.
 *   - The caller owns every buffer, including workspaces (size them with the *_workspace_bytes query).
 *     The library allocates nothing per call and frees nothing of the caller's.
 *   - `stream` is a cudaStream_t passed as void* (NULL = default stream).  Calls only enqueue work;
 *     they never synchronise.
 *   - Return value: 0 on success, negative on failure (AETHER_E_*); aether_last_error() then holds a
 *     message for the calling thread.  Nothing is launched when an argument check fails.
 *   - Kernels that wait on hardware barriers give up after about two seconds and record a code that
 *     aether_device_status() returns after the stream has been synchronised (0 = no such event).
 */
#ifndef AETHER_B200_H
#define AETHER_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define AETHER_E_BAD_ARG (-1)
#define AETHER_E_UNSUPPORTED (-2)
#define AETHER_E_CUDA (-3)
#define AETHER_E_DEVICE_TIMEOUT (-4)

/* Operand precision of the convolution GEMMs (accumulation is always fp32). */
#define AETHER_MATH_BF16 0 /* bf16 operands on the tensor cores (tcgen05 kind::f16)            */
#define AETHER_MATH_TF32 1 /* tf32 operands on the tensor cores (tcgen05 kind::tf32)           */
#define AETHER_MATH_FP32 2 /* fp32 FMA on the CUDA cores (also used for shapes the tensor path   */
                           /* does not take: stride > 1, Cin or Cout < 16 or not a multiple of 4) */

#define AETHER_POOL_MAX 0
#define AETHER_POOL_AVG 1

/* Geometry of one Conv_Layer (constructor arguments at CNN_classes_cupy.py:38-45 plus the batch).
 * padH/padW are the zero padding on each side: (fH-1)/2 on BOTH axes for padding="same" (:78-81),
 * 0 for "valid".  Output size is (H + 2*padH - fH)/sH + 1 (:84-85). */
typedef struct AetherConvDesc {
    int32_t S, H, W, Cin, Cout;
    int32_t fH, fW, sH, sW, padH, padW;
    int32_t math_mode; /* AETHER_MATH_* */
} AetherConvDesc;

int aether_version(void);
/* Message of the last failed call on this thread ("" if none). */
const char* aether_last_error(void);
/* Number of kernels this library has launched since it was loaded (all threads). */
uint64_t aether_launch_count(void);
/* Code recorded by a kernel that abandoned a bounded wait (0 = none).  Read after synchronising. */
int aether_device_status(void);
void aether_device_status_clear(void);
/* Self-test of that give-up path (no counterpart in the reference, which has no device-side waits): launches one
 * thread that waits, with the kernels' own bounded wait, on a barrier nothing completes; after `limit_cycles`
 * SM clock cycles (1 .. 2e9) it records code 5 and the kernel ends by itself.  After the stream is synchronised
 * aether_device_status() returns 5 and the convolution entry points return AETHER_E_DEVICE_TIMEOUT until
 * aether_device_status_clear() is called. */
int aether_selftest_bounded_wait(int64_t limit_cycles, void* stream);

/* Optional kernel timing for benchmarks (off by default).  aether_profile_enable(n), n >= 1, creates a fixed
 * pool of CUDA events once and resets the counters; while enabled, events are recorded on the launch
 * stream around every n-th launch of each kind of convolution kernel (an event record takes a few
 * microseconds of stream time itself, so timing every launch slows short steps measurably);
 * aether_profile_enable(0) switches it off.  aether_profile_read waits for the recorded events and
 * returns the summed duration and the number of timed launches of one kind:
 * 0 = forward implicit GEMM, 1 = dX implicit GEMM, 2 = dW kernel, 3 = operand (bf16) cast kernels. */
int aether_profile_enable(int on);
int aether_profile_read(int kind, double* total_ms, int* launches);
void aether_profile_reset(void);

/* ---- Conv_Layer ------------------------------------------------------------------------------ */

/* Bytes of scratch one layer needs for forward + backward (shadow copies of the operands in the MMA
 * precision, split-K partial sums).  The same buffer should be passed to the forward and the
 * backward call of a layer. */
size_t aether_conv2d_workspace_bytes(const AetherConvDesc* desc);

/* Conv_Layer.forward, CNN_classes_cupy.py:70-120: y = conv(x, w) + b with zero padding.
 * x (S,H,W,Cin), w (fH,fW,Cin,Cout), b (Cout) or NULL, y (S,Ho,Wo,Cout). */
int aether_conv2d_fwd(const AetherConvDesc* desc, const float* x, const float* w, const float* b, float* y, void* ws,
                      size_t ws_bytes, void* stream);

/* Conv_Layer.forward with the Batch_Norm statistics of its output taken in the kernel's epilogue: the reference
 * computes them in a separate pass over the layer output (Batch_Norm.forward, CNN_classes_cupy.py:467-470, mean and
 * var over all axes but the last).  `stats` receives aether_conv2d_bnstats_blocks(desc) blocks of [3][Cout] floats:
 * (count, mean, M2 = sum of squared deviations) of y over the rows each block covered; hand them to
 * aether_bn_fwd_train_partials.  aether_conv2d_bnstats_blocks returns 0 when the forward kernel that serves the
 * shape does not produce statistics; then aether_conv2d_fwd_bnstats fails with AETHER_E_UNSUPPORTED and the
 * caller uses aether_conv2d_fwd + aether_bn_fwd_train. */
int64_t aether_conv2d_bnstats_blocks(const AetherConvDesc* desc);
int aether_conv2d_fwd_bnstats(const AetherConvDesc* desc, const float* x, const float* w, const float* b, float* y,
                              float* stats, size_t stats_bytes, void* ws, size_t ws_bytes, void* stream);

/* Conv_Layer.backward, CNN_classes_cupy.py:123-154: db = sum dy (:132), dw = windows^T dy (:134),
 * dx = scatter-add of dy w^T (:138-146) with the padding border removed (:149-153; returned
 * contiguous).  Any of dx, dw, db may be NULL to skip it.  x_shadow_valid is a bit mask about the operand copies
 * that the last aether_conv2d_fwd / aether_conv2d_fwd_bnstats call with this `ws` left in it: bit 0 = the copy of x
 * is still the copy of this x (saves one pass over x), bit 1 = w has not changed since, so the copy of the filter
 * that dX multiplies by is reused (saves one pass over w).  0 is always safe: everything is rebuilt. */
int aether_conv2d_bwd(const AetherConvDesc* desc, const float* x, const float* dy, const float* w, float* dx, float* dw,
                      float* db, void* ws, size_t ws_bytes, int x_shadow_valid, void* stream);

/* Operand-copy hand-off between neighbouring layers.  The reference passes fp32 activations from layer to layer
 * (Pooling.output -> Conv_Layer.forward :70-120; Batch_Norm.backward :484-508 -> Conv_Layer.backward :123-154); the
 * bf16 tensor-core kernels here read a bf16 copy of x and of dy that a cast pass makes from them.  The kernel that
 * PRODUCES such an activation can write that copy itself, straight into the consuming layer's workspace, and the
 * consumer is then told to skip its cast pass:
 *   aether_conv2d_operand_layout: where in `ws` (byte offsets) the copies live and how wide their rows are (channels
 *     padded to a multiple of 64).  Returns 1 and fills `out` when this shape runs on the bf16 tensor-core path,
 *     0 otherwise (no copies are read: nothing to hand in).  The copy of x is [S*H*W][x_copy_ld] bf16, the copy of dy
 *     [S*Ho*Wo][dy_copy_ld] bf16 (padding channels zero); with the copy of dy the producer also hands in per-block
 *     column sums of dy for the bias gradient (:132), float [rows][Cout] at dy_colsum_offset, rows <= dy_colsum_rows_max.
 *   aether_conv2d_fwd_ex: aether_conv2d_fwd (stats == NULL) / aether_conv2d_fwd_bnstats (stats given) with flags:
 *     AETHER_CONV_X_COPY_READY = the copy of x is already in ws.
 *   aether_conv2d_bwd_ex: aether_conv2d_bwd whose bit mask may also carry AETHER_CONV_DY_COPY_READY = the copy of dy
 *     and dy_colsum_rows rows of column sums are already in ws.
 * These entry points have no counterpart in the reference. */
typedef struct AetherOperandLayout {
    size_t x_copy_offset;
    int32_t x_copy_ld;
    size_t dy_copy_offset;
    int32_t dy_copy_ld;
    size_t dy_colsum_offset;
    int32_t dy_colsum_rows_max;
} AetherOperandLayout;
enum { AETHER_CONV_X_COPY_READY = 1, AETHER_CONV_W_COPY_READY = 2, AETHER_CONV_DY_COPY_READY = 4 };
int aether_conv2d_operand_layout(const AetherConvDesc* desc, AetherOperandLayout* out);
int aether_conv2d_fwd_ex(const AetherConvDesc* desc, const float* x, const float* w, const float* b, float* y, float* stats,
                         size_t stats_bytes, void* ws, size_t ws_bytes, int flags, void* stream);
int aether_conv2d_bwd_ex(const AetherConvDesc* desc, const float* x, const float* dy, const float* w, float* dx, float* dw,
                         float* db, void* ws, size_t ws_bytes, int x_shadow_valid, int dy_colsum_rows, void* stream);

/* ---- Batch_Norm (CNN_classes_cupy.py:430-526); x is [rows][C], rows = product of leading axes --- */
size_t aether_bn_workspace_bytes(int64_t rows, int C);
/* Training forward :467-476.  Writes batch_mean/batch_var (biased), y, and updates running_* in place
 * as momentum*old + (1-momentum)*batch. */
int aether_bn_fwd_train(const float* x, const float* gamma, const float* beta, float* running_mean, float* running_var,
                        float* batch_mean, float* batch_var, float* y, int64_t rows, int C, float eps, float momentum,
                        void* ws, size_t ws_bytes, void* stream);
/* Training forward :467-476 from per-block partial statistics [nblocks][3][C] = (count, mean, M2) that the producer
 * of x already wrote (aether_conv2d_fwd_bnstats): merges them (double precision), then normalises.  x is read once.
 * ws: at least 2*C floats. */
int aether_bn_fwd_train_partials(const float* x, const float* partials, int64_t nblocks, const float* gamma,
                                 const float* beta, float* running_mean, float* running_var, float* batch_mean,
                                 float* batch_var, float* y, int64_t rows, int C, float eps, float momentum, void* ws,
                                 size_t ws_bytes, void* stream);
/* Same result as aether_bn_fwd_train, for callers that have no way to provide the workspace.  (No counterpart
 * in the reference: its Batch_Norm lets CuPy allocate temporaries freely.)  Some hosts of this library must not
 * or cannot allocate device memory around a call -- a process whose whole device-memory budget was handed to
 * another pool at start-up, a plug-in that may touch only the arrays its host gave it, a step function that has
 * to keep its memory footprint fixed -- so this variant keeps its scratch (per-block partial statistics and the
 * per-channel coefficients) in a fixed array inside the library image, about 1.8 MB that every GPU loading the
 * library holds until the process exits.  It performs no cudaMalloc/cudaFree and calls no allocating routine.
 *   - Limit: C <= AETHER_BN_STATIC_MAX_CHANNELS; larger C is rejected with AETHER_E_UNSUPPORTED.
 *   - The FIRST call on each device looks up the array's device address (the device must be current); make
 *     that first call before any stream capture begins.
 *   - All calls on a device share the one array and it keeps whatever the last call left there.  Nothing needs
 *     clearing (every element is rewritten before it is read), but two calls whose kernels can overlap on the
 *     GPU (different streams without ordering) race on it: serialise them. */
#define AETHER_BN_STATIC_MAX_CHANNELS 1024
int aether_bn_fwd_train_static(const float* x, const float* gamma, const float* beta, float* running_mean,
                               float* running_var, float* batch_mean, float* batch_var, float* y, int64_t rows, int C,
                               float eps, float momentum, void* stream);
/* Inference forward :478-480 (ws: at least 2*C floats). */
int aether_bn_fwd_eval(const float* x, const float* gamma, const float* beta, const float* running_mean,
                       const float* running_var, float* y, int64_t rows, int C, float eps, void* ws, size_t ws_bytes,
                       void* stream);
/* Backward :484-508: dx, dgamma (= dweights), dbeta (= dbiases). */
int aether_bn_bwd(const float* x, const float* dy, const float* gamma, const float* batch_mean, const float* batch_var,
                  float* dx, float* dgamma, float* dbeta, int64_t rows, int C, float eps, void* ws, size_t ws_bytes,
                  void* stream);
/* Batch_Norm immediately followed by ReLU / Leaky_ReLU (:406-428), both applied in the same passes over the data:
 * y = act(bn(x)) with act(v) = v > 0 ? v : alpha*v (alpha = 0 is ReLU, 0 <= alpha < 1); the normalised but not yet
 * activated tensor is never written.  The reference runs them as two layers with one more read and write of the
 * activation each way.
 *   aether_bn_act_fwd_train: Batch_Norm.forward (training) + activation.  `partials` may be NULL (x is reduced here)
 *     or [nblocks][3][C] partial statistics from aether_conv2d_fwd_bnstats.  ws: aether_bn_workspace_bytes(rows, C).
 *   aether_bn_act_fwd_eval: the same with the running statistics (ws: 2*C floats).
 *   aether_bn_act_bwd: dy is the gradient w.r.t. y = act(bn(x)).  The activation's derivative is taken at the
 *     pre-activation v = gamma*xhat + beta, recomputed from x while x is read for the Batch_Norm sums (y is not
 *     read): alpha where v < 0, else 1 -- the gradient passes at v == 0 exactly as ReLU.backward (:412-414,
 *     dvalues[inputs < 0] = 0) and Leaky_ReLU.backward (:424-428) do.
 *   channel_scale (C floats >= 0, or NULL): the mask / keep_prob of a Layer_Dropout_Spatial (:384-404) that follows
 *     the activation; y = act(bn(x)) * channel_scale[c] and the backward treats dy as the gradient w.r.t. that y.
 *     (Folded into the per-channel coefficients: act(v) * m = act(m * v) for m >= 0.) */
int aether_bn_act_fwd_train(const float* x, const float* partials, int64_t nblocks, const float* gamma, const float* beta,
                            float* running_mean, float* running_var, float* batch_mean, float* batch_var, float* y,
                            int64_t rows, int C, float eps, float momentum, float alpha, const float* channel_scale,
                            void* ws, size_t ws_bytes, void* stream);
int aether_bn_act_fwd_eval(const float* x, const float* gamma, const float* beta, const float* running_mean,
                           const float* running_var, float* y, int64_t rows, int C, float eps, float alpha, void* ws,
                           size_t ws_bytes, void* stream);
int aether_bn_act_bwd(const float* x, const float* beta, const float* dy, const float* gamma, const float* batch_mean,
                      const float* batch_var, float* dx, float* dgamma, float* dbeta, int64_t rows, int C, float eps,
                      float alpha, const float* channel_scale, void* ws, size_t ws_bytes, void* stream);

/* The whole tail of a convolution block in one pass each way: Batch_Norm (:430-526), ReLU / Leaky_ReLU (:406-428),
 * optional Layer_Dropout_Spatial (:384-404, channel_scale = mask / keep_prob or NULL) and a max Pooling (:204-312) with
 * fH x fW windows of stride (fH, fW) that tile the input (H % fH == 0, W % fW == 0; C % 4 == 0).  The activated tensor
 * between convolution and pooling is never written.
 *   aether_bn_act_pool_fwd: x (S,H,W,C) -> pooled (S,H/fH,W/fW,C) and one argmax byte per pooled element (window-local
 *     index i*fW+j of the first maximum, as aether_pool_fwd).  training != 0: batch statistics (from `partials` of
 *     aether_conv2d_fwd_bnstats, or reduced here when NULL), running statistics updated, batch_mean/var written;
 *     training == 0: running statistics, channel_scale ignored.  ws: aether_bn_workspace_bytes(S*H*W, C).
 *   aether_bn_act_pool_bwd: dpooled is the gradient w.r.t. that pooled tensor; returns dx (S,H,W,C), dgamma, dbeta.
 *     The activation's derivative is recomputed from x (pre-activation gamma*xhat + beta), so it equals
 *     ReLU/Leaky_ReLU.backward exactly (the gradient passes where the pre-activation is 0). */
int aether_bn_act_pool_fwd(const float* x, const float* partials, int64_t nblocks, const float* gamma, const float* beta,
                           float* running_mean, float* running_var, float* batch_mean, float* batch_var, float* pooled,
                           uint8_t* argmax, int S, int H, int W, int C, int fH, int fW, float eps, float momentum,
                           float alpha, const float* channel_scale, int training, void* ws, size_t ws_bytes, void* stream);
int aether_bn_act_pool_bwd(const float* x, const float* dpooled, const uint8_t* argmax, const float* gamma,
                           const float* beta, const float* batch_mean, const float* batch_var, float* dx, float* dgamma,
                           float* dbeta, int S, int H, int W, int C, int fH, int fW, float eps, float alpha,
                           const float* channel_scale, void* ws, size_t ws_bytes, void* stream);
/* The same two passes writing, from the values they already hold, the bf16 operand copy the neighbouring convolution
 * reads (see aether_conv2d_operand_layout):
 *   ..._fwd_copy: operand_copy (nullable) = the next layer's copy of x, [S*(H/fH)*(W/fW)][copy_ld] bf16, copy_ld >= C.
 *   ..._bwd_copy: operand_copy (nullable) = the previous convolution's copy of dy, [S*H*W][copy_ld] bf16, together
 *     with one row of column sums of dx per thread block in colsum_part [*colsum_rows <= colsum_rows_max][C]
 *     (needs C/4 to divide 256).  With operand_copy == NULL they are the calls above.  With an operand copy the fp32
 *     result itself (pooled / dx) may be NULL: a caller whose next kernel reads only the copy saves that write.
 *   selected_x (nullable, float, shaped like the pooled tensor): the forward pass stores x at every window's selected
 *     cell; given back to the backward pass, its statistics pass reads that and dpooled (half of |x|) instead of
 *     gathering all of x.  Same sums: only the selected cell of a window has a gradient. */
int aether_bn_act_pool_fwd_copy(const float* x, const float* partials, int64_t nblocks, const float* gamma,
                                const float* beta, float* running_mean, float* running_var, float* batch_mean,
                                float* batch_var, float* pooled, uint8_t* argmax, int S, int H, int W, int C, int fH, int fW,
                                float eps, float momentum, float alpha, const float* channel_scale, int training,
                                void* operand_copy, int copy_ld, float* selected_x, void* ws, size_t ws_bytes, void* stream);
int aether_bn_act_pool_bwd_copy(const float* x, const float* dpooled, const uint8_t* argmax, const float* gamma,
                                const float* beta, const float* batch_mean, const float* batch_var, float* dx, float* dgamma,
                                float* dbeta, int S, int H, int W, int C, int fH, int fW, float eps, float alpha,
                                const float* channel_scale, void* operand_copy, int copy_ld, float* colsum_part,
                                int colsum_rows_max, int* colsum_rows, const float* selected_x, void* ws, size_t ws_bytes,
                                void* stream);

/* ---- Pooling, 'valid' padding (CNN_classes_cupy.py:204-312) ---------------------------------- */
/* Forward :212-273.  argmax (uint8, same shape as y; max pooling only) receives i*fW+j of the first
 * maximum of each window in row-major order (:259-265). */
int aether_pool_fwd(const float* x, float* y, uint8_t* argmax, int S, int H, int W, int C, int fH, int fW, int sH, int sW,
                    int kind, void* stream);
/* Backward :275-312 (max: routes dy to the argmax cell; average: dy/(fH*fW) to every cell, kernel :163-202). */
int aether_pool_bwd(const float* dy, const uint8_t* argmax, float* dx, int S, int H, int W, int C, int fH, int fW, int sH,
                    int sW, int kind, void* stream);

/* ---- ReLU :406-415 (alpha = 0) and Leaky_ReLU :417-428 --------------------------------------- */
int aether_leaky_relu_fwd(const float* x, float* y, int64_t n, float alpha, void* stream);
/* dx = dy where x >= 0, alpha*dy where x < 0. */
int aether_leaky_relu_bwd(const float* x, const float* dy, float* dx, int64_t n, float alpha, void* stream);

/* ---- Layer_Dropout_Spatial :384-404: y = x * scale[c], scale = channel mask / keep_prob (C floats);
 *      the same call with dy gives the backward. */
int aether_channel_scale(const float* x, const float* scale, float* y, int64_t n, int C, void* stream);
/* ---- Layer_Dropout :364-382: mask = Bernoulli(keep_prob)/keep_prob drawn from Philox(seed, offset),
 *      y = x * mask; the mask is stored for the backward (aether_mul(dy, mask)). */
int aether_dropout_fwd(const float* x, float* y, float* mask, int64_t n, float keep_prob, uint64_t seed, uint64_t offset,
                       void* stream);
int aether_mul(const float* a, const float* b, float* y, int64_t n, void* stream);

/* ---- Optimizer_Adam.update_parameters :702-734 over one flat buffer.  bias_corr = 1 - beta^(it+1);
 *      epsilon is added outside the square root; grad_scale multiplies g first (1/world for the
 *      data-parallel average). */
int aether_adam_step(float* p, const float* g, float* m, float* v, int64_t n, float lr, float beta1, float beta2,
                     float eps, float bias_corr1, float bias_corr2, float grad_scale, void* stream);
/* ---- Variants for a train step captured in a CUDA graph.  A replayed graph cannot change kernel arguments, so
 *      whatever the reference changes on the host from step to step is read from device memory instead: one int64
 *      counter that the caller increments once per step (a device-side add inside the graph).
 *   aether_adam_step_dev: Optimizer_Adam.pre_update_parameters + update_parameters (:705-734) with
 *      iterations = *iterations_dev: lr = lr0 / (1 + decay*iterations), bias_corr = 1 - beta^(iterations+1).
 *   aether_dropout_fwd_dev: Layer_Dropout.forward (:364-382) on Philox stream offset + (*calls_dev << 40).
 *   aether_channel_mask_dev: the (C,) mask of Layer_Dropout_Spatial.forward (:392-397), Bernoulli(keep_prob)/keep_prob
 *      per channel, drawn on the device (the reference draws it with NumPy on the host); apply it with
 *      aether_channel_scale. */
int aether_adam_step_dev(float* p, const float* g, float* m, float* v, int64_t n, float lr0, float decay, float beta1,
                         float beta2, float eps, float grad_scale, const int64_t* iterations_dev, void* stream);
int aether_dropout_fwd_dev(const float* x, float* y, float* mask, int64_t n, float keep_prob, uint64_t seed,
                           uint64_t offset, const int64_t* calls_dev, void* stream);
int aether_channel_mask_dev(float* mask, int C, float keep_prob, uint64_t seed, const int64_t* calls_dev, void* stream);
/* L1/L2 terms of Layer_Dense.backward :337-351: g += l1*sign(w) + 2*l2*w. */
int aether_regularizer_grad(const float* w, float* g, int64_t n, float l1, float l2, void* stream);
/* Loss.regularization_loss :593-609: out[0] += l1*sum|w| + l2*sum w^2. */
int aether_regularizer_loss(const float* w, int64_t n, float l1, float l2, float* out, void* stream);

/* ---- SoftMax.forward :542-547 + Loss_CategoricalCrossEntropy.forward :615-632 + combined backward
 *      :666-680.  z [rows][classes]; labels int32 [rows] or NULL; any of prob, loss (per sample), dz,
 *      correct (1 where argmax == label) may be NULL.  smooth_fwd / smooth_bwd are the label smoothing
 *      applied to the loss and to the gradient.  input_is_prob != 0: z already holds probabilities
 *      (the reference's loss classes take the softmax OUTPUT), so the softmax itself is skipped. */
int aether_softmax_cce(const float* z, const int32_t* labels, float* prob, float* loss, float* dz, int32_t* correct,
                       int rows, int classes, float smooth_fwd, float smooth_bwd, int input_is_prob, void* stream);
/* The same with rows of target probabilities, float [rows][classes], instead of class indices: one-hot rows or soft
 * targets, used as they are (after label smoothing) by the loss and its gradient (:625-637, :644-650, :672-680);
 * `correct` compares arg-maxes. */
int aether_softmax_cce_targets(const float* z, const float* targets, float* prob, float* loss, float* dz, int32_t* correct,
                               int rows, int classes, float smooth_fwd, float smooth_bwd, int input_is_prob, void* stream);
/* SoftMax.backward on its own (:549-560, the per-sample Jacobian loop): dinputs = p * (dvalues - sum_k p_k dvalues_k)
 * per row; p is the softmax output. */
int aether_softmax_bwd(const float* p, const float* dvalues, float* dinputs, int rows, int classes, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* AETHER_B200_H */
