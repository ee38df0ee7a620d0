/*
 * b200conv.h -- C ABI of the B200 (sm_100a) convolution hot-path library (libb200conv.so).
 *
 * Drop-in boundary for the tensor-math layer of da-nie/CUDA-CNN-GAN-VAE: every entry point below
 * replaces one static method of the reference's CTensorConv / CTensorMath / CTensorApplyFunc
 * classes (the reference file:line is cited on each).  The reference has no C ABI of its own; its
 * header-only templates call CUDA kernels directly, so the binding a maintainer adds is a thin
 * header whose static methods forward to these functions (shipped in host/ of this package).
 *
 * Conventions
 *  - All tensors are dense fp32 in the reference layout W,Z,Y,X (W = batch, Z = channels), i.e.
 *    NCHW; every pointer is a DEVICE pointer unless a name ends in _host.  Position tensors of
 *    max-pooling are pairs {uint32 X, uint32 Y} (the reference's SPos).
 *  - Every operand carries its own W count and is indexed with (w % count): the reference's
 *    W-broadcast rule (cpu/ctensorconv.h:113-116).
 *  - Convolution weights are [Wk][K][C*kh*kw], a filter row ordered c*kh*kw + ky*kw + kx
 *    (cpu/ctensorconv.h:138); bias is [Wb][K].
 *  - `stream` is a cudaStream_t passed as void*.  Calls are asynchronous on that stream; they
 *    never exit the process and never throw.  Return value 0 = success, otherwise a B200_E_* code;
 *    b200_last_error() gives the text of the last failure on the calling thread.
 *  - Scratch memory (packed operands, split-K partial sums) comes from a per-device arena that the
 *    library grows with cudaMalloc on demand and releases in b200_shutdown().
 *  - Threads: the reference is a single-threaded program and so is this library's state.  Use ONE host thread per device,
 *    and one stream at a time per device for the stateless entry points (they share the device's scratch arena; a layer
 *    context owns its buffers and serves one stream at a time).  The precision mode and the profiling switch are
 *    process-wide.  Calls from several threads on the same device must be serialised by the caller.
 *  - Alignment: tensors may start at any 4-byte boundary (the vector code paths are taken only when the pointers allow);
 *    the position tensor of max-pooling must be 8-byte aligned.
 */
#ifndef B200CONV_H
#define B200CONV_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
    B200_OK = 0,
    B200_E_SHAPE = 1,      /* inconsistent sizes (the reference throws a C string here)            */
    B200_E_ARG = 2,        /* null pointer / unsupported value                                      */
    B200_E_CUDA = 3,       /* a CUDA runtime or driver call failed                                  */
    B200_E_TIMEOUT = 4,    /* a bounded device-side wait gave up; the context stays usable          */
    B200_E_NOMEM = 5,      /* a fixed-size scratch area is too small for this call                  */
    B200_E_NCCL = 6        /* reserved (the library's own exchange reports B200_E_CUDA / B200_E_TIMEOUT)          */
};

/* Arithmetic of the tensor-core contractions.  B200_TF32X3 (default) splits every operand into a
 * TF32 high and low part and issues three MMAs per product (error ~2^-21, meets 1e-4 against the
 * fp32 CPU backend); B200_TF32 issues one (error ~2^-11, 2e-3); B200_FP32 forces the CUDA-core
 * fp32 kernels for every shape. */
enum { B200_TF32X3 = 0, B200_TF32 = 1, B200_FP32 = 2 };

/* Which implementation the last convolution / GEMM call on this thread used. */
enum { B200_PATH_NONE = 0, B200_PATH_SIMT = 1, B200_PATH_TCGEN05 = 2 };

/* Geometry of one convolution layer, named as in the reference signatures
 * (cuda/ctensorconv.cu.h:63-66).  out_y/out_x are the spatial size of the forward output
 * ((in - kernel + 2*padding)/stride + 1); for the backward pass in_y/in_x is the size of the
 * tensor being produced. */
typedef struct b200_conv_geom {
    int in_z, in_y, in_x;          /* image channels, height, width                               */
    int kernel_amount;             /* number of filters K                                          */
    int kernel_y, kernel_x;
    int stride_y, stride_x;
    int padding_y, padding_x;
    int out_y, out_x;
} b200_conv_geom;

/* Activation codes (netlayer/neuron.cu.h NEURON_FUNCTION_*; scalar definitions
 * cpu/ctensorapplyfunc.h:128-257).  LEAKY_RELU uses the slope given to the call, a double multiplied
 * in double precision as the reference does with its constant 0.1. */
enum { B200_ACT_SIGMOID = 0, B200_ACT_RELU = 1, B200_ACT_LEAKY_RELU = 2, B200_ACT_LINEAR = 3,
       B200_ACT_TANH = 4, B200_ACT_GELU = 5 };

/* ---- library control ------------------------------------------------------------------------ */
const char *b200_last_error(void);
int b200_last_path(void);
int b200_set_precision(int mode);
int b200_get_precision(void);
/* Frees the scratch arena of every device.  Safe to call more than once. */
int b200_shutdown(void);
/* Bytes currently held by the scratch arena of the current device. */
size_t b200_scratch_bytes(void);
/* Waits for `stream` and reports what the kernels recorded: B200_OK, B200_E_CUDA if the stream
 * failed, B200_E_TIMEOUT if a bounded device-side wait (mbarrier) gave up.  The reference's
 * counterpart is the cudaDeviceSynchronize + HANDLE_ERROR pair after every launch
 * (cuda/ctensormath.cu.h:1980-1981, cuda/handle_error.cu.h:7-18), minus the exit(). */
int b200_stream_status(void *stream);
/* Test aid with no reference counterpart: writes `code` into the current device's status word FROM THE HOST, exactly where a
 * device-side wait that gave up would have recorded it, so that a caller's handling of B200_E_TIMEOUT can be exercised
 * without making any kernel wait.  The next b200_stream_status() on the device reports and clears it. */
int b200_debug_set_status(unsigned code);

/* Number of kernels this library has launched in this process (all devices, all threads). */
unsigned long long b200_launch_count(void);
/* Measurement aid with no reference counterpart: when enabled, every launch of the tcgen05 kernel
 * is bracketed by a pair of CUDA events on its stream; b200_profile_read() waits for the recorded
 * launches and returns their summed duration in milliseconds and their number, then forgets them. */
int b200_profile_tensor_core(int enable);
int b200_profile_read(double *total_ms, int *launches);

/* ---- convolution trio ------------------------------------------------------------------------ */

/* CTensorConv::ForwardConvolution (cuda/ctensorconv.cu.h:276-315, cpu/ctensorconv.h:84-148):
 * out[w,k,oy,ox] = bias[w%Wb,k] + sum_{ky,kx,c} kernel[w%Wk,k,c,ky,kx] * image[w%Wi,c,s*oy+ky-p,s*ox+kx-p]. */
int b200_conv_forward(const b200_conv_geom *g, float *out, int out_w,
                      const float *image, int image_w, const float *kernel, int kernel_w,
                      const float *bias, int bias_w, void *stream);

/* CTensorConv::BackwardConvolution (cuda/ctensorconv.cu.h:683-725, cpu/ctensorconv.h:196-266):
 * out_delta[w,c,y,x] = sum_{ky,kx,f} kernel[f,c,kh-1-ky,kw-1-kx] * delta[w,f,(y+ky-p')/s,(x+kx-p')/s]
 * over taps where the division is exact and in range, p' = k-1-p.  Also the forward pass of the
 * transposed-convolution layer.  `bias` may be NULL; if given it is added once per contributing tap
 * and filter, which is what the reference CPU backend does (every reference caller passes zeros). */
int b200_conv_backward(const b200_conv_geom *g, float *out_delta, int out_w,
                       const float *delta, int delta_w, const float *kernel, int kernel_w,
                       const float *bias, int bias_w, void *stream);

/* CTensorConv::CreateDeltaWeightAndBias (cuda/ctensorconv.cu.h:1168-1211, cpu/ctensorconv.h:319-386):
 * for every w < dkernel_w:  dkernel[w] += wgrad(image[w%Wi], delta[w%Wd]),  dbias[w%Wb] += sum delta.
 * Accumulates into the existing contents. */
int b200_conv_wgrad(const b200_conv_geom *g, float *dkernel, int dkernel_w, float *dbias, int dbias_w,
                    const float *image, int image_w, const float *delta, int delta_w, void *stream);

/* CTensorConv::CreateBackDeltaWeightAndBias (cuda/ctensorconv.cu.h:1218-1222): the same with image
 * and delta exchanged (`image` = layer input with kernel_amount channels of size out_y x out_x,
 * `delta` = error of the layer output with in_z channels of size in_y x in_x); dbias is zeroed. */
int b200_conv_back_wgrad(const b200_conv_geom *g, float *dkernel, int dkernel_w, float *dbias, int dbias_w,
                         const float *image, int image_w, const float *delta, int delta_w, void *stream);

/* Batch-summed weight gradient used by the layers: what CNetLayerConvolution::TrainingBackward
 * obtains from CreateDeltaWeightAndBias into a per-sample tensor followed by two AddSumW passes
 * (netlayer/cnetlayerconvolution.cu.h:501-508), without materialising the per-sample tensor:
 *   dkernel[K][C*kh*kw] (+)= sum_w wgrad(image[w], delta[w]),  dbias[K] (+)= sum_w sum_yx delta[w].
 * accumulate = 0 overwrites, 1 adds to the existing contents.  dbias may be NULL. */
int b200_conv_wgrad_batch(const b200_conv_geom *g, float *dkernel, float *dbias, int accumulate,
                          const float *image, const float *delta, int batch, void *stream);

/* ---- layer-level calls ------------------------------------------------------------------------- */

/* The Forward / TrainingBackward pair of the reference's convolution layer
 * (netlayer/cnetlayerconvolution.cu.h:310-318 and 484-515) and, with transposed != 0, of its
 * transposed-convolution layer (netlayer/cnetlayerbackconvolution.cu.h:303-313 and 475-497), on a
 * context object that owns the packed operands: the packed layer input made by the forward call is
 * reused by the weight gradient, and the packed output error is shared by the input-error and the
 * weight-gradient kernels.  `g` always describes the underlying convolution; for a transposed layer the
 * layer input has kernel_amount channels of out_y x out_x and the layer output in_z channels of
 * in_y x in_x.  One context serves one layer and one stream at a time; create/destroy allocate and free
 * device memory (buffers grow on first use).  The forward call also prepares the re-laid-out weights of the backward pass:
 * `kernel` must not change between a layer's forward call and the backward call that follows it (TrainingUpdateWeight runs
 * after all backward passes in every training loop of the reference). */
typedef struct b200_conv_layer b200_conv_layer;
int b200_conv_layer_create(b200_conv_layer **layer, const b200_conv_geom *g, int batch, int transposed);
int b200_conv_layer_destroy(b200_conv_layer *layer);
/* out = conv(input) + bias (convolution layer) or the transposed convolution of input (transposed layer;
 * its bias is ignored, as in the reference's CUDA backend). */
int b200_conv_layer_forward(b200_conv_layer *layer, float *out, const float *input, const float *kernel, const float *bias,
                            void *stream);
/* Forward with the function layers around the convolution layer folded in (CNetLayerFunction::Forward,
 * netlayer/cnetlayerfunction.cu.h:202: H = f(input of the function layer)):
 *   input_func  >= 0: the layer's input is f_in(input) -- the function layer IN FRONT of this layer; f_in is applied while
 *                     the input is re-laid out for the tensor cores, so the activated tensor need not exist.  input_act_out,
 *                     if not NULL, also receives f_in(input) (same shape as input).
 *   output_func >= 0: out = f_out(conv + bias) -- the function layer BEHIND this layer, applied in the epilogue of the
 *                     convolution kernel.  output_pre, if not NULL, receives conv + bias (what that function layer keeps
 *                     for its derivative in SetOutputError, :347-358).
 * -1 switches a side off; both off (or fusion == NULL) is b200_conv_layer_forward.  The results are bit-identical to the
 * separate calls b200_activation -> b200_conv_layer_forward -> b200_activation in the same precision mode.  A later
 * b200_conv_layer_backward must be given, as `input`, f_in(input) if it has to re-pack (it does not when it follows this
 * call in the same precision mode on a tensor-core path; pass input_act_out to be safe in B200_FP32 mode). */
typedef struct b200_conv_fusion {
    int input_func;
    double input_slope;
    float *input_act_out;
    int output_func;
    double output_slope;
    float *output_pre;
} b200_conv_fusion;
int b200_conv_layer_forward_fused(b200_conv_layer *layer, float *out, const float *input, const float *kernel, const float *bias,
                                  const b200_conv_fusion *fusion, void *stream);
/* The weights of several layers re-laid out for the tensor cores in ONE launch, for the next forward call of each (the
 * reference has no counterpart: its layers read the weights as they are; netlayer/cnetlayerconvolution.cu.h:310).  A training
 * step that calls this once for all layers of its nets, before their forward passes, saves one launch per layer.  kernels[i]
 * is the kernel tensor that layer i's next b200_conv_layer_forward(_fused) call will be given.  The mark is good for that one
 * forward call (and the backward call after it) in the current precision mode; a forward call without it packs the weights
 * itself, so calling this is never required -- but the weights must not change between this call and the forward call. */
int b200_conv_layers_prepack(b200_conv_layer *const *layers, const float *const *kernels, int count, void *stream);
/* input_delta (may be NULL) = error of the layer input; dkernel / dbias (may be NULL) (+)= batch-summed
 * gradients (dbias of a transposed layer is cleared, as the reference does).  `input` must hold what the
 * forward call saw: it is only read when the kept pack cannot be used (no forward call yet, precision
 * mode changed, or the CUDA-core path).  The call may be split in two on the same output_delta -- gradients only
 * (input_delta NULL), then input error only (dkernel and dbias NULL) -- so that the caller can start reducing the
 * gradients across devices while the input error is computed; the second call then reuses the packed error of the
 * first, provided nothing else was called on the layer in between and output_delta was not modified. */
int b200_conv_layer_backward(b200_conv_layer *layer, float *input_delta, float *dkernel, float *dbias, int accumulate,
                             const float *output_delta, const float *input, const float *kernel, void *stream);

/* Allocation-free form of b200_conv_wgrad_batch (no counterpart in the reference, which allocates
 * its per-sample gradient tensors up front in the layer objects).  For callers that must not allocate
 * device memory where they call the library: hosts that hand out all device memory from their own pool
 * at start-up, loops that cannot take the device-wide stall of cudaMalloc/cudaFree, and program phases
 * in which the CUDA runtime refuses allocations.  Same arguments and result as b200_conv_wgrad_batch
 * (fp32 CUDA-core arithmetic in the reference summation order, whatever the precision mode), but the
 * per-sample scratch lives in a fixed 16 MiB array inside the library image (b200_static_scratch_bytes(),
 * held by every GPU that loads the library until the process exits): batch * (K*C*kh*kw + K) floats must
 * fit, otherwise the call returns B200_E_NOMEM and does nothing.  It calls no cudaMalloc / cudaFree.
 * The first call on each device looks up the array's device address; make that first call outside any
 * stream capture, with the device current.  All calls on a device share the array, which keeps the last
 * call's contents (this call clears what it needs first): two calls whose kernels overlap on the GPU
 * (different streams, no ordering between them) race on it. */
int b200_conv_wgrad_batch_static(const b200_conv_geom *g, float *dkernel, float *dbias, int accumulate,
                                 const float *image, const float *delta, int batch, void *stream);
size_t b200_static_scratch_bytes(void);

/* ---- dense products -------------------------------------------------------------------------- */

/* CTensorMath::Mul (cuda/ctensormath.cu.h:2237, cpu/ctensormath.h:531-595) when transpose_left = 0:
 *   out[w,z] (LY x RX) = left[w%Lw,z] (LY x LX) * right[w%Rw,z] (LX x RX);
 * CTensorMath::TransponseMul (:2249, cpu :643-712) when transpose_left = 1:
 *   out[w,z] (LX x RX) = left[w%Lw,z]^T (left is LY x LX) * right[w%Rw,z] (LY x RX). */
int b200_mul(float *out, int out_w, const float *left, int left_w, const float *right, int right_w,
             int z, int ly, int lx, int rx, int transpose_left, void *stream);

/* ---- element-wise, reductions ---------------------------------------------------------------- */

/* CTensorMath::Add / Sub (cuda/ctensormath.cu.h:837,1021; cpu :235,314): out[w] = ls*left[w%Lw] +/- rs*right[w%Rw];
 * n = Z*Y*X elements per w. */
int b200_add(float *out, int out_w, const float *left, int left_w, const float *right, int right_w,
             size_t n, float ls, float rs, int subtract, void *stream);
/* CTensorMath::AddSumW (cuda :914, cpu :273): out[0] = ls*sum_w left + rs*sum_w right, out[w>0] = 0.
 * out may alias left or right. */
int b200_add_sum_w(float *out, int out_w, const float *left, int left_w, const float *right, int right_w,
                   size_t n, float ls, float rs, void *stream);
/* CTensorMath::AddBias (cuda :1328, cpu :352): t[w,z,:,:] += bias[w%Bw,z]. */
int b200_add_bias(float *t, int t_w, int z, size_t yx, const float *bias, int bias_w, void *stream);
/* CTensorMath::SummXY (cuda :1396, cpu :455): out[w,z] = sum_{y,x} in[w%Iw,z,:,:]. */
int b200_summ_xy(float *out, int out_w, const float *in, int in_w, int z, size_t yx, void *stream);
/* CTensorMath::Pow2 (op 0: i*i*a), SQRT (op 1: sqrt(i+b)*a), Inv (op 2: 1/i), Mul by scalar (op 3: i*a)
 * (cuda :1196,1262,702,2291; cpu :387,421,163,721); AddValue / SubValue / Set (op 4: i*a+b; cuda :986,1061,1127),
 * Clip (op 5: min(max(i,a),b); cuda :2807), Signum (op 6; cuda :2865); input W-broadcast. */
int b200_unary(float *out, int out_w, const float *in, int in_w, size_t n, int op, float a, float b, void *stream);
/* CTensorMath::Div (cuda :738-800, cpu :197): out[w] = (ls*left[w%Lw]) / (rs*right[w%Rw]). */
int b200_div(float *out, int out_w, const float *left, int left_w, const float *right, int right_w,
             size_t n, float ls, float rs, void *stream);
/* CTensorMath::ConcatecationZ (cuda/ctensormath.cu.h:502): out[w] = the planes of a[w % a_w] followed by those of b[w % b_w];
 * CTensorMath::SplitZ (:569): the first a_z planes of in[w] to out_a[w], the other b_z to out_b[w].  yx = Y*X. */
int b200_concat_z(float *out, int out_w, const float *a, int a_w, int a_z, const float *b, int b_w, int b_z, size_t yx, void *stream);
int b200_split_z(float *out_a, int a_z, float *out_b, int b_z, const float *in, int w, size_t yx, void *stream);
/* CTensorMath::Transponse (cuda :2345-2390, cpu :787): every (w,z) plane rows x cols -> cols x rows. */
int b200_transpose(float *out, const float *in, int planes, int rows, int cols, void *stream);
/* CTensorMath::TensorItemProduction (cuda :2425, cpu :822). */
int b200_item_product(float *out, int out_w, const float *left, int left_w, const float *right, int right_w,
                      size_t n, void *stream);
/* CTensorMath::Fill (cuda :637, cpu :154). */
int b200_fill(float *out, size_t n, float value, void *stream);

/* CTensorApplyFunc::Apply* / ApplyDifferential* (cuda/ctensorapplyfunc.cu.h:325-866): out = f(in) or f'(in). */
int b200_activation(float *out, const float *in, size_t n, int func, int derivative, double leaky_slope, void *stream);
/* CNetLayerFunction::SetOutputError (netlayer/cnetlayerfunction.cu.h:347-358) fused: out = f'(z) * error. */
int b200_activation_backward(float *out, const float *z, const float *error, size_t n, int func, double leaky_slope,
                             void *stream);
/* AddBias followed by an activation in one pass: t[w,z,:,:] = f(t + bias[z]) (cuda/ctensormath.cu.h:1328 +
 * ctensorapplyfunc.cu.h Apply*).  pre may be NULL; if given it receives t + bias (the value the
 * activation layer keeps for its derivative). */
int b200_bias_activation(float *t, float *pre, int t_w, int z, size_t yx, const float *bias, int func,
                         double leaky_slope, void *stream);

/* ---- pooling / resampling -------------------------------------------------------------------- */

/* CTensorMath::MaxPooling (cuda :2693, cpu :955-1013): window max and absolute argmax {X,Y}; ties keep the
 * first element of the row-major scan. */
int b200_maxpool(float *out, uint32_t *pos, const float *in, int w, int z, int in_y, int in_x, int pool_x, int pool_y,
                 void *stream);
/* CTensorMath::MaxPoolingBackward (cuda :2767, cpu :1019-1055): out zeroed, out[argmax] = delta. */
int b200_maxpool_backward(float *out, const uint32_t *pos, const float *delta, int w, int z, int out_y, int out_x,
                          int pool_x, int pool_y, void *stream);
/* CTensorMath::UpSampling (cuda :2518, cpu :868) and DownSampling (cuda :2600, cpu :908; mean, used as the
 * backward of UpSampling). */
int b200_upsample(float *out, const float *in, int w, int z, int in_y, int in_x, int ux, int uy, void *stream);
int b200_downsample(float *out, const float *in, int w, int z, int in_y, int in_x, int dx, int dy, void *stream);

/* ---- fused layer kernels --------------------------------------------------------------------- */

/* CNetLayerBatchNormalization::Forward, training mode (netlayer/cnetlayerbatchnormalization.cu.h:301-379):
 * statistics per (z,y,x) element over the batch W; n = Z*Y*X.  Writes y, xhat (W*n each), ivar, mean,
 * var (n each); if new_mean/new_var are non-NULL they are updated as m*old + (1-m)*batch statistic. */
int b200_bn_forward(float *y, float *xhat, float *ivar, float *mean, float *var, float *new_mean, float *new_var,
                    const float *x, const float *gamma, const float *beta, int w, size_t n, float momentum, float eps,
                    void *stream);
/* CNetLayerBatchNormalization::TrainingBackward (:578-604): dx, and dgamma += sum_w dy*xhat,
 * dbeta += sum_w dy when create_delta_weight != 0. */
int b200_bn_backward(float *dx, float *dgamma, float *dbeta, const float *dy, const float *xhat, const float *ivar,
                     const float *gamma, int w, size_t n, int create_delta_weight, void *stream);
/* The batch-normalisation layer together with the function layer that follows it (CNetLayerFunction::Forward and
 * SetOutputError, netlayer/cnetlayerfunction.cu.h:347-358), same arithmetic as the two layers in sequence:
 * forward writes out = f(gamma*xhat + beta) (the normalisation's own output is not stored); backward takes the error
 * above the function layer, forms f'(gamma*xhat + beta) * error (the output recomputed from xhat) and continues as
 * b200_bn_backward.  func is a B200_ACT_* code. */
int b200_bn_act_forward(float *out, float *xhat, float *ivar, float *mean, float *var, float *new_mean, float *new_var,
                        const float *x, const float *gamma, const float *beta, int w, size_t n, float momentum, float eps,
                        int func, double leaky_slope, void *stream);
int b200_bn_act_backward(float *dx, float *dgamma, float *dbeta, const float *error, const float *xhat, const float *ivar,
                         const float *gamma, const float *beta, int w, size_t n, int create_delta_weight, int func,
                         double leaky_slope, void *stream);
/* CNetLayerVAECoderOutput::Forward (netlayer/cnetlayervaecoderoutput.cu.h:251-280) with the noise eps
 * supplied by the caller: z = mu + exp(clamp(logvar,-10,10)/2)*eps; *kl_host (host pointer, may be NULL;
 * the call synchronises the stream if given) receives -0.5/batch * sum(1+lv-mu^2-exp(lv)). */
int b200_vae_forward(float *z, const float *mu, const float *logvar, const float *eps, int batch, size_t n,
                     float *kl_host, void *stream);
/* CNetLayerVAECoderOutput::SetOutputError (:424-455). */
int b200_vae_backward(float *d_mu, float *d_logvar, const float *delta, const float *mu, const float *logvar,
                      const float *eps, size_t total, float kl_speed, void *stream);
/* CTensorMath::Adam (cuda :2978-3022, cpu :1119-1165).  iteration is used as given (the CPU backend's rule).  The moments m
 * and v are bit-identical to the CPU backend's; the step is evaluated in fp32 instead of double, so an updated weight may
 * differ from the CPU backend's in its last bit. */
int b200_adam(float *weight, const float *dweight, float *m, float *v, size_t n, uint32_t batch_size, double speed,
              double beta1, double beta2, double epsilon, double iteration, void *stream);
/* The same update with the two bias corrections {1 - beta1^t, 1 - beta2^t} read from device memory (two doubles) instead of
 * being formed from `iteration` on the host: every argument of the launch is then fixed, so a step that ends in Adam can be
 * replayed from a CUDA graph while the caller refreshes the two numbers before each replay.  No reference counterpart. */
int b200_adam_prepared(float *weight, const float *dweight, float *m, float *v, size_t n, uint32_t batch_size, double speed,
                       double beta1, double beta2, double epsilon, const double *corrections, void *stream);
/* ---- helpers of the diffusion model and the drop-out layer ------------------------------------- */

/* CTensorMath::SetTimeStep (cuda/ctensormath.cu.h:3029-3096; the forward pass of CNetLayerTimeEmbedding,
 * netlayer/cnetlayertimeembedding.cu.h:224-227): out[w,pos] = in[w,pos] + (pos even ? sin : cos)(t[w] / 10000^(pos/n)), pos the
 * linear index inside one sample of n = Z*Y*X elements, t a DEVICE array of w uint32 time steps. */
int b200_set_time_step(float *out, const float *in, const uint32_t *time_step, int w, size_t n, void *stream);
/* CTensorMath::SetNormalNoise (cuda/ctensormath.cu.h:3161-3210): standard normal numbers.  The reference seeds cuRAND states
 * with rand(); here the caller gives the seed of a counter-based Philox4x32-10 stream (same seed, same tensor). */
int b200_normal_noise(float *out, size_t n, unsigned long long seed, void *stream);
/* CTensorMath::CreateDropOutMatrix (cuda/ctensormath.cu.h:3101-3156): 0 with probability drop_out, else 1 / (1 - drop_out). */
int b200_dropout_mask(float *out, size_t n, float drop_out, unsigned long long seed, void *stream);
/* CTensorMath::GetNoiseImageAndNoise (cuda/ctensormath.cu.h:3216-3294): noisy[w] = sqrt_alpha_bar[w] * image[w] +
 * sqrt_one_minus_alpha_bar[w] * noise[w] (the two coefficient arrays hold one float per sample).  generate != 0: the noise
 * is drawn (seed) and written to `noise` in the same pass, as the reference does; generate == 0: `noise` is an input. */
int b200_noisy_image(float *noisy, float *noise, const float *image, const float *sqrt_alpha_bar, const float *sqrt_one_minus_alpha_bar,
                     int w, size_t n, int generate, unsigned long long seed, void *stream);

/* Adam followed by the exponential moving average of the updated weights that the reference's layers keep when EMA is
 * enabled (netlayer/cnetlayerconvolution.cu.h:547-551: Add(W_EMA, W_EMA, W, EMA_K, 1 - EMA_K) after the update), in the same
 * pass over the parameters: ema = ema_k * ema + (1 - ema_k) * weight.  ema may be NULL (plain Adam).  corrections, when
 * non-NULL, replaces `iteration` as in b200_adam_prepared. */
int b200_adam_ema(float *weight, const float *dweight, float *m, float *v, float *ema, size_t n, uint32_t batch_size, double speed,
                  double beta1, double beta2, double epsilon, double iteration, const double *corrections, double ema_k, void *stream);

/* ---- data-parallel exchange over NVLink peer memory -------------------------------------------- */

/* The reference is a single-GPU program; what it has is the reduction of per-sample gradients over W (AddSumW,
 * netlayer/cnetlayerconvolution.cu.h:507-508) and the batch_scale argument of TrainingUpdateWeight (netlayer/inetlayer.cu.h:87).
 * Here each rank (one process, or one host thread, per GPU) reduces its shard inside the weight-gradient kernel and the
 * shards are summed across GPUs by the calls below, which read and write the peers' memory directly over NVLink.
 *
 * A communicator owns one device allocation: a signal pad and a data region of `bytes` bytes (b200_comm_buffer) in which the
 * caller places the arenas to be exchanged (gradients, weights), at the same offsets on every rank.  Set-up: every rank calls
 * b200_comm_create, then b200_comm_handle, carries the B200_COMM_HANDLE_BYTES-byte handles of all ranks to all ranks by any
 * means, and calls b200_comm_connect with them in rank order.  Ranks in different processes are mapped with CUDA IPC, ranks
 * that share a process by enabling peer access.  Destroy only after every rank has finished its last exchange.
 * Exchanges on one channel (0..3) of a communicator must be issued in the same order by every rank and are serialised by
 * the stream order of each rank; exchanges that may overlap on a GPU (different streams) need different channels.
 * Every device-side wait is bounded (about a second); a rank whose peers do not arrive reports B200_E_TIMEOUT through
 * b200_stream_status and its results are invalid. */
#define B200_COMM_HANDLE_BYTES 128
typedef struct b200_comm b200_comm;
int b200_comm_create(b200_comm **comm, int rank, int world, size_t bytes);
int b200_comm_handle(b200_comm *comm, void *handle);
int b200_comm_connect(b200_comm *comm, const void *handles);
void *b200_comm_buffer(b200_comm *comm);
size_t b200_comm_buffer_bytes(b200_comm *comm);
int b200_comm_destroy(b200_comm *comm);
/* The slice [begin, end) (in floats) of an arena of n floats that rank `rank` of `world` reduces and updates.  Host
 * arithmetic only. */
int b200_comm_slice(size_t n, int rank, int world, size_t *begin, size_t *end);
/* In-place sum over the ranks of the n floats at float offset `offset` of the data region (n and offset multiples of 4):
 * each rank adds its slice from all ranks in rank order and writes the sum to all ranks. */
int b200_allreduce(b200_comm *comm, size_t offset, size_t n, int channel, void *stream);
/* Reduce-scatter + Adam + all-gather in one kernel: rank r sums slice r of the gradient arenas (at grad_offset) of all ranks,
 * applies CTensorMath::Adam (as b200_adam; batch_size is the global batch) to slice r of its weights (at weight_offset) and of
 * its local moment arrays m, v (n floats each, only slice r is touched), and writes the new weights of slice r into the
 * weight arenas of all ranks.  On return of the kernel every rank holds the same, fully updated weights; the gradient arenas
 * keep their per-rank contents.  corrections: as in b200_adam_prepared (may be NULL). */
int b200_allreduce_adam(b200_comm *comm, size_t grad_offset, size_t weight_offset, float *m, float *v, size_t n, uint32_t batch_size,
                        double speed, double beta1, double beta2, double epsilon, double iteration, const double *corrections, int channel,
                        void *stream);

/* The same for up to four arenas (the networks of one training step) in ONE launch: one pair of barriers and one launch
 * instead of one per network.  All arenas lie in the communicator's buffer; Adam's arguments are shared. */
typedef struct b200_exchange_segment {
    size_t grad_offset, weight_offset, n;      /* floats, multiples of 4 */
    float *m, *v;                               /* local Adam moments of the arena (n floats each) */
} b200_exchange_segment;
int b200_allreduce_adam_multi(b200_comm *comm, int count, const b200_exchange_segment *segments, uint32_t batch_size, double speed,
                              double beta1, double beta2, double epsilon, double iteration, const double *corrections, int channel,
                              void *stream);

#ifdef __cplusplus
}
#endif
#endif /* B200CONV_H */
