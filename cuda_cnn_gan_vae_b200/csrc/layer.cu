// Layer-level entry points: the pair Forward / TrainingBackward of the reference's convolution
// layer (netlayer/cnetlayerconvolution.cu.h:310-318, 484-515) and of its transposed-convolution
// layer (netlayer/cnetlayerbackconvolution.cu.h:303-313, 475-497) as two calls on a small context
// object.  What the context adds over the stateless tensor-math entry points is operand reuse: the
// packed copy of the layer input made for the forward pass also feeds the weight gradient, and the
// packed output error is made once for both the input error and the weight gradient.
#include "common.cuh"
#include "kernels.h"
#include <cstdlib>
#include <cstring>
#include <new>

struct b200_conv_layer {
    b200_conv_geom g;
    int batch;
    int transposed;
    int device;
    enum { IN_HI, IN_LO, ER_HI, ER_LO, W_HI, W_LO, W2_HI, W2_LO, PARTIAL, DB_TMP, COL_HI, COL_LO, TMP, DK_TMP, KSPLIT, ACT_TMP, MIRROR_W, MIRROR_DW, NBUF };
    float *buf[NBUF];
    size_t cap[NBUF];            // bytes
    int in_valid;                // the kept input pack matches the last forward call
    int in_precision;
    int col_valid;               // the kept im2col copy of the layer input matches the last forward call (few-channel layers)
    int col_precision;
    int er_valid;                // the packed output error of a weights-only backward call may serve the input-only call that follows
    int er_precision;
    const float *er_ptr;
    // how the last forward call got its input when a neuron function was fused in front of the layer: 0 the caller's tensor
    // is the layer input; 1 only the packed copy holds f(input); 2 f(input) also lies in the ACT_TMP buffer; 3 in the caller's
    // input_act_out.  The backward call reads its `input` argument only when it must re-pack, and then needs f(input).
    int fused_input;
    // The forward call packs the weights for both passes in one launch: W_HI/W_LO hold the orientation of the pass that
    // packed, W2_HI/W2_LO the other one, valid for the backward call that follows (same kernel pointer, same precision mode).
    int w_slot;                  // W_HI or W2_HI: the pack the next contraction reads
    int w2_valid, w2_precision;
    const float *w2_kernel;
    // b200_conv_layers_prepack packed both orientations for the NEXT forward call (same kernel pointer, same precision mode);
    // that call consumes the mark, so a forward call without a fresh prepack packs the weights itself.
    int prepacked, prepacked_precision;
    const float *prepacked_kernel;
    // A convolution layer with few filters (an RGB output layer) computes its input error and its weight gradient on the
    // mirrored problem, which has few input channels: a second context with the mirrored geometry (NULL for other layers).
    b200_conv_layer *mirror;
    // set on a mirror context around its backward call: the packed output error it would make already exists (it is the
    // owner's packed layer input)
    const float *lent_er_hi, *lent_er_lo;
};

namespace b200 {

static int ensure(b200_conv_layer *l, int which, size_t bytes, cudaStream_t s)
{
    if (l->cap[which] >= bytes) return B200_OK;
    if (l->buf[which]) {
        B200_CUDA(cudaStreamSynchronize(s));
        B200_CUDA(cudaFree(l->buf[which]));
        l->buf[which] = nullptr;
        l->cap[which] = 0;
    }
    void *p = nullptr;
    cudaError_t e = cudaMalloc(&p, bytes);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(B200_E_NOMEM, "conv layer: cudaMalloc(%zu) failed: %s", bytes, cudaGetErrorString(e));
    }
    l->buf[which] = (float *)p;
    l->cap[which] = bytes;
    return B200_OK;
}

// Shapes of the two packs of a layer.  "in" is what the layer's forward pass gathers, "er" what its
// backward pass gathers.
static ActPack in_shape(const b200_conv_layer *l)
{
    const b200_conv_geom &g = l->g;
    return l->transposed ? act_pack_shape(l->batch, g.kernel_amount, g.out_y, g.out_x, 1, 1)
                         : act_pack_shape(l->batch, g.in_z, g.in_y, g.in_x, g.stride_y, g.stride_x);
}
static ActPack er_shape(const b200_conv_layer *l)
{
    const b200_conv_geom &g = l->g;
    return l->transposed ? act_pack_shape(l->batch, g.in_z, g.in_y, g.in_x, g.stride_y, g.stride_x)
                         : act_pack_shape(l->batch, g.kernel_amount, g.out_y, g.out_x, 1, 1);
}

// rowsum_runs != NULL: the pack also leaves partial plane sums of src in the DB_TMP buffer (first stage of the bias gradient)
static int pack_into(b200_conv_layer *l, int hi_slot, ActPack &pk, const float *src, bool x3, cudaStream_t s, int *rowsum_runs = nullptr,
                     const PackFunction *pf = nullptr)
{
    int r;
    const size_t bytes = sizeof(float) * pk.elems() + kPackPad;
    if ((r = ensure(l, hi_slot, bytes, s))) return r;
    if (x3 && (r = ensure(l, hi_slot + 1, bytes, s))) return r;
    pk.hi = l->buf[hi_slot];
    pk.lo = x3 ? l->buf[hi_slot + 1] : nullptr;
    if (!rowsum_runs) return act_pack_fill(pk, src, s, pf);
    if ((r = ensure(l, b200_conv_layer::DB_TMP, sizeof(float) * act_pack_rowsum_elems(pk), s))) return r;
    return act_pack_fill_with_sums(pk, src, l->buf[b200_conv_layer::DB_TMP], rowsum_runs, s);
}

// first_of_step: the forward call; it also leaves the pack of the other orientation for the backward call that follows.
// The weights must not change between a layer's forward call and the backward call after it (no training loop of the
// reference changes them there: TrainingUpdateWeight runs after all backward passes).
static int pack_weights(b200_conv_layer *l, bool backward, const float *kernel, bool x3, cudaStream_t s, bool first_of_step = false)
{
    int r;
    static const bool both = !(getenv("B200CONV_PACK_BOTH") && getenv("B200CONV_PACK_BOTH")[0] == '0');      // debug switch
    const int prec = x3 ? B200_TF32X3 : B200_TF32;
    if (first_of_step) {
        const bool ready = l->prepacked && l->prepacked_kernel == kernel && l->prepacked_precision == prec;
        l->prepacked = 0;
        if (ready) {
            // packed by b200_conv_layers_prepack: this pass's orientation lies in W_HI/W_LO, the other one in W2_HI/W2_LO
            l->w_slot = b200_conv_layer::W_HI;
            l->w2_valid = 1; l->w2_precision = prec; l->w2_kernel = kernel;
            return B200_OK;
        }
    }
    if (!first_of_step && l->w2_valid && l->w2_kernel == kernel && l->w2_precision == prec) {
        l->w_slot = b200_conv_layer::W2_HI;          // packed by the forward call
        return B200_OK;
    }
    l->w2_valid = 0;
    l->w_slot = b200_conv_layer::W_HI;
    const size_t bytes = sizeof(float) * weight_pack_elems(l->g, backward);
    if ((r = ensure(l, b200_conv_layer::W_HI, bytes, s))) return r;
    if (x3 && (r = ensure(l, b200_conv_layer::W_LO, bytes, s))) return r;
    if (!first_of_step || !both)
        return weight_pack_fill(l->g, backward, kernel, l->buf[b200_conv_layer::W_HI], x3 ? l->buf[b200_conv_layer::W_LO] : nullptr, s);
    const size_t other = sizeof(float) * weight_pack_elems(l->g, !backward);
    if ((r = ensure(l, b200_conv_layer::W2_HI, other, s))) return r;
    if (x3 && (r = ensure(l, b200_conv_layer::W2_LO, other, s))) return r;
    float *mine_hi = l->buf[b200_conv_layer::W_HI], *mine_lo = x3 ? l->buf[b200_conv_layer::W_LO] : nullptr;
    float *other_hi = l->buf[b200_conv_layer::W2_HI], *other_lo = x3 ? l->buf[b200_conv_layer::W2_LO] : nullptr;
    r = backward ? weight_pack_fill_both(l->g, kernel, other_hi, other_lo, mine_hi, mine_lo, s)
                 : weight_pack_fill_both(l->g, kernel, mine_hi, mine_lo, other_hi, other_lo, s);
    if (r) return r;
    l->w2_valid = 1; l->w2_precision = prec; l->w2_kernel = kernel;
    return B200_OK;
}

// conv_gemm with the layer's split-K scratch (sized on first use; none for layers whose output is large)
static int layer_conv_gemm(b200_conv_layer *l, bool backward, const b200_conv_geom &g, float *out, const ActPack &act, const float *bias, bool x3,
                           cudaStream_t s, const EpilogueFunction *ef = nullptr)
{
    const size_t elems = conv_gemm_partial_elems(backward, g, l->batch);
    if (elems) {
        int r = ensure(l, b200_conv_layer::KSPLIT, sizeof(float) * elems, s);
        if (r) return r;
    }
    return conv_gemm(backward, g, out, act, l->buf[l->w_slot], l->buf[l->w_slot + 1], bias, x3, s,
                     elems ? l->buf[b200_conv_layer::KSPLIT] : nullptr, elems, ef);
}

// ---- few-channel layers (smallc.cu): taps folded into the channel dimension, contractions as 1x1 convolutions ------------
static bool use_smallc(const b200_conv_layer *l)
{
    static const bool enabled = !(getenv("B200CONV_SMALLC") && getenv("B200CONV_SMALLC")[0] == '0');      // debug switch
    return enabled && smallc_applies(l->g);
}

static ActPack col_shape(const b200_conv_layer *l)
{
    const b200_conv_geom &g = l->g;
    return act_pack_shape(l->batch, g.in_z * g.kernel_x * g.kernel_y, g.out_y, g.out_x, 1, 1);
}

// im2col copy of `src` (the tensor with the few channels) into the COL buffers
static int col_into(b200_conv_layer *l, ActPack &col, const float *src, bool x3, cudaStream_t s)
{
    int r;
    col = col_shape(l);
    const size_t bytes = sizeof(float) * col.elems() + kPackPad;
    if ((r = ensure(l, b200_conv_layer::COL_HI, bytes, s))) return r;
    if (x3 && (r = ensure(l, b200_conv_layer::COL_LO, bytes, s))) return r;
    col.hi = l->buf[b200_conv_layer::COL_HI];
    col.lo = x3 ? l->buf[b200_conv_layer::COL_LO] : nullptr;
    return im2col_pack(l->g, col, src, l->batch, s);
}

static int smallc_weights_into(b200_conv_layer *l, const float *kernel, int pitch, bool transposed, bool x3, cudaStream_t s)
{
    int r;
    const b200_conv_geom &g = l->g;
    const size_t rows = transposed ? (size_t)g.in_z * g.kernel_x * g.kernel_y : (size_t)g.kernel_amount;
    const size_t bytes = sizeof(float) * rows * pitch + kPackPad;
    if ((r = ensure(l, b200_conv_layer::W_HI, bytes, s))) return r;
    if (x3 && (r = ensure(l, b200_conv_layer::W_LO, bytes, s))) return r;
    l->w_slot = b200_conv_layer::W_HI;
    l->w2_valid = 0;
    return smallc_weights(g, kernel, l->buf[b200_conv_layer::W_HI], x3 ? l->buf[b200_conv_layer::W_LO] : nullptr, pitch, transposed, s);
}

// out[n, k, oy, ox] = sum_c' W'[k][c'] col[n, oy, ox, c'] (+ bias): the convolution of the few-channel tensor
static int smallc_conv(b200_conv_layer *l, float *out, const ActPack &col, const float *kernel, const float *bias, bool x3, cudaStream_t s,
                       const EpilogueFunction *ef = nullptr)
{
    int r;
    if ((r = smallc_weights_into(l, kernel, col.cp, false, x3, s))) return r;
    return layer_conv_gemm(l, false, smallc_geom(l->g), out, col, bias, x3, s, ef);
}

// dx = col2im(W''^T delta): the transposed convolution towards the few-channel tensor; `many` is the pack of the
// many-channel tensor (kernel_amount channels on the out_y x out_x plane)
static int smallc_tconv(b200_conv_layer *l, float *dx, const ActPack &many, const float *kernel, bool x3, cudaStream_t s)
{
    int r;
    const b200_conv_geom &g = l->g;
    const int cc = g.in_z * g.kernel_x * g.kernel_y;
    if ((r = smallc_weights_into(l, kernel, many.cp, true, x3, s))) return r;
    if ((r = ensure(l, b200_conv_layer::TMP, sizeof(float) * (size_t)l->batch * cc * g.out_y * g.out_x, s))) return r;
    b200_conv_geom q = smallc_geom(g);
    q.in_z = g.kernel_amount;
    q.kernel_amount = cc;
    if ((r = layer_conv_gemm(l, false, q, l->buf[b200_conv_layer::TMP], many, nullptr, x3, s))) return r;
    return col2im_gather(g, dx, l->buf[b200_conv_layer::TMP], l->batch, s);
}

// dkernel (+)= sum over positions of many x col, re-ordered into the reference's [k][c*taps + tap]
static int smallc_wgrad(b200_conv_layer *l, float *dkernel, int accumulate, const ActPack &col, const ActPack &many, bool x3, cudaStream_t s)
{
    int r;
    const b200_conv_geom &g = l->g;
    const b200_conv_geom q = smallc_geom(g);
    if ((r = ensure(l, b200_conv_layer::PARTIAL, sizeof(float) * wgrad_partial_elems(q, l->batch), s))) return r;
    if ((r = ensure(l, b200_conv_layer::DK_TMP, sizeof(float) * (size_t)g.kernel_amount * q.in_z, s))) return r;
    if ((r = wgrad_gemm(q, l->buf[b200_conv_layer::DK_TMP], 0, col, many, l->buf[b200_conv_layer::PARTIAL], x3, s))) return r;
    return smallc_dkernel(g, dkernel, l->buf[b200_conv_layer::DK_TMP], accumulate, s);
}

}  // namespace b200

using namespace b200;

extern "C" {

int b200_conv_layer_create(b200_conv_layer **layer, const b200_conv_geom *g, int batch, int transposed)
{
    if (!layer || !g) return fail(B200_E_ARG, "null argument");
    if (batch <= 0 || g->kernel_amount <= 0 || g->in_z <= 0 || g->in_y <= 0 || g->in_x <= 0 || g->kernel_x <= 0 ||
        g->kernel_y <= 0 || g->stride_x <= 0 || g->stride_y <= 0 || g->padding_x < 0 || g->padding_y < 0)
        return fail(B200_E_SHAPE, "non-positive convolution geometry");
    const int ox = (g->in_x - g->kernel_x + 2 * g->padding_x) / g->stride_x + 1;
    const int oy = (g->in_y - g->kernel_y + 2 * g->padding_y) / g->stride_y + 1;
    if (ox != g->out_x || oy != g->out_y || ox <= 0 || oy <= 0)
        return fail(B200_E_SHAPE, "wrong output size for convolution: expected %dx%d, got %dx%d", oy, ox, g->out_y, g->out_x);
    b200_conv_layer *l = new (std::nothrow) b200_conv_layer;
    if (!l) return fail(B200_E_NOMEM, "host allocation failed");
    memset(l, 0, sizeof(*l));
    l->g = *g;
    l->batch = batch;
    l->transposed = transposed != 0;
    l->w_slot = b200_conv_layer::W_HI;
    cudaGetDevice(&l->device);
    static const bool mirrors = !(getenv("B200CONV_MIRROR") && getenv("B200CONV_MIRROR")[0] == '0');      // debug switch
    if (mirrors && !l->transposed && mirror_applies(*g)) {
        const b200_conv_geom q = mirror_geom(*g);
        const int r = b200_conv_layer_create(&l->mirror, &q, batch, 0);
        if (r) { delete l; return r; }
    }
    *layer = l;
    return B200_OK;
}

int b200_conv_layer_destroy(b200_conv_layer *l)
{
    if (!l) return B200_OK;
    for (int i = 0; i < b200_conv_layer::NBUF; i++)
        if (l->buf[i]) cudaFree(l->buf[i]);
    if (l->mirror) b200_conv_layer_destroy(l->mirror);
    delete l;
    return B200_OK;
}

int b200_conv_layers_prepack(b200_conv_layer *const *layers, const float *const *kernels, int count, void *stream)
{
    cudaStream_t s = (cudaStream_t)stream;
    if (count < 0 || (count && (!layers || !kernels))) return fail(B200_E_ARG, "null argument");
    const int prec = precision();
    if (prec == B200_FP32) return B200_OK;                 // the CUDA-core path reads the weights as they are
    const bool x3 = prec == B200_TF32X3;
    WeightPackJobs jobs;
    jobs.count = 0;
    int r;
    for (int i = 0; i < count; i++) {
        b200_conv_layer *l = layers[i];
        if (!l || !kernels[i]) return fail(B200_E_ARG, "null layer or kernel in the list");
        l->prepacked = 0;
        if (use_smallc(l)) continue;                       // few-channel layers fold their weights per call
        // the forward call of a transposed-convolution layer reads the rotated pack: that one goes to W_HI/W_LO
        const int f_slot = l->transposed ? b200_conv_layer::W2_HI : b200_conv_layer::W_HI;
        const int b_slot = l->transposed ? b200_conv_layer::W_HI : b200_conv_layer::W2_HI;
        const size_t f_bytes = sizeof(float) * weight_pack_elems(l->g, false), b_bytes = sizeof(float) * weight_pack_elems(l->g, true);
        if ((r = ensure(l, f_slot, f_bytes, s)) || (r = ensure(l, b_slot, b_bytes, s))) return r;
        if (x3 && ((r = ensure(l, f_slot + 1, f_bytes, s)) || (r = ensure(l, b_slot + 1, b_bytes, s)))) return r;
        WeightPackJob job;
        if (!weight_pack_job(l->g, kernels[i], l->buf[f_slot], x3 ? l->buf[f_slot + 1] : nullptr, l->buf[b_slot], x3 ? l->buf[b_slot + 1] : nullptr, &job))
            continue;
        jobs.job[jobs.count++] = job;
        l->prepacked = 1; l->prepacked_precision = prec; l->prepacked_kernel = kernels[i];
        l->w2_valid = 0;
        if (jobs.count == kMaxPackJobs) {
            if ((r = weight_pack_fill_many(jobs, s))) return r;
            jobs.count = 0;
        }
    }
    return weight_pack_fill_many(jobs, s);
}

// Forward pass with the optional fusions.  The tensor-core paths apply f->input_func while they pack the layer input and
// f->output_func in the epilogue; where a path cannot (few-channel layers pack through im2col, the transposed few-channel
// layer finishes in a gather kernel, the CUDA-core path), the same results are produced with separate activation launches.
static int layer_forward(b200_conv_layer *l, float *out, const float *input, const float *kernel, const float *bias, const b200_conv_fusion *f,
                         void *stream)
{
    cudaStream_t s = (cudaStream_t)stream;
    const int prec = precision();
    const b200_conv_geom &g = l->g;
    l->in_valid = 0;
    int r = TC_UNSUPPORTED;
    l->col_valid = 0;
    l->er_valid = 0;
    const bool in_act = f && f->input_func >= 0, out_act = f && f->output_func >= 0;
    l->fused_input = in_act ? (f->input_act_out ? 3 : 1) : 0;
    const size_t in_count = (size_t)l->batch * (l->transposed ? (size_t)g.kernel_amount * g.out_y * g.out_x : (size_t)g.in_z * g.in_y * g.in_x);
    const size_t out_count = (size_t)l->batch * (l->transposed ? (size_t)g.in_z * g.in_y * g.in_x : (size_t)g.kernel_amount * g.out_y * g.out_x);
    // the activated input as a tensor of its own (paths that cannot apply the function while packing)
    const float *plain_input = input;
    bool input_materialised = false;
    auto materialise_input = [&]() -> int {
        if (!in_act || input_materialised) return B200_OK;
        float *dst = f->input_act_out;
        if (!dst) {
            int e = ensure(l, b200_conv_layer::ACT_TMP, sizeof(float) * in_count, s);
            if (e) return e;
            dst = l->buf[b200_conv_layer::ACT_TMP];
            l->fused_input = 2;
        }
        int e = b200_activation(dst, input, in_count, f->input_func, 0, f->input_slope, stream);
        if (e) return e;
        plain_input = dst;
        input_materialised = true;
        return B200_OK;
    };
    // the neuron function behind the layer as a launch of its own: the convolution goes to output_pre (or in place)
    auto finish_output = [&](float *conv_out) -> int {
        if (!out_act) return B200_OK;
        return b200_activation(out, conv_out, out_count, f->output_func, 0, f->output_slope, stream);
    };
    float *unfused_out = (out_act && f->output_pre) ? f->output_pre : out;
    EpilogueFunction ef = {out_act ? f->output_func : -1, out_act ? f->output_slope : 0.0, out_act ? f->output_pre : nullptr};
    const EpilogueFunction *efp = out_act ? &ef : nullptr;

    if (prec != B200_FP32 && use_smallc(l)) {
        const bool x3 = prec == B200_TF32X3;
        if ((r = materialise_input())) return r;
        if (!l->transposed) {
            ActPack col;
            if ((r = col_into(l, col, plain_input, x3, s)) == B200_OK) r = smallc_conv(l, out, col, kernel, bias, x3, s, efp);
            if (r == B200_OK) { l->col_valid = 1; l->col_precision = prec; }
        } else {
            ActPack in = in_shape(l);
            if ((r = pack_into(l, b200_conv_layer::IN_HI, in, plain_input, x3, s)) == B200_OK) r = smallc_tconv(l, unfused_out, in, kernel, x3, s);
            if (r == B200_OK) r = finish_output(unfused_out);
            if (r == B200_OK) { l->in_valid = 1; l->in_precision = prec; }
        }
        if (r == B200_OK) { set_path(B200_PATH_TCGEN05); return r; }
        if (r != TC_UNSUPPORTED) return r;
        l->in_valid = l->col_valid = 0;
    }
    if (prec != B200_FP32) {
        const bool x3 = prec == B200_TF32X3;
        // a layer with few filters forms its weight gradient on the mirrored problem, which reads the layer input as a tensor
        if (l->mirror && in_act && !f->input_act_out && (r = materialise_input())) return r;
        ActPack in = in_shape(l);
        PackFunction pf = {in_act ? f->input_func : -1, in_act ? f->input_slope : 0.0, in_act ? f->input_act_out : nullptr};
        const bool fuse_pack = in_act && !input_materialised;
        if ((r = pack_into(l, b200_conv_layer::IN_HI, in, plain_input, x3, s, nullptr, fuse_pack ? &pf : nullptr)) == B200_OK &&
            (r = pack_weights(l, l->transposed, kernel, x3, s, true)) == B200_OK)
            r = layer_conv_gemm(l, l->transposed, g, out, in, l->transposed ? nullptr : bias, x3, s, efp);
        if (r == B200_OK) {
            l->in_valid = 1;
            l->in_precision = prec;
            set_path(B200_PATH_TCGEN05);
            return r;
        }
        if (r != TC_UNSUPPORTED) return r;
    }
    // general path: the stateless tensor-math entry points
    if ((r = materialise_input())) return r;
    if (!l->transposed) r = b200_conv_forward(&g, unfused_out, l->batch, plain_input, l->batch, kernel, 1, bias, 1, stream);
    else r = b200_conv_backward(&g, unfused_out, l->batch, plain_input, l->batch, kernel, 1, nullptr, 0, stream);
    if (r) return r;
    return finish_output(unfused_out);
}

int b200_conv_layer_forward(b200_conv_layer *l, float *out, const float *input, const float *kernel, const float *bias, void *stream)
{
    if (!l || !out || !input || !kernel) return fail(B200_E_ARG, "null argument");
    return layer_forward(l, out, input, kernel, bias, nullptr, stream);
}

int b200_conv_layer_forward_fused(b200_conv_layer *l, float *out, const float *input, const float *kernel, const float *bias,
                                  const b200_conv_fusion *fusion, void *stream)
{
    if (!l || !out || !input || !kernel) return fail(B200_E_ARG, "null argument");
    if (fusion) {
        if (fusion->input_func > B200_ACT_GELU || fusion->output_func > B200_ACT_GELU) return fail(B200_E_ARG, "unknown neuron function");
        if (fusion->output_pre == out && fusion->output_func >= 0) return fail(B200_E_ARG, "output_pre must not alias the output");
    }
    return layer_forward(l, out, input, kernel, bias, fusion, stream);
}

int b200_conv_layer_backward(b200_conv_layer *l, float *input_delta, float *dkernel, float *dbias, int accumulate,
                             const float *output_delta, const float *input, const float *kernel, void *stream)
{
    cudaStream_t s = (cudaStream_t)stream;
    if (!l || !output_delta || !input || !kernel) return fail(B200_E_ARG, "null argument");
    if (!input_delta && !dkernel) return B200_OK;
    const b200_conv_geom &g = l->g;
    const int prec = precision();
    int r = TC_UNSUPPORTED;
    // after a forward call with a neuron function fused in front, the layer input f(x) may exist only inside the library
    if (l->fused_input == 2) input = l->buf[b200_conv_layer::ACT_TMP];
    if (l->fused_input == 1 && dkernel) {
        const bool kept = prec != B200_FP32 && ((use_smallc(l) && !l->transposed) ? (l->col_valid && l->col_precision == prec) : (l->in_valid && l->in_precision == prec));
        if (!kept)
            return fail(B200_E_ARG, "the layer input of the fused forward call was kept only in packed form for another precision mode: "
                                    "pass input_act_out to b200_conv_layer_forward_fused and hand that tensor to the backward call");
    }
    // A weights-only call followed by an input-only call on the same output error (the order that lets a caller start the
    // all-reduce of the gradients while the input error is still being computed) packs the error once.
    const bool reuse_er = l->er_valid && l->er_ptr == output_delta && l->er_precision == prec && !dkernel && input_delta;
    l->er_valid = 0;
    // Few filters: both products on the mirrored problem (few input channels, taps folded into the channel dimension).  The
    // layer input must exist as a tensor for the weight gradient (not only as the pack of a fused forward call).
    if (prec != B200_FP32 && l->mirror && use_smallc(l->mirror) && !(l->fused_input == 1 && dkernel)) {
        b200_conv_layer *m = l->mirror;
        const size_t w_count = (size_t)g.kernel_amount * g.in_z * g.kernel_x * g.kernel_y;
        m->col_valid = 0;                  // whatever the mirror gathered belongs to an earlier output error
        r = ensure(l, b200_conv_layer::MIRROR_W, sizeof(float) * w_count, s);
        if (r == B200_OK) r = mirror_weights(g, l->buf[b200_conv_layer::MIRROR_W], kernel, 0, 0, s);
        // input error = the mirrored layer's forward pass over the output error
        if (r == B200_OK && input_delta) r = layer_forward(m, input_delta, output_delta, l->buf[b200_conv_layer::MIRROR_W], nullptr, nullptr, stream);
        if (r == B200_OK && dkernel) {
            // weight gradient = the mirrored layer's, image and error exchanged, put back into this layer's order
            if ((r = ensure(l, b200_conv_layer::MIRROR_DW, sizeof(float) * w_count, s)) == B200_OK) {
                // the mirror's packed output error is this layer's packed input, kept by the forward call
                if (l->in_valid && l->in_precision == prec) {
                    m->lent_er_hi = l->buf[b200_conv_layer::IN_HI];
                    m->lent_er_lo = prec == B200_TF32X3 ? l->buf[b200_conv_layer::IN_LO] : nullptr;
                }
                r = b200_conv_layer_backward(m, nullptr, l->buf[b200_conv_layer::MIRROR_DW], nullptr, 0, input, output_delta,
                                             l->buf[b200_conv_layer::MIRROR_W], stream);
                m->lent_er_hi = m->lent_er_lo = nullptr;
            }
            if (r == B200_OK) r = mirror_weights(g, dkernel, l->buf[b200_conv_layer::MIRROR_DW], 1, accumulate, s);
            if (r == B200_OK && dbias && (r = ensure(l, b200_conv_layer::DB_TMP, sizeof(float) * (size_t)l->batch * g.kernel_amount, s)) == B200_OK)
                r = dbias_batch(dbias, accumulate, output_delta, l->batch, g.kernel_amount, (size_t)g.out_y * g.out_x, l->buf[b200_conv_layer::DB_TMP], s);
        }
        m->col_valid = 0;
        if (r == B200_OK) { set_path(B200_PATH_TCGEN05); return r; }
        return r;
    }
    if (prec != B200_FP32 && use_smallc(l)) {
        const bool x3 = prec == B200_TF32X3;
        if (!l->transposed) {
            // the output error has the many channels: packed once (with the bias gradient's plane sums) for both products
            ActPack er = er_shape(l), col;
            int sum_runs = 0;
            const bool want_sums = dkernel && dbias;
            if (l->lent_er_hi && !want_sums && (!x3 || l->lent_er_lo)) {
                er.hi = const_cast<float *>(l->lent_er_hi);
                er.lo = x3 ? const_cast<float *>(l->lent_er_lo) : nullptr;
                r = B200_OK;
            } else {
                r = pack_into(l, b200_conv_layer::ER_HI, er, output_delta, x3, s, want_sums ? &sum_runs : nullptr);
            }
            if (r == B200_OK && input_delta) r = smallc_tconv(l, input_delta, er, kernel, x3, s);
            if (r == B200_OK && dkernel) {
                if (l->col_valid && l->col_precision == prec) {
                    col = col_shape(l);
                    col.hi = l->buf[b200_conv_layer::COL_HI];
                    col.lo = x3 ? l->buf[b200_conv_layer::COL_LO] : nullptr;
                } else {
                    r = col_into(l, col, input, x3, s);
                }
                if (r == B200_OK) r = smallc_wgrad(l, dkernel, accumulate, col, er, x3, s);
                if (r == B200_OK && dbias) {
                    if (sum_runs > 0) r = dbias_from_rowsums(dbias, accumulate, l->buf[b200_conv_layer::DB_TMP], l->batch, g.kernel_amount, sum_runs, s);
                    else if ((r = ensure(l, b200_conv_layer::DB_TMP, sizeof(float) * (size_t)l->batch * g.kernel_amount, s)) == B200_OK)
                        r = dbias_batch(dbias, accumulate, output_delta, l->batch, g.kernel_amount, (size_t)g.out_y * g.out_x,
                                        l->buf[b200_conv_layer::DB_TMP], s);
                }
            }
        } else {
            // the output error has the few channels: its im2col copy serves the input error and the weight gradient
            ActPack col, in = in_shape(l);
            r = col_into(l, col, output_delta, x3, s);
            if (r == B200_OK && input_delta) r = smallc_conv(l, input_delta, col, kernel, nullptr, x3, s);
            if (r == B200_OK && dkernel) {
                if (l->in_valid && l->in_precision == prec) {
                    in.hi = l->buf[b200_conv_layer::IN_HI];
                    in.lo = x3 ? l->buf[b200_conv_layer::IN_LO] : nullptr;
                } else {
                    r = pack_into(l, b200_conv_layer::IN_HI, in, input, x3, s);
                }
                if (r == B200_OK) r = smallc_wgrad(l, dkernel, accumulate, col, in, x3, s);
                // the reference clears the bias gradient of this layer (cuda/ctensorconv.cu.h:1221)
                if (r == B200_OK && dbias && !accumulate) B200_CUDA(cudaMemsetAsync(dbias, 0, sizeof(float) * g.kernel_amount, s));
            }
        }
        if (r == B200_OK) { set_path(B200_PATH_TCGEN05); return r; }
        if (r != TC_UNSUPPORTED) return r;
    }
    if (prec != B200_FP32) {
        const bool x3 = prec == B200_TF32X3;
        ActPack in = in_shape(l), er = er_shape(l);
        // a convolution layer's bias gradient is the plane sum of the output error: its first stage rides on the pack
        int sum_runs = 0;
        static const bool fuse_sums = !(getenv("B200CONV_FUSE_DBIAS") && getenv("B200CONV_FUSE_DBIAS")[0] == '0');   // debug switch
        const bool want_sums = fuse_sums && !l->transposed && dkernel && dbias;
        if (reuse_er) {
            er.hi = l->buf[b200_conv_layer::ER_HI];
            er.lo = x3 ? l->buf[b200_conv_layer::ER_LO] : nullptr;
            r = B200_OK;
        } else {
            r = pack_into(l, b200_conv_layer::ER_HI, er, output_delta, x3, s, want_sums ? &sum_runs : nullptr);
        }
        if (r == B200_OK && input_delta) {
            // error of the layer input: BackwardConvolution for a convolution layer, ForwardConvolution
            // (zero bias) for a transposed-convolution layer
            if ((r = pack_weights(l, !l->transposed, kernel, x3, s)) == B200_OK)
                r = layer_conv_gemm(l, !l->transposed, g, input_delta, er, nullptr, x3, s);
        }
        if (r == B200_OK && dkernel) {
            if (l->in_valid && l->in_precision == prec) {
                in.hi = l->buf[b200_conv_layer::IN_HI];
                in.lo = x3 ? l->buf[b200_conv_layer::IN_LO] : nullptr;
            } else {
                r = pack_into(l, b200_conv_layer::IN_HI, in, input, x3, s);      // forward was not run in this mode
            }
            if (r == B200_OK) r = ensure(l, b200_conv_layer::PARTIAL, sizeof(float) * wgrad_partial_elems(g, l->batch), s);
            // image role / delta role of the weight gradient: (input, error) for a convolution layer,
            // (error, input) for a transposed-convolution layer
            if (r == B200_OK)
                r = l->transposed ? wgrad_gemm(g, dkernel, accumulate, er, in, l->buf[b200_conv_layer::PARTIAL], x3, s)
                                  : wgrad_gemm(g, dkernel, accumulate, in, er, l->buf[b200_conv_layer::PARTIAL], x3, s);
            if (r == B200_OK && dbias) {
                if (l->transposed) {
                    // the reference clears the bias gradient of this layer (cuda/ctensorconv.cu.h:1221)
                    if (!accumulate) B200_CUDA(cudaMemsetAsync(dbias, 0, sizeof(float) * g.kernel_amount, s));
                } else if (sum_runs > 0) {
                    r = dbias_from_rowsums(dbias, accumulate, l->buf[b200_conv_layer::DB_TMP], l->batch, g.kernel_amount, sum_runs, s);
                } else if ((r = ensure(l, b200_conv_layer::DB_TMP, sizeof(float) * (size_t)l->batch * g.kernel_amount, s)) == B200_OK) {
                    r = dbias_batch(dbias, accumulate, output_delta, l->batch, g.kernel_amount, (size_t)g.out_y * g.out_x,
                                    l->buf[b200_conv_layer::DB_TMP], s);
                }
            }
        }
        if (r == B200_OK) {
            if (dkernel && !input_delta) { l->er_valid = 1; l->er_precision = prec; l->er_ptr = output_delta; }
            set_path(B200_PATH_TCGEN05);
            return r;
        }
        if (r != TC_UNSUPPORTED) return r;
    }
    // general path
    if (input_delta) {
        r = l->transposed ? b200_conv_forward(&g, input_delta, l->batch, output_delta, l->batch, kernel, 1, nullptr, 0, stream)
                          : b200_conv_backward(&g, input_delta, l->batch, output_delta, l->batch, kernel, 1, nullptr, 0, stream);
        if (r) return r;
    }
    if (dkernel) {
        r = l->transposed ? b200_conv_wgrad_batch(&g, dkernel, nullptr, accumulate, output_delta, input, l->batch, stream)
                          : b200_conv_wgrad_batch(&g, dkernel, dbias, accumulate, input, output_delta, l->batch, stream);
        if (r) return r;
        if (l->transposed && dbias && !accumulate) B200_CUDA(cudaMemsetAsync(dbias, 0, sizeof(float) * g.kernel_amount, s));
    }
    return B200_OK;
}

}  // extern "C"
