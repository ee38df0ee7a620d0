// C-ABI wrapper around the UNMODIFIED reference CPU backend (cpu/tensor.h of
// da-nie/CUDA-CNN-GAN-VAE), compiled in place from the reference tree by oracle/build.py into
// oracle/_ref/libref.so.  Test infrastructure only: it validates the plain-C oracle, generates the
// golden fixtures and serves as the timed CPU baseline.  No reference source is copied here; this
// file only includes the reference headers and moves raw float buffers in and out of CTensor.
#include <cstring>
#include <string>
#include <algorithm>
#include <cstdint>
#include <cmath>
#include <cstdio>

#include "cpu/tensor.h"

// The VAE output layer of the reference (netlayer/cnetlayervaecoderoutput.cu.h) compiles against its CPU
// backend (-DUSE_CPU, set by oracle/build.py).  Its noise tensor, its two error tensors and the current
// Kullback-Leibler weight are private members with no accessor; the checker reads them directly.
#define private public
#include "netlayer/cnetlayervaecoderoutput.cu.h"
#undef private
#include "netlayer/cnetlayerconvolutioninput.cu.h"

typedef CTensor<float> T;

static void put(T &t, const float *src)
{
    size_t n = (size_t)t.GetSizeW() * t.GetSizeZ() * t.GetSizeY() * t.GetSizeX();
    std::memcpy(t.GetColumnPtr(0, 0, 0), src, n * sizeof(float));
}
static void get(T &t, float *dst)
{
    size_t n = (size_t)t.GetSizeW() * t.GetSizeZ() * t.GetSizeY() * t.GetSizeX();
    std::memcpy(dst, t.GetColumnPtr(0, 0, 0), n * sizeof(float));
}

#define GUARD(...)                                    \
    try { __VA_ARGS__; return 0; }                    \
    catch (const char *msg) { std::fprintf(stderr, "reference threw: %s\n", msg); return 100; }

extern "C" {

int ref_conv_forward(float *out, int out_w, int out_y, int out_x,
                     const float *image, int image_w, int in_z, int in_y, int in_x,
                     const float *kernel, int kernel_w, int kernel_x, int kernel_y, int kernel_amount,
                     const float *bias, int bias_w, int sx, int sy, int px, int py)
{
    GUARD({
        T o(out_w, kernel_amount, out_y, out_x), i(image_w, in_z, in_y, in_x),
            k(kernel_w, 1, kernel_amount, kernel_x * kernel_y * in_z), b(bias_w, kernel_amount, 1, 1);
        put(i, image); put(k, kernel); put(b, bias);
        CTensorConv<float>::ForwardConvolution(o, i, k, kernel_x, kernel_y, in_z, kernel_amount, b, sx, sy, px, py);
        get(o, out);
    })
}

int ref_conv_backward(float *out, int out_w, int out_z, int out_y, int out_x,
                      const float *delta, int delta_w, int d_y, int d_x,
                      const float *kernel, int kernel_w, int kernel_x, int kernel_y, int kernel_amount,
                      const float *bias, int bias_w, int sx, int sy, int px, int py)
{
    GUARD({
        T o(out_w, out_z, out_y, out_x), d(delta_w, kernel_amount, d_y, d_x),
            k(kernel_w, 1, kernel_amount, kernel_x * kernel_y * out_z), b(bias_w, kernel_amount, 1, 1);
        put(d, delta); put(k, kernel); put(b, bias);
        CTensorConv<float>::BackwardConvolution(o, d, k, kernel_x, kernel_y, out_z, kernel_amount, b, sx, sy, px, py);
        get(o, out);
    })
}

int ref_conv_wgrad(float *dkernel, int dkernel_w, int kernel_x, int kernel_y, int kernel_z, int kernel_amount,
                   float *dbias, int dbias_w,
                   const float *image, int image_w, int image_y, int image_x,
                   const float *delta, int delta_w, int delta_y, int delta_x,
                   int sx, int sy, int px, int py, int back_variant)
{
    GUARD({
        T dk(dkernel_w, 1, kernel_amount, kernel_x * kernel_y * kernel_z), db(dbias_w, kernel_amount, 1, 1);
        put(dk, dkernel); put(db, dbias);
        if (!back_variant) {
            T i(image_w, kernel_z, image_y, image_x), d(delta_w, kernel_amount, delta_y, delta_x);
            put(i, image); put(d, delta);
            CTensorConv<float>::CreateDeltaWeightAndBias(dk, kernel_x, kernel_y, kernel_z, kernel_amount, db, i, d, sx, sy, px, py);
        } else {
            // back variant: "image" plays the delta role (kernel_amount channels), "delta" the image role
            T i(image_w, kernel_amount, image_y, image_x), d(delta_w, kernel_z, delta_y, delta_x);
            put(i, image); put(d, delta);
            CTensorConv<float>::CreateBackDeltaWeightAndBias(dk, kernel_x, kernel_y, kernel_z, kernel_amount, db, i, d, sx, sy, px, py);
        }
        get(dk, dkernel); get(db, dbias);
    })
}

int ref_mul(float *out, int out_w, const float *left, int left_w, const float *right, int right_w,
            int Z, int LY, int LX, int RX, int transpose_left)
{
    GUARD({
        if (!transpose_left) {
            T o(out_w, Z, LY, RX), l(left_w, Z, LY, LX), r(right_w, Z, LX, RX);
            put(l, left); put(r, right);
            CTensorMath<float>::Mul(o, l, r);
            get(o, out);
        } else {  // left is LY x LX (LY = shared dim), out is LX x RX
            T o(out_w, Z, LX, RX), l(left_w, Z, LY, LX), r(right_w, Z, LY, RX);
            put(l, left); put(r, right);
            CTensorMath<float>::TransponseMul(o, l, r);
            get(o, out);
        }
    })
}

// op: 0 Add, 1 Sub, 2 AddSumW, 3 TensorItemProduction
int ref_binary(float *out, int out_w, const float *left, int left_w, const float *right, int right_w,
               int Z, int Y, int X, float ls, float rs, int op)
{
    GUARD({
        T o(out_w, Z, Y, X), l(left_w, Z, Y, X), r(right_w, Z, Y, X);
        put(l, left); put(r, right);
        if (op == 0) CTensorMath<float>::Add(o, l, r, ls, rs);
        else if (op == 1) CTensorMath<float>::Sub(o, l, r, ls, rs);
        else if (op == 2) CTensorMath<float>::AddSumW(o, l, r, ls, rs);
        else CTensorMath<float>::TensorItemProduction(o, l, r);
        get(o, out);
    })
}

// op: 0 Pow2(a), 1 SQRT(a,b), 2 Inv, 3 Mul by scalar a
int ref_unary(float *out, int out_w, const float *in, int in_w, int Z, int Y, int X, int op, float a, float b)
{
    GUARD({
        T o(out_w, Z, Y, X), i(in_w, Z, Y, X);
        put(i, in);
        if (op == 0) CTensorMath<float>::Pow2(o, i, a);
        else if (op == 1) CTensorMath<float>::SQRT(o, i, a, b);
        else if (op == 2) CTensorMath<float>::Inv(o, i);
        else CTensorMath<float>::Mul(o, i, a);
        get(o, out);
    })
}

int ref_add_bias(float *t, int t_w, int Z, int Y, int X, const float *bias, int bias_w)
{
    GUARD({
        T o(t_w, Z, Y, X), b(bias_w, Z, 1, 1);
        put(o, t); put(b, bias);
        CTensorMath<float>::AddBias(o, b);
        get(o, t);
    })
}

int ref_summ_xy(float *out, int out_w, const float *in, int in_w, int Z, int Y, int X)
{
    GUARD({
        T o(out_w, Z, 1, 1), i(in_w, Z, Y, X);
        put(i, in);
        CTensorMath<float>::SummXY(o, i);
        get(o, out);
    })
}

int ref_maxpool(float *out, uint32_t *pos, const float *in, int W, int Z, int in_y, int in_x, int pool_x, int pool_y)
{
    GUARD({
        int oy = in_y / pool_y; int ox = in_x / pool_x;
        T o(W, Z, oy, ox), i(W, Z, in_y, in_x);
        CTensor<SPos> p(W, Z, oy, ox);
        put(i, in);
        CTensorMath<float>::MaxPooling(o, p, i, pool_x, pool_y);
        get(o, out);
        std::memcpy(pos, p.GetColumnPtr(0, 0, 0), sizeof(SPos) * (size_t)W * Z * oy * ox);
    })
}

int ref_maxpool_backward(float *out, const uint32_t *pos, const float *delta, int W, int Z, int out_y, int out_x,
                         int pool_x, int pool_y)
{
    GUARD({
        int dy = out_y / pool_y; int dx = out_x / pool_x;
        T o(W, Z, out_y, out_x), d(W, Z, dy, dx);
        CTensor<SPos> p(W, Z, dy, dx);
        put(d, delta);
        std::memcpy(p.GetColumnPtr(0, 0, 0), pos, sizeof(SPos) * (size_t)W * Z * dy * dx);
        CTensorMath<float>::MaxPoolingBackward(o, p, d, pool_x, pool_y);
        get(o, out);
    })
}

int ref_resample(float *out, const float *in, int W, int Z, int in_y, int in_x, int out_y, int out_x,
                 int fx, int fy, int down)
{
    GUARD({
        T o(W, Z, out_y, out_x), i(W, Z, in_y, in_x);
        put(i, in);
        if (down) CTensorMath<float>::DownSampling(o, i, fx, fy);
        else CTensorMath<float>::UpSampling(o, i, fx, fy);
        get(o, out);
    })
}

// func: 0 sigmoid, 1 ReLU, 2 LeakyReLU, 3 linear, 4 tanh, 5 GeLU
int ref_activation(float *out, const float *in, int W, int Z, int Y, int X, int func, int derivative)
{
    GUARD({
        T o(W, Z, Y, X), i(W, Z, Y, X);
        put(i, in);
        typedef CTensorApplyFunc<float> F;
        if (!derivative) {
            switch (func) {
            case 0: F::ApplySigmoid(o, i); break;
            case 1: F::ApplyReLU(o, i); break;
            case 2: F::ApplyLeakyReLU(o, i); break;
            case 3: F::ApplyLinear(o, i); break;
            case 4: F::ApplyTangence(o, i); break;
            default: F::ApplyGeLU(o, i); break;
            }
        } else {
            switch (func) {
            case 0: F::ApplyDifferentialSigmoid(o, i); break;
            case 1: F::ApplyDifferentialReLU(o, i); break;
            case 2: F::ApplyDifferentialLeakyReLU(o, i); break;
            case 3: F::ApplyDifferentialLinear(o, i); break;
            case 4: F::ApplyDifferentialTangence(o, i); break;
            default: F::ApplyDifferentialGeLU(o, i); break;
            }
        }
        get(o, out);
    })
}

int ref_adam(float *weight, const float *dweight, float *m, float *v, int n, uint32_t batch_size,
             double speed, double beta1, double beta2, double epsilon, double iteration)
{
    GUARD({
        T w(1, 1, 1, n), dw(1, 1, 1, n), mm(1, 1, 1, n), vv(1, 1, 1, n);
        put(w, weight); put(dw, dweight); put(mm, m); put(vv, v);
        CTensorMath<float>::Adam(w, dw, mm, vv, batch_size, speed, beta1, beta2, epsilon, iteration);
        get(w, weight); get(mm, m); get(vv, v);
    })
}

// Batch-normalisation layer, training-mode forward pass.  The layer class itself does not compile at the
// reference's head revision, so this drives the reference's own CTensorMath<float> routines in the order,
// with the operands, scale arguments and temporaries of netlayer/cnetlayerbatchnormalization.cu.h:301-379
// (momentum is a type_t member there, EPSILON a double constant passed to a type_t parameter).
// n-element statistics are [1,Z,Y,X]; x, y, xhat are [W,Z,Y,X].
int ref_bn_forward(float *y, float *xhat, float *ivar, float *mean, float *var, float *new_mean, float *new_var,
                   const float *x, const float *gamma, const float *beta, int W, int Z, int Y, int X, float momentum, double eps)
{
    GUARD({
        typedef CTensorMath<float> M;
        T in(W, Z, Y, X), H(W, Z, Y, X), XHAT(W, Z, Y, X), TmpA_H(W, Z, Y, X);
        T TmpA(1, Z, Y, X), VAR(1, Z, Y, X), SQRTVAR(1, Z, Y, X), IVAR(1, Z, Y, X), NewMean(1, Z, Y, X), NewVariable(1, Z, Y, X),
            Gamma(1, Z, Y, X), Beta(1, Z, Y, X);
        put(in, x); put(Gamma, gamma); put(Beta, beta);
        if (new_mean) put(NewMean, new_mean); else M::Fill(NewMean, 0);
        if (new_var) put(NewVariable, new_var); else M::Fill(NewVariable, 0);
        float N = static_cast<float>(W);
        float Momentum = momentum;
        M::Fill(TmpA, 0);
        M::AddSumW(TmpA, TmpA, in, 1, 1.0 / N);
        M::Add(NewMean, NewMean, TmpA, Momentum, 1.0 - Momentum);
        M::Sub(XHAT, in, TmpA, 1.0, 1.0);
        M::Fill(VAR, 0);
        M::Pow2(TmpA_H, XHAT, 1);
        M::AddSumW(VAR, VAR, TmpA_H, 1, 1.0 / N);
        M::Add(NewVariable, NewVariable, VAR, Momentum, 1.0 - Momentum);
        M::SQRT(SQRTVAR, VAR, 1, eps);
        M::Inv(IVAR, SQRTVAR);
        M::TensorItemProduction(XHAT, XHAT, IVAR);
        M::TensorItemProduction(TmpA_H, Gamma, XHAT);
        M::Add(H, TmpA_H, Beta);
        get(H, y); get(XHAT, xhat); get(IVAR, ivar); get(TmpA, mean); get(VAR, var);
        if (new_mean) get(NewMean, new_mean);
        if (new_var) get(NewVariable, new_var);
    })
}

// Batch-normalisation layer, TrainingBackward: the reference's CTensorMath<float> calls of
// netlayer/cnetlayerbatchnormalization.cu.h:578-604 in their order.  dgamma / dbeta are accumulated into.
int ref_bn_backward(float *dx, float *dgamma, float *dbeta, const float *dy, const float *xhat, const float *ivar,
                    const float *gamma, int W, int Z, int Y, int X, int create_delta_weight)
{
    GUARD({
        typedef CTensorMath<float> M;
        T Delta(W, Z, Y, X), XHAT(W, Z, Y, X), DXHAT(W, Z, Y, X), TmpA_H(W, Z, Y, X), Prev(W, Z, Y, X);
        T TmpB(1, Z, Y, X), TmpC(1, Z, Y, X), IVAR(1, Z, Y, X), Gamma(1, Z, Y, X), dGamma(1, Z, Y, X), dBeta(1, Z, Y, X);
        put(Delta, dy); put(XHAT, xhat); put(IVAR, ivar); put(Gamma, gamma); put(dGamma, dgamma); put(dBeta, dbeta);
        float N = static_cast<float>(W);
        M::Fill(TmpB, 0);
        M::Fill(TmpC, 0);
        M::TensorItemProduction(DXHAT, Delta, Gamma);
        M::AddSumW(TmpB, TmpB, DXHAT);
        M::TensorItemProduction(TmpA_H, DXHAT, XHAT);
        M::AddSumW(TmpC, TmpC, TmpA_H);
        if (create_delta_weight) {
            M::TensorItemProduction(TmpA_H, Delta, XHAT);
            M::AddSumW(dGamma, dGamma, TmpA_H);
            M::AddSumW(dBeta, dBeta, Delta);
        }
        M::Mul(Prev, DXHAT, N);
        M::TensorItemProduction(TmpA_H, XHAT, TmpC);
        M::Sub(Prev, Prev, TmpA_H);
        M::Sub(Prev, Prev, TmpB);
        M::TensorItemProduction(Prev, Prev, IVAR);
        M::Mul(Prev, Prev, 1.0 / N);
        get(Prev, dx); get(dGamma, dgamma); get(dBeta, dbeta);
    })
}

// The reference's own CNetLayerVAECoderOutput<float> (unmodified): Forward draws its noise from a
// random_device-seeded generator, so the noise it used is handed back (eps_out) together with the layer
// output; SetOutputError then runs on the same object with the Kullback-Leibler weight kl_speed and the
// two errors it hands to the mean / log-variance layers are returned.  mu, logvar, delta: [W,Z,Y,X].
int ref_vae_layer(float *z_out, float *eps_out, float *d_mu, float *d_logvar, const float *mu, const float *logvar,
                  const float *delta, int W, int Z, int Y, int X, float kl_speed)
{
    GUARD({
        CNetLayerConvolutionInput<float> mu_layer(Z, Y, X, W), lv_layer(Z, Y, X, W);
        T m(W, Z, Y, X), l(W, Z, Y, X), d(W, Z, Y, X);
        put(m, mu); put(l, logvar); put(d, delta);
        mu_layer.SetOutput(m);
        lv_layer.SetOutput(l);
        CNetLayerVAECoderOutput<float> layer(kl_speed, &mu_layer, &lv_layer, W);
        layer.TrainingStart();
        layer.Forward();
        get(layer.cTensor_H, z_out);
        get(layer.cTensor_Epsilon, eps_out);
        layer.KLSpeedCurrent = kl_speed;
        layer.SetOutputError(d);
        get(layer.cTensor_PrevLayerError_Mu, d_mu);
        get(layer.cTensor_PrevLayerError_LogVar, d_logvar);
        layer.TrainingStop();
    })
}

}  // extern "C"
