/*
 * CPU oracle for the convolution hot path.  TEST INFRASTRUCTURE ONLY: it is the checker the
 * CUDA library is compared with (tests, the smoke check and the CPU-baseline leg of the bench);
 * the product library never links, loads or calls it.
 *
 * Every function is a plain-C restatement of one routine of the reference CPU backend
 * (da-nie/CUDA-CNN-GAN-VAE, directory cpu/ and netlayer/); the reference file:line each one
 * follows is cited above it.  Loop order and float arithmetic follow the reference so that the
 * results are bit-identical to it (checked against the compiled reference and against the
 * known-answer vectors of cuda/ctensortest.cu.h by the CPU test-suite: parity is pinned).
 *
 * Tensors are dense fp32 in W,Z,Y,X order (W=batch, Z=channel), exactly the reference layout.
 * Every operand carries its own W count and is indexed with w % W (reference W-broadcast rule).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define IDX4(w, z, y, x, Z, Y, X) ((((size_t)(w) * (Z) + (z)) * (Y) + (y)) * (X) + (x))

/* cpu/ctensorconv.h:84-148  CTensorConv::ForwardConvolution */
int orc_conv_forward(float *out, int out_w, int out_y, int out_x,
                     const float *image, int image_w, int in_z, int in_y, int in_x,
                     const float *kernel, int kernel_w, int kernel_x, int kernel_y, int kernel_amount,
                     const float *bias, int bias_w,
                     int stride_x, int stride_y, int padding_x, int padding_y)
{
    if (kernel_amount == 0) return 1;
    if (out_x != (in_x - kernel_x + 2 * padding_x) / stride_x + 1) return 2;
    if (out_y != (in_y - kernel_y + 2 * padding_y) / stride_y + 1) return 2;
    const int klen = in_z * kernel_x * kernel_y;
    for (int w = 0; w < out_w; w++) {
        const float *img = image + (size_t)(w % image_w) * in_z * in_y * in_x;
        const float *ker = kernel + (size_t)(w % kernel_w) * kernel_amount * klen;
        const float *bs = bias + (size_t)(w % bias_w) * kernel_amount;
        for (int k = 0; k < kernel_amount; k++)
            for (int y = 0; y < out_y; y++)
                for (int x = 0; x < out_x; x++) {
                    float sum = bs[k];
                    for (int ky = 0; ky < kernel_y; ky++) {
                        int y0 = stride_y * y + ky - padding_y;
                        if (y0 < 0 || y0 >= in_y) continue;
                        for (int kx = 0; kx < kernel_x; kx++) {
                            int x0 = stride_x * x + kx - padding_x;
                            if (x0 < 0 || x0 >= in_x) continue;
                            for (int z = 0; z < in_z; z++) {
                                float kv = ker[(size_t)k * klen + z * kernel_x * kernel_y + ky * kernel_x + kx];
                                float iv = img[((size_t)z * in_y + y0) * in_x + x0];
                                sum += kv * iv;
                            }
                        }
                    }
                    out[IDX4(w, k, y, x, kernel_amount, out_y, out_x)] = sum;
                }
    }
    return 0;
}

/* cpu/ctensorconv.h:196-266  CTensorConv::BackwardConvolution (also the forward pass of the
 * transposed-convolution layer).  The bias term is added once per contributing tap and filter,
 * as the reference does; every caller passes a zero bias. */
int orc_conv_backward(float *out, int out_w, int out_z, int out_y, int out_x,
                      const float *delta, int delta_w, int d_y, int d_x,
                      const float *kernel, int kernel_w, int kernel_x, int kernel_y, int kernel_amount,
                      const float *bias, int bias_w,
                      int stride_x, int stride_y, int padding_x, int padding_y)
{
    if (kernel_amount == 0) return 1;
    padding_x = kernel_x - 1 - padding_x;
    padding_y = kernel_y - 1 - padding_y;
    const int klen = out_z * kernel_x * kernel_y;
    for (int w = 0; w < out_w; w++) {
        const float *dl = delta + (size_t)(w % delta_w) * kernel_amount * d_y * d_x;
        const float *ker = kernel + (size_t)(w % kernel_w) * kernel_amount * klen;
        const float *bs = bias + (size_t)(w % bias_w) * kernel_amount;
        for (int y = 0; y < out_y; y++)
            for (int x = 0; x < out_x; x++)
                for (int z = 0; z < out_z; z++) {
                    float summ = 0;
                    for (int ky = 0; ky < kernel_y; ky++) {
                        int y0 = y + ky - padding_y;
                        if (y0 % stride_y != 0) continue;
                        int dy0 = y0 / stride_y;
                        if (dy0 < 0 || dy0 >= d_y) continue;
                        for (int kx = 0; kx < kernel_x; kx++) {
                            int x0 = x + kx - padding_x;
                            if (x0 % stride_x != 0) continue;
                            int dx0 = x0 / stride_x;
                            if (dx0 < 0 || dx0 >= d_x) continue;
                            for (int f = 0; f < kernel_amount; f++) {
                                summ += bs[f];
                                float kv = ker[(size_t)f * klen + z * kernel_x * kernel_y +
                                               (kernel_y - 1 - ky) * kernel_x + (kernel_x - 1 - kx)];
                                float dv = dl[((size_t)f * d_y + dy0) * d_x + dx0];
                                summ += kv * dv;
                            }
                        }
                    }
                    out[IDX4(w, z, y, x, out_z, out_y, out_x)] = summ;
                }
    }
    return 0;
}

/* cpu/ctensorconv.h:319-386  CTensorConv::CreateDeltaWeightAndBias.  Accumulates (+=) into the
 * existing dkernel / dbias contents, one dkernel per w < dkernel_w. */
int orc_conv_wgrad(float *dkernel, int dkernel_w, int kernel_x, int kernel_y, int kernel_z, int kernel_amount,
                   float *dbias, int dbias_w,
                   const float *image, int image_w, int image_y, int image_x,
                   const float *delta, int delta_w, int delta_y, int delta_x,
                   int stride_x, int stride_y, int padding_x, int padding_y)
{
    if (kernel_amount == 0) return 1;
    const int klen = kernel_z * kernel_x * kernel_y;
    const int new_dx = stride_x * (delta_x - 1) + 1;
    const int new_dy = stride_y * (delta_y - 1) + 1;
    for (int w = 0; w < dkernel_w; w++) {
        float *dk = dkernel + (size_t)w * kernel_amount * klen;
        float *db = dbias + (size_t)(w % dbias_w) * kernel_amount;
        const float *img = image + (size_t)(w % image_w) * kernel_z * image_y * image_x;
        const float *dl = delta + (size_t)(w % delta_w) * kernel_amount * delta_y * delta_x;
        for (int f = 0; f < kernel_amount; f++)
            for (int y = 0; y < new_dy; y++) {
                if (y % stride_y != 0) continue;
                for (int x = 0; x < new_dx; x++) {
                    if (x % stride_x != 0) continue;
                    float d = dl[((size_t)f * delta_y + y / stride_y) * delta_x + x / stride_x];
                    for (int i = 0; i < kernel_y; i++) {
                        int i0 = i + y - padding_y;
                        if (i0 < 0 || i0 >= image_y) continue;
                        for (int j = 0; j < kernel_x; j++) {
                            int j0 = j + x - padding_x;
                            if (j0 < 0 || j0 >= image_x) continue;
                            for (int c = 0; c < kernel_z; c++) {
                                size_t o = (size_t)f * klen + c * kernel_x * kernel_y + i * kernel_x + j;
                                float v = dk[o];
                                v += d * img[((size_t)c * image_y + i0) * image_x + j0];
                                dk[o] = v;
                            }
                        }
                    }
                    db[f] += d;
                }
            }
    }
    return 0;
}

/* cpu/ctensorconv.h:392-396  CTensorConv::CreateBackDeltaWeightAndBias: the same routine with
 * image and delta exchanged, after which the bias gradient is cleared. */
int orc_conv_back_wgrad(float *dkernel, int dkernel_w, int kernel_x, int kernel_y, int kernel_z, int kernel_amount,
                        float *dbias, int dbias_w,
                        const float *image, int image_w, int image_y, int image_x,
                        const float *delta, int delta_w, int delta_y, int delta_x,
                        int stride_x, int stride_y, int padding_x, int padding_y)
{
    int r = orc_conv_wgrad(dkernel, dkernel_w, kernel_x, kernel_y, kernel_z, kernel_amount, dbias, dbias_w,
                           delta, delta_w, delta_y, delta_x, image, image_w, image_y, image_x,
                           stride_x, stride_y, padding_x, padding_y);
    memset(dbias, 0, sizeof(float) * (size_t)dbias_w * kernel_amount);
    return r;
}

/* cpu/ctensormath.h:531-595  CTensorMath::Mul: out[w,z] = left[w%Lw,z] (LY x LX) * right[w%Rw,z]
 * (LX x RX), 32x32x32 cache blocking in the order yy,kk,xx / y,k,x. */
void orc_mul(float *out, int out_w, const float *left, int left_w, const float *right, int right_w,
             int Z, int LY, int LX, int RX)
{
    memset(out, 0, sizeof(float) * (size_t)out_w * Z * LY * RX);
    const int BS = 32;
    for (int w = 0; w < out_w; w++)
        for (int z = 0; z < Z; z++) {
            const float *lb = left + ((size_t)(w % left_w) * Z + z) * LY * LX;
            const float *rb = right + ((size_t)(w % right_w) * Z + z) * LX * RX;
            float *ob = out + ((size_t)w * Z + z) * LY * RX;
            for (int yy = 0; yy < LY; yy += BS)
                for (int kk = 0; kk < LX; kk += BS)
                    for (int xx = 0; xx < RX; xx += BS) {
                        int ye = yy + BS < LY ? yy + BS : LY;
                        int ke = kk + BS < LX ? kk + BS : LX;
                        int xe = xx + BS < RX ? xx + BS : RX;
                        for (int y = yy; y < ye; y++)
                            for (int k = kk; k < ke; k++) {
                                float lv = lb[(size_t)y * LX + k];
                                for (int x = xx; x < xe; x++) ob[(size_t)y * RX + x] += lv * rb[(size_t)k * RX + x];
                            }
                    }
        }
}

/* cpu/ctensormath.h:643-712  CTensorMath::TransponseMul: out[w,z] = left[w%Lw,z]^T * right[w%Rw,z],
 * left is KD x LX, right is KD x RX, out is LX x RX; blocking order kk,yy,xx / k,y,x. */
void orc_tmul(float *out, int out_w, const float *left, int left_w, const float *right, int right_w,
              int Z, int KD, int LX, int RX)
{
    memset(out, 0, sizeof(float) * (size_t)out_w * Z * LX * RX);
    const int BS = 32;
    for (int w = 0; w < out_w; w++)
        for (int z = 0; z < Z; z++) {
            const float *lb = left + ((size_t)(w % left_w) * Z + z) * KD * LX;
            const float *rb = right + ((size_t)(w % right_w) * Z + z) * KD * RX;
            float *ob = out + ((size_t)w * Z + z) * LX * RX;
            for (int kk = 0; kk < KD; kk += BS)
                for (int yy = 0; yy < LX; yy += BS)
                    for (int xx = 0; xx < RX; xx += BS) {
                        int ke = kk + BS < KD ? kk + BS : KD;
                        int ye = yy + BS < LX ? yy + BS : LX;
                        int xe = xx + BS < RX ? xx + BS : RX;
                        for (int k = kk; k < ke; k++)
                            for (int y = yy; y < ye; y++) {
                                float lv = lb[(size_t)k * LX + y];
                                for (int x = xx; x < xe; x++) ob[(size_t)y * RX + x] += lv * rb[(size_t)k * RX + x];
                            }
                    }
        }
}

/* cpu/ctensormath.h:235-267 Add, :314-347 Sub: out[w] = ls*left[w%Lw] (+|-) rs*right[w%Rw]; n = Z*Y*X. */
void orc_add(float *out, int out_w, const float *left, int left_w, const float *right, int right_w,
             size_t n, float ls, float rs, int subtract)
{
    for (int w = 0; w < out_w; w++) {
        const float *l = left + (size_t)(w % left_w) * n;
        const float *r = right + (size_t)(w % right_w) * n;
        float *o = out + (size_t)w * n;
        if (subtract) for (size_t i = 0; i < n; i++) o[i] = (ls * l[i]) - (rs * r[i]);
        else          for (size_t i = 0; i < n; i++) o[i] = (ls * l[i]) + (rs * r[i]);
    }
}

/* cpu/ctensormath.h:273-308  AddSumW: out[0] = ls*sum_w left + rs*sum_w right, out[w>0] = 0.
 * out may alias left (the sum is formed before the store, as in the reference). */
void orc_add_sum_w(float *out, int out_w, const float *left, int left_w, const float *right, int right_w,
                   size_t n, float ls, float rs)
{
    for (size_t i = 0; i < n; i++) {
        float sl = 0, sr = 0;
        for (int w = 0; w < left_w; w++) sl += left[(size_t)w * n + i];
        sl *= ls;
        for (int w = 0; w < right_w; w++) sr += right[(size_t)w * n + i];
        sr *= rs;
        out[i] = sl + sr;
        for (int w = 1; w < out_w; w++) out[(size_t)w * n + i] = 0;
    }
}

/* cpu/ctensormath.h:352-381  AddBias: t[w,z,:,:] += bias[w%Bw,z]. */
void orc_add_bias(float *t, int t_w, int Z, size_t yx, const float *bias, int bias_w)
{
    for (int w = 0; w < t_w; w++)
        for (int z = 0; z < Z; z++) {
            float b = bias[(size_t)(w % bias_w) * Z + z];
            float *p = t + ((size_t)w * Z + z) * yx;
            for (size_t i = 0; i < yx; i++) p[i] += b;
        }
}

/* cpu/ctensormath.h:455-483  SummXY: out[w,z] = sum over y,x of in[w%Iw,z,:,:] (sequential fp32 sum). */
void orc_summ_xy(float *out, int out_w, const float *in, int in_w, int Z, size_t yx)
{
    for (int w = 0; w < out_w; w++)
        for (int z = 0; z < Z; z++) {
            const float *p = in + ((size_t)(w % in_w) * Z + z) * yx;
            float s = 0;
            for (size_t i = 0; i < yx; i++) s += p[i];
            out[(size_t)w * Z + z] = s;
        }
}

/* Unary element-wise routines with W-broadcast of the input:
 * op 0: Pow2  o=i*i*a          cpu/ctensormath.h:387-415
 * op 1: SQRT  o=sqrt(i+b)*a    cpu/ctensormath.h:421-449
 * op 2: Inv   o=1/i            cpu/ctensormath.h:163-191
 * op 3: Mul by scalar o=i*a    cpu/ctensormath.h:721-781 */
void orc_unary(float *out, int out_w, const float *in, int in_w, size_t n, int op, float a, float b)
{
    for (int w = 0; w < out_w; w++) {
        const float *p = in + (size_t)(w % in_w) * n;
        float *o = out + (size_t)w * n;
        for (size_t i = 0; i < n; i++) {
            float v = p[i];
            switch (op) {
            case 0: o[i] = v * v * a; break;
            case 1: o[i] = (float)(sqrt(v + b)) * a; break;
            case 2: o[i] = (float)(1.0 / v); break;
            default: o[i] = v * a; break;
            }
        }
    }
}

/* cpu/ctensormath.h:822-851  TensorItemProduction: out[w] = left[w%Lw] .* right[w%Rw]. */
void orc_item_product(float *out, int out_w, const float *left, int left_w, const float *right, int right_w, size_t n)
{
    for (int w = 0; w < out_w; w++) {
        const float *l = left + (size_t)(w % left_w) * n;
        const float *r = right + (size_t)(w % right_w) * n;
        float *o = out + (size_t)w * n;
        for (size_t i = 0; i < n; i++) o[i] = l[i] * r[i];
    }
}

/* cpu/ctensormath.h:955-1013  MaxPooling: window max, argmax as absolute (X,Y) of the input,
 * ties keep the first element of a row-major scan (strict >).  pos holds pairs {X,Y} of uint32. */
void orc_maxpool(float *out, uint32_t *pos, const float *in, int W, int Z, int in_y, int in_x, int pool_x, int pool_y)
{
    int oy = in_y / pool_y, ox = in_x / pool_x;
    for (int w = 0; w < W; w++)
        for (int z = 0; z < Z; z++) {
            const float *p = in + ((size_t)w * Z + z) * in_y * in_x;
            for (int y = 0; y < oy; y++)
                for (int x = 0; x < ox; x++) {
                    int ix = x * pool_x, iy = y * pool_y;
                    float m = p[(size_t)iy * in_x + ix];
                    uint32_t mx = ix, my = iy;
                    for (int py = 0; py < pool_y; py++)
                        for (int px = 0; px < pool_x; px++) {
                            float e = p[(size_t)(iy + py) * in_x + ix + px];
                            if (e > m) { m = e; mx = ix + px; my = iy + py; }
                        }
                    size_t o = (((size_t)w * Z + z) * oy + y) * ox + x;
                    out[o] = m;
                    pos[2 * o] = mx;
                    pos[2 * o + 1] = my;
                }
        }
}

/* cpu/ctensormath.h:1019-1055  MaxPoolingBackward: out (W,Z,out_y,out_x) cleared, then
 * out[argmax] = delta (plain store, last writer wins as in the reference). */
void orc_maxpool_backward(float *out, const uint32_t *pos, const float *delta, int W, int Z, int out_y, int out_x,
                          int pool_x, int pool_y)
{
    int dy = out_y / pool_y, dx = out_x / pool_x;
    memset(out, 0, sizeof(float) * (size_t)W * Z * out_y * out_x);
    for (int w = 0; w < W; w++)
        for (int z = 0; z < Z; z++)
            for (int y = 0; y < dy; y++)
                for (int x = 0; x < dx; x++) {
                    size_t i = (((size_t)w * Z + z) * dy + y) * dx + x;
                    out[((size_t)w * Z + z) * out_y * out_x + (size_t)pos[2 * i + 1] * out_x + pos[2 * i]] = delta[i];
                }
}

/* cpu/ctensormath.h:868-902  UpSampling: nearest-neighbour replication, zero where the source
 * index leaves the input. */
void orc_upsample(float *out, const float *in, int W, int Z, int in_y, int in_x, int out_y, int out_x, int ux, int uy)
{
    for (int w = 0; w < W; w++)
        for (int z = 0; z < Z; z++)
            for (int y = 0; y < out_y; y++)
                for (int x = 0; x < out_x; x++) {
                    int iy = y / uy, ix = x / ux;
                    float v = 0;
                    if (ix < in_x && iy < in_y) v = in[(((size_t)w * Z + z) * in_y + iy) * in_x + ix];
                    out[(((size_t)w * Z + z) * out_y + y) * out_x + x] = v;
                }
}

/* cpu/ctensormath.h:908-949  DownSampling: mean over the dx*dy window (sum order dx outer, dy
 * inner; divisor is always dx*dy).  Used as the backward pass of UpSampling. */
void orc_downsample(float *out, const float *in, int W, int Z, int in_y, int in_x, int out_y, int out_x, int dsx, int dsy)
{
    for (int w = 0; w < W; w++)
        for (int z = 0; z < Z; z++)
            for (int y = 0; y < out_y; y++)
                for (int x = 0; x < out_x; x++) {
                    int ix = x * dsx, iy = y * dsy;
                    float s = 0;
                    for (int dx = 0; dx < dsx; dx++) {
                        int xp = ix + dx;
                        if (xp >= in_x) continue;
                        for (int dy = 0; dy < dsy; dy++) {
                            int yp = iy + dy;
                            if (yp >= in_y) continue;
                            s += in[(((size_t)w * Z + z) * in_y + yp) * in_x + xp];
                        }
                    }
                    s /= (float)(dsx * dsy);
                    out[(((size_t)w * Z + z) * out_y + y) * out_x + x] = s;
                }
}

/* cpu/ctensorapplyfunc.h:128-257 scalar activations and derivatives.
 * func: 0 sigmoid, 1 ReLU, 2 LeakyReLU(0.1), 3 linear, 4 tanh, 5 GeLU.  The clamp constants and
 * the double-precision intermediate of sigmoid follow the reference. */
static float act_sigmoid(float v) { if (v > 30) v = 29.99999f; if (v < -30) v = -29.99999f; return (float)(1.0 / (1.0 + expf(-v))); }
static float act_tanh(float v) { if (v > 30) v = 29.99999f; if (v < -30) v = -29.99999f; return tanhf(v); }
static float act_gelu(float v)
{
    const float PI = 3.141592654f;
    float ft = (float)(sqrtf(2 / PI) * (v + 0.044715 * v * v * v));
    ft = tanhf(ft);
    return (float)(0.5 * v * (1 + ft));
}
static float act_dgelu(float v)
{
    const float PI = 3.141592654f;
    float ft = (float)(sqrtf(2 / PI) * (v + 0.044715 * v * v * v));
    float fa = (float)(sqrtf(2 / PI) * (1 + 3 * 0.044715 * v * v));
    float sech = 1 / coshf(ft);
    return (float)(0.5 * ((1 + tanhf(ft)) + 0.5 * v * sech * sech) * fa);
}
float orc_act_scalar(float v, int func, int derivative)
{
    if (!derivative) {
        switch (func) {
        case 0: return act_sigmoid(v);
        case 1: return v > 0 ? v : 0;
        case 2: return v > 0 ? v : (float)(0.1 * v);
        case 3: return v;
        case 4: return act_tanh(v);
        default: return act_gelu(v);
        }
    }
    switch (func) {
    case 0: { float s = act_sigmoid(v); return (float)((1.0 - s) * s); }
    case 1: return v >= 0 ? 1.f : 0.f;
    case 2: return v >= 0 ? 1.f : 0.1f;
    case 3: return 1.f;
    case 4: { float t = act_tanh(v); return 1 - t * t; }
    default: return act_dgelu(v);
    }
}
/* cpu/ctensorapplyfunc.h Apply* / ApplyDifferential*: element-wise over the whole tensor. */
void orc_activation(float *out, const float *in, size_t n, int func, int derivative)
{
    for (size_t i = 0; i < n; i++) out[i] = orc_act_scalar(in[i], func, derivative);
}

/* netlayer/cnetlayerbatchnormalization.cu.h:301-379  training-mode forward of the batch-norm
 * layer, restated as the same sequence of tensor routines: statistics are taken per (z,y,x)
 * element over the batch W only.  n = Z*Y*X.  Outputs: y, xhat (W x n), ivar, mean, var (n).
 * new_mean/new_var are the running statistics updated with `momentum` (may be NULL). */
void orc_bn_forward(float *y, float *xhat, float *ivar, float *mean, float *var,
                    float *new_mean, float *new_var,
                    const float *x, const float *gamma, const float *beta,
                    int W, size_t n, float momentum, float eps)
{
    float N = (float)W;
    float *tmp = (float *)malloc(sizeof(float) * (size_t)W * n);
    float *sq = (float *)malloc(sizeof(float) * n);
    memset(mean, 0, sizeof(float) * n);
    orc_add_sum_w(mean, 1, mean, 1, x, W, n, 1.f, (float)(1.0 / N));
    if (new_mean) orc_add(new_mean, 1, new_mean, 1, mean, 1, n, momentum, (float)(1.0 - momentum), 0);
    orc_add(xhat, W, x, W, mean, 1, n, 1.f, 1.f, 1);
    memset(var, 0, sizeof(float) * n);
    orc_unary(tmp, W, xhat, W, n, 0, 1.f, 0.f);
    orc_add_sum_w(var, 1, var, 1, tmp, W, n, 1.f, (float)(1.0 / N));
    if (new_var) orc_add(new_var, 1, new_var, 1, var, 1, n, momentum, (float)(1.0 - momentum), 0);
    orc_unary(sq, 1, var, 1, n, 1, 1.f, eps);
    orc_unary(ivar, 1, sq, 1, n, 2, 0.f, 0.f);
    orc_item_product(xhat, W, xhat, W, ivar, 1, n);
    orc_item_product(tmp, W, gamma, 1, xhat, W, n);
    orc_add(y, W, tmp, W, beta, 1, n, 1.f, 1.f, 0);
    free(tmp);
    free(sq);
}

/* netlayer/cnetlayerbatchnormalization.cu.h:578-604  backward of the batch-norm layer:
 * dx = ivar/N * (N*dxhat - xhat*sum_w(dxhat*xhat) - sum_w(dxhat)), dgamma += sum_w(dy*xhat),
 * dbeta += sum_w(dy); the operation order of the reference sequence is kept. */
void orc_bn_backward(float *dx, float *dgamma, float *dbeta,
                     const float *dy, const float *xhat, const float *ivar, const float *gamma,
                     int W, size_t n, int create_delta_weight)
{
    float N = (float)W;
    float *dxhat = (float *)malloc(sizeof(float) * (size_t)W * n);
    float *tmp = (float *)malloc(sizeof(float) * (size_t)W * n);
    float *sb = (float *)calloc(n, sizeof(float));
    float *sc = (float *)calloc(n, sizeof(float));
    orc_item_product(dxhat, W, dy, W, gamma, 1, n);
    orc_add_sum_w(sb, 1, sb, 1, dxhat, W, n, 1.f, 1.f);
    orc_item_product(tmp, W, dxhat, W, xhat, W, n);
    orc_add_sum_w(sc, 1, sc, 1, tmp, W, n, 1.f, 1.f);
    if (create_delta_weight) {
        orc_item_product(tmp, W, dy, W, xhat, W, n);
        orc_add_sum_w(dgamma, 1, dgamma, 1, tmp, W, n, 1.f, 1.f);
        orc_add_sum_w(dbeta, 1, dbeta, 1, dy, W, n, 1.f, 1.f);
    }
    orc_unary(dx, W, dxhat, W, n, 3, N, 0.f);
    orc_item_product(tmp, W, xhat, W, sc, 1, n);
    orc_add(dx, W, dx, W, tmp, W, n, 1.f, 1.f, 1);
    orc_add(dx, W, dx, W, sb, 1, n, 1.f, 1.f, 1);
    orc_item_product(dx, W, dx, W, ivar, 1, n);
    orc_unary(dx, W, dx, W, n, 3, (float)(1.0 / N), 0.f);
    free(dxhat); free(tmp); free(sb); free(sc);
}

/* netlayer/cnetlayervaecoderoutput.cu.h:251-280  reparameterisation z = mu + exp(clamp(logvar)/2)*eps
 * with eps supplied by the caller (the reference draws it from an unseedable generator);
 * returns the KL term -0.5/batch * sum(1 + lv - mu^2 - exp(lv)) accumulated in float. */
float orc_vae_forward(float *z, const float *mu, const float *logvar, const float *eps, int batch, size_t n)
{
    float kl = 0;
    for (size_t i = 0; i < (size_t)batch * n; i++) {
        float lv = logvar[i];
        if (lv > 10) lv = 10;
        if (lv < -10) lv = -10;
        float e = (float)exp(lv / 2.0);
        z[i] = mu[i] + e * eps[i];
        kl += 1 + lv - mu[i] * mu[i] - expf(lv);
    }
    kl *= -0.5f;
    kl /= batch;
    return kl;
}

/* netlayer/cnetlayervaecoderoutput.cu.h:424-455  error split of the VAE output layer:
 * d_logvar = delta*0.5*eps*exp(lv/2) - 0.5*(1-exp(lv))*k,  d_mu = delta + mu*k  (no clamp here,
 * as in the reference). */
void orc_vae_backward(float *d_mu, float *d_logvar, const float *delta, const float *mu, const float *logvar,
                      const float *eps, size_t total, float k)
{
    for (size_t i = 0; i < total; i++) {
        float lv = logvar[i];
        float diff = (float)(1.0 / 2.0 * eps[i] * exp(lv / 2.0));
        float o = delta[i] * diff;
        o += (float)(-1.0 / 2.0 * (1 - expf(lv)) * k);
        d_logvar[i] = o;
        float m = delta[i] * 1;
        m += (float)(-1.0 / 2.0 * (0 - 2 * mu[i]) * k);
        d_mu[i] = m;
    }
}

/* cuda/ctensormath.cu.h:3029-3058  SetTimeStep (the reference has this routine on its CUDA backend only, so this
 * restatement follows the kernel's arithmetic and is NOT pinned to a reference run: parity unpinned for this routine):
 * out[w,pos] = in[w,pos] + (pos even ? sin : cos)(t[w] / 10000^(pos/n)), float arithmetic. */
void orc_set_time_step(float *out, const float *in, const uint32_t *time_step, int W, size_t n)
{
    for (int w = 0; w < W; w++)
        for (size_t pos = 0; pos < n; pos++) {
            float t = (float)time_step[w];
            float angle = t / powf(10000.0f, (float)pos / (float)n);
            float value = in[(size_t)w * n + pos];
            if ((pos & 1) == 0) value += sinf(angle);
            else value += cosf(angle);
            out[(size_t)w * n + pos] = value;
        }
}

/* cuda/ctensormath.cu.h:3216-3245  GetNoiseImageAndNoise with the noise supplied (CUDA backend only, parity unpinned):
 * noisy = sqrt_alpha_bar[w]*image + sqrt_one_minus_alpha_bar[w]*noise. */
void orc_noisy_image(float *noisy, const float *image, const float *noise, const float *sa, const float *so, int W, size_t n)
{
    for (int w = 0; w < W; w++)
        for (size_t i = 0; i < n; i++) {
            size_t k = (size_t)w * n + i;
            noisy[k] = sa[w] * image[k] + so[w] * noise[k];
        }
}

/* cpu/ctensormath.h:1119-1165  Adam step (the CPU variant: bias correction with `iteration` as given). */
void orc_adam(float *weight, const float *dweight, float *m, float *v, size_t n, uint32_t batch_size,
              double speed, double beta1, double beta2, double epsilon, double iteration)
{
    for (size_t i = 0; i < n; i++) {
        float dw = dweight[i], mm = m[i], vv = v[i];
        dw /= (float)batch_size;
        mm = (float)(beta1 * mm + (1.0 - beta1) * dw);
        vv = (float)(beta2 * vv + (1.0 - beta2) * dw * dw);
        float mc = (float)(mm / (1.0 - pow(beta1, iteration)));
        float vc = (float)(vv / (1.0 - pow(beta2, iteration)));
        dw = (float)(speed * mc / (sqrt(vc) + epsilon));
        m[i] = mm;
        v[i] = vv;
        weight[i] = weight[i] - dw;
    }
}
