// CTensorMath::Adam (cpu/ctensormath.h:1119-1165) for one parameter, shared by the stand-alone optimiser kernel and by the
// kernel that fuses the gradient reduction across devices with the update.
//
// The reference evaluates the two moment updates in double precision and rounds them to float; that part is kept
// operation for operation (double multiplies and adds, no divisions), so m and v are bit-identical.  The two bias
// corrections become multiplications by reciprocals formed once on the host, and the step speed * mc / (sqrt(vc) + epsilon)
// is evaluated in IEEE fp32 (relative error ~2e-7 of a step that is itself ~1e-4 of a weight): the updated weight equals
// the reference's except, rarely, in its last bit.  What this buys: no double-precision division or square root per
// element, which is what held the kernel at 0.42 of the HBM bandwidth.
#pragma once
#include <cuda_runtime.h>

namespace b200 {

struct AdamArgs {
    float batch, inv_batch;     // gradient divisor; inv_batch != 0 when the reciprocal is exact (power of two)
    double beta1, beta2, omb1, omb2, inv_c1, inv_c2;
    float speed, epsilon;
    float ema_k, ema_k1;        // exponential moving average of the weights: ema = ema_k * ema + ema_k1 * weight
};

inline AdamArgs adam_args(unsigned batch_size, double speed, double beta1, double beta2, double epsilon, double c1, double c2, double ema_k)
{
    AdamArgs a;
    a.batch = (float)batch_size;
    a.inv_batch = (batch_size & (batch_size - 1)) == 0 ? 1.0f / (float)batch_size : 0.f;
    a.beta1 = beta1; a.beta2 = beta2; a.omb1 = 1.0 - beta1; a.omb2 = 1.0 - beta2;
    a.inv_c1 = 1.0 / c1; a.inv_c2 = 1.0 / c2;
    a.speed = (float)speed; a.epsilon = (float)epsilon;
    a.ema_k = (float)ema_k; a.ema_k1 = (float)(1.0 - ema_k);
    return a;
}

__device__ __forceinline__ float adam_element(float w, float g, float &m, float &v, const AdamArgs &a)
{
    const float dw = a.inv_batch != 0.f ? __fmul_rn(g, a.inv_batch) : __fdiv_rn(g, a.batch);
    const double dwd = (double)dw;
    const float mm = (float)__dadd_rn(__dmul_rn(a.beta1, (double)m), __dmul_rn(a.omb1, dwd));
    const float vv = (float)__dadd_rn(__dmul_rn(a.beta2, (double)v), __dmul_rn(__dmul_rn(a.omb2, dwd), dwd));
    const float mc = (float)__dmul_rn((double)mm, a.inv_c1);
    const float vc = (float)__dmul_rn((double)vv, a.inv_c2);
    const float step = __fdiv_rn(__fmul_rn(a.speed, mc), __fadd_rn(__fsqrt_rn(vc), a.epsilon));
    m = mm;
    v = vv;
    return __fsub_rn(w, step);
}

__device__ __forceinline__ float ema_element(float ema, float w, const AdamArgs &a)
{
    // CTensorMath::Add(ema, ema, weight, EMA_K, 1 - EMA_K) (netlayer/cnetlayerconvolution.cu.h:547-551, cpu/ctensormath.h:235)
    return __fadd_rn(__fmul_rn(a.ema_k, ema), __fmul_rn(a.ema_k1, w));
}

}  // namespace b200
