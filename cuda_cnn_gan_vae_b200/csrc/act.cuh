// The neuron functions of the reference (cpu/ctensorapplyfunc.h:128-257: sigmoid and tanh with the argument clamped to +-30,
// LeakyReLU multiplied in double precision, derivative 1 at zero for ReLU and LeakyReLU) as device functions shared by the
// element-wise kernels, the operand packs and the epilogue of the tensor-core kernel, so that an activation gives the same
// bits wherever it is applied.
#pragma once
#include <cuda_runtime.h>
#include "../../include/b200conv.h"

namespace b200 {

__device__ __forceinline__ float act_sigmoid(float v)
{
    if (v > 30.f) v = 29.99999f;
    if (v < -30.f) v = -29.99999f;
    return 1.0f / (1.0f + expf(-v));
}
__device__ __forceinline__ float act_tanh(float v)
{
    if (v > 30.f) v = 29.99999f;
    if (v < -30.f) v = -29.99999f;
    return tanhf(v);
}
__device__ __forceinline__ float act_apply(float v, int func, double slope)
{
    switch (func) {
    case B200_ACT_SIGMOID: return act_sigmoid(v);
    case B200_ACT_RELU: return v > 0.f ? v : 0.f;
    case B200_ACT_LEAKY_RELU: return v > 0.f ? v : (float)(slope * (double)v);   // the reference multiplies in double
    case B200_ACT_LINEAR: return v;
    case B200_ACT_TANH: return act_tanh(v);
    default: {
        const float c = 0.7978845608f;  // sqrt(2/pi)
        float ft = tanhf(c * (v + 0.044715f * v * v * v));
        return 0.5f * v * (1.f + ft);
    }
    }
}
__device__ __forceinline__ float act_derivative(float v, int func, double slope)
{
    switch (func) {
    case B200_ACT_SIGMOID: { float s = act_sigmoid(v); return (1.0f - s) * s; }
    case B200_ACT_RELU: return v >= 0.f ? 1.f : 0.f;
    case B200_ACT_LEAKY_RELU: return v >= 0.f ? 1.f : (float)slope;
    case B200_ACT_LINEAR: return 1.f;
    case B200_ACT_TANH: { float t = act_tanh(v); return 1.f - t * t; }
    default: {
        const float c = 0.7978845608f;
        float ft = c * (v + 0.044715f * v * v * v);
        float fa = c * (1.f + 3.f * 0.044715f * v * v);
        float sech = 1.f / coshf(ft);
        return 0.5f * ((1.f + tanhf(ft)) + 0.5f * v * sech * sech) * fa;
    }
    }
}

}  // namespace b200
