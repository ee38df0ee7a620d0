// CUDA-core fp32 convolution kernels for arbitrary geometry and W-broadcast (per-sample kernels,
// ragged sizes, any stride/padding).  They follow the summation order of the reference CPU backend
// (cpu/ctensorconv.h:111-148, 224-266, 345-385) with separate multiply and add, so their results
// are bit-identical to it.  The tensor-core kernels take over for the shapes they support; these
// are the general path behind the same entry points.
#include "common.cuh"
#include "kernels.h"

namespace b200 {

__global__ void simt_conv_forward_kernel(b200_conv_geom g, float *__restrict__ out, int out_w,
                                         const float *__restrict__ image, int image_w,
                                         const float *__restrict__ kernel, int kernel_w,
                                         const float *__restrict__ bias, int bias_w)
{
    grid_dependency_wait();
    const size_t total = (size_t)out_w * g.kernel_amount * g.out_y * g.out_x;
    const int klen = g.in_z * g.kernel_y * g.kernel_x;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        int x = idx % g.out_x;
        size_t t = idx / g.out_x;
        int y = t % g.out_y; t /= g.out_y;
        int k = t % g.kernel_amount;
        int w = t / g.kernel_amount;
        const float *img = image + (size_t)(w % image_w) * g.in_z * g.in_y * g.in_x;
        const float *ker = kernel + ((size_t)(w % kernel_w) * g.kernel_amount + k) * klen;
        float sum = bias ? bias[(size_t)(w % bias_w) * g.kernel_amount + k] : 0.f;
        for (int ky = 0; ky < g.kernel_y; ky++) {
            int y0 = g.stride_y * y + ky - g.padding_y;
            if (y0 < 0 || y0 >= g.in_y) continue;
            for (int kx = 0; kx < g.kernel_x; kx++) {
                int x0 = g.stride_x * x + kx - g.padding_x;
                if (x0 < 0 || x0 >= g.in_x) continue;
                const float *ip = img + (size_t)y0 * g.in_x + x0;
                const float *kp = ker + ky * g.kernel_x + kx;
                for (int z = 0; z < g.in_z; z++)
                    sum = __fadd_rn(sum, __fmul_rn(kp[z * g.kernel_y * g.kernel_x], ip[(size_t)z * g.in_y * g.in_x]));
            }
        }
        out[idx] = sum;
    }
}

__global__ void simt_conv_backward_kernel(b200_conv_geom g, float *__restrict__ out, int out_w,
                                          const float *__restrict__ delta, int delta_w,
                                          const float *__restrict__ kernel, int kernel_w,
                                          const float *__restrict__ bias, int bias_w)
{
    grid_dependency_wait();
    const size_t total = (size_t)out_w * g.in_z * g.in_y * g.in_x;
    const int klen = g.in_z * g.kernel_y * g.kernel_x;
    const int pad_y = g.kernel_y - 1 - g.padding_y, pad_x = g.kernel_x - 1 - g.padding_x;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        int x = idx % g.in_x;
        size_t t = idx / g.in_x;
        int y = t % g.in_y; t /= g.in_y;
        int z = t % g.in_z;
        int w = t / g.in_z;
        const float *dl = delta + (size_t)(w % delta_w) * g.kernel_amount * g.out_y * g.out_x;
        const float *ker = kernel + (size_t)(w % kernel_w) * g.kernel_amount * klen + z * g.kernel_y * g.kernel_x;
        const float *bs = bias ? bias + (size_t)(w % bias_w) * g.kernel_amount : nullptr;
        float summ = 0.f;
        for (int ky = 0; ky < g.kernel_y; ky++) {
            int y0 = y + ky - pad_y;
            if (y0 % g.stride_y != 0) continue;
            int dy0 = y0 / g.stride_y;
            if (dy0 < 0 || dy0 >= g.out_y) continue;
            for (int kx = 0; kx < g.kernel_x; kx++) {
                int x0 = x + kx - pad_x;
                if (x0 % g.stride_x != 0) continue;
                int dx0 = x0 / g.stride_x;
                if (dx0 < 0 || dx0 >= g.out_x) continue;
                const float *kp = ker + (g.kernel_y - 1 - ky) * g.kernel_x + (g.kernel_x - 1 - kx);
                const float *dp = dl + (size_t)dy0 * g.out_x + dx0;
                for (int f = 0; f < g.kernel_amount; f++) {
                    if (bs) summ = __fadd_rn(summ, bs[f]);
                    summ = __fadd_rn(summ, __fmul_rn(kp[(size_t)f * klen], dp[(size_t)f * g.out_y * g.out_x]));
                }
            }
        }
        out[idx] = summ;
    }
}

// One thread per (w, f, c, i, j) weight element; sums over the delta plane in y,x order starting
// from the existing value, exactly the order in which the CPU loop touches that element.
__global__ void simt_conv_wgrad_kernel(b200_conv_geom g, float *__restrict__ dkernel, int dkernel_w,
                                       const float *__restrict__ image, int image_w,
                                       const float *__restrict__ delta, int delta_w)
{
    grid_dependency_wait();
    const int klen = g.in_z * g.kernel_y * g.kernel_x;
    const size_t total = (size_t)dkernel_w * g.kernel_amount * klen;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        int e = idx % klen;
        size_t t = idx / klen;
        int f = t % g.kernel_amount;
        int w = t / g.kernel_amount;
        int j = e % g.kernel_x;
        int i = (e / g.kernel_x) % g.kernel_y;
        int c = e / (g.kernel_x * g.kernel_y);
        const float *img = image + ((size_t)(w % image_w) * g.in_z + c) * g.in_y * g.in_x;
        const float *dl = delta + ((size_t)(w % delta_w) * g.kernel_amount + f) * g.out_y * g.out_x;
        float v = dkernel[idx];
        for (int oy = 0; oy < g.out_y; oy++) {
            int i0 = i + oy * g.stride_y - g.padding_y;
            if (i0 < 0 || i0 >= g.in_y) continue;
            for (int ox = 0; ox < g.out_x; ox++) {
                int j0 = j + ox * g.stride_x - g.padding_x;
                if (j0 < 0 || j0 >= g.in_x) continue;
                v = __fadd_rn(v, __fmul_rn(dl[(size_t)oy * g.out_x + ox], img[(size_t)i0 * g.in_x + j0]));
            }
        }
        dkernel[idx] = v;
    }
}

// dbias[wb][f] += sum over every w < dkernel_w with w % dbias_w == wb (in increasing w) of the
// delta plane summed in y,x order: the CPU order.
__global__ void simt_conv_dbias_kernel(int kernel_amount, int plane, float *__restrict__ dbias, int dbias_w,
                                       int dkernel_w, const float *__restrict__ delta, int delta_w)
{
    grid_dependency_wait();
    int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= dbias_w * kernel_amount) return;
    int f = idx % kernel_amount, wb = idx / kernel_amount;
    float b = dbias[idx];
    for (int w = wb; w < dkernel_w; w += dbias_w) {
        const float *dl = delta + ((size_t)(w % delta_w) * kernel_amount + f) * plane;
        for (int p = 0; p < plane; p++) b = __fadd_rn(b, dl[p]);
    }
    dbias[idx] = b;
}

static int grid_for(size_t total, int block)
{
    size_t blocks = (total + block - 1) / block;
    size_t cap = (size_t)sm_count() * 32;
    return (int)(blocks < cap ? (blocks ? blocks : 1) : cap);
}

int simt_conv_forward(const b200_conv_geom &g, float *out, int out_w, const float *image, int image_w,
                      const float *kernel, int kernel_w, const float *bias, int bias_w, cudaStream_t s)
{
    size_t total = (size_t)out_w * g.kernel_amount * g.out_y * g.out_x;
    if (!total) return B200_OK;
    Launch(grid_for(total, 256), 256, 0, s)(simt_conv_forward_kernel, g, out, out_w, image, image_w, kernel, kernel_w, bias, bias_w);
    B200_LAUNCH_CHECK();
    return B200_OK;
}

int simt_conv_backward(const b200_conv_geom &g, float *out, int out_w, const float *delta, int delta_w,
                       const float *kernel, int kernel_w, const float *bias, int bias_w, cudaStream_t s)
{
    size_t total = (size_t)out_w * g.in_z * g.in_y * g.in_x;
    if (!total) return B200_OK;
    Launch(grid_for(total, 256), 256, 0, s)(simt_conv_backward_kernel, g, out, out_w, delta, delta_w, kernel, kernel_w, bias, bias_w);
    B200_LAUNCH_CHECK();
    return B200_OK;
}

int simt_conv_wgrad(const b200_conv_geom &g, float *dkernel, int dkernel_w, float *dbias, int dbias_w,
                    const float *image, int image_w, const float *delta, int delta_w, cudaStream_t s)
{
    size_t total = (size_t)dkernel_w * g.kernel_amount * g.in_z * g.kernel_y * g.kernel_x;
    if (!total) return B200_OK;
    Launch(grid_for(total, 128), 128, 0, s)(simt_conv_wgrad_kernel, g, dkernel, dkernel_w, image, image_w, delta, delta_w);
    B200_LAUNCH_CHECK();
    if (dbias) {
        int n = dbias_w * g.kernel_amount;
        Launch(ceil_div(n, 128), 128, 0, s)(simt_conv_dbias_kernel, g.kernel_amount, g.out_y * g.out_x, dbias, dbias_w,
                                                               dkernel_w, delta, delta_w);
        B200_LAUNCH_CHECK();
    }
    return B200_OK;
}

}  // namespace b200
