// Memory-bound kernels of the hot path and their C-ABI entry points: element-wise arithmetic with
// W-broadcast, reductions over W and over the Y,X plane, activations, pooling, resampling, fused
// batch-norm, the VAE reparameterisation and Adam.  All of them stream through HBM once with
// 128-bit accesses where the alignment allows; grids are sized in multiples of the SM count.
#include "common.cuh"
#include "kernels.h"
#include "tc_ptx.cuh"
#include "adam.cuh"
#include "act.cuh"
#include <cmath>

namespace b200 {

static inline int stream_grid(size_t work_items, int block)
{
    size_t blocks = (work_items + block - 1) / block;
    size_t cap = (size_t)sm_count() * 16;
    if (blocks < 1) blocks = 1;
    return (int)(blocks < cap ? blocks : cap);
}

static inline bool aligned16(const void *p) { return ((uintptr_t)p & 15) == 0; }

// ---------------------------------------------------------------------------------------------
// element-wise with W-broadcast: out[w][i] = F(left[w%Lw][i], right[w%Rw][i])
// ---------------------------------------------------------------------------------------------
struct OpAdd { float ls, rs; __device__ float operator()(float l, float r) const { return __fadd_rn(__fmul_rn(ls, l), __fmul_rn(rs, r)); } };
struct OpSub { float ls, rs; __device__ float operator()(float l, float r) const { return __fsub_rn(__fmul_rn(ls, l), __fmul_rn(rs, r)); } };
struct OpMul { __device__ float operator()(float l, float r) const { return __fmul_rn(l, r); } };
struct OpDiv { float ls, rs; __device__ float operator()(float l, float r) const { return __fdiv_rn(__fmul_rn(l, ls), __fmul_rn(r, rs)); } };

// out[p] (cols x rows) = in[p]^T (rows x cols) for every (w,z) plane p; 32x32 shared-memory tiles
__global__ void transpose_kernel(float *__restrict__ out, const float *__restrict__ in, int rows, int cols)
{
    grid_dependency_wait();
    __shared__ float tile[32][33];
    const size_t plane = (size_t)blockIdx.z * rows * cols;
    const int x0 = blockIdx.x * 32, y0 = blockIdx.y * 32;
    for (int i = threadIdx.y; i < 32; i += blockDim.y) {
        int y = y0 + i, x = x0 + threadIdx.x;
        tile[i][threadIdx.x] = (y < rows && x < cols) ? in[plane + (size_t)y * cols + x] : 0.f;
    }
    __syncthreads();
    for (int i = threadIdx.y; i < 32; i += blockDim.y) {
        int x = x0 + i, y = y0 + threadIdx.x;
        if (x < cols && y < rows) out[plane + (size_t)x * rows + y] = tile[threadIdx.x][i];
    }
}

template <class F, bool VEC>
__global__ void binary_kernel(float *__restrict__ out, int out_w, const float *left, int left_w,
                              const float *right, int right_w, size_t n, F f)
{
    grid_dependency_wait();
    const size_t per_w = VEC ? n / 4 : n;
    const size_t total = per_w * out_w;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        size_t w = idx / per_w, i = idx - w * per_w;
        if (VEC) {
            float4 l = reinterpret_cast<const float4 *>(left + (w % left_w) * n)[i];
            float4 r = reinterpret_cast<const float4 *>(right + (w % right_w) * n)[i];
            float4 o = make_float4(f(l.x, r.x), f(l.y, r.y), f(l.z, r.z), f(l.w, r.w));
            reinterpret_cast<float4 *>(out + w * n)[i] = o;
        } else {
            out[w * n + i] = f(left[(w % left_w) * n + i], right[(w % right_w) * n + i]);
        }
    }
}

template <class F>
static int launch_binary(float *out, int out_w, const float *left, int left_w, const float *right, int right_w,
                         size_t n, F f, cudaStream_t s)
{
    if (!out || !left || !right) return fail(B200_E_ARG, "null tensor pointer");
    if (out_w <= 0 || left_w <= 0 || right_w <= 0) return fail(B200_E_SHAPE, "non-positive W count");
    if (!n) return B200_OK;
    bool vec = (n % 4 == 0) && aligned16(out) && aligned16(left) && aligned16(right);
    size_t total = (vec ? n / 4 : n) * out_w;
    if (vec) Launch(stream_grid(total, 256), 256, 0, s)(binary_kernel<F, true>, out, out_w, left, left_w, right, right_w, n, f);
    else Launch(stream_grid(total, 256), 256, 0, s)(binary_kernel<F, false>, out, out_w, left, left_w, right, right_w, n, f);
    B200_LAUNCH_CHECK();
    return B200_OK;
}

// ---------------------------------------------------------------------------------------------
// unary with W-broadcast of the input
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float unary_apply(float v, int op, float a, float b)
{
    switch (op) {
    case 0: return __fmul_rn(__fmul_rn(v, v), a);
    case 1: return __fmul_rn(__fsqrt_rn(__fadd_rn(v, b)), a);
    case 2: return __fdiv_rn(1.0f, v);
    case 3: return __fmul_rn(v, a);
    case 4: return __fadd_rn(__fmul_rn(v, a), b);
    case 5: return v > b ? b : (v < a ? a : v);
    default: return v > 0.f ? 1.f : (v < 0.f ? -1.f : v);
    }
}

__global__ void unary_kernel(float *__restrict__ out, int out_w, const float *in, int in_w, size_t n, int op, float a, float b)
{
    grid_dependency_wait();
    const size_t total = n * out_w;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        size_t w = idx / n, i = idx - w * n;
        out[idx] = unary_apply(in[(w % in_w) * n + i], op, a, b);
    }
}

__global__ void fill_kernel(float *__restrict__ out, size_t n, float v)
{
    grid_dependency_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) out[i] = v;
}

// ---------------------------------------------------------------------------------------------
// AddSumW: out[0][i] = ls*sum_w left[w][i] + rs*sum_w right[w][i]; out[w>0][i] = 0.  One thread per
// element walks W sequentially (the reference order); neighbouring threads read neighbouring
// addresses, so every pass over a w-slice is fully coalesced.
// ---------------------------------------------------------------------------------------------
__global__ void add_sum_w_kernel(float *out, int out_w, const float *left, int left_w, const float *right, int right_w,
                                 size_t n, float ls, float rs)
{
    grid_dependency_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        float sl = 0.f, sr = 0.f;
        for (int w = 0; w < left_w; w++) sl = __fadd_rn(sl, left[(size_t)w * n + i]);
        sl = __fmul_rn(sl, ls);
        for (int w = 0; w < right_w; w++) sr = __fadd_rn(sr, right[(size_t)w * n + i]);
        sr = __fmul_rn(sr, rs);
        out[i] = __fadd_rn(sl, sr);
        for (int w = 1; w < out_w; w++) out[(size_t)w * n + i] = 0.f;
    }
}

// ---------------------------------------------------------------------------------------------
// AddBias (+ optional activation): t[w,z,:,:] = f(t + bias[w%Bw,z])
// ---------------------------------------------------------------------------------------------
template <bool VEC>
__global__ void bias_act_kernel(float *t, float *pre, int t_w, int z, size_t yx, const float *__restrict__ bias, int bias_w,
                                int func, double slope)
{
    grid_dependency_wait();
    const size_t per_plane = VEC ? yx / 4 : yx;
    const size_t total = per_plane * z * t_w;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        size_t plane = idx / per_plane;
        int zz = plane % z;
        size_t w = plane / z;
        float b = bias[(w % bias_w) * z + zz];
        if (VEC) {
            float4 v = reinterpret_cast<float4 *>(t)[idx];
            v.x = __fadd_rn(v.x, b); v.y = __fadd_rn(v.y, b); v.z = __fadd_rn(v.z, b); v.w = __fadd_rn(v.w, b);
            if (pre) reinterpret_cast<float4 *>(pre)[idx] = v;
            if (func != B200_ACT_LINEAR) {
                v.x = act_apply(v.x, func, slope); v.y = act_apply(v.y, func, slope);
                v.z = act_apply(v.z, func, slope); v.w = act_apply(v.w, func, slope);
            }
            reinterpret_cast<float4 *>(t)[idx] = v;
        } else {
            float v = __fadd_rn(t[idx], b);
            if (pre) pre[idx] = v;
            t[idx] = func != B200_ACT_LINEAR ? act_apply(v, func, slope) : v;
        }
    }
}

__global__ void activation_kernel(float *__restrict__ out, const float *__restrict__ in, const float *__restrict__ err,
                                  size_t n, int func, int derivative, double slope)
{
    grid_dependency_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        float v = in[i];
        float r = derivative ? act_derivative(v, func, slope) : act_apply(v, func, slope);
        out[i] = err ? r * err[i] : r;
    }
}

// the same with 16-byte accesses (n4 = n / 4 vectors; all pointers 16-byte aligned)
__global__ void activation_vec_kernel(float4 *__restrict__ out, const float4 *__restrict__ in, const float4 *__restrict__ err,
                                      size_t n4, int func, int derivative, double slope)
{
    grid_dependency_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (size_t)gridDim.x * blockDim.x) {
        const float4 v = in[i];
        float4 r;
        if (derivative) {
            r.x = act_derivative(v.x, func, slope); r.y = act_derivative(v.y, func, slope);
            r.z = act_derivative(v.z, func, slope); r.w = act_derivative(v.w, func, slope);
        } else {
            r.x = act_apply(v.x, func, slope); r.y = act_apply(v.y, func, slope);
            r.z = act_apply(v.z, func, slope); r.w = act_apply(v.w, func, slope);
        }
        if (err) {
            const float4 e = err[i];
            r.x *= e.x; r.y *= e.y; r.z *= e.z; r.w *= e.w;
        }
        out[i] = r;
    }
}

static void launch_activation(float *out, const float *in, const float *err, size_t n, int func, int derivative, double slope,
                              cudaStream_t s)
{
    if (n % 4 == 0 && aligned16(out) && aligned16(in) && (!err || aligned16(err)))
        Launch(stream_grid(n / 4, 256), 256, 0, s)(activation_vec_kernel, reinterpret_cast<float4 *>(out), reinterpret_cast<const float4 *>(in),
                                                                     reinterpret_cast<const float4 *>(err), n / 4, func, derivative, slope);
    else
        Launch(stream_grid(n, 256), 256, 0, s)(activation_kernel, out, in, err, n, func, derivative, slope);
}

// ---------------------------------------------------------------------------------------------
// SummXY: out[w,z] = sum of one Y,X plane.  One warp (small planes) or one block (large planes)
// per plane; float4 loads, warp-shuffle tree, fixed order => reproducible run to run.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float warp_sum(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__global__ void summ_xy_kernel(float *__restrict__ out, int out_w, const float *__restrict__ in, int in_w, int z, size_t yx)
{
    grid_dependency_wait();
    __shared__ float part[32];
    const int planes = out_w * z;
    for (int p = blockIdx.x; p < planes; p += gridDim.x) {
        int w = p / z, zz = p % z;
        const float *src = in + ((size_t)(w % in_w) * z + zz) * yx;
        float s = 0.f;
        if ((yx % 4 == 0) && (((uintptr_t)src & 15) == 0)) {
            const float4 *s4 = reinterpret_cast<const float4 *>(src);
            for (size_t i = threadIdx.x; i < yx / 4; i += blockDim.x) { float4 v = s4[i]; s += (v.x + v.y) + (v.z + v.w); }
        } else {
            for (size_t i = threadIdx.x; i < yx; i += blockDim.x) s += src[i];
        }
        s = warp_sum(s);
        if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = s;
        __syncthreads();
        if (threadIdx.x < 32) {
            float v = threadIdx.x < (blockDim.x >> 5) ? part[threadIdx.x] : 0.f;
            v = warp_sum(v);
            if (threadIdx.x == 0) out[p] = v;
        }
        __syncthreads();
    }
}

// ---------------------------------------------------------------------------------------------
// pooling / resampling
// ---------------------------------------------------------------------------------------------
__global__ void maxpool_kernel(float *__restrict__ out, uint2 *__restrict__ pos, const float *__restrict__ in,
                               size_t planes, int in_y, int in_x, int pool_x, int pool_y, int vec2)
{
    grid_dependency_wait();
    const int oy = in_y / pool_y, ox = in_x / pool_x;
    const size_t total = planes * oy * ox;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        int x = idx % ox;
        size_t t = idx / ox;
        int y = t % oy;
        size_t pl = t / oy;
        const float *p = in + pl * in_y * in_x;
        int ix = x * pool_x, iy = y * pool_y;
        float m = p[(size_t)iy * in_x + ix];
        uint32_t mx = ix, my = iy;
        if (vec2) {      // 2x2 windows, even rows, 8-byte aligned input: two 8-byte loads per window
            float2 r0 = *reinterpret_cast<const float2 *>(p + (size_t)iy * in_x + ix);
            float2 r1 = *reinterpret_cast<const float2 *>(p + (size_t)(iy + 1) * in_x + ix);
            if (r0.y > m) { m = r0.y; mx = ix + 1; my = iy; }
            if (r1.x > m) { m = r1.x; mx = ix; my = iy + 1; }
            if (r1.y > m) { m = r1.y; mx = ix + 1; my = iy + 1; }
        } else {
            for (int py = 0; py < pool_y; py++)
                for (int px = 0; px < pool_x; px++) {
                    float e = p[(size_t)(iy + py) * in_x + ix + px];
                    if (e > m) { m = e; mx = ix + px; my = iy + py; }
                }
        }
        out[idx] = m;
        pos[idx] = make_uint2(mx, my);
    }
}

// Backward of max-pooling as a gather over the OUTPUT (race-free, writes every element once):
// out[y,x] = delta of the window that owns (y,x) if that window's argmax is (x,y), else 0.
__global__ void maxpool_backward_kernel(float *__restrict__ out, const uint2 *__restrict__ pos, const float *__restrict__ delta,
                                        size_t planes, int out_y, int out_x, int pool_x, int pool_y)
{
    grid_dependency_wait();
    const int dy = out_y / pool_y, dx = out_x / pool_x;
    const size_t total = planes * out_y * out_x;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        int x = idx % out_x;
        size_t t = idx / out_x;
        int y = t % out_y;
        size_t pl = t / out_y;
        int wy = y / pool_y, wx = x / pool_x;
        float v = 0.f;
        if (wy < dy && wx < dx) {
            size_t i = (pl * dy + wy) * dx + wx;
            uint2 ps = pos[i];
            if (ps.x == (uint32_t)x && ps.y == (uint32_t)y) v = delta[i];
        }
        out[idx] = v;
    }
}

// 2x2 windows that tile the plane exactly: one thread per window; it reads its position and delta once and writes the
// window's two rows as 8-byte stores (consecutive threads write consecutive addresses).
__global__ void maxpool_backward_2x2_kernel(float *__restrict__ out, const uint2 *__restrict__ pos, const float *__restrict__ delta,
                                            unsigned rows, unsigned dx)
{
    grid_dependency_wait();
    // rows = planes * dy window rows; each owns two output rows of 2*dx floats
    const size_t total = (size_t)rows * dx;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const unsigned wx = (unsigned)(i % dx);
        const size_t row = i / dx;
        const uint2 ps = pos[i];
        const float d = delta[i];
        const unsigned px = ps.x - 2 * wx, py = ps.y & 1u;      // position inside the window (y is absolute within the plane, windows start at even rows)
        float2 r0 = make_float2(0.f, 0.f), r1 = r0;
        if (py == 0) { if (px == 0) r0.x = d; else r0.y = d; }
        else { if (px == 0) r1.x = d; else r1.y = d; }
        float2 *o = reinterpret_cast<float2 *>(out + (row * 2) * (size_t)(2 * dx)) + wx;
        o[0] = r0;
        o[dx] = r1;
    }
}

// factor 2 in both directions: one thread per input element, two 8-byte stores
__global__ void upsample_2x2_kernel(float *__restrict__ out, const float *__restrict__ in, unsigned rows, unsigned in_x)
{
    grid_dependency_wait();
    const size_t total = (size_t)rows * in_x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const unsigned x = (unsigned)(i % in_x);
        const size_t row = i / in_x;
        const float v = in[i];
        float2 *o = reinterpret_cast<float2 *>(out + (row * 2) * (size_t)(2 * in_x)) + x;
        o[0] = make_float2(v, v);
        o[in_x] = make_float2(v, v);
    }
}

// factor 2 in both directions, even input sizes: one thread per output, two 8-byte loads; the four values are added in
// the reference's order (column by column, rows inside)
__global__ void downsample_2x2_kernel(float *__restrict__ out, const float *__restrict__ in, unsigned rows, unsigned out_x)
{
    grid_dependency_wait();
    const size_t total = (size_t)rows * out_x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const unsigned x = (unsigned)(i % out_x);
        const size_t row = i / out_x;
        const float2 *p = reinterpret_cast<const float2 *>(in + (row * 2) * (size_t)(2 * out_x)) + x;
        const float2 a = p[0], b = p[out_x];
        float s = __fadd_rn(0.f, a.x);
        s = __fadd_rn(s, b.x);
        s = __fadd_rn(s, a.y);
        s = __fadd_rn(s, b.y);
        out[i] = __fdiv_rn(s, 4.0f);
    }
}

__global__ void upsample_kernel(float *__restrict__ out, const float *__restrict__ in, size_t planes, int in_y, int in_x,
                                int out_y, int out_x, int ux, int uy)
{
    grid_dependency_wait();
    const size_t total = planes * out_y * out_x;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        int x = idx % out_x;
        size_t t = idx / out_x;
        int y = t % out_y;
        size_t pl = t / out_y;
        int iy = y / uy, ix = x / ux;
        out[idx] = (ix < in_x && iy < in_y) ? in[(pl * in_y + iy) * in_x + ix] : 0.f;
    }
}

__global__ void downsample_kernel(float *__restrict__ out, const float *__restrict__ in, size_t planes, int in_y, int in_x,
                                  int out_y, int out_x, int dsx, int dsy)
{
    grid_dependency_wait();
    const size_t total = planes * out_y * out_x;
    const float div = (float)(dsx * dsy);
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        int x = idx % out_x;
        size_t t = idx / out_x;
        int y = t % out_y;
        size_t pl = t / out_y;
        float s = 0.f;
        for (int dx = 0; dx < dsx; dx++) {
            int xp = x * dsx + dx;
            if (xp >= in_x) continue;
            for (int dy = 0; dy < dsy; dy++) {
                int yp = y * dsy + dy;
                if (yp >= in_y) continue;
                s = __fadd_rn(s, in[(pl * in_y + yp) * in_x + xp]);
            }
        }
        out[idx] = __fdiv_rn(s, div);
    }
}

// ---------------------------------------------------------------------------------------------
// fused batch-norm (statistics per element over W).  One thread per (z,y,x) element; the W column is
// walked three times (mean, variance, normalise) and stays in L1/L2 between the passes, so HBM sees
// one read of x and one write each of y and xhat.  Arithmetic follows the reference sequence.
// ---------------------------------------------------------------------------------------------
__global__ void bn_forward_kernel(float *__restrict__ y, float *__restrict__ xhat, float *__restrict__ ivar,
                                  float *__restrict__ mean, float *__restrict__ var, float *new_mean, float *new_var,
                                  const float *__restrict__ x, const float *__restrict__ gamma, const float *__restrict__ beta,
                                  int W, size_t n, float momentum, float eps)
{
    grid_dependency_wait();
    const float invN = (float)(1.0 / (double)(float)W);
    const float om = (float)(1.0 - (double)momentum);
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        float s = 0.f;
        for (int w = 0; w < W; w++) s = __fadd_rn(s, x[(size_t)w * n + i]);
        float mu = __fadd_rn(0.f, __fmul_rn(s, invN));
        float q = 0.f;
        for (int w = 0; w < W; w++) {
            float d = __fsub_rn(x[(size_t)w * n + i], mu);
            q = __fadd_rn(q, __fmul_rn(__fmul_rn(d, d), 1.0f));
        }
        float vr = __fadd_rn(0.f, __fmul_rn(q, invN));
        float iv = __fdiv_rn(1.0f, __fmul_rn(__fsqrt_rn(__fadd_rn(vr, eps)), 1.0f));
        mean[i] = mu; var[i] = vr; ivar[i] = iv;
        if (new_mean) new_mean[i] = __fadd_rn(__fmul_rn(momentum, new_mean[i]), __fmul_rn(om, mu));
        if (new_var) new_var[i] = __fadd_rn(__fmul_rn(momentum, new_var[i]), __fmul_rn(om, vr));
        float g = gamma[i], b = beta[i];
        for (int w = 0; w < W; w++) {
            float h = __fmul_rn(__fsub_rn(x[(size_t)w * n + i], mu), iv);
            xhat[(size_t)w * n + i] = h;
            y[(size_t)w * n + i] = __fadd_rn(__fmul_rn(g, h), b);
        }
    }
}

// The same arithmetic with the W column of an element held in registers (W <= WMAX): every load of a pass is independent
// of the others and x is read from HBM exactly once, whatever the tensor's size relative to L2.
template <int WMAX>
__global__ void __launch_bounds__(128) bn_forward_reg_kernel(float *__restrict__ y, float *__restrict__ xhat, float *__restrict__ ivar,
                                      float *__restrict__ mean, float *__restrict__ var, float *new_mean, float *new_var,
                                      const float *__restrict__ x, const float *__restrict__ gamma, const float *__restrict__ beta,
                                      int W, size_t n, float momentum, float eps)
{
    grid_dependency_wait();
    const float invN = (float)(1.0 / (double)(float)W);
    const float om = (float)(1.0 - (double)momentum);
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        float v[WMAX];
#pragma unroll
        for (int w = 0; w < WMAX; w++) v[w] = w < W ? x[(size_t)w * n + i] : 0.f;
        float s = 0.f;
#pragma unroll
        for (int w = 0; w < WMAX; w++) if (w < W) s = __fadd_rn(s, v[w]);
        const float mu = __fadd_rn(0.f, __fmul_rn(s, invN));
        float q = 0.f;
#pragma unroll
        for (int w = 0; w < WMAX; w++) if (w < W) {
            const float d = __fsub_rn(v[w], mu);
            q = __fadd_rn(q, __fmul_rn(__fmul_rn(d, d), 1.0f));
        }
        const float vr = __fadd_rn(0.f, __fmul_rn(q, invN));
        const float iv = __fdiv_rn(1.0f, __fmul_rn(__fsqrt_rn(__fadd_rn(vr, eps)), 1.0f));
        mean[i] = mu; var[i] = vr; ivar[i] = iv;
        if (new_mean) new_mean[i] = __fadd_rn(__fmul_rn(momentum, new_mean[i]), __fmul_rn(om, mu));
        if (new_var) new_var[i] = __fadd_rn(__fmul_rn(momentum, new_var[i]), __fmul_rn(om, vr));
        const float g = gamma[i], b = beta[i];
#pragma unroll
        for (int w = 0; w < WMAX; w++) if (w < W) {
            const float h = __fmul_rn(__fsub_rn(v[w], mu), iv);
            xhat[(size_t)w * n + i] = h;
            y[(size_t)w * n + i] = __fadd_rn(__fmul_rn(g, h), b);
        }
    }
}

template <int WMAX>
__global__ void __launch_bounds__(128) bn_backward_reg_kernel(float *dx, float *dgamma, float *dbeta, const float *dy,   // dy may be dx
                                       const float *__restrict__ xhat, const float *__restrict__ ivar, const float *__restrict__ gamma,
                                       int W, size_t n, int create_delta_weight)
{
    grid_dependency_wait();
    const float N = (float)W;
    const float invN = (float)(1.0 / (double)N);
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        float d[WMAX], h[WMAX];
#pragma unroll
        for (int w = 0; w < WMAX; w++) {
            d[w] = w < W ? dy[(size_t)w * n + i] : 0.f;
            h[w] = w < W ? xhat[(size_t)w * n + i] : 0.f;
        }
        const float g = gamma[i], iv = ivar[i];
        float sb = 0.f, sc = 0.f, sg = 0.f, sbeta = 0.f;
#pragma unroll
        for (int w = 0; w < WMAX; w++) if (w < W) {
            const float dh = __fmul_rn(d[w], g);
            sb = __fadd_rn(sb, dh);
            sc = __fadd_rn(sc, __fmul_rn(dh, h[w]));
            sg = __fadd_rn(sg, __fmul_rn(d[w], h[w]));
            sbeta = __fadd_rn(sbeta, d[w]);
        }
        if (create_delta_weight) {
            dgamma[i] = __fadd_rn(dgamma[i], sg);
            dbeta[i] = __fadd_rn(dbeta[i], sbeta);
        }
#pragma unroll
        for (int w = 0; w < WMAX; w++) if (w < W) {
            float v = __fmul_rn(__fmul_rn(d[w], g), N);
            v = __fsub_rn(v, __fmul_rn(h[w], sc));
            v = __fsub_rn(v, sb);
            v = __fmul_rn(v, iv);
            dx[(size_t)w * n + i] = __fmul_rn(v, invN);
        }
    }
}

// ---- batch-norm with the W column block staged in shared memory by bulk copies ---------------------------------------
// One block of TW threads per tile of TW consecutive elements x all W samples.  Thread 0 issues one cp.async.bulk per batch
// row (TW*4 bytes; all rows of the tile in flight at once) and the block waits on one mbarrier.  Each thread then walks its
// own column in shared memory in the reference's order (bit-identical results) and stores coalesced rows.  Several blocks
// are resident per SM, so the loads of one overlap the arithmetic and stores of the others (measured: better than
// persistent double-buffered blocks, which leave too few threads per SM for the dependent additions of a column).
// Needs n % 4 == 0 (16-byte aligned rows).  The wait is bounded; on a time-out the block reports through the status word
// and returns.
__device__ __forceinline__ void bulk_load_row(uint32_t dst, const float *src, uint32_t bytes, uint32_t bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

__device__ __forceinline__ bool bounded_wait(uint32_t bar, uint32_t parity, unsigned *status)
{
    const long long t0 = clock64();
    while (!ptx::mbar_try_wait(bar, parity)) {
        if (clock64() - t0 > 2000000000LL) {
            atomicExch(status, 0x500u + B200_E_TIMEOUT);
            __threadfence_system();
            return false;
        }
    }
    return true;
}

// rows of `arrays` tensors (1 or 2) for the tile starting at element i0 into one stage buffer [array][W][TW]
template <int TW>
__device__ __forceinline__ void bn_issue_tile(float *buf, uint32_t bar, const float *a0, const float *a1, int arrays, int W, size_t n, size_t i0)
{
    const uint32_t cols = (uint32_t)min((size_t)TW, n - i0);
    ptx::mbar_arrive_expect_tx(bar, (uint32_t)arrays * (uint32_t)W * cols * 4u);
    for (int w = 0; w < W; w++) {
        bulk_load_row(ptx::smem_u32(buf + (size_t)w * TW), a0 + (size_t)w * n + i0, cols * 4u, bar);
        if (arrays == 2) bulk_load_row(ptx::smem_u32(buf + (size_t)(W + w) * TW), a1 + (size_t)w * n + i0, cols * 4u, bar);
    }
}

template <int TW>
__global__ void __launch_bounds__(TW) bn_forward_smem_kernel(float *__restrict__ y, float *__restrict__ xhat, float *__restrict__ ivar,
                                      float *__restrict__ mean, float *__restrict__ var, float *new_mean, float *new_var,
                                      const float *__restrict__ x, const float *__restrict__ gamma, const float *__restrict__ beta,
                                      int W, size_t n, float momentum, float eps, unsigned *status, int func, double slope)
{
    grid_dependency_wait();
    // func >= 0: the activation of the function layer that follows is applied to the output (y = f(gamma*xhat + beta))
    extern __shared__ __align__(128) float xs[];          // [W][TW]
    __shared__ __align__(8) unsigned long long bar_storage;
    const uint32_t bar0 = ptx::smem_u32(&bar_storage);
    const int t = threadIdx.x;
    const size_t tile = blockIdx.x;
    if (t == 0) {
        ptx::mbar_init(bar0, 1);
        ptx::fence_barrier_init();
        bn_issue_tile<TW>(xs, bar0, x, nullptr, 1, W, n, tile * TW);
    }
    __syncthreads();
    const float invN = (float)(1.0 / (double)(float)W);
    const float om = (float)(1.0 - (double)momentum);
    {
        if (!bounded_wait(bar0, 0, status)) return;
        const float *col = xs + t;
        const size_t i = tile * TW + t;
        if (i < n) {
            float s = 0.f;
            for (int w = 0; w < W; w++) s = __fadd_rn(s, col[w * TW]);
            const float mu = __fadd_rn(0.f, __fmul_rn(s, invN));
            float q = 0.f;
            for (int w = 0; w < W; w++) {
                const float d = __fsub_rn(col[w * TW], mu);
                q = __fadd_rn(q, __fmul_rn(__fmul_rn(d, d), 1.0f));
            }
            const float vr = __fadd_rn(0.f, __fmul_rn(q, invN));
            const float iv = __fdiv_rn(1.0f, __fmul_rn(__fsqrt_rn(__fadd_rn(vr, eps)), 1.0f));
            mean[i] = mu; var[i] = vr; ivar[i] = iv;
            if (new_mean) new_mean[i] = __fadd_rn(__fmul_rn(momentum, new_mean[i]), __fmul_rn(om, mu));
            if (new_var) new_var[i] = __fadd_rn(__fmul_rn(momentum, new_var[i]), __fmul_rn(om, vr));
            const float g = gamma[i], b = beta[i];
#pragma unroll 8
            for (int w = 0; w < W; w++) {
                const float h = __fmul_rn(__fsub_rn(col[w * TW], mu), iv);
                xhat[(size_t)w * n + i] = h;
                const float o = __fadd_rn(__fmul_rn(g, h), b);
                y[(size_t)w * n + i] = func < 0 ? o : act_apply(o, func, slope);
            }
        }
    }
}

// Two threads per element (2*TW threads per block): the four sums of the first pass are independent chains, so one thread of
// the pair forms sum(dxhat) and sum(dxhat*xhat), the other the two weight gradients; the second pass is split by even/odd
// sample.  Every chain keeps the reference's order of additions.
template <int TW>
__global__ void __launch_bounds__(2 * TW) bn_backward_smem_kernel(float *__restrict__ dx, float *dgamma, float *dbeta, const float *__restrict__ dy,
                                       const float *__restrict__ xhat, const float *__restrict__ ivar, const float *__restrict__ gamma,
                                       int W, size_t n, int create_delta_weight, unsigned *status, const float *__restrict__ beta, int func,
                                       double slope)
{
    grid_dependency_wait();
    // func >= 0: dy is the error above the function layer that follows this one; it is first multiplied by f'(gamma*xhat + beta)
    // (the layer's output, recomputed from xhat), which is what that function layer would have handed down
    extern __shared__ __align__(128) float xs[];          // dy rows [W][TW], xhat rows [W][TW]
    __shared__ __align__(8) unsigned long long bar_storage;
    __shared__ float sums[2][TW];
    const uint32_t bar0 = ptx::smem_u32(&bar_storage);
    const int t = threadIdx.x % TW, half = threadIdx.x / TW;
    const size_t tile = blockIdx.x;
    if (threadIdx.x == 0) {
        ptx::mbar_init(bar0, 1);
        ptx::fence_barrier_init();
        bn_issue_tile<TW>(xs, bar0, dy, xhat, 2, W, n, tile * TW);
    }
    __syncthreads();
    const float N = (float)W;
    const float invN = (float)(1.0 / (double)N);
    const bool ok = bounded_wait(bar0, 0, status);
    const float *ds = xs + t, *hs = ds + (size_t)W * TW;
    const size_t i = tile * TW + t;
    const bool live = ok && i < n;
    float g = 0.f, iv = 0.f;
    if (func >= 0) {
        if (live) {
            float *dw = xs + t;
            const float gg = gamma[i], bb = beta[i];
            for (int w = half; w < W; w += 2) {
                const float o = __fadd_rn(__fmul_rn(gg, hs[w * TW]), bb);
                dw[w * TW] = act_derivative(o, func, slope) * dw[w * TW];
            }
        }
        __syncthreads();
    }
    if (live) {
        g = gamma[i]; iv = ivar[i];
        if (half == 0) {
            float sb = 0.f, sc = 0.f;
            for (int w = 0; w < W; w++) {
                const float dh = __fmul_rn(ds[w * TW], g);
                sb = __fadd_rn(sb, dh);
                sc = __fadd_rn(sc, __fmul_rn(dh, hs[w * TW]));
            }
            sums[0][t] = sb; sums[1][t] = sc;
        } else if (create_delta_weight) {
            float sg = 0.f, sbeta = 0.f;
            for (int w = 0; w < W; w++) {
                const float d = ds[w * TW];
                sg = __fadd_rn(sg, __fmul_rn(d, hs[w * TW]));
                sbeta = __fadd_rn(sbeta, d);
            }
            dgamma[i] = __fadd_rn(dgamma[i], sg);
            dbeta[i] = __fadd_rn(dbeta[i], sbeta);
        }
    }
    __syncthreads();
    if (!live) return;
    const float sb = sums[0][t], sc = sums[1][t];
#pragma unroll 8
    for (int w = half; w < W; w += 2) {
        const float d = ds[w * TW], h = hs[w * TW];
        float v = __fmul_rn(__fmul_rn(d, g), N);
        v = __fsub_rn(v, __fmul_rn(h, sc));
        v = __fsub_rn(v, sb);
        v = __fmul_rn(v, iv);
        dx[(size_t)w * n + i] = __fmul_rn(v, invN);
    }
}

__global__ void bn_backward_kernel(float *dx, float *dgamma, float *dbeta, const float *dy,      // dy may be dx (in place)
                                   const float *__restrict__ xhat, const float *__restrict__ ivar, const float *__restrict__ gamma,
                                   int W, size_t n, int create_delta_weight)
{
    grid_dependency_wait();
    const float N = (float)W;
    const float invN = (float)(1.0 / (double)N);
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        float g = gamma[i], iv = ivar[i];
        float sb = 0.f, sc = 0.f, sg = 0.f, sbeta = 0.f;
        for (int w = 0; w < W; w++) {
            float d = dy[(size_t)w * n + i], h = xhat[(size_t)w * n + i];
            float dh = __fmul_rn(d, g);
            sb = __fadd_rn(sb, dh);
            sc = __fadd_rn(sc, __fmul_rn(dh, h));
            sg = __fadd_rn(sg, __fmul_rn(d, h));
            sbeta = __fadd_rn(sbeta, d);
        }
        if (create_delta_weight) {
            dgamma[i] = __fadd_rn(dgamma[i], sg);
            dbeta[i] = __fadd_rn(dbeta[i], sbeta);
        }
        for (int w = 0; w < W; w++) {
            float d = dy[(size_t)w * n + i], h = xhat[(size_t)w * n + i];
            float v = __fmul_rn(__fmul_rn(d, g), N);
            v = __fsub_rn(v, __fmul_rn(h, sc));
            v = __fsub_rn(v, sb);
            v = __fmul_rn(v, iv);
            dx[(size_t)w * n + i] = __fmul_rn(v, invN);
        }
    }
}

// ---------------------------------------------------------------------------------------------
// VAE output layer
// ---------------------------------------------------------------------------------------------
__global__ void vae_forward_kernel(float *__restrict__ z, const float *__restrict__ mu, const float *__restrict__ logvar,
                                   const float *__restrict__ eps, size_t total, float *kl_partial)
{
    grid_dependency_wait();
    __shared__ float part[32];
    float kl = 0.f;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        float lv = logvar[i], m = mu[i];
        lv = fminf(fmaxf(lv, -10.f), 10.f);
        z[i] = m + expf(lv * 0.5f) * eps[i];
        kl += 1.f + lv - m * m - expf(lv);
    }
    kl = warp_sum(kl);
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = kl;
    __syncthreads();
    if (threadIdx.x < 32) {
        float v = threadIdx.x < (blockDim.x >> 5) ? part[threadIdx.x] : 0.f;
        v = warp_sum(v);
        if (threadIdx.x == 0 && kl_partial) kl_partial[blockIdx.x] = v;
    }
}

__global__ void vae_backward_kernel(float *__restrict__ d_mu, float *__restrict__ d_logvar, const float *__restrict__ delta,
                                    const float *__restrict__ mu, const float *__restrict__ logvar, const float *__restrict__ eps,
                                    size_t total, float k)
{
    grid_dependency_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        float lv = logvar[i], d = delta[i];
        d_logvar[i] = d * (0.5f * eps[i] * expf(lv * 0.5f)) - 0.5f * (1.f - expf(lv)) * k;
        d_mu[i] = d + mu[i] * k;
    }
}

// One pass over the parameter arena: 16-byte accesses on the four (five with the moving average) streams; the bias
// corrections 1 - beta^t come from the launch arguments or, when `corrections` is given, from device memory (a launch
// with fixed arguments, replayable from a CUDA graph while the step number advances).
template <bool EMA>
__global__ void __launch_bounds__(256) adam_kernel(float *__restrict__ weight, const float *__restrict__ dweight, float *__restrict__ m,
                                                   float *__restrict__ v, float *__restrict__ ema, size_t n, AdamArgs a,
                                                   const double *__restrict__ corrections, int vec)
{
    grid_dependency_wait();
    if (corrections) { a.inv_c1 = 1.0 / corrections[0]; a.inv_c2 = 1.0 / corrections[1]; }
    const size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x, stride = (size_t)gridDim.x * blockDim.x;
    const size_t n4 = vec ? n / 4 : 0;
    for (size_t i = tid; i < n4; i += stride) {
        float4 w = reinterpret_cast<float4 *>(weight)[i];
        const float4 g = reinterpret_cast<const float4 *>(dweight)[i];
        float4 mm = reinterpret_cast<float4 *>(m)[i], vv = reinterpret_cast<float4 *>(v)[i];
        w.x = adam_element(w.x, g.x, mm.x, vv.x, a); w.y = adam_element(w.y, g.y, mm.y, vv.y, a);
        w.z = adam_element(w.z, g.z, mm.z, vv.z, a); w.w = adam_element(w.w, g.w, mm.w, vv.w, a);
        reinterpret_cast<float4 *>(weight)[i] = w;
        reinterpret_cast<float4 *>(m)[i] = mm;
        reinterpret_cast<float4 *>(v)[i] = vv;
        if (EMA) {
            float4 e = reinterpret_cast<float4 *>(ema)[i];
            e.x = ema_element(e.x, w.x, a); e.y = ema_element(e.y, w.y, a); e.z = ema_element(e.z, w.z, a); e.w = ema_element(e.w, w.w, a);
            reinterpret_cast<float4 *>(ema)[i] = e;
        }
    }
    for (size_t i = n4 * 4 + tid; i < n; i += stride) {
        float mm = m[i], vv = v[i];
        const float w = adam_element(weight[i], dweight[i], mm, vv, a);
        weight[i] = w; m[i] = mm; v[i] = vv;
        if (EMA) ema[i] = ema_element(ema[i], w, a);
    }
}

static int launch_adam(float *weight, const float *dweight, float *m, float *v, float *ema, size_t n, const AdamArgs &a,
                       const double *corrections, cudaStream_t s)
{
    const int vec = aligned16(weight) && aligned16(dweight) && aligned16(m) && aligned16(v) && (!ema || aligned16(ema));
    const int grid = stream_grid(vec ? (n + 3) / 4 : n, 256);
    if (ema) Launch(grid, 256, 0, s)(adam_kernel<true>, weight, dweight, m, v, ema, n, a, corrections, vec);
    else Launch(grid, 256, 0, s)(adam_kernel<false>, weight, dweight, m, v, nullptr, n, a, corrections, vec);
    B200_LAUNCH_CHECK();
    return B200_OK;
}

// ---------------------------------------------------------------------------------------------
// CUDA-core GEMM with W-broadcast (general shapes; k summed in increasing order like the CPU backend)
// ---------------------------------------------------------------------------------------------
__global__ void simt_mul_kernel(float *__restrict__ out, int out_w, const float *__restrict__ left, int left_w,
                                const float *__restrict__ right, int right_w, int Z, int LY, int LX, int RX, int tl)
{
    grid_dependency_wait();
    // tl == 0: out (LY x RX) = left (LY x LX) * right (LX x RX)
    // tl == 1: out (LX x RX) = left^T, left is (LY x LX), right (LY x RX)
    const int OR = tl ? LX : LY, KD = tl ? LY : LX;
    const size_t total = (size_t)out_w * Z * OR * RX;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        int x = idx % RX;
        size_t t = idx / RX;
        int y = t % OR; t /= OR;
        int z = t % Z;
        int w = t / Z;
        const float *lb = left + ((size_t)(w % left_w) * Z + z) * LY * LX;
        const float *rb = right + ((size_t)(w % right_w) * Z + z) * (size_t)KD * RX;
        float acc = 0.f;
        if (!tl) for (int k = 0; k < KD; k++) acc = __fadd_rn(acc, __fmul_rn(lb[(size_t)y * LX + k], rb[(size_t)k * RX + x]));
        else     for (int k = 0; k < KD; k++) acc = __fadd_rn(acc, __fmul_rn(lb[(size_t)k * LX + y], rb[(size_t)k * RX + x]));
        out[idx] = acc;
    }
}

// Matrix-times-column products (RX == 1, not transposed: out[w,z,y] = <row y of left, right>), one warp per output
// element: both operands are contiguous along the contraction, the lanes stride over it with 16-byte loads and combine
// with a shuffle tree.  The order of the additions differs from the CPU backend's, so the bit-exact FP32 mode does
// not use it; it serves the tensor-core modes when a product has too few outputs for a tensor-core tile (a Linear
// layer with a handful of neurons).
__global__ void warp_dot_kernel(float *__restrict__ out, int out_w, const float *__restrict__ left, int left_w,
                                const float *__restrict__ right, int right_w, int Z, int LY, int LX)
{
    grid_dependency_wait();
    const int lane = threadIdx.x & 31;
    const size_t warps = ((size_t)gridDim.x * blockDim.x) >> 5;
    const size_t total = (size_t)out_w * Z * LY;
    const bool vec = (LX % 4 == 0) && ((((uintptr_t)left) | ((uintptr_t)right)) % 16 == 0);
    for (size_t idx = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; idx < total; idx += warps) {
        const int y = idx % LY;
        size_t t = idx / LY;
        const int z = t % Z;
        const int w = t / Z;
        const float *a = left + (((size_t)(w % left_w) * Z + z) * LY + y) * LX;
        const float *b = right + ((size_t)(w % right_w) * Z + z) * LX;
        float acc = 0.f;
        if (vec) {
            const float4 *a4 = reinterpret_cast<const float4 *>(a), *b4 = reinterpret_cast<const float4 *>(b);
            for (int k = lane; k < LX / 4; k += 32) {
                const float4 u = a4[k], v = b4[k];
                acc += u.x * v.x + u.y * v.y + u.z * v.z + u.w * v.w;
            }
        } else {
            for (int k = lane; k < LX; k += 32) acc += a[k] * b[k];
        }
        acc = warp_sum(acc);
        if (lane == 0) out[idx] = acc;
    }
}

// The same product with one BLOCK per output element: for a handful of long dot products (the discriminator's last layer:
// 64 outputs of 8192 terms) one warp per output leaves the GPU idle and walks each row in 64 dependent steps.
__global__ void __launch_bounds__(256) block_dot_kernel(float *__restrict__ out, int out_w, const float *__restrict__ left, int left_w,
                                                        const float *__restrict__ right, int right_w, int Z, int LY, int LX)
{
    grid_dependency_wait();
    __shared__ float part[8];
    const size_t idx = blockIdx.x;
    const int y = idx % LY;
    const size_t t = idx / LY;
    const int z = t % Z;
    const int w = t / Z;
    const float *a = left + (((size_t)(w % left_w) * Z + z) * LY + y) * LX;
    const float *b = right + ((size_t)(w % right_w) * Z + z) * LX;
    float acc = 0.f;
    if ((LX % 4 == 0) && ((((uintptr_t)a) | ((uintptr_t)b)) % 16 == 0)) {
        const float4 *a4 = reinterpret_cast<const float4 *>(a), *b4 = reinterpret_cast<const float4 *>(b);
        for (int k = threadIdx.x; k < LX / 4; k += 256) {
            const float4 u = a4[k], v = b4[k];
            acc += u.x * v.x + u.y * v.y + u.z * v.z + u.w * v.w;
        }
    } else {
        for (int k = threadIdx.x; k < LX; k += 256) acc += a[k] * b[k];
    }
    acc = warp_sum(acc);
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
        float s = part[0];
        for (int i = 1; i < 8; i++) s += part[i];
        out[idx] = s;
    }
}

int warp_dot_mul(float *out, int out_w, const float *left, int left_w, const float *right, int right_w, int z, int ly, int lx,
                 cudaStream_t s)
{
    const size_t total = (size_t)out_w * z * ly;
    if (!total) return B200_OK;
    if (total <= (size_t)sm_count() * 8 && lx >= 1024) {
        Launch((unsigned)total, 256, 0, s)(block_dot_kernel, out, out_w, left, left_w, right, right_w, z, ly, lx);
        B200_LAUNCH_CHECK();
        return B200_OK;
    }
    Launch(stream_grid(total * 32, 256), 256, 0, s)(warp_dot_kernel, out, out_w, left, left_w, right, right_w, z, ly, lx);
    B200_LAUNCH_CHECK();
    return B200_OK;
}

int simt_mul(float *out, int out_w, const float *left, int left_w, const float *right, int right_w,
             int z, int ly, int lx, int rx, int transpose_left, cudaStream_t s)
{
    size_t total = (size_t)out_w * z * (transpose_left ? lx : ly) * rx;
    if (!total) return B200_OK;
    Launch(stream_grid(total, 256), 256, 0, s)(simt_mul_kernel, out, out_w, left, left_w, right, right_w, z, ly, lx, rx, transpose_left);
    B200_LAUNCH_CHECK();
    return B200_OK;
}

}  // namespace b200

using namespace b200;

#define ST(s) ((cudaStream_t)(s))

extern "C" {

int b200_add(float *out, int out_w, const float *left, int left_w, const float *right, int right_w,
             size_t n, float ls, float rs, int subtract, void *stream)
{
    if (subtract) return launch_binary(out, out_w, left, left_w, right, right_w, n, OpSub{ls, rs}, ST(stream));
    return launch_binary(out, out_w, left, left_w, right, right_w, n, OpAdd{ls, rs}, ST(stream));
}

int b200_div(float *out, int out_w, const float *left, int left_w, const float *right, int right_w,
             size_t n, float ls, float rs, void *stream)
{
    return launch_binary(out, out_w, left, left_w, right, right_w, n, OpDiv{ls, rs}, ST(stream));
}

// out[w][z] = a[w % aw][z] for z < za, b[w % bw][z - za] otherwise (split == 0), or the reverse copy: the first za planes
// of in[w] go to a[w], the rest to b[w] (split != 0).  yx = Y*X elements per plane.
__global__ void concat_split_z_kernel(float *cat, int cat_w, float *a, int aw, int za, float *b, int bw, int zb, size_t yx, int split)
{
    grid_dependency_wait();
    const int z_all = za + zb;
    const size_t total = (size_t)cat_w * z_all * yx;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        const size_t e = idx % yx;
        const size_t plane = idx / yx;
        const int z = (int)(plane % z_all);
        const int w = (int)(plane / z_all);
        float *part = z < za ? a + ((size_t)(w % aw) * za + z) * yx + e : b + ((size_t)(w % bw) * zb + (z - za)) * yx + e;
        if (split) *part = cat[idx]; else cat[idx] = *part;
    }
}

int b200_concat_z(float *out, int out_w, const float *a, int a_w, int a_z, const float *b, int b_w, int b_z, size_t yx, void *stream)
{
    if (!out || !a || !b) return fail(B200_E_ARG, "null tensor pointer");
    if (out_w <= 0 || a_w <= 0 || b_w <= 0 || a_z <= 0 || b_z <= 0) return fail(B200_E_SHAPE, "non-positive size");
    const size_t total = (size_t)out_w * (a_z + b_z) * yx;
    if (!total) return B200_OK;
    Launch(stream_grid(total, 256), 256, 0, ST(stream))(concat_split_z_kernel, out, out_w, const_cast<float *>(a), a_w, a_z, const_cast<float *>(b), b_w, b_z, yx, 0);
    B200_LAUNCH_CHECK();
    return B200_OK;
}

int b200_split_z(float *out_a, int a_z, float *out_b, int b_z, const float *in, int w, size_t yx, void *stream)
{
    if (!out_a || !out_b || !in) return fail(B200_E_ARG, "null tensor pointer");
    if (w <= 0 || a_z <= 0 || b_z <= 0) return fail(B200_E_SHAPE, "non-positive size");
    const size_t total = (size_t)w * (a_z + b_z) * yx;
    if (!total) return B200_OK;
    Launch(stream_grid(total, 256), 256, 0, ST(stream))(concat_split_z_kernel, const_cast<float *>(in), w, out_a, w, a_z, out_b, w, b_z, yx, 1);
    B200_LAUNCH_CHECK();
    return B200_OK;
}

int b200_transpose(float *out, const float *in, int planes, int rows, int cols, void *stream)
{
    if (!out || !in) return fail(B200_E_ARG, "null tensor pointer");
    if (planes <= 0 || rows <= 0 || cols <= 0) return fail(B200_E_SHAPE, "non-positive matrix size");
    if (planes > 65535) return fail(B200_E_SHAPE, "too many planes for one transpose call");
    dim3 grid((cols + 31) / 32, (rows + 31) / 32, planes), block(32, 8);
    Launch(grid, block, 0, ST(stream))(transpose_kernel, out, in, rows, cols);
    B200_LAUNCH_CHECK();
    return B200_OK;
}

int b200_item_product(float *out, int out_w, const float *left, int left_w, const float *right, int right_w,
                      size_t n, void *stream)
{
    return launch_binary(out, out_w, left, left_w, right, right_w, n, OpMul{}, ST(stream));
}

int b200_add_sum_w(float *out, int out_w, const float *left, int left_w, const float *right, int right_w,
                   size_t n, float ls, float rs, void *stream)
{
    if (!out || !left || !right) return fail(B200_E_ARG, "null tensor pointer");
    if (out_w <= 0 || left_w <= 0 || right_w <= 0) return fail(B200_E_SHAPE, "non-positive W count");
    if (!n) return B200_OK;
    Launch(stream_grid(n, 128), 128, 0, ST(stream))(add_sum_w_kernel, out, out_w, left, left_w, right, right_w, n, ls, rs);
    B200_LAUNCH_CHECK();
    return B200_OK;
}

static int bias_act_launch(float *t, float *pre, int t_w, int z, size_t yx, const float *bias, int bias_w, int func,
                           double leaky_slope, cudaStream_t s)
{
    if (!t || !bias) return fail(B200_E_ARG, "null tensor pointer");
    if (t_w <= 0 || z <= 0 || bias_w <= 0) return fail(B200_E_SHAPE, "non-positive size");
    if (func < 0 || func > 5) return fail(B200_E_ARG, "unknown activation %d", func);
    if (!yx) return B200_OK;
    bool vec = (yx % 4 == 0) && aligned16(t) && (!pre || aligned16(pre));
    size_t total = (vec ? yx / 4 : yx) * z * t_w;
    if (vec) Launch(stream_grid(total, 256), 256, 0, s)(bias_act_kernel<true>, t, pre, t_w, z, yx, bias, bias_w, func, leaky_slope);
    else Launch(stream_grid(total, 256), 256, 0, s)(bias_act_kernel<false>, t, pre, t_w, z, yx, bias, bias_w, func, leaky_slope);
    B200_LAUNCH_CHECK();
    return B200_OK;
}

int b200_add_bias(float *t, int t_w, int z, size_t yx, const float *bias, int bias_w, void *stream)
{
    return bias_act_launch(t, nullptr, t_w, z, yx, bias, bias_w, B200_ACT_LINEAR, 0.0, ST(stream));
}

int b200_bias_activation(float *t, float *pre, int t_w, int z, size_t yx, const float *bias, int func,
                         double leaky_slope, void *stream)
{
    return bias_act_launch(t, pre, t_w, z, yx, bias, 1, func, leaky_slope, ST(stream));
}

int b200_summ_xy(float *out, int out_w, const float *in, int in_w, int z, size_t yx, void *stream)
{
    if (!out || !in) return fail(B200_E_ARG, "null tensor pointer");
    if (out_w <= 0 || in_w <= 0 || z <= 0) return fail(B200_E_SHAPE, "non-positive size");
    int planes = out_w * z;
    int block = yx >= 4096 ? 256 : (yx >= 512 ? 128 : 32);
    int grid = planes < sm_count() * 16 ? planes : sm_count() * 16;
    Launch(grid, block, 0, ST(stream))(summ_xy_kernel, out, out_w, in, in_w, z, yx);
    B200_LAUNCH_CHECK();
    return B200_OK;
}

int b200_unary(float *out, int out_w, const float *in, int in_w, size_t n, int op, float a, float b, void *stream)
{
    if (!out || !in) return fail(B200_E_ARG, "null tensor pointer");
    if (out_w <= 0 || in_w <= 0 || op < 0 || op > 6) return fail(B200_E_ARG, "bad unary arguments");
    if (!n) return B200_OK;
    Launch(stream_grid(n * out_w, 256), 256, 0, ST(stream))(unary_kernel, out, out_w, in, in_w, n, op, a, b);
    B200_LAUNCH_CHECK();
    return B200_OK;
}

int b200_fill(float *out, size_t n, float value, void *stream)
{
    if (!out) return fail(B200_E_ARG, "null tensor pointer");
    if (!n) return B200_OK;
    Launch(stream_grid(n, 256), 256, 0, ST(stream))(fill_kernel, out, n, value);
    B200_LAUNCH_CHECK();
    return B200_OK;
}

int b200_activation(float *out, const float *in, size_t n, int func, int derivative, double leaky_slope, void *stream)
{
    if (!out || !in) return fail(B200_E_ARG, "null tensor pointer");
    if (func < 0 || func > 5) return fail(B200_E_ARG, "unknown activation %d", func);
    if (!n) return B200_OK;
    launch_activation(out, in, nullptr, n, func, derivative, leaky_slope, ST(stream));
    B200_LAUNCH_CHECK();
    return B200_OK;
}

int b200_activation_backward(float *out, const float *z, const float *error, size_t n, int func, double leaky_slope,
                             void *stream)
{
    if (!out || !z || !error) return fail(B200_E_ARG, "null tensor pointer");
    if (func < 0 || func > 5) return fail(B200_E_ARG, "unknown activation %d", func);
    if (!n) return B200_OK;
    launch_activation(out, z, error, n, func, 1, leaky_slope, ST(stream));
    B200_LAUNCH_CHECK();
    return B200_OK;
}

int b200_maxpool(float *out, uint32_t *pos, const float *in, int w, int z, int in_y, int in_x, int pool_x, int pool_y,
                 void *stream)
{
    if (!out || !pos || !in) return fail(B200_E_ARG, "null tensor pointer");
    if (pool_x <= 0 || pool_y <= 0 || in_y < pool_y || in_x < pool_x) return fail(B200_E_SHAPE, "bad pooling geometry");
    size_t planes = (size_t)w * z;
    size_t total = planes * (in_y / pool_y) * (in_x / pool_x);
    if (!total) return B200_OK;
    // positions are {X, Y} pairs stored with one 8-byte access each
    if ((uintptr_t)pos & 7) return fail(B200_E_ARG, "max-pooling: the position tensor must be 8-byte aligned");
    const int vec2 = pool_x == 2 && pool_y == 2 && in_x % 2 == 0 && ((uintptr_t)in & 7) == 0;
    Launch(stream_grid(total, 256), 256, 0, ST(stream))(maxpool_kernel, out, reinterpret_cast<uint2 *>(pos), in, planes, in_y, in_x, pool_x, pool_y, vec2);
    B200_LAUNCH_CHECK();
    return B200_OK;
}

int b200_maxpool_backward(float *out, const uint32_t *pos, const float *delta, int w, int z, int out_y, int out_x,
                          int pool_x, int pool_y, void *stream)
{
    if (!out || !pos || !delta) return fail(B200_E_ARG, "null tensor pointer");
    if (pool_x <= 0 || pool_y <= 0) return fail(B200_E_SHAPE, "bad pooling geometry");
    size_t planes = (size_t)w * z;
    size_t total = planes * out_y * out_x;
    if (!total) return B200_OK;
    if ((uintptr_t)pos & 7) return fail(B200_E_ARG, "max-pooling: the position tensor must be 8-byte aligned");
    if (pool_x == 2 && pool_y == 2 && out_x % 2 == 0 && out_y % 2 == 0 && ((uintptr_t)out % 8) == 0 && planes * (size_t)(out_y / 2) < 0xFFFFFFFFull)
        Launch(stream_grid(total / 4, 256), 256, 0, ST(stream))(maxpool_backward_2x2_kernel, out, reinterpret_cast<const uint2 *>(pos), delta,
                                                                                       (unsigned)(planes * (out_y / 2)), (unsigned)(out_x / 2));
    else
        Launch(stream_grid(total, 256), 256, 0, ST(stream))(maxpool_backward_kernel, out, reinterpret_cast<const uint2 *>(pos), delta, planes,
                                                                               out_y, out_x, pool_x, pool_y);
    B200_LAUNCH_CHECK();
    return B200_OK;
}

int b200_upsample(float *out, const float *in, int w, int z, int in_y, int in_x, int ux, int uy, void *stream)
{
    if (!out || !in) return fail(B200_E_ARG, "null tensor pointer");
    if (ux <= 0 || uy <= 0) return fail(B200_E_SHAPE, "bad upsampling factor");
    size_t planes = (size_t)w * z;
    size_t total = planes * in_y * uy * in_x * ux;
    if (!total) return B200_OK;
    if (ux == 2 && uy == 2 && ((uintptr_t)out % 8) == 0 && planes * (size_t)in_y < 0xFFFFFFFFull)
        Launch(stream_grid(total / 4, 256), 256, 0, ST(stream))(upsample_2x2_kernel, out, in, (unsigned)(planes * in_y), (unsigned)in_x);
    else
        Launch(stream_grid(total, 256), 256, 0, ST(stream))(upsample_kernel, out, in, planes, in_y, in_x, in_y * uy, in_x * ux, ux, uy);
    B200_LAUNCH_CHECK();
    return B200_OK;
}

int b200_downsample(float *out, const float *in, int w, int z, int in_y, int in_x, int dx, int dy, void *stream)
{
    if (!out || !in) return fail(B200_E_ARG, "null tensor pointer");
    if (dx <= 0 || dy <= 0) return fail(B200_E_SHAPE, "bad downsampling factor");
    size_t planes = (size_t)w * z;
    size_t total = planes * (in_y / dy) * (in_x / dx);
    if (!total) return B200_OK;
    if (dx == 2 && dy == 2 && in_x % 2 == 0 && in_y % 2 == 0 && ((uintptr_t)in % 8) == 0 && planes * (size_t)(in_y / 2) < 0xFFFFFFFFull)
        Launch(stream_grid(total, 256), 256, 0, ST(stream))(downsample_2x2_kernel, out, in, (unsigned)(planes * (in_y / 2)), (unsigned)(in_x / 2));
    else
        Launch(stream_grid(total, 256), 256, 0, ST(stream))(downsample_kernel, out, in, planes, in_y, in_x, in_y / dy, in_x / dx, dx, dy);
    B200_LAUNCH_CHECK();
    return B200_OK;
}

static int bn_forward_impl(float *y, float *xhat, float *ivar, float *mean, float *var, float *new_mean, float *new_var,
                           const float *x, const float *gamma, const float *beta, int w, size_t n, float momentum, float eps,
                           int func, double leaky_slope, void *stream)
{
    if (!y || !xhat || !ivar || !mean || !var || !x || !gamma || !beta) return fail(B200_E_ARG, "null tensor pointer");
    if (w <= 0) return fail(B200_E_SHAPE, "non-positive batch");
    if (!n) return B200_OK;
    {
        // staged through shared memory when the rows are 16-byte aligned and the column block fits
        const size_t smem = (size_t)w * 128 * sizeof(float);
        if (n % 4 == 0 && aligned16(x) && w >= 8 && smem <= 200 * 1024) {
            unsigned *status = nullptr;
            int r = status_word(&status);
            if (r) return r;
            B200_CUDA(cudaFuncSetAttribute(bn_forward_smem_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            Launch((unsigned)((n + 127) / 128), 128, smem, ST(stream))(bn_forward_smem_kernel<128>, 
                y, xhat, ivar, mean, var, new_mean, new_var, x, gamma, beta, w, n, momentum, eps, status, func, leaky_slope);
            B200_LAUNCH_CHECK();
            return B200_OK;
        }
    }
#define B200_BN_FWD(WMAX) Launch(stream_grid(n, 128), 128, 0, ST(stream))(bn_forward_reg_kernel<WMAX>, y, xhat, ivar, mean, var, new_mean, new_var, x, gamma, beta, w, n, momentum, eps)
    if (w <= 16) B200_BN_FWD(16);
    else if (w <= 32) B200_BN_FWD(32);
    else if (w <= 64) B200_BN_FWD(64);
    else if (w <= 128) B200_BN_FWD(128);
    else Launch(stream_grid(n, 128), 128, 0, ST(stream))(bn_forward_kernel, y, xhat, ivar, mean, var, new_mean, new_var, x, gamma, beta,
                                                                       w, n, momentum, eps);
#undef B200_BN_FWD
    B200_LAUNCH_CHECK();
    // the general kernels leave the plain output; the function layer's activation follows as its own pass
    if (func >= 0) launch_activation(y, y, nullptr, (size_t)w * n, func, 0, leaky_slope, ST(stream));
    return B200_OK;
}

int b200_bn_forward(float *y, float *xhat, float *ivar, float *mean, float *var, float *new_mean, float *new_var,
                    const float *x, const float *gamma, const float *beta, int w, size_t n, float momentum, float eps,
                    void *stream)
{
    return bn_forward_impl(y, xhat, ivar, mean, var, new_mean, new_var, x, gamma, beta, w, n, momentum, eps, -1, 0.0, stream);
}

int b200_bn_act_forward(float *out, float *xhat, float *ivar, float *mean, float *var, float *new_mean, float *new_var,
                        const float *x, const float *gamma, const float *beta, int w, size_t n, float momentum, float eps,
                        int func, double leaky_slope, void *stream)
{
    if (func < 0 || func > 5) return fail(B200_E_ARG, "unknown activation %d", func);
    return bn_forward_impl(out, xhat, ivar, mean, var, new_mean, new_var, x, gamma, beta, w, n, momentum, eps, func, leaky_slope, stream);
}

// dx[w][i] = f'(gamma[i]*xhat[w][i] + beta[i]) * error[w][i]: what the function layer above would hand down
__global__ void bn_act_delta_kernel(float *dx, const float *error, const float *__restrict__ xhat, const float *__restrict__ gamma,
                                    const float *__restrict__ beta, size_t total, size_t n, int func, double slope)
{
    grid_dependency_wait();
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        const size_t i = idx % n;
        const float o = __fadd_rn(__fmul_rn(gamma[i], xhat[idx]), beta[i]);
        dx[idx] = act_derivative(o, func, slope) * error[idx];
    }
}

static int bn_backward_impl(float *dx, float *dgamma, float *dbeta, const float *dy, const float *xhat, const float *ivar,
                            const float *gamma, int w, size_t n, int create_delta_weight, const float *beta, int func, double leaky_slope,
                            void *stream)
{
    if (!dx || !dy || !xhat || !ivar || !gamma) return fail(B200_E_ARG, "null tensor pointer");
    if (create_delta_weight && (!dgamma || !dbeta)) return fail(B200_E_ARG, "null gradient pointer");
    if (w <= 0) return fail(B200_E_SHAPE, "non-positive batch");
    if (!n) return B200_OK;
    {
        // 64-element tiles here: two tensors are staged, and six blocks per SM stay resident at batch 64
        const size_t smem = 2 * (size_t)w * 64 * sizeof(float);
        if (n % 4 == 0 && aligned16(dy) && aligned16(xhat) && w >= 8 && smem <= 200 * 1024) {
            unsigned *status = nullptr;
            int r = status_word(&status);
            if (r) return r;
            B200_CUDA(cudaFuncSetAttribute(bn_backward_smem_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            Launch((unsigned)((n + 63) / 64), 128, smem, ST(stream))(bn_backward_smem_kernel<64>, 
                dx, dgamma, dbeta, dy, xhat, ivar, gamma, w, n, create_delta_weight, status, beta, func, leaky_slope);
            B200_LAUNCH_CHECK();
            return B200_OK;
        }
    }
    if (func >= 0) {
        // general kernels: the error is first turned into the function layer's delta, in place in dx
        Launch(stream_grid((size_t)w * n, 256), 256, 0, ST(stream))(bn_act_delta_kernel, dx, dy, xhat, gamma, beta, (size_t)w * n, n, func, leaky_slope);
        B200_LAUNCH_CHECK();
        dy = dx;
    }
#define B200_BN_BWD(WMAX) Launch(stream_grid(n, 128), 128, 0, ST(stream))(bn_backward_reg_kernel<WMAX>, dx, dgamma, dbeta, dy, xhat, ivar, gamma, w, n, create_delta_weight)
    if (w <= 16) B200_BN_BWD(16);
    else if (w <= 32) B200_BN_BWD(32);
    else if (w <= 64) B200_BN_BWD(64);
    else Launch(stream_grid(n, 128), 128, 0, ST(stream))(bn_backward_kernel, dx, dgamma, dbeta, dy, xhat, ivar, gamma, w, n, create_delta_weight);
#undef B200_BN_BWD
    B200_LAUNCH_CHECK();
    return B200_OK;
}

int b200_bn_backward(float *dx, float *dgamma, float *dbeta, const float *dy, const float *xhat, const float *ivar,
                     const float *gamma, int w, size_t n, int create_delta_weight, void *stream)
{
    return bn_backward_impl(dx, dgamma, dbeta, dy, xhat, ivar, gamma, w, n, create_delta_weight, nullptr, -1, 0.0, stream);
}

int b200_bn_act_backward(float *dx, float *dgamma, float *dbeta, const float *error, const float *xhat, const float *ivar,
                         const float *gamma, const float *beta, int w, size_t n, int create_delta_weight, int func, double leaky_slope,
                         void *stream)
{
    if (func < 0 || func > 5) return fail(B200_E_ARG, "unknown activation %d", func);
    if (!beta) return fail(B200_E_ARG, "null tensor pointer");
    return bn_backward_impl(dx, dgamma, dbeta, error, xhat, ivar, gamma, w, n, create_delta_weight, beta, func, leaky_slope, stream);
}

int b200_vae_forward(float *z, const float *mu, const float *logvar, const float *eps, int batch, size_t n,
                     float *kl_host, void *stream)
{
    if (!z || !mu || !logvar || !eps) return fail(B200_E_ARG, "null tensor pointer");
    if (batch <= 0) return fail(B200_E_SHAPE, "non-positive batch");
    size_t total = (size_t)batch * n;
    if (!total) return B200_OK;
    int grid = stream_grid(total, 256);
    float *partial = nullptr;
    if (kl_host) {
        int r = arena_reserve(sizeof(float) * grid, ST(stream));
        if (r) return r;
        arena_reset();
        partial = (float *)arena_take(sizeof(float) * grid);
    }
    Launch(grid, 256, 0, ST(stream))(vae_forward_kernel, z, mu, logvar, eps, total, partial);
    B200_LAUNCH_CHECK();
    if (kl_host) {
        float *h = (float *)malloc(sizeof(float) * grid);
        if (!h) return fail(B200_E_NOMEM, "host allocation failed");
        cudaError_t e = cudaMemcpyAsync(h, partial, sizeof(float) * grid, cudaMemcpyDeviceToHost, ST(stream));
        if (e == cudaSuccess) e = cudaStreamSynchronize(ST(stream));
        if (e != cudaSuccess) { free(h); return fail(B200_E_CUDA, "kl readback failed: %s", cudaGetErrorString(e)); }
        double kl = 0;
        for (int i = 0; i < grid; i++) kl += h[i];
        free(h);
        *kl_host = (float)(-0.5 * kl / batch);
    }
    return B200_OK;
}

int b200_vae_backward(float *d_mu, float *d_logvar, const float *delta, const float *mu, const float *logvar,
                      const float *eps, size_t total, float kl_speed, void *stream)
{
    if (!d_mu || !d_logvar || !delta || !mu || !logvar || !eps) return fail(B200_E_ARG, "null tensor pointer");
    if (!total) return B200_OK;
    Launch(stream_grid(total, 256), 256, 0, ST(stream))(vae_backward_kernel, d_mu, d_logvar, delta, mu, logvar, eps, total, kl_speed);
    B200_LAUNCH_CHECK();
    return B200_OK;
}

int b200_adam(float *weight, const float *dweight, float *m, float *v, size_t n, uint32_t batch_size, double speed,
              double beta1, double beta2, double epsilon, double iteration, void *stream)
{
    return b200_adam_ema(weight, dweight, m, v, nullptr, n, batch_size, speed, beta1, beta2, epsilon, iteration, nullptr, 0.0, stream);
}

int b200_adam_prepared(float *weight, const float *dweight, float *m, float *v, size_t n, uint32_t batch_size, double speed,
                       double beta1, double beta2, double epsilon, const double *corrections, void *stream)
{
    if (!corrections) return fail(B200_E_ARG, "null tensor pointer");
    return b200_adam_ema(weight, dweight, m, v, nullptr, n, batch_size, speed, beta1, beta2, epsilon, 0.0, corrections, 0.0, stream);
}

int b200_adam_ema(float *weight, const float *dweight, float *m, float *v, float *ema, size_t n, uint32_t batch_size, double speed,
                  double beta1, double beta2, double epsilon, double iteration, const double *corrections, double ema_k, void *stream)
{
    if (!weight || !dweight || !m || !v) return fail(B200_E_ARG, "null tensor pointer");
    if (!batch_size) return fail(B200_E_ARG, "batch_size must be positive");
    if (!n) return B200_OK;
    const double c1 = corrections ? 1.0 : 1.0 - pow(beta1, iteration), c2 = corrections ? 1.0 : 1.0 - pow(beta2, iteration);
    if (!corrections && (c1 == 0.0 || c2 == 0.0)) return fail(B200_E_ARG, "Adam: iteration must be positive");
    return launch_adam(weight, dweight, m, v, ema, n, adam_args(batch_size, speed, beta1, beta2, epsilon, c1, c2, ema_k), corrections, ST(stream));
}

}  // extern "C"
