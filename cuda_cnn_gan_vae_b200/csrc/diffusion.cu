// Helpers of the reference's diffusion model and drop-out layer: the sinusoidal time-step embedding, the forward noising
// step, a normal-noise generator and the drop-out mask.  All are single passes over a tensor (bound: HBM).  The reference
// has these on its CUDA backend only (cuda/ctensormath.cu.h:3029-3291); its random numbers come from cuRAND states seeded
// with rand(), so the streams are not reproducible there either -- here they are a counter-based Philox4x32-10 generator
// (Salmon et al., "Parallel random numbers: as easy as 1, 2, 3", 2011) keyed by a caller-supplied seed: the same seed gives
// the same tensor whatever the launch geometry.
#include "common.cuh"
#include "kernels.h"

namespace b200 {

static inline int grid_for(size_t items)
{
    size_t blocks = (items + 255) / 256, cap = (size_t)sm_count() * 16;
    if (blocks < 1) blocks = 1;
    return (int)(blocks < cap ? blocks : cap);
}

// out[w, pos] = in[w, pos] + (pos even ? sin : cos)(t[w] / 10000^(pos / n)),  pos = linear index inside one sample
__global__ void time_step_kernel(float *__restrict__ out, const float *__restrict__ in, const uint32_t *__restrict__ time_step, int W, size_t n)
{
    grid_dependency_wait();
    const size_t total = (size_t)W * n;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        const size_t w = idx / n;
        const uint32_t pos = (uint32_t)(idx - w * n);
        const float t = (float)time_step[w];
        const float angle = t / powf(10000.0f, (float)pos / (float)(uint32_t)n);
        out[idx] = in[idx] + ((pos & 1u) ? cosf(angle) : sinf(angle));
    }
}

struct Philox { uint32_t c[4]; };

__device__ __forceinline__ Philox philox4x32_10(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3, uint32_t k0, uint32_t k1)
{
#pragma unroll
    for (int r = 0; r < 10; r++) {
        const uint32_t hi0 = __umulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
        const uint32_t hi1 = __umulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
        const uint32_t n0 = hi1 ^ c1 ^ k0, n2 = hi0 ^ c3 ^ k1;
        c0 = n0; c1 = lo1; c2 = n2; c3 = lo0;
        k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
    }
    Philox p;
    p.c[0] = c0; p.c[1] = c1; p.c[2] = c2; p.c[3] = c3;
    return p;
}

// uniform in (0, 1]: never zero, so that its logarithm is finite
__device__ __forceinline__ float u01(uint32_t x) { return ((float)(x >> 8) + 1.0f) * (1.0f / 16777216.0f); }

// Four consecutive elements per counter value.  MODE 0: standard normal numbers (Box-Muller on two pairs of uniforms);
// MODE 1: the same, and noisy = sa[w] * image + so[w] * noise; MODE 2: drop-out mask (0 with probability p, else 1/(1-p)).
template <int MODE>
__global__ void __launch_bounds__(256) random_kernel(float *__restrict__ out, float *__restrict__ noisy, const float *__restrict__ image,
                                                     const float *__restrict__ sa, const float *__restrict__ so, size_t n_per_w, size_t total,
                                                     unsigned long long seed, float p, float keep_scale)
{
    grid_dependency_wait();
    const size_t groups = (total + 3) / 4;
    for (size_t g = (size_t)blockIdx.x * blockDim.x + threadIdx.x; g < groups; g += (size_t)gridDim.x * blockDim.x) {
        const Philox r = philox4x32_10((uint32_t)g, (uint32_t)(g >> 32), 0u, 0u, (uint32_t)seed, (uint32_t)(seed >> 32));
        float v[4];
        if (MODE == 2) {
#pragma unroll
            for (int j = 0; j < 4; j++) v[j] = u01(r.c[j]) > p ? keep_scale : 0.f;
        } else {
#pragma unroll
            for (int j = 0; j < 2; j++) {
                const float radius = sqrtf(-2.0f * logf(u01(r.c[2 * j])));
                float sn, cs;
                sincospif(2.0f * u01(r.c[2 * j + 1]), &sn, &cs);
                v[2 * j] = radius * cs;
                v[2 * j + 1] = radius * sn;
            }
        }
        const size_t base = g * 4;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const size_t i = base + j;
            if (i >= total) break;
            out[i] = v[j];
            if (MODE == 1) {
                const size_t w = i / n_per_w;
                noisy[i] = __fadd_rn(__fmul_rn(sa[w], image[i]), __fmul_rn(so[w], v[j]));
            }
        }
    }
}

__global__ void noisy_image_kernel(float *__restrict__ noisy, const float *__restrict__ image, const float *__restrict__ noise,
                                   const float *__restrict__ sa, const float *__restrict__ so, size_t n_per_w, size_t total)
{
    grid_dependency_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t w = i / n_per_w;
        noisy[i] = __fadd_rn(__fmul_rn(sa[w], image[i]), __fmul_rn(so[w], noise[i]));
    }
}

}  // namespace b200

using namespace b200;
#define ST(s) ((cudaStream_t)(s))

extern "C" {

int b200_set_time_step(float *out, const float *in, const uint32_t *time_step, int w, size_t n, void *stream)
{
    if (!out || !in || !time_step) return fail(B200_E_ARG, "null tensor pointer");
    if (w <= 0 || n > 0xFFFFFFFFull) return fail(B200_E_SHAPE, "CTensor::SetTimeStep: bad sizes");
    if (!n) return B200_OK;
    Launch(grid_for((size_t)w * n), 256, 0, ST(stream))(time_step_kernel, out, in, time_step, w, n);
    B200_LAUNCH_CHECK();
    return B200_OK;
}

int b200_normal_noise(float *out, size_t n, unsigned long long seed, void *stream)
{
    if (!out) return fail(B200_E_ARG, "null tensor pointer");
    if (!n) return B200_OK;
    Launch(grid_for((n + 3) / 4), 256, 0, ST(stream))(random_kernel<0>, out, nullptr, nullptr, nullptr, nullptr, n, n, seed, 0.f, 0.f);
    B200_LAUNCH_CHECK();
    return B200_OK;
}

int b200_dropout_mask(float *out, size_t n, float drop_out, unsigned long long seed, void *stream)
{
    if (!out) return fail(B200_E_ARG, "null tensor pointer");
    if (!(drop_out >= 0.f && drop_out < 1.f)) return fail(B200_E_ARG, "drop-out probability must lie in [0, 1)");
    if (!n) return B200_OK;
    Launch(grid_for((n + 3) / 4), 256, 0, ST(stream))(random_kernel<2>, out, nullptr, nullptr, nullptr, nullptr, n, n, seed, drop_out,
                                                                   (float)(1.0 / (1.0 - drop_out)));
    B200_LAUNCH_CHECK();
    return B200_OK;
}

int b200_noisy_image(float *noisy, float *noise, const float *image, const float *sqrt_alpha_bar, const float *sqrt_one_minus_alpha_bar,
                     int w, size_t n, int generate, unsigned long long seed, void *stream)
{
    if (!noisy || !noise || !image || !sqrt_alpha_bar || !sqrt_one_minus_alpha_bar) return fail(B200_E_ARG, "null tensor pointer");
    if (w <= 0) return fail(B200_E_SHAPE, "CTensor::GetNoiseImageAndNoise: bad sizes");
    const size_t total = (size_t)w * n;
    if (!total) return B200_OK;
    if (generate)
        Launch(grid_for((total + 3) / 4), 256, 0, ST(stream))(random_kernel<1>, noise, noisy, image, sqrt_alpha_bar, sqrt_one_minus_alpha_bar, n, total,
                                                                           seed, 0.f, 0.f);
    else
        Launch(grid_for(total), 256, 0, ST(stream))(noisy_image_kernel, noisy, image, noise, sqrt_alpha_bar, sqrt_one_minus_alpha_bar, n, total);
    B200_LAUNCH_CHECK();
    return B200_OK;
}

}  // extern "C"
