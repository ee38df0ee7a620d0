// Internal launcher prototypes shared by the translation units of the library.
#pragma once
#include <cuda_runtime.h>
#include "../../include/b200conv.h"

namespace b200 {

// simt_conv.cu -- CUDA-core fp32 convolution, any geometry, bit-identical to the CPU backend
int simt_conv_forward(const b200_conv_geom &g, float *out, int out_w, const float *image, int image_w,
                      const float *kernel, int kernel_w, const float *bias, int bias_w, cudaStream_t s);
int simt_conv_backward(const b200_conv_geom &g, float *out, int out_w, const float *delta, int delta_w,
                       const float *kernel, int kernel_w, const float *bias, int bias_w, cudaStream_t s);
int simt_conv_wgrad(const b200_conv_geom &g, float *dkernel, int dkernel_w, float *dbias, int dbias_w,
                    const float *image, int image_w, const float *delta, int delta_w, cudaStream_t s);

// simt_math.cu
int simt_mul(float *out, int out_w, const float *left, int left_w, const float *right, int right_w,
             int z, int ly, int lx, int rx, int transpose_left, cudaStream_t s);

// tc_conv.cu -- tcgen05 implicit-GEMM convolution and dense GEMM.  Each returns B200_OK when it ran,
// a negative value (TC_UNSUPPORTED) when the shape is not covered so the caller falls through to the
// CUDA-core kernels, or a positive B200_E_* code on failure.
enum { TC_UNSUPPORTED = -1 };
int tc_conv_forward(const b200_conv_geom &g, float *out, const float *image, const float *kernel, const float *bias,
                    int batch, int precision, cudaStream_t s);
int tc_conv_backward(const b200_conv_geom &g, float *out_delta, const float *delta, const float *kernel, int batch,
                     int precision, cudaStream_t s);
int tc_conv_wgrad_batch(const b200_conv_geom &g, float *dkernel, float *dbias, int accumulate, const float *image,
                        const float *delta, int batch, int precision, cudaStream_t s);
int tc_gemm(float *out, const float *a, const float *b, int m, int n, int k, int a_mn_major, int b_mn_major,
            int precision, cudaStream_t s);

// Status word written by device-side waits that gave up (0 = none); clear != 0 resets it.
unsigned tc_read_status(int clear);

void tc_profile_enable(int on);
int tc_profile_read(double *total_ms, int *launches);

}  // namespace b200
