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
// matrix times column (rx == 1, not transposed), one warp per output element; not in the CPU backend's summation order
int warp_dot_mul(float *out, int out_w, const float *left, int left_w, const float *right, int right_w, int z, int ly, int lx,
                 cudaStream_t s);

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

// Packed operands of the tensor-core kernels (tc_conv.cu): a phase-split NHWC copy of an activation
// tensor, TF32-rounded high part `hi` and (3xTF32 only) remainder `lo`.  Buffers hold elems() floats
// plus kPackPad bytes (the blocked tensor maps of MN-major operands may read that far past the end).
struct ActPack {
    float *hi = nullptr, *lo = nullptr;
    int n = 0, c = 0, h = 0, w = 0;          // the source tensor
    int cp = 0, sy = 1, sx = 1, hs = 0, ws = 0;
    size_t elems() const { return (size_t)sy * sx * n * hs * ws * cp; }
};
constexpr size_t kPackPad = 256;
ActPack act_pack_shape(int n, int c, int h, int w, int sy, int sx);
// A neuron function applied while an operand is packed (the function layer in front of a convolution layer): func is a
// B200_ACT_* code; act_out, if not NULL, also receives f(src) in the source layout.
struct PackFunction { int func; double slope; float *act_out; };
// A neuron function applied to out + bias in the epilogue of the convolution (the function layer behind it): pre_out, if not
// NULL, receives the value before the function (what the function layer keeps for its derivative).
struct EpilogueFunction { int func; double slope; float *pre_out; };
int act_pack_fill(const ActPack &pk, const float *src, cudaStream_t s, const PackFunction *pf = nullptr);
// The same pack with the first stage of a bias gradient fused in: rowsum (act_pack_rowsum_elems floats) receives partial
// plane sums [n][c][runs]; *runs == 0 on return means the shape took the scalar pack kernel and no sums were produced.
size_t act_pack_rowsum_elems(const ActPack &pk);
int act_pack_fill_with_sums(const ActPack &pk, const float *src, float *rowsum, int *runs, cudaStream_t s);
int dbias_from_rowsums(float *dbias, int accumulate, const float *rowsum, int batch, int K, int runs, cudaStream_t s);
size_t weight_pack_elems(const b200_conv_geom &g, bool backward);
// The weight packs of several layers in one launch: weight_pack_job fills a job (false: this geometry is packed by the
// per-layer kernels only), weight_pack_fill_many launches them.
struct WeightPackJob {
    const float *src;
    float *f_hi, *f_lo, *b_hi, *b_lo;      // forward and rotated (backward) pack, high / low plane (low NULL in plain TF32)
    int K, C, taps, ip_f, ip_b, n_forward, blocks, block_begin;
};
constexpr int kMaxPackJobs = 16;
struct WeightPackJobs { WeightPackJob job[kMaxPackJobs]; int count; };
bool weight_pack_job(const b200_conv_geom &g, const float *kernel, float *f_hi, float *f_lo, float *b_hi, float *b_lo, WeightPackJob *job);
int weight_pack_fill_many(WeightPackJobs &jobs, cudaStream_t s);
int weight_pack_fill(const b200_conv_geom &g, bool backward, const float *kernel, float *hi, float *lo, cudaStream_t s);
// the forward pack (f_*) and the rotated pack of the backward pass (b_*) in one launch
int weight_pack_fill_both(const b200_conv_geom &g, const float *kernel, float *f_hi, float *f_lo, float *b_hi, float *b_lo, cudaStream_t s);
// kpartial (optional): scratch of conv_gemm_partial_elems() floats that allows splitting the contraction of small layers
size_t conv_gemm_partial_elems(bool backward, const b200_conv_geom &g, int batch);
int conv_gemm(bool backward, const b200_conv_geom &g, float *out, const ActPack &act, const float *w_hi, const float *w_lo,
              const float *bias, bool x3, cudaStream_t s, float *kpartial = nullptr, size_t kpartial_elems = 0, const EpilogueFunction *ef = nullptr);
size_t wgrad_partial_elems(const b200_conv_geom &g, int batch);
int wgrad_gemm(const b200_conv_geom &g, float *dkernel, int accumulate, const ActPack &x, const ActPack &d, float *partial,
               bool x3, cudaStream_t s);
int dbias_batch(float *dbias, int accumulate, const float *delta, int batch, int K, size_t plane, float *db_tmp, cudaStream_t s);

// smallc.cu -- layers with very few channels on one side: the taps are folded into the channel dimension (explicit
// im2col, C' = taps*C) and the contractions run as 1x1 convolutions on the tensor-core kernel
bool smallc_applies(const b200_conv_geom &g);
b200_conv_geom smallc_geom(const b200_conv_geom &g);          // in_z = C', 1x1 kernel on the out_y x out_x plane
int im2col_pack(const b200_conv_geom &g, const ActPack &col, const float *x, int batch, cudaStream_t s);
int smallc_weights(const b200_conv_geom &g, const float *kernel, float *hi, float *lo, int pitch, bool transposed, cudaStream_t s);
int col2im_gather(const b200_conv_geom &g, float *dx, const float *t, int batch, cudaStream_t s);
int smallc_dkernel(const b200_conv_geom &g, float *dkernel, const float *dk, int accumulate, cudaStream_t s);
// layers with few filters: the same problem read backwards has few channels (g is the layer's own geometry in all three)
bool mirror_applies(const b200_conv_geom &g);
b200_conv_geom mirror_geom(const b200_conv_geom &g);
int mirror_weights(const b200_conv_geom &g, float *dst, const float *src, int back, int accumulate, cudaStream_t s);

// Status word written by device-side waits that gave up (0 = none); clear != 0 resets it.
unsigned tc_read_status(int clear);
// host-side write of the status word (what a device-side wait that gave up would have written); for tests of the decoding
void tc_write_status(unsigned code);
// device pointer of the per-device status word (pinned, mapped host memory) that bounded device-side waits report into
int status_word(unsigned **dev);

void tc_profile_enable(int on);
int tc_profile_read(double *total_ms, int *launches);

}  // namespace b200
