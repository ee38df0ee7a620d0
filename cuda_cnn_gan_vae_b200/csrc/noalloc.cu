// Allocation-free variant of the batch-summed weight gradient.
//
// Who needs it: code that is not allowed to allocate device memory at the point where it calls
// the library -- a host whose device memory is handed out once at start-up by its own pool, a loop
// that must not hit the implicit device synchronisation of cudaMalloc/cudaFree, or a section of a
// program in which the CUDA runtime forbids allocation.  b200_conv_wgrad_batch() grows a scratch
// arena with cudaMalloc when a call needs more than earlier calls did; this entry point never does.
//
// The scratch (one weight gradient and one bias gradient per sample, reduced over the batch at the
// end) lives in the fixed array below, which belongs to the library image: every GPU that loads the
// library holds its 16 MiB until the process exits.  Calls whose scratch would not fit are rejected.
#include "common.cuh"
#include "kernels.h"

namespace b200 {

constexpr size_t kStaticScratchFloats = (size_t)4 << 20;   // 4 Mi floats = 16 MiB per device

static __device__ __align__(256) float g_static_scratch[kStaticScratchFloats];

// In host code `g_static_scratch` is only a handle for the runtime, not a device address; the address
// a kernel may use is looked up once per device, with that device current.
static float *g_static_scratch_addr[64];

static int static_scratch(float **out)
{
    int dev = 0;
    B200_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return fail(B200_E_ARG, "device index %d out of range", dev);
    if (!g_static_scratch_addr[dev]) {
        void *p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_static_scratch);
        if (e != cudaSuccess || !p)
            return fail(B200_E_CUDA, "cudaGetSymbolAddress(static scratch) failed on device %d: %s", dev, cudaGetErrorString(e));
        g_static_scratch_addr[dev] = (float *)p;
    }
    *out = g_static_scratch_addr[dev];
    return B200_OK;
}

}  // namespace b200

using namespace b200;

extern "C" {

size_t b200_static_scratch_bytes(void) { return kStaticScratchFloats * sizeof(float); }

int b200_conv_wgrad_batch_static(const b200_conv_geom *g, float *dkernel, float *dbias, int accumulate,
                                 const float *image, const float *delta, int batch, void *stream)
{
    cudaStream_t s = (cudaStream_t)stream;
    if (!g) return fail(B200_E_ARG, "null geometry");
    if (!dkernel || !image || !delta) return fail(B200_E_ARG, "null tensor pointer");
    if (batch <= 0 || g->kernel_amount <= 0 || g->in_z <= 0 || g->kernel_x <= 0 || g->kernel_y <= 0 || g->stride_x <= 0 ||
        g->stride_y <= 0 || g->in_y <= 0 || g->in_x <= 0 || g->out_y <= 0 || g->out_x <= 0 || g->padding_x < 0 || g->padding_y < 0)
        return fail(B200_E_SHAPE, "non-positive convolution geometry");
    if (g->out_x != (g->in_x - g->kernel_x + 2 * g->padding_x) / g->stride_x + 1 || g->out_y != (g->in_y - g->kernel_y + 2 * g->padding_y) / g->stride_y + 1)
        return fail(B200_E_SHAPE, "wrong output size for convolution: %dx%d does not follow from the image, kernel, stride and padding", g->out_y, g->out_x);
    const size_t klen = (size_t)g->kernel_amount * g->in_z * g->kernel_y * g->kernel_x;
    const size_t dk_floats = (size_t)batch * klen;
    const size_t db_floats = (size_t)batch * g->kernel_amount;
    if (dk_floats + db_floats > kStaticScratchFloats)
        return fail(B200_E_NOMEM,
                    "b200_conv_wgrad_batch_static: batch %d x %zu weights needs %zu scratch floats, the fixed scratch holds %zu; "
                    "use b200_conv_wgrad_batch or a smaller batch",
                    batch, klen, dk_floats + db_floats, kStaticScratchFloats);
    float *scratch = nullptr;
    int r = static_scratch(&scratch);
    if (r) return r;
    float *dk = scratch, *db = scratch + dk_floats;
    // the per-sample kernel accumulates, and the array still holds whatever the previous call left
    B200_CUDA(cudaMemsetAsync(scratch, 0, sizeof(float) * (dk_floats + db_floats), s));
    if ((r = simt_conv_wgrad(*g, dk, batch, db, batch, image, batch, delta, batch, s))) return r;
    if (!accumulate) {
        B200_CUDA(cudaMemsetAsync(dkernel, 0, sizeof(float) * klen, s));
        if (dbias) B200_CUDA(cudaMemsetAsync(dbias, 0, sizeof(float) * g->kernel_amount, s));
    }
    if ((r = b200_add_sum_w(dkernel, 1, dkernel, 1, dk, batch, klen, 1.f, 1.f, stream))) return r;
    if (dbias && (r = b200_add_sum_w(dbias, 1, dbias, 1, db, batch, (size_t)g->kernel_amount, 1.f, 1.f, stream))) return r;
    set_path(B200_PATH_SIMT);
    return B200_OK;
}

}  // extern "C"
