// Shared host-side helpers of the library: per-thread error text, status codes, the per-device
// scratch arena, and small launch utilities.
#pragma once
#include <cuda_runtime.h>
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include "../../include/b200conv.h"

namespace b200 {

void set_error(const char *fmt, ...);
int fail(int code, const char *fmt, ...);
void set_path(int path);
int precision();

#define B200_CUDA(expr)                                                                              \
    do {                                                                                             \
        cudaError_t e__ = (expr);                                                                    \
        if (e__ != cudaSuccess)                                                                      \
            return ::b200::fail(B200_E_CUDA, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(e__), \
                                __FILE__, __LINE__);                                                 \
    } while (0)

// Every kernel launch of the library goes through this check, which also counts it.
void count_launch();
#define B200_LAUNCH_CHECK()                    \
    do {                                       \
        ::b200::count_launch();                \
        B200_CUDA(::b200::take_launch_error()); \
        B200_CUDA(cudaGetLastError());         \
    } while (0)

// Programmatic dependent launch.  Every kernel of the library begins with grid_dependency_wait() (before its first access
// to global memory: it returns once the kernels before it in the stream have completed and their writes are visible) and is
// launched with the programmatic-stream-serialisation attribute, so its blocks are set up while the previous kernel drains
// instead of after it has retired.  The training steps are chains of a hundred short launches; the hand-over between two of
// them is a sizeable part of each.  No kernel signals early, so the order of all memory accesses is that of plain stream
// order.  (Letting every kernel trigger its dependents right after its own wait was measured too: the next kernel's blocks then
// wait on the SMs beside the running one, and the VAE step took 5.98 ms instead of 5.86 ms.)  B200CONV_PDL=0 in the environment launches without the attribute (the wait is then a no-op).
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
bool dependent_launch_enabled();
void note_launch_error(cudaError_t e);
cudaError_t take_launch_error();

struct Launch {
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute attr[2];
    Launch(dim3 grid, dim3 block, size_t smem = 0, cudaStream_t stream = 0)
    {
        cfg = cudaLaunchConfig_t{};
        cfg.gridDim = grid;
        cfg.blockDim = block;
        cfg.dynamicSmemBytes = smem;
        cfg.stream = stream;
        cfg.attrs = attr;
        cfg.numAttrs = 0;
        if (dependent_launch_enabled()) {
            attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
            attr[0].val.programmaticStreamSerializationAllowed = 1;
            cfg.numAttrs = 1;
        }
    }
    // thread-block cluster of `x` CTAs (the CTA-pair kernels)
    Launch &cluster(unsigned x)
    {
        if (x > 1) {
            cudaLaunchAttribute &a = attr[cfg.numAttrs++];
            a.id = cudaLaunchAttributeClusterDimension;
            a.val.clusterDim.x = x;
            a.val.clusterDim.y = 1;
            a.val.clusterDim.z = 1;
        }
        return *this;
    }
    template <typename... KArgs, typename... Args>
    void operator()(void (*kernel)(KArgs...), Args &&...args) const
    {
        const cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
        if (e != cudaSuccess) note_launch_error(e);
    }
};

// Scratch arena: one growing cudaMalloc block per device, carved by bump allocation for the
// duration of one library call.  The stream order of the call protects reuse between calls on the
// same stream; callers that use several streams concurrently must serialise library calls.
struct Arena {
    char *base = nullptr;
    size_t cap = 0;
    size_t used = 0;
};
int arena_reserve(size_t bytes, cudaStream_t stream);  // make sure cap >= bytes (may synchronise + reallocate)
void *arena_take(size_t bytes);                        // bump-allocate (256-byte aligned); call after arena_reserve
void arena_reset();

inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }
inline int ceil_div(int a, int b) { return (a + b - 1) / b; }
int sm_count();

}  // namespace b200
