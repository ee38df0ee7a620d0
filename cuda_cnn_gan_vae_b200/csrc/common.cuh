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
#define B200_LAUNCH_CHECK()          \
    do {                             \
        ::b200::count_launch();      \
        B200_CUDA(cudaGetLastError()); \
    } while (0)

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
