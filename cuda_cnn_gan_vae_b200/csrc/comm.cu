// Data-parallel exchange over NVLink peer memory: the sum of the weight-gradient arenas of all ranks, alone or fused
// with the optimiser step.
//
// One process per GPU.  Every rank owns a "communicator": one device allocation (signal pad + data region) that it
// exports as a CUDA IPC handle; the caller carries the handles between the ranks (any channel: MPI, a file, a socket,
// torch.distributed) and every rank maps the others' allocations.  The gradient and weight arenas of a network live in the
// data region, so the weight-gradient kernels write where the peers will read: no staging copy.
//
// The kernel is a two-shot exchange in which rank r owns slice r of the arena:
//   1. ready barrier  -- per CTA and peer: "my gradients are complete" flags, written into the peers' signal pads with
//                        system-scope release stores, polled locally;
//   2. reduce-scatter -- the CTA reads its part of slice r from every rank (plain 16-byte peer loads, fixed rank order, so
//                        the sum is reproducible) and either writes the sum back into every rank's arena (all-reduce) or
//                        applies Adam to its slice of the weights and moments and writes the NEW WEIGHTS into every
//                        rank's weight arena (reduce-scatter + Adam + all-gather: the optimiser touches 1/world of the
//                        parameters per rank, the summed gradient never travels back);
//   3. done barrier   -- nobody leaves before every peer has finished reading its gradients and writing its weights.
// No multicast load of any kind is used (plain loads and stores on mapped peer pointers).  Every wait is bounded (about a
// second): a rank whose peers never arrive records B200_E_TIMEOUT in the status word that b200_stream_status() reads, skips
// the remaining waits and returns normally, so the context stays usable.
#include "common.cuh"
#include "kernels.h"
#include "adam.cuh"
#include <cstdlib>
#include <cstring>
#include <new>
#include <unistd.h>

namespace b200 {

constexpr int kCommMaxWorld = 16;
constexpr int kCommMaxCtas = 256;
constexpr int kCommChannels = 4;
constexpr long long kCommWaitCycles = 2000000000LL;

// One channel of a signal pad.  ready/done[p][b]: written by rank p's CTA b, polled by this rank's CTA b.
struct CommChannel {
    unsigned epoch;            // number of exchanges completed on this channel (advanced by the last CTA to finish)
    unsigned finished;         // CTAs of the running exchange that have finished
    unsigned pad[62];
    unsigned ready[kCommMaxWorld][kCommMaxCtas];
    unsigned done[kCommMaxWorld][kCommMaxCtas];
};
constexpr size_t kPadBytes = sizeof(CommChannel) * kCommChannels;      // data region starts here (a multiple of 256 bytes)

struct CommHandle {            // what travels between the ranks (B200_COMM_HANDLE_BYTES)
    cudaIpcMemHandle_t ipc;
    long long pid;
    unsigned long long address;    // the allocation's address in the exporting process (used when both ranks share a process)
    unsigned long long bytes;
    int rank, device;
    char reserved[128 - sizeof(cudaIpcMemHandle_t) - 8 - 8 - 8 - 4 - 4];
};
static_assert(sizeof(CommHandle) == 128, "handle size is part of the ABI");

struct CommPeers {
    char *base[kCommMaxWorld];
};

constexpr int kCommMaxSegments = 4;

// One arena of an exchange: several (the arenas of several networks) share the launch and its two barriers.
struct ExchangeSegment {
    size_t first, second;      // float offsets into the data region: (gradients, weights) or (buffer, unused)
    size_t n4;                 // 16-byte groups in the arena
    float *m, *v;              // local Adam moments (full-size arrays; only this rank's slice is touched)
};

struct ExchangeParams {
    CommPeers peers;
    int rank, world, channel, segments;
    ExchangeSegment seg[kCommMaxSegments];
    AdamArgs adam;
    const double *corrections;
    unsigned *status;
};

__device__ __forceinline__ void st_release_sys(unsigned *p, unsigned v)
{
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned *p)
{
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ unsigned ld_relaxed_sys(const unsigned *p)
{
    unsigned v;
    asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void fence_acquire_sys() { asm volatile("fence.acq_rel.sys;" ::: "memory"); }

// Waits until *flag >= epoch (flags only grow).  Gives up after kCommWaitCycles or when another thread of the CTA did.
__device__ __forceinline__ bool wait_flag(const unsigned *flag, unsigned epoch, volatile int *abort_flag, unsigned *status, unsigned code)
{
    // relaxed polls, one acquire fence once the flag is there
    if ((int)(ld_relaxed_sys(flag) - epoch) < 0) {
        const long long t0 = clock64();
        while ((int)(ld_relaxed_sys(flag) - epoch) < 0) {
            if (*abort_flag) return false;
            if (clock64() - t0 > kCommWaitCycles) {
                *abort_flag = 1;
                atomicExch(status, code);
                __threadfence_system();
                return false;
            }
        }
    }
    fence_acquire_sys();
    return true;
}

template <bool ADAM>
__global__ void __launch_bounds__(512) exchange_kernel(const ExchangeParams p)
{
    __shared__ unsigned s_epoch;
    __shared__ int s_abort;
    CommChannel *mine = reinterpret_cast<CommChannel *>(p.peers.base[p.rank]) + p.channel;
    if (threadIdx.x == 0) {
        s_epoch = ld_acquire_sys(&mine->epoch) + 1u;
        s_abort = 0;
    }
    __syncthreads();
#ifdef B200_COMM_TIMING
    auto stamp = [&](int k) { if (blockIdx.x == 0 && threadIdx.x == 0) { unsigned long long t; asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t)); mine->pad[k] = (unsigned)t; } };
    stamp(0);
#else
    auto stamp = [&](int) {};
#endif
    const unsigned epoch = s_epoch;
    const int b = blockIdx.x;
    const bool peer_lane = (int)threadIdx.x < p.world && (int)threadIdx.x != p.rank;
    CommChannel *theirs = peer_lane ? reinterpret_cast<CommChannel *>(p.peers.base[threadIdx.x]) + p.channel : nullptr;

    // 1. ready barrier: the kernels that produced this rank's gradients finished before this one started (stream order)
    if (peer_lane) {
        st_release_sys(&theirs->ready[p.rank][b], epoch);
        wait_flag(&mine->ready[threadIdx.x][b], epoch, &s_abort, p.status, 0x500u + B200_E_TIMEOUT);
    }
    __syncthreads();
    stamp(1);

    // 2. this rank's slice, in 16-byte groups
    if (!s_abort) {
        AdamArgs a = p.adam;
        if (ADAM && p.corrections) { a.inv_c1 = 1.0 / p.corrections[0]; a.inv_c2 = 1.0 / p.corrections[1]; }
        const size_t data0 = kPadBytes / sizeof(float4);
      for (int sg = 0; sg < p.segments; sg++) {
        const ExchangeSegment &q = p.seg[sg];
        const size_t per = (q.n4 + p.world - 1) / p.world;
        const size_t begin = per * p.rank < q.n4 ? per * p.rank : q.n4;
        const size_t end = begin + per < q.n4 ? begin + per : q.n4;
        // Two groups per thread and trip, and the loads from up to eight ranks issued together before the first addition: a
        // remote load takes a few microseconds, so a thread keeps 2 x world of them in flight instead of paying one round trip
        // per rank.  The additions stay in rank order (reproducible, and equal to a sequential sum over the ranks).
        // (Measured on 2 GPUs: a lighter variant -- 256 threads, one group per trip, up to 256 CTAs -- that could share SMs
        // with the convolution kernels of another stream was 15-30 % slower and gave the DCGAN step nothing.)
        constexpr int U = 2, R = 8;
        const size_t stride = (size_t)gridDim.x * blockDim.x;
        for (size_t i0 = begin + (size_t)b * blockDim.x + threadIdx.x; i0 < end; i0 += U * stride) {
            float4 s[U];
            for (int r0 = 0; r0 < p.world; r0 += R) {
                float4 t[U][R];
#pragma unroll
                for (int u = 0; u < U; u++) {
                    const size_t i = i0 + u * stride;
#pragma unroll
                    for (int rr = 0; rr < R; rr++)
                        if (r0 + rr < p.world && i < end)
                            t[u][rr] = __ldcg(reinterpret_cast<const float4 *>(p.peers.base[r0 + rr]) + data0 + q.first / 4 + i);
                }
#pragma unroll
                for (int u = 0; u < U; u++) {
#pragma unroll
                    for (int rr = 0; rr < R; rr++) {
                        if (r0 + rr >= p.world) continue;
                        if (r0 + rr == 0) { s[u] = t[u][0]; continue; }
                        s[u].x = __fadd_rn(s[u].x, t[u][rr].x); s[u].y = __fadd_rn(s[u].y, t[u][rr].y);
                        s[u].z = __fadd_rn(s[u].z, t[u][rr].z); s[u].w = __fadd_rn(s[u].w, t[u][rr].w);
                    }
                }
            }
#pragma unroll
            for (int u = 0; u < U; u++) {
                const size_t i = i0 + u * stride;
                if (i >= end) break;
                const size_t gi = data0 + q.first / 4 + i;
                if (ADAM) {
                    const size_t wi = data0 + q.second / 4 + i;
                    float4 w = reinterpret_cast<const float4 *>(p.peers.base[p.rank])[wi];
                    float4 mm = reinterpret_cast<float4 *>(q.m)[i], vv = reinterpret_cast<float4 *>(q.v)[i];
                    w.x = adam_element(w.x, s[u].x, mm.x, vv.x, a); w.y = adam_element(w.y, s[u].y, mm.y, vv.y, a);
                    w.z = adam_element(w.z, s[u].z, mm.z, vv.z, a); w.w = adam_element(w.w, s[u].w, mm.w, vv.w, a);
                    reinterpret_cast<float4 *>(q.m)[i] = mm;
                    reinterpret_cast<float4 *>(q.v)[i] = vv;
                    for (int r = 0; r < p.world; r++) reinterpret_cast<float4 *>(p.peers.base[r])[wi] = w;
                } else {
                    for (int r = 0; r < p.world; r++) reinterpret_cast<float4 *>(p.peers.base[r])[gi] = s[u];
                }
            }
        }
      }
    }

    // 3. done barrier: my stores into the peers' arenas are visible before the flag is, and nobody's gradients are
    //    overwritten by its next step while a peer still reads them
    stamp(2);
    // The CTA barrier orders every thread's stores before the flag threads' release stores, whose system-scope release is
    // cumulative over them: one fence per flag instead of one per thread.
    __syncthreads();
    stamp(3);
    if (peer_lane && !s_abort) {
        st_release_sys(&theirs->done[p.rank][b], epoch);
        wait_flag(&mine->done[threadIdx.x][b], epoch, &s_abort, p.status, 0x600u + B200_E_TIMEOUT);
    }
    __syncthreads();
    stamp(4);
    // the last CTA of this rank to finish publishes the new epoch (every CTA read the old one at its start)
    if (threadIdx.x == 0) {
        __threadfence();
        const unsigned c = atomicAdd(&mine->finished, 1u);
        if (c == gridDim.x - 1) {
            mine->finished = 0;
            __threadfence();
            st_release_sys(&mine->epoch, epoch);
        }
    }
}

}  // namespace b200

using namespace b200;

struct b200_comm {
    int rank, world, device;
    size_t bytes;              // data region
    char *base;                // this rank's allocation (pad + data)
    char *peer[kCommMaxWorld]; // mapped allocations of all ranks (peer[rank] == base)
    bool opened[kCommMaxWorld];
    bool connected;
};

static int exchange_grid(size_t n4, int world, int threads)
{
    // the same on every rank: enough CTAs to keep the links busy, no more than the flags of a channel, none idle
    const size_t per = (n4 + world - 1) / world;
    size_t g = (per + threads - 1) / threads;
    // tuning aid: B200CONV_EXCHANGE_CTAS=<n> caps the grid (read once; must be the same on every rank)
    static const int cap = [] { const char *e = getenv("B200CONV_EXCHANGE_CTAS"); int v = e ? atoi(e) : 0; return (v >= 1 && v <= kCommMaxCtas) ? v : 144; }();
    if (g > (size_t)cap) g = (size_t)cap;
    if (g < 1) g = 1;
    return (int)g;
}

static int launch_exchange(b200_comm *c, bool adam, int count, const b200_exchange_segment *segs, const AdamArgs &a, const double *corrections,
                           int channel, cudaStream_t s)
{
    if (!c) return fail(B200_E_ARG, "null communicator");
    if (!c->connected) return fail(B200_E_ARG, "communicator is not connected");
    if (channel < 0 || channel >= kCommChannels) return fail(B200_E_ARG, "channel must lie in [0, %d)", kCommChannels);
    if (count < 1 || count > kCommMaxSegments || !segs) return fail(B200_E_ARG, "an exchange takes 1 to %d arenas", kCommMaxSegments);
    ExchangeParams p;
    memset(&p, 0, sizeof(p));
    size_t largest = 0, total = 0;
    for (int i = 0; i < count; i++) {
        const b200_exchange_segment &g = segs[i];
        if ((g.n % 4) || (g.grad_offset % 4) || (g.weight_offset % 4)) return fail(B200_E_ARG, "arena offsets and sizes must be multiples of 4 floats");
        if ((g.grad_offset + g.n) * sizeof(float) > c->bytes || (adam && (g.weight_offset + g.n) * sizeof(float) > c->bytes))
            return fail(B200_E_SHAPE, "arena reaches beyond the communicator's buffer");
        if (adam && (!g.m || !g.v)) return fail(B200_E_ARG, "null Adam moments");
        if (adam && (((uintptr_t)g.m | (uintptr_t)g.v) & 15)) return fail(B200_E_ARG, "Adam moments must be 16-byte aligned");
        p.seg[i].first = g.grad_offset; p.seg[i].second = g.weight_offset; p.seg[i].n4 = g.n / 4;
        p.seg[i].m = g.m; p.seg[i].v = g.v;
        if (g.n / 4 > largest) largest = g.n / 4;
        total += g.n;
    }
    if (!total) return B200_OK;
    int dev = 0;
    B200_CUDA(cudaGetDevice(&dev));
    if (dev != c->device) return fail(B200_E_ARG, "communicator belongs to device %d, current device is %d", c->device, dev);
    for (int r = 0; r < c->world; r++) p.peers.base[r] = c->peer[r];
    p.rank = c->rank; p.world = c->world; p.channel = channel; p.segments = count;
    p.adam = a; p.corrections = corrections;
    int r = status_word(&p.status);
    if (r) return r;
    // The fused exchange runs alone at the end of a step: 512-thread CTAs keep the most loads in flight.  The plain sum is
    // what a caller overlaps with a convolution of another stream: at ~120 registers a 512-thread CTA needs a whole register
    // file and could not share an SM with a tensor-core CTA (it then waits for the convolution to end, or delays part of its
    // persistent grid); 256 threads fit beside one.
    // (tuning aid: B200CONV_EXCHANGE_THREADS=256|512 forces either; read once, must be the same on every rank)
    static const int forced = [] { const char *e = getenv("B200CONV_EXCHANGE_THREADS"); const int v = e ? atoi(e) : 0; return (v == 256 || v == 512) ? v : 0; }();
    const int threads = forced ? forced : (adam ? 512 : 256);
    const int grid = exchange_grid(largest, c->world, threads);
    if (adam) exchange_kernel<true><<<grid, threads, 0, s>>>(p);
    else exchange_kernel<false><<<grid, threads, 0, s>>>(p);
    B200_LAUNCH_CHECK();
    return B200_OK;
}

extern "C" {

int b200_comm_slice(size_t n, int rank, int world, size_t *begin, size_t *end)
{
    if (!begin || !end || world < 1 || rank < 0 || rank >= world || (n % 4)) return fail(B200_E_ARG, "bad slice request");
    const size_t n4 = n / 4, per = (n4 + world - 1) / world;
    const size_t b = per * rank < n4 ? per * rank : n4;
    const size_t e = b + per < n4 ? b + per : n4;
    *begin = b * 4;
    *end = e * 4;
    return B200_OK;
}

int b200_comm_create(b200_comm **comm, int rank, int world, size_t bytes)
{
    if (!comm) return fail(B200_E_ARG, "null argument");
    if (world < 1 || world > kCommMaxWorld || rank < 0 || rank >= world) return fail(B200_E_ARG, "rank %d of %d is out of range (at most %d ranks)", rank, world, kCommMaxWorld);
    b200_comm *c = new (std::nothrow) b200_comm;
    if (!c) return fail(B200_E_NOMEM, "host allocation failed");
    memset(c, 0, sizeof(*c));
    c->rank = rank; c->world = world;
    c->bytes = align_up(bytes, 256);
    cudaError_t e = cudaGetDevice(&c->device);
    void *p = nullptr;
    if (e == cudaSuccess) e = cudaMalloc(&p, kPadBytes + c->bytes);
    if (e == cudaSuccess) e = cudaMemset(p, 0, kPadBytes + c->bytes);
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    if (e != cudaSuccess) {
        cudaGetLastError();
        if (p) cudaFree(p);
        delete c;
        return fail(B200_E_NOMEM, "communicator: allocation of %zu bytes failed: %s", kPadBytes + bytes, cudaGetErrorString(e));
    }
    c->base = (char *)p;
    c->peer[rank] = c->base;
    c->connected = world == 1;
    *comm = c;
    return B200_OK;
}

int b200_comm_handle(b200_comm *c, void *handle)
{
    if (!c || !handle) return fail(B200_E_ARG, "null argument");
    CommHandle h;
    memset(&h, 0, sizeof(h));
    B200_CUDA(cudaIpcGetMemHandle(&h.ipc, c->base));
    h.pid = (long long)getpid();
    h.address = (unsigned long long)(uintptr_t)c->base;
    h.bytes = kPadBytes + c->bytes;
    h.rank = c->rank;
    h.device = c->device;
    memcpy(handle, &h, sizeof(h));
    return B200_OK;
}

int b200_comm_connect(b200_comm *c, const void *handles)
{
    if (!c || !handles) return fail(B200_E_ARG, "null argument");
    if (c->connected) return B200_OK;
    const CommHandle *h = (const CommHandle *)handles;
    for (int r = 0; r < c->world; r++) {
        if (h[r].rank != r) return fail(B200_E_ARG, "handle %d belongs to rank %d: pass the handles in rank order", r, h[r].rank);
        if (h[r].bytes != kPadBytes + c->bytes) return fail(B200_E_SHAPE, "rank %d created its communicator with another size", r);
    }
    for (int r = 0; r < c->world; r++) {
        if (r == c->rank) continue;
        if (h[r].pid == (long long)getpid()) {
            // ranks that share a process (one thread per device): the address is valid here once peer access is enabled
            int can = 0;
            B200_CUDA(cudaDeviceCanAccessPeer(&can, c->device, h[r].device));
            if (!can) return fail(B200_E_CUDA, "device %d cannot access device %d", c->device, h[r].device);
            cudaError_t e = cudaDeviceEnablePeerAccess(h[r].device, 0);
            if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled) return fail(B200_E_CUDA, "cudaDeviceEnablePeerAccess: %s", cudaGetErrorString(e));
            cudaGetLastError();
            c->peer[r] = (char *)(uintptr_t)h[r].address;
        } else {
            void *p = nullptr;
            cudaError_t e = cudaIpcOpenMemHandle(&p, h[r].ipc, cudaIpcMemLazyEnablePeerAccess);
            if (e != cudaSuccess) {
                cudaGetLastError();
                return fail(B200_E_CUDA, "cudaIpcOpenMemHandle for rank %d failed: %s", r, cudaGetErrorString(e));
            }
            c->peer[r] = (char *)p;
            c->opened[r] = true;
        }
    }
    c->connected = true;
    return B200_OK;
}

void *b200_comm_buffer(b200_comm *c) { return c ? (void *)(c->base + kPadBytes) : nullptr; }
size_t b200_comm_buffer_bytes(b200_comm *c) { return c ? c->bytes : 0; }

int b200_comm_destroy(b200_comm *c)
{
    if (!c) return B200_OK;
    cudaDeviceSynchronize();
    for (int r = 0; r < c->world; r++)
        if (c->opened[r]) cudaIpcCloseMemHandle(c->peer[r]);
    if (c->base) cudaFree(c->base);
    delete c;
    return B200_OK;
}

int b200_allreduce(b200_comm *c, size_t offset, size_t n, int channel, void *stream)
{
    if (c && c->world == 1) return B200_OK;
    AdamArgs a;
    memset(&a, 0, sizeof(a));
    b200_exchange_segment g = {offset, 0, n, nullptr, nullptr};
    return launch_exchange(c, false, 1, &g, a, nullptr, channel, (cudaStream_t)stream);
}

int b200_allreduce_adam(b200_comm *c, size_t grad_offset, size_t weight_offset, float *m, float *v, size_t n, uint32_t batch_size,
                        double speed, double beta1, double beta2, double epsilon, double iteration, const double *corrections, int channel,
                        void *stream)
{
    b200_exchange_segment g = {grad_offset, weight_offset, n, m, v};
    return b200_allreduce_adam_multi(c, 1, &g, batch_size, speed, beta1, beta2, epsilon, iteration, corrections, channel, stream);
}

int b200_allreduce_adam_multi(b200_comm *c, int count, const b200_exchange_segment *segments, uint32_t batch_size, double speed, double beta1,
                              double beta2, double epsilon, double iteration, const double *corrections, int channel, void *stream)
{
    if (!c || !segments) return fail(B200_E_ARG, "null argument");
    if (!batch_size) return fail(B200_E_ARG, "batch_size must be positive");
    const double c1 = corrections ? 1.0 : 1.0 - pow(beta1, iteration), c2 = corrections ? 1.0 : 1.0 - pow(beta2, iteration);
    if (!corrections && (c1 == 0.0 || c2 == 0.0)) return fail(B200_E_ARG, "Adam: iteration must be positive");
    return launch_exchange(c, true, count, segments, adam_args(batch_size, speed, beta1, beta2, epsilon, c1, c2, 0.0), corrections, channel,
                           (cudaStream_t)stream);
}

}  // extern "C"
