// tcgen05 implicit-GEMM kernels for sm_100a: forward convolution, backward-data convolution
// (= transposed convolution), batch-summed weight gradient and the dense GEMM of the Linear layer.
//
// One warp-specialised persistent kernel serves all four problems.  Per CTA (one per SM, 224 threads):
//   warps 0, 6  TMA producers (alternate stages): stream 128 x 32 (A) and BN x 32 (B) TF32 tiles into a ring of
//               shared-memory stages with cp.async.bulk.tensor (128-byte swizzle); zero fill of
//               out-of-range coordinates implements the convolution padding and every ragged edge;
//   warp 1      MMA issuer: one thread issues tcgen05.mma kind::tf32 (M=128, N=BN, K=8), four per
//               stage (twelve in 3xTF32 mode), accumulating in tensor memory; two accumulator
//               stages let the epilogue of tile i overlap the main loop of tile i+1;
//   warps 2-5   epilogue: tcgen05.ld of the accumulator (lane = output row), bias, coalesced stores.
// A stage holds one or two K blocks of 32 (two when three such stages fit).  In CTA-pair mode (template CTAS = 2) a
// cluster of two CTAs shares one 256-row MMA issued by the leader (tcgen05 cta_group::2): each CTA stages its own 128
// rows of A and half of B's rows, which halves the B bytes per flop.
// The problems differ only in how a (tile, step) pair maps to TMA coordinates and in the epilogue:
//   CONV   rows = 128 output pixels (a BI x BH x BW box of the NHWC activation pack), columns =
//          filters, K = (tap, 32-channel chunk).  Strided convolutions read a phase-split pack (one
//          sub-image per (y mod s, x mod s)), strided backward convolutions run one stride-1
//          problem per output phase, so no structural zero is ever multiplied.
//   WGRAD  rows = filters, columns = input channels, K = output pixels (batch folded into K), both
//          operands MN-major straight from the NHWC packs; split-K partial sums go to scratch and a
//          second kernel reduces them in a fixed order (run-to-run reproducible).
//   GEMM   plain C = A*B with either operand K-major or MN-major.
// Every mbarrier wait is bounded: after ~1 s of polling the kernel records a status code in
// host-visible memory, tells the other warps to stop and returns normally.
#include "common.cuh"
#include "kernels.h"
#include "tc_ptx.cuh"
#include "act.cuh"
#include <cstdlib>
#include <cstring>
#include <vector>

namespace b200 {

enum { MODE_CONV = 0, MODE_WGRAD = 1, MODE_GEMM = 2 };

constexpr int kThreads = 224;            // warps: 0 and 6 TMA producers, 1 MMA issuer, 2-5 epilogue
constexpr int kABytes = 128 * 128;        // 128 rows x 32 tf32
constexpr int kMaxTaps = 64;
constexpr int kMaxPhases = 16;
constexpr long long kWaitCycles = 2000000000LL;

struct TapEntry { int8_t dy, dx; uint8_t in_phase, wtap; };
struct TapGroup { uint8_t count, tap[4], unused[3]; };      // WGRAD with packed taps: the taps (of one stride phase) of a work item

struct PhaseInfo {
    int tile_begin;            // first M-tile of this output phase
    int pair_begin;            // first M-tile pair of this phase (CTA-pair kernels)
    int tiles_x, tiles_y, tiles_i;
    int ext_y, ext_x;          // output extent of the phase (rows / columns it owns)
    int off_y, off_x;          // position of the phase inside the full output
    int tap_begin, tap_count;
};

struct TcParams {
    int stages, BN, acc_stride, tmem_cols;
    int acc_stages;            // accumulator sets in tensor memory: 2 (epilogue of tile i overlaps the main loop of tile i+1) or 1
    int acc_set_stride;        // columns from one accumulator set to the next
    int small_off;             // 3xTF32: column offset, inside a set, of the accumulator of the two small product terms
    int a_boxes, b_boxes;
    uint32_t a_box_bytes, b_box_bytes, b_bytes, mini_bytes, stage_bytes;
    int ksub;                  // 32-wide K blocks per pipeline stage (each block = one set of operand boxes)
    uint32_t a_lbo, a_sbo, a_kadv, a_layout, b_lbo, b_sbo, b_kadv, b_layout, idesc;
    int num_tiles;             // work items of the kernel: tiles, or tile pairs for the CTA-pair kernel
    unsigned *status;
    // CONV
    int n_tiles_n, c_chunks, phases, BW, BH, BI, n_img, k_out, OH, OW, out_stride_y, out_stride_x;
    PhaseInfo phase[kMaxPhases];
    TapEntry taps[kMaxTaps];
    float *out;
    const float *bias;
    int act_func;              // CONV: neuron function applied to out + bias in the epilogue (B200_ACT_*), -1 = none
    double act_slope;
    float *pre_out;            // CONV: optional second output, the value before the neuron function
    int ksplit;                // CONV: the K steps of a tile are divided over ksplit work items (1 = no split)
    float *kpartial;           // ksplit > 1: partial outputs [split][n][k][y][x], summed by conv_ksplit_reduce_kernel
    long long out_elems;
    // WGRAD
    int ft_n, ct_n, taps_n, splits, chunks_x, chunks_y, chunks_i, k_rows, c_cols, wg_ctas;
    long long chunks_total;
    float *partial;
    // WGRAD with few filters: the 128 rows of the MMA hold `members` taps x `tapm` filters (tapm = filters padded to 32 or 64;
    // 0 = one tap per work item), a work item covers a group of taps of one stride phase
    int tapm, members, items_n;
    uint32_t member_bytes;
    TapGroup groups[kMaxTaps];
    // GEMM
    int M, N, K, ldc, a_mn, b_mn;
#ifdef B200_TC_TIMING
    long long *dbg;            // per-CTA cycle counters: [0] producer waiting, [1] issuer waiting for data, [2] issuer waiting for TMEM, [3] issuer total, [4] epilogue waiting, [5] epilogue total
#endif
};

struct TileCtx {
    int nsteps;
    int nt;                    // CONV/GEMM: n tile
    int ph, tx, ty, ig;        // CONV
    int step_begin;            // CONV: first K step of this work item (split-K)
    int ft, tap, ct, split;    // WGRAD (split also CONV)
    long long chunk_begin;     // WGRAD
    int mt;                    // GEMM
};

// CTA-pair convolution: work item `pair` = two neighbouring M-tiles of one output phase, CTA `rank`
// takes the rank-th of them.  A phase with an odd tile count ends in a pair whose second tile lies
// outside the batch: its loads are zero-filled and its stores masked.
// Division by a small runtime value is some twenty dependent instructions, and the three roles of the kernel run ONE warp
// each: for layers with a short contraction the decode and the epilogue's index arithmetic per tile weighed as much as the
// tile's MMAs.  The common divisors (no split-K, one column tile, one tile per row / plane) are therefore branched around.
__device__ __forceinline__ void div_mod(int v, int d, int &q, int &r)
{
    if (d == 1) { q = v; r = 0; } else { q = v / d; r = v - q * d; }
}

__device__ __forceinline__ TileCtx decode_pair(const TcParams &p, int pair, int rank)
{
    TileCtx c;
    div_mod(pair, p.ksplit, pair, c.split);
    int mp;
    div_mod(pair, p.n_tiles_n, mp, c.nt);
    int ph = 0;
    while (ph + 1 < p.phases && mp >= p.phase[ph + 1].pair_begin) ph++;
    const PhaseInfo &pi = p.phase[ph];
    int local = (mp - pi.pair_begin) * 2 + rank;
    c.ph = ph;
    {
        const int total = pi.tap_count * p.c_chunks;
        if (p.ksplit == 1) { c.step_begin = 0; c.nsteps = total; }
        else {
            c.step_begin = total * c.split / p.ksplit;
            c.nsteps = total * (c.split + 1) / p.ksplit - c.step_begin;
        }
    }
    if (local < pi.tiles_x * pi.tiles_y * pi.tiles_i) {
        int rest;
        div_mod(local, pi.tiles_x, rest, c.tx);
        div_mod(rest, pi.tiles_y, c.ig, c.ty);
    } else {
        c.tx = 0; c.ty = 0; c.ig = pi.tiles_i;
    }
    return c;
}

template <int MODE>
__device__ __forceinline__ TileCtx decode_tile(const TcParams &p, int tile, int rank = 0)
{
    TileCtx c;
    if (MODE == MODE_CONV) {
        div_mod(tile, p.ksplit, tile, c.split);
        int mt;
        div_mod(tile, p.n_tiles_n, mt, c.nt);
        int ph = 0;
        while (ph + 1 < p.phases && mt >= p.phase[ph + 1].tile_begin) ph++;
        const PhaseInfo &pi = p.phase[ph];
        int local = mt - pi.tile_begin;
        c.ph = ph;
        int rest;
        div_mod(local, pi.tiles_x, rest, c.tx);
        div_mod(rest, pi.tiles_y, c.ig, c.ty);
        const int total = pi.tap_count * p.c_chunks;
        if (p.ksplit == 1) { c.step_begin = 0; c.nsteps = total; }
        else {
            c.step_begin = total * c.split / p.ksplit;
            c.nsteps = total * (c.split + 1) / p.ksplit - c.step_begin;
        }
    } else if (MODE == MODE_WGRAD) {
        // The tap varies fastest: the CTAs that run side by side work on the taps of ONE range of output pixels, so the error
        // chunk they all read and the (shifted) image chunks come from HBM once and from L2 for the other taps.  With the
        // split fastest instead, every tap streamed both tensors from HBM again (9 or 16 times the traffic, which is what
        // bounds this kernel on layers with few channels).
        c.tap = tile % p.items_n;                        // a tap, or a group of taps
        int rest = tile / p.items_n;
        c.split = rest % p.splits; rest /= p.splits;
        c.ct = rest % p.ct_n;
        c.ft = (rest / p.ct_n) * p.wg_ctas + rank;       // CTA pair: the pair owns two neighbouring filter tiles
        long long b = p.chunks_total * c.split / p.splits;
        long long e = p.chunks_total * (c.split + 1) / p.splits;
        c.chunk_begin = b;
        c.nsteps = (int)(e - b);
    } else {
        c.split = tile % p.ksplit;
        tile /= p.ksplit;
        c.nt = tile % p.n_tiles_n;
        c.mt = tile / p.n_tiles_n;
        const int total = (p.K + 31) / 32;
        c.step_begin = total * c.split / p.ksplit;
        c.nsteps = total * (c.split + 1) / p.ksplit - c.step_begin;
    }
    return c;
}

__device__ __forceinline__ bool wait_bar(uint32_t bar, uint32_t parity, volatile int *abort_flag, unsigned *status, unsigned code)
{
    if (ptx::mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    while (true) {
#pragma unroll 1
        for (int i = 0; i < 128; i++)
            if (ptx::mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
        if (clock64() - t0 > kWaitCycles) {
            *abort_flag = 1;
            atomicExch(status, code);
            __threadfence_system();
            return false;
        }
    }
}

// ACT: the CONV epilogue also applies a neuron function and / or writes the value before it (instantiated separately so that
// the plain epilogue keeps its short store loop).
template <int MODE, bool X3, int CTAS, bool ACT>
__global__ void __launch_bounds__(kThreads, 1)
tc_kernel(const __grid_constant__ CUtensorMap mapA_hi, const __grid_constant__ CUtensorMap mapA_lo,
          const __grid_constant__ CUtensorMap mapB_hi, const __grid_constant__ CUtensorMap mapB_lo,
          const __grid_constant__ TcParams p)
{
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + (size_t)p.stages * p.stage_bytes);
    // barrier layout: full[stages], empty[stages], tfull[2], tempty[2]
    const uint32_t bar_base = ptx::smem_u32(bars);
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (p.stages + s); };
    auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * p.stages + a); };
    auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * p.stages + 2 + a); };
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * p.stages + 4);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // CTA pair: both CTAs run the producer and the epilogue on their own 128 rows; the leader (rank 0)
    // alone issues the 256-row MMAs.  full[] and tempty[] live in the leader, empty[] and tfull[] in
    // each CTA (signalled in both by the leader's tcgen05.commit).
    const uint32_t rank = CTAS == 2 ? ptx::cluster_ctarank() : 0u;
    const int work_begin = CTAS == 2 ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
    const int work_step = CTAS == 2 ? (int)(gridDim.x >> 1) : (int)gridDim.x;

    if (threadIdx.x == 0) {
        for (int s = 0; s < p.stages; s++) { ptx::mbar_init(full_bar(s), 1); ptx::mbar_init(empty_bar(s), 1); }
        for (int a = 0; a < 2; a++) { ptx::mbar_init(tfull_bar(a), 1); ptx::mbar_init(tempty_bar(a), 4 * CTAS); }
        *abort_flag = 0;
        ptx::fence_barrier_init();
        ptx::prefetch_tensormap(&mapA_hi);
        ptx::prefetch_tensormap(&mapB_hi);
        if (X3) { ptx::prefetch_tensormap(&mapA_lo); ptx::prefetch_tensormap(&mapB_lo); }
    }
    if (warp == 1) {
        if (CTAS == 2) { ptx::tmem_alloc_pair(ptx::smem_u32(tmem_slot), (uint32_t)p.tmem_cols); ptx::tmem_relinquish_pair(); }
        else { ptx::tmem_alloc(ptx::smem_u32(tmem_slot), (uint32_t)p.tmem_cols); ptx::tmem_relinquish(); }
    }
    ptx::tc_fence_before();
    __syncthreads();
    if (CTAS == 2) ptx::cluster_sync();      // the peer's barriers are initialised before anything signals them
    ptx::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // barriers, tensor memory and descriptors are set up while the previous kernel of the stream drains; nothing above
    // touches global memory
    grid_dependency_wait();

    const uint32_t a_bytes = kABytes;
    const uint32_t off_a_lo = a_bytes;
    const uint32_t off_b_hi = X3 ? 2 * a_bytes : a_bytes;
    const uint32_t off_b_lo = off_b_hi + p.b_bytes;
    const uint32_t stage_tx = p.stage_bytes * (uint32_t)CTAS;    // bytes of both CTAs land on the leader's barrier

    if (warp == 0 || warp == 6) {
        // ------------------------------------------------------------------ TMA producers
        // Two producer warps take alternate stages (a stage hand-shake plus its TMA issue keeps one warp
        // busy for several hundred cycles, more than the MMAs of a stage take).
        // The whole warp walks the tile/step sequence; lane 0 owns the barrier handshake and each box
        // of a stage is issued by its own lane, so a stage of many small boxes (MN-major operands,
        // 3xTF32 planes) costs one issue slot instead of one per box.
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        // Fixed role of this lane: which K block of a stage (my_m), which operand and plane, where in the
        // stage it lands.  One warp-wide TMA instruction then fills a whole stage.
        const int planes = X3 ? 2 : 1;
        const int a_parts = (MODE == MODE_WGRAD && p.tapm) ? p.members : 1;      // packed taps: one box per member tap
        const int n_boxes = (a_parts + 1) * planes;              // A (parts) and B, high (and low) plane
        const bool active = lane < n_boxes * p.ksub;
        const int my_m = lane / n_boxes, my_box = lane - my_m * n_boxes;
        const bool is_a = my_box < a_parts * planes;
        const bool is_lo = (my_box & 1) && X3;
        const int my_part = is_a ? my_box / planes : 0;
        const uint32_t my_off = (uint32_t)my_m * p.mini_bytes + (is_a ? (is_lo ? off_a_lo : 0u) + (uint32_t)my_part * p.member_bytes : (is_lo ? off_b_lo : off_b_hi));
        const CUtensorMap *my_map = is_a ? (is_lo ? &mapA_lo : &mapA_hi) : (is_lo ? &mapB_lo : &mapB_hi);
        const uint32_t smem0 = ptx::smem_u32(smem);
        const uint32_t my_turn = warp == 0 ? 0u : 1u;
        uint32_t iter = 0;
#ifdef B200_TC_TIMING
        long long dbg_pw = 0;
#endif
        for (int tile = work_begin; ok && tile < p.num_tiles; tile += work_step) {
            const TileCtx c = (CTAS == 2 && MODE == MODE_CONV) ? decode_pair(p, tile, (int)rank) : decode_tile<MODE>(p, tile, (int)rank);
            // running decomposition of this lane's K-block index st = step + my_m
            int st = my_m, ti = 0, cc = 0, cx = 0, cy = 0, ci = 0;
            int tap_begin = 0, base1 = 0, base2 = 0, base3 = 0, bcoord = 0;
            if (MODE == MODE_CONV) {
                const PhaseInfo &pi = p.phase[c.ph];
                const int g0 = c.step_begin + my_m;
                ti = g0 / p.c_chunks; cc = g0 - ti * p.c_chunks;
                tap_begin = pi.tap_begin;
                base1 = c.tx * p.BW; base2 = c.ty * p.BH; base3 = c.ig * p.BI;
                bcoord = c.nt * p.BN + (int)rank * (p.BN / 2) * (CTAS - 1);
            } else if (MODE == MODE_WGRAD) {
                const long long q = c.chunk_begin + my_m;
                cx = (int)(q % p.chunks_x);
                const long long r = q / p.chunks_x;
                cy = (int)(r % p.chunks_y);
                ci = (int)(r / p.chunks_y);
            }
            for (int step = 0; step < c.nsteps; step += p.ksub, iter++) {
              if ((iter & 1u) == my_turn) {
#ifdef B200_TC_TIMING
                const long long tw0 = clock64();
#endif
                if (lane == 0) ok = wait_bar(empty_bar(stage), phase ^ 1u, abort_flag, p.status, 0x100u + B200_E_TIMEOUT);
#ifdef B200_TC_TIMING
                if (lane == 0) dbg_pw += clock64() - tw0;
#endif
                ok = __shfl_sync(0xffffffffu, ok, 0);
                if (!ok) break;
                const uint32_t fb = full_bar(stage);
                if (lane == 0 && rank == 0) ptx::mbar_arrive_expect_tx(fb, stage_tx);
                __syncwarp();
                if (active) {
                    const bool pad = st >= c.nsteps;      // filler block of the last stage: coordinates out of range => zeros
                    int c0, c1, c2, c3, c4;
                    if (MODE == MODE_CONV) {
                        const TapEntry t = p.taps[tap_begin + (pad ? 0 : ti)];
                        if (is_a) { c0 = cc * 32; c1 = base1 + t.dx; c2 = base2 + t.dy; c3 = pad ? p.n_img + p.BI : base3; c4 = t.in_phase; }
                        else { c0 = cc * 32; c1 = t.wtap; c2 = bcoord; c3 = 0; c4 = 0; }
                    } else if (MODE == MODE_WGRAD && p.tapm) {
                        // The image chunk is taken unshifted from its phase plane and every member tap brings the error chunk
                        // that meets it: pixel X of the plane pairs with output pixel X - d of the tap.  Members a short group
                        // lacks, and filler blocks, read past the batch (zeros, same byte count).
                        const TapGroup &grp = p.groups[c.tap];
                        const bool absent = my_part >= grp.count;
                        const TapEntry t = p.taps[grp.tap[absent ? 0 : my_part]];
                        if (is_a) { c0 = 0; c1 = cx * p.BW - t.dx; c2 = cy * p.BH - t.dy; c3 = (pad || absent) ? (p.chunks_i + 1) * p.BI : ci * p.BI; c4 = 0; }
                        else { c0 = 0; c1 = cx * p.BW; c2 = cy * p.BH; c3 = t.in_phase * p.n_img + ci * p.BI; c4 = c.ct * (p.BN / 32); }
                    } else if (MODE == MODE_WGRAD) {
                        const TapEntry t = p.taps[c.tap];
                        // coordinate 4 walks the 32-channel blocks, so one box brings all blocks of the operand
                        if (is_a) { c0 = 0; c1 = cx * p.BW; c2 = cy * p.BH; c3 = pad ? (p.chunks_i + 1) * p.BI : ci * p.BI; c4 = c.ft * 4; }
                        else { c0 = 0; c1 = cx * p.BW + t.dx; c2 = cy * p.BH + t.dy; c3 = t.in_phase * p.n_img + ci * p.BI; c4 = c.ct * (p.BN / 32) + (int)rank * (p.BN / 64) * (CTAS - 1); }
                    } else {
                        // a filler block (and everything past K) reads beyond the matrix: zero-filled
                        const int k0 = pad ? ((p.K + 31) / 32 + 1) * 32 : (c.step_begin + st) * 32;
                        c2 = c3 = c4 = 0;
                        if (is_a) { if (p.a_mn) { c0 = 0; c1 = k0; c4 = c.mt * 4; } else { c0 = k0; c1 = c.mt * 128; } }
                        else { if (p.b_mn) { c0 = 0; c1 = k0; c4 = c.nt * (p.BN / 32); } else { c0 = k0; c1 = c.nt * p.BN; } }
                    }
                    const uint32_t dst = smem0 + (uint32_t)stage * p.stage_bytes + my_off;
                    if (CTAS == 2) ptx::tma_load_5d_pair(dst, my_map, fb, c0, c1, c2, c3, c4);
                    else ptx::tma_load_5d(dst, my_map, fb, c0, c1, c2, c3, c4);
                }
              }
                // advance this lane's K-block index by the blocks of one stage
                st += p.ksub;
                if (MODE == MODE_CONV) {
                    cc += p.ksub;
                    while (cc >= p.c_chunks) { cc -= p.c_chunks; ti++; }
                } else if (MODE == MODE_WGRAD) {
                    cx += p.ksub;
                    while (cx >= p.chunks_x) { cx -= p.chunks_x; if (++cy == p.chunks_y) { cy = 0; ci++; } }
                }
                if (++stage == p.stages) { stage = 0; phase ^= 1u; }
            }
        }
#ifdef B200_TC_TIMING
        if (lane == 0 && p.dbg) p.dbg[blockIdx.x * 8 + (warp == 0 ? 0 : 6)] = dbg_pw;
#endif
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0 && rank == 0) {
            int stage = 0;
            uint32_t phase = 0;
            int tile_iter = 0;
            bool ok = true;
            const uint32_t s0 = ptx::smem_u32(smem);
            const uint64_t a_hi0 = ptx::smem_desc(s0, p.a_lbo, p.a_sbo, p.a_layout);
            const uint64_t a_lo0 = ptx::smem_desc(s0 + off_a_lo, p.a_lbo, p.a_sbo, p.a_layout);
            const uint64_t b_hi0 = ptx::smem_desc(s0 + off_b_hi, p.b_lbo, p.b_sbo, p.b_layout);
            const uint64_t b_lo0 = ptx::smem_desc(s0 + off_b_lo, p.b_lbo, p.b_sbo, p.b_layout);
            const uint64_t stage16 = p.stage_bytes >> 4, mini16 = p.mini_bytes >> 4, ak16 = p.a_kadv >> 4, bk16 = p.b_kadv >> 4;
            const uint32_t idesc = p.idesc;
#ifdef B200_TC_TIMING
            long long dbg_mw = 0, dbg_mt = 0;
            const long long dbg_m0 = clock64();
#endif
            auto issue = [&](uint32_t dd, uint64_t ad, uint64_t bd, uint32_t acc_in) {
                if (CTAS == 2) ptx::mma_tf32_pair(dd, ad, bd, idesc, acc_in); else ptx::mma_tf32(dd, ad, bd, idesc, acc_in);
            };
            for (int tile = work_begin; ok && tile < p.num_tiles; tile += work_step, tile_iter++) {
                const TileCtx c = (CTAS == 2 && MODE == MODE_CONV) ? decode_pair(p, tile, 0) : decode_tile<MODE>(p, tile, 0);
                const int acc = p.acc_stages == 2 ? (tile_iter & 1) : 0;
                const uint32_t acc_phase = (uint32_t)(p.acc_stages == 2 ? (tile_iter >> 1) : tile_iter) & 1u;
#ifdef B200_TC_TIMING
                const long long te0 = clock64();
#endif
                if (!wait_bar(tempty_bar(acc), acc_phase ^ 1u, abort_flag, p.status, 0x200u + B200_E_TIMEOUT)) break;
#ifdef B200_TC_TIMING
                dbg_mt += clock64() - te0;
#endif
                ptx::tc_fence_after();
                const uint32_t d = tmem_base + (uint32_t)(acc * p.acc_set_stride);
                // 3xTF32 with small_off != 0 (optional): the two small product terms go to an accumulator of their own.  The tensor
                // core adds into its fp32 accumulator without rounding to nearest, an error proportional to the accumulator's
                // magnitude per MMA; kept apart, the small terms (2^-11 of the product) add next to nothing to it, and the large
                // accumulator sees one MMA per K step instead of three.  The epilogue adds the two.
                const uint32_t d_small = d + (uint32_t)p.small_off;
                for (int step = 0; step < c.nsteps; step += p.ksub) {
#ifdef B200_TC_TIMING
                    const long long tf0 = clock64();
#endif
                    if (!wait_bar(full_bar(stage), phase, abort_flag, p.status, 0x300u + B200_E_TIMEOUT)) { ok = false; break; }
#ifdef B200_TC_TIMING
                    dbg_mw += clock64() - tf0;
#endif
                    ptx::tc_fence_after();
                    // descriptors of this stage: the precomputed stage-0 descriptors plus the stage offset; only
                    // the 14-bit address field changes (shared memory ends below 256 KB, so it cannot carry out)
                    for (int m = 0; m < p.ksub; m++) {
                        const uint64_t so = (uint64_t)stage * stage16 + (uint64_t)m * mini16;
                        const uint64_t a_hi = a_hi0 + so, b_hi = b_hi0 + so;
#pragma unroll
                        for (int k = 0; k < 4; k++) {
                            const uint32_t acc_in = (step > 0 || m > 0 || k > 0) ? 1u : 0u;
                            if (X3) {
                                const uint64_t a_lo = a_lo0 + so, b_lo = b_lo0 + so;
                                issue(d_small, a_lo + k * ak16, b_hi + k * bk16, acc_in);      // small terms first
                                issue(d_small, a_hi + k * ak16, b_lo + k * bk16, 1u);
                                issue(d, a_hi + k * ak16, b_hi + k * bk16, p.small_off ? acc_in : 1u);
                            } else {
                                issue(d, a_hi + k * ak16, b_hi + k * bk16, acc_in);
                            }
                        }
                    }
                    if (CTAS == 2) ptx::mma_commit_pair(empty_bar(stage)); else ptx::mma_commit(empty_bar(stage));
                    if (++stage == p.stages) { stage = 0; phase ^= 1u; }
                }
                if (ok) { if (CTAS == 2) ptx::mma_commit_pair(tfull_bar(acc)); else ptx::mma_commit(tfull_bar(acc)); }
            }
#ifdef B200_TC_TIMING
            if (p.dbg) { p.dbg[blockIdx.x * 8 + 1] = dbg_mw; p.dbg[blockIdx.x * 8 + 2] = dbg_mt; p.dbg[blockIdx.x * 8 + 3] = clock64() - dbg_m0; }
#endif
        }
    } else {
        // ------------------------------------------------------------------ epilogue (warps 2..5)
        const int q = warp & 3;
        const int row = q * 32 + lane;
        // CONV: this thread's pixel inside a tile (the same for every tile)
        const int row_bx = MODE == MODE_CONV ? row % p.BW : 0;
        const int row_by = MODE == MODE_CONV ? (row / p.BW) % p.BH : 0;
        const int row_bi = MODE == MODE_CONV ? row / (p.BW * p.BH) : 0;
        int tile_iter = 0;
#ifdef B200_TC_TIMING
        long long dbg_ew = 0;
        const long long dbg_e0 = clock64();
#endif
        for (int tile = work_begin; tile < p.num_tiles; tile += work_step, tile_iter++) {
            const TileCtx c = (CTAS == 2 && MODE == MODE_CONV) ? decode_pair(p, tile, (int)rank) : decode_tile<MODE>(p, tile, (int)rank);
            const int acc = p.acc_stages == 2 ? (tile_iter & 1) : 0;
            const uint32_t acc_phase = (uint32_t)(p.acc_stages == 2 ? (tile_iter >> 1) : tile_iter) & 1u;
#ifdef B200_TC_TIMING
            const long long tq0 = clock64();
#endif
            bool ok = wait_bar(tfull_bar(acc), acc_phase, abort_flag, p.status, 0x400u + B200_E_TIMEOUT);
#ifdef B200_TC_TIMING
            dbg_ew += clock64() - tq0;
#endif
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            ptx::tc_fence_after();
            const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * p.acc_set_stride);
            float v[16];
            // 16 columns of the tile: the accumulator, plus in 3xTF32 mode the accumulator of the small terms
            auto load16 = [&](int c0) {
                ptx::tmem_ld16(taddr + c0, v);
                if (X3 && p.small_off) {
                    float u[16];
                    ptx::tmem_ld16(taddr + (uint32_t)p.small_off + c0, u);
#pragma unroll
                    for (int j = 0; j < 16; j++) v[j] = __fadd_rn(v[j], u[j]);
                }
            };
            if (MODE == MODE_CONV) {
                const PhaseInfo &pi = p.phase[c.ph];
                const int n = c.ig * p.BI + row_bi, yy = c.ty * p.BH + row_by, xx = c.tx * p.BW + row_bx;
                const bool valid = n < p.n_img && yy < pi.ext_y && xx < pi.ext_x;
                const size_t plane = (size_t)p.OH * p.OW;
                float *obase = p.ksplit > 1 ? p.kpartial + (size_t)c.split * (size_t)p.out_elems : p.out;
                const float *bias = p.ksplit > 1 ? nullptr : p.bias;       // split-K: bias and neuron function are applied by the reduction
                const size_t off = (size_t)n * p.k_out * plane + (size_t)(yy * p.out_stride_y + pi.off_y) * p.OW + (xx * p.out_stride_x + pi.off_x);
                float *dst = obase + off;
                float *pre = (!ACT || p.ksplit > 1 || !p.pre_out) ? nullptr : p.pre_out + off;
                const int func = (!ACT || p.ksplit > 1) ? -1 : p.act_func;
                for (int c0 = 0; ACT && c0 < p.BN; c0 += 16) {
                    load16(c0);
                    const int k0 = c.nt * p.BN + c0;
                    const int live = valid ? p.k_out - k0 : 0;
                    float *q0 = dst + (size_t)k0 * plane, *q1 = pre ? pre + (size_t)k0 * plane : nullptr;
#pragma unroll
                    for (int j = 0; j < 16; j++, q0 += plane) {
                        if (j < live) {
                            float val = bias ? __fadd_rn(v[j], __ldg(bias + k0 + j)) : v[j];
                            if (q1) q1[(size_t)j * plane] = val;
                            if (func >= 0) val = act_apply(val, func, p.act_slope);      // the function layer fused into the epilogue
                            *q0 = val;
                        }
                    }
                }
                if (!ACT && !(X3 && p.small_off)) {
                    // plain epilogue, software-pipelined: the tensor-memory load of the next 16 columns is in flight while
                    // the current 16 are stored (a load-wait-store sequence per 16 columns left the stores idle half the time)
                    uint32_t ra[16], rb[16];
                    // 16 columns = 16 channel planes of this thread's pixel: the plane pointer is stepped, the number of real
                    // columns is one subtraction, and the bias values come through the read-only path before the stores
                    auto store16 = [&](const uint32_t *r, int c0) {
                        const int k0 = c.nt * p.BN + c0;
                        const int live = valid ? p.k_out - k0 : 0;          // columns j < live are stored
                        if (live <= 0) return;
                        float *q0 = dst + (size_t)k0 * plane;
                        if (bias) {
                            float bv[16];
#pragma unroll
                            for (int j = 0; j < 16; j++) bv[j] = j < live ? __ldg(bias + k0 + j) : 0.f;
#pragma unroll
                            for (int j = 0; j < 16; j++, q0 += plane)
                                if (j < live) *q0 = __fadd_rn(__uint_as_float(r[j]), bv[j]);
                        } else {
#pragma unroll
                            for (int j = 0; j < 16; j++, q0 += plane)
                                if (j < live) *q0 = __uint_as_float(r[j]);
                        }
                    };
                    ptx::tmem_ld16_issue(taddr, ra);
                    for (int c0 = 0; c0 < p.BN; c0 += 32) {
                        ptx::tmem_ld_wait(ra);
                        if (c0 + 16 < p.BN) ptx::tmem_ld16_issue(taddr + c0 + 16, rb);
                        store16(ra, c0);
                        if (c0 + 16 < p.BN) {
                            ptx::tmem_ld_wait(rb);
                            if (c0 + 32 < p.BN) ptx::tmem_ld16_issue(taddr + c0 + 32, ra);
                            store16(rb, c0 + 16);
                        }
                    }
                } else if (!ACT) {
                    for (int c0 = 0; c0 < p.BN; c0 += 16) {
                        load16(c0);
#pragma unroll
                        for (int j = 0; j < 16; j++) {
                            const int k = c.nt * p.BN + c0 + j;
                            if (valid && k < p.k_out) dst[(size_t)k * plane] = bias ? __fadd_rn(v[j], bias[k]) : v[j];
                        }
                    }
                }
            } else if (MODE == MODE_WGRAD) {
                int f = c.ft * 128 + row, tap = c.tap;
                bool row_ok = f < p.k_rows;
                if (p.tapm) {
                    // packed taps: row = member * tapm + filter
                    const TapGroup &grp = p.groups[c.tap];
                    const int member = row / p.tapm;
                    f = row - member * p.tapm;
                    row_ok = member < grp.count && f < p.k_rows;
                    tap = grp.tap[member < grp.count ? member : 0];
                }
                float *dst = p.partial + (((size_t)c.split * p.taps_n + tap) * p.c_cols) * p.k_rows + f;
                for (int c0 = 0; c0 < p.BN; c0 += 16) {
                    load16(c0);
                    const int ch0 = c.ct * p.BN + c0;
                    const int live = row_ok ? p.c_cols - ch0 : 0;
                    float *q0 = dst + (size_t)ch0 * p.k_rows;
#pragma unroll
                    for (int j = 0; j < 16; j++, q0 += p.k_rows)
                        if (j < live) *q0 = v[j];
                }
            } else {
                const int m = c.mt * 128 + row;
                float *dst = (p.ksplit > 1 ? p.kpartial + (size_t)c.split * (size_t)p.out_elems : p.out) + (size_t)m * p.ldc + c.nt * p.BN;
                for (int c0 = 0; c0 < p.BN; c0 += 16) {
                    load16(c0);
#pragma unroll
                    for (int j = 0; j < 16; j++) {
                        const int n = c.nt * p.BN + c0 + j;
                        if (m < p.M && n < p.N) dst[c0 + j] = v[j];
                    }
                }
            }
            ptx::tc_fence_before();
            __syncwarp();
            if (lane == 0) { if (CTAS == 2) ptx::mbar_arrive_remote(tempty_bar(acc), 0u); else ptx::mbar_arrive(tempty_bar(acc)); }
        }
#ifdef B200_TC_TIMING
        if (threadIdx.x == 64 && p.dbg) { p.dbg[blockIdx.x * 8 + 4] = dbg_ew; p.dbg[blockIdx.x * 8 + 5] = clock64() - dbg_e0; }
#endif
    }

    if (*abort_flag) {   // give TMA copies still in flight time to land before the CTA's shared memory is released
        const long long t0 = clock64();
        while (clock64() - t0 < 200000) __nanosleep(200);
    }
    ptx::tc_fence_before();
    __syncthreads();
    if (CTAS == 2) ptx::cluster_sync();      // neither CTA leaves while its partner may still touch its shared memory or barriers
    if (warp == 1) {
        ptx::tc_fence_after();
        if (CTAS == 2) ptx::tmem_dealloc_pair(tmem_base, (uint32_t)p.tmem_cols);
        else ptx::tmem_dealloc(tmem_base, (uint32_t)p.tmem_cols);
    }
}

// ---------------------------------------------------------------------------------------------------
// operand packing (memory-bound pre-passes)
// ---------------------------------------------------------------------------------------------------

// NCHW fp32 -> phase-split NHWC, TF32-rounded high part and (optionally) TF32-rounded remainder:
//   dst[ph][n][h/sy][w/sx][c],  ph = (h % sy) * sx + (w % sx),  channel pitch Cp (multiple of 4).
// func >= 0: the neuron function is applied to every element on the way (the function layer in front of a convolution
// layer fused into the layer's pack); act_out, if given, also receives the activated tensor in the source layout.
__global__ void pack_act_kernel(const float *__restrict__ src, float *__restrict__ hi, float *__restrict__ lo,
                                int N, int C, int H, int W, int Cp, int sy, int sx, int Hs, int Ws, int func, double slope, float *__restrict__ act_out)
{
    grid_dependency_wait();
    __shared__ float tile[32][33];
    const int n = blockIdx.z, h = blockIdx.y, w0 = blockIdx.x * 32;
    const int tx = threadIdx.x, ty = threadIdx.y;
    const bool row_ok = h < H;
    const int hq = h / sy, hr = h % sy;
    for (int c0 = 0; c0 < Cp; c0 += 32) {
#pragma unroll
        for (int i = 0; i < 4; i++) {
            int c = c0 + ty + 8 * i, w = w0 + tx;
            float v = 0.f;
            if (row_ok && c < C && w < W) {
                const size_t at = (((size_t)n * C + c) * H + h) * W + w;
                v = src[at];
                if (func >= 0) { v = act_apply(v, func, slope); if (act_out) act_out[at] = v; }
            }
            tile[ty + 8 * i][tx] = v;
        }
        __syncthreads();
        const int c = c0 + tx;
        if (c < Cp) {
#pragma unroll
            for (int i = 0; i < 4; i++) {
                int wl = ty + 8 * i, w = w0 + wl;
                if (w < Ws * sx) {
                    int ph = hr * sx + (w % sx);
                    size_t o = ((((size_t)ph * N + n) * Hs + hq) * Ws + (w / sx)) * Cp + c;
                    float v = tile[tx][wl];
                    float vh = ptx::to_tf32(v);
                    hi[o] = vh;
                    if (lo) lo[o] = ptx::to_tf32(v - vh);
                }
            }
        }
        __syncthreads();
    }
}

// Same re-layout with 128-bit accesses: a block moves 4 rows x 32 pixels x 32 channels per iteration, per row one
// float4 load (4 pixels of one channel) and one float4 store per plane (4 channels of one pixel) per thread.  Needs
// W % 4 == 0 and a 16-byte aligned source.
// The four loads of an iteration are issued together: with one load in flight per thread the resident threads of an SM
// could not cover the latency of the memory, and the four rows of a channel are neighbours in the source (512 contiguous
// bytes for a 32-pixel row) instead of lone 128-byte pieces.
// (ROWS = 1 or 2 for tensors too small to give every block four rows: fewer registers, more resident blocks.)
constexpr int kPackRows = 4;
template <int ROWS>
__global__ void __launch_bounds__(256)
pack_act_vec_kernel(const float *__restrict__ src, float *__restrict__ hi, float *__restrict__ lo,
                    int N, int C, int H, int W, int Cp, int sy, int sx, int Hs, int Ws, int rows_per_block, float *__restrict__ rowsum,
                    int func, double slope, float *__restrict__ act_out)
{
    grid_dependency_wait();
    __shared__ float tile[ROWS][32][33];
    const int n = blockIdx.z, h0 = blockIdx.y * rows_per_block, w0 = blockIdx.x * 32;
    const int h1 = min(h0 + rows_per_block, Hs * sy);
    const int tid = threadIdx.x;
    const int lc = tid >> 3, lq = tid & 7;          // load role: channel lc of the chunk, pixel quad lq
    const int sp = tid >> 3, sq = tid & 7;          // store role: pixel sp of the tile, channel quad sq
    const int wl = w0 + 4 * lq;
    const int ws = w0 + sp;
    for (int c0 = 0; c0 < Cp; c0 += 32) {
        const int c = c0 + lc;
        const int cq = c0 + 4 * sq;
        float acc = 0.f;                            // this thread's share of the plane sum of channel c (bias gradient)
        for (int hb = h0; hb < h1; hb += ROWS) {
            float4 v[ROWS];
#pragma unroll
            for (int j = 0; j < ROWS; j++) {
                const int h = hb + j;
                v[j] = make_float4(0.f, 0.f, 0.f, 0.f);
                if (h < h1 && h < H && c < C && wl < W) v[j] = *reinterpret_cast<const float4 *>(src + (((size_t)n * C + c) * H + h) * W + wl);
            }
#pragma unroll
            for (int j = 0; j < ROWS; j++) {
                const int h = hb + j;
                if (func >= 0 && h < h1 && h < H && c < C && wl < W) {
                    v[j].x = act_apply(v[j].x, func, slope); v[j].y = act_apply(v[j].y, func, slope);
                    v[j].z = act_apply(v[j].z, func, slope); v[j].w = act_apply(v[j].w, func, slope);
                    if (act_out) *reinterpret_cast<float4 *>(act_out + (((size_t)n * C + c) * H + h) * W + wl) = v[j];
                }
                if (h >= h1) break;                     // the same for every thread of the block
                acc += (v[j].x + v[j].y) + (v[j].z + v[j].w);
                tile[j][lc][4 * lq + 0] = v[j].x; tile[j][lc][4 * lq + 1] = v[j].y; tile[j][lc][4 * lq + 2] = v[j].z; tile[j][lc][4 * lq + 3] = v[j].w;
            }
            __syncthreads();
            if (ws < Ws * sx && cq < Cp) {
#pragma unroll
                for (int j = 0; j < ROWS; j++) {
                    const int h = hb + j;
                    if (h >= h1) break;
                    const int hq = h / sy, hr = h % sy;
                    const int ph = hr * sx + (ws % sx);
                    const size_t obase = ((((size_t)ph * N + n) * Hs + hq) * Ws + (ws / sx)) * Cp;
                    float4 a = make_float4(tile[j][4 * sq + 0][sp], tile[j][4 * sq + 1][sp], tile[j][4 * sq + 2][sp], tile[j][4 * sq + 3][sp]);
                    float4 b = make_float4(ptx::to_tf32(a.x), ptx::to_tf32(a.y), ptx::to_tf32(a.z), ptx::to_tf32(a.w));
                    *reinterpret_cast<float4 *>(hi + obase + cq) = b;
                    if (lo)
                        *reinterpret_cast<float4 *>(lo + obase + cq) =
                            make_float4(ptx::to_tf32(a.x - b.x), ptx::to_tf32(a.y - b.y), ptx::to_tf32(a.z - b.z), ptx::to_tf32(a.w - b.w));
                }
            }
            __syncthreads();
        }
        if (rowsum) {
            // first stage of the bias gradient: the 8 threads that hold channel c are neighbours in a warp; one partial sum
            // per block and channel goes to rowsum[n][c][row group][x block]
            acc += __shfl_xor_sync(0xffffffffu, acc, 1);
            acc += __shfl_xor_sync(0xffffffffu, acc, 2);
            acc += __shfl_xor_sync(0xffffffffu, acc, 4);
            if (lq == 0 && c < C) rowsum[(((size_t)n * C + c) * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x] = acc;
        }
    }
}

// Weights [K][C][taps] -> rows x taps x inner (pitch ip):
//   forward  (rot = 0): dst[k][tap][c] = W[k][c][tap]
//   backward (rot = 1): dst[c][tap][k] = W[k][c][taps-1-tap]   (kernel rotated by 180 degrees)
__global__ void pack_weight_kernel(const float *__restrict__ src, float *__restrict__ hi, float *__restrict__ lo,
                                   int K, int C, int taps, int ip, int rot)
{
    grid_dependency_wait();
    const int rows = rot ? C : K, inner = rot ? K : C;
    const size_t total = (size_t)rows * taps * ip;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        int i = idx % ip;
        size_t t = idx / ip;
        int tap = t % taps;
        int r = t / taps;
        float v = 0.f;
        if (i < inner) v = rot ? src[((size_t)i * C + r) * taps + (taps - 1 - tap)] : src[((size_t)r * C + i) * taps + tap];
        float vh = ptx::to_tf32(v);
        hi[idx] = vh;
        if (lo) lo[idx] = ptx::to_tf32(v - vh);
    }
}

__global__ void split_tf32_kernel(const float *__restrict__ src, float *__restrict__ hi, float *__restrict__ lo, size_t n)
{
    grid_dependency_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        float v = src[i];
        float vh = ptx::to_tf32(v);
        hi[i] = vh;
        if (lo) lo[i] = ptx::to_tf32(v - vh);
    }
}

// two tensors in one launch: the first `blocks_a` blocks split a, the others b
__global__ void split_tf32_pair_kernel(const float *__restrict__ a, float *__restrict__ a_hi, float *__restrict__ a_lo, size_t na,
                                       const float *__restrict__ b, float *__restrict__ b_hi, float *__restrict__ b_lo, size_t nb, int blocks_a)
{
    grid_dependency_wait();
    const bool first = (int)blockIdx.x < blocks_a;
    const float *src = first ? a : b;
    float *hi = first ? a_hi : b_hi, *lo = first ? a_lo : b_lo;
    const size_t n = first ? na : nb;
    const size_t block = first ? blockIdx.x : blockIdx.x - blocks_a, blocks = first ? blocks_a : gridDim.x - blocks_a;
    for (size_t i = block * blockDim.x + threadIdx.x; i < n; i += blocks * blockDim.x) {
        const float v = src[i];
        const float vh = ptx::to_tf32(v);
        hi[i] = vh;
        if (lo) lo[i] = ptx::to_tf32(v - vh);
    }
}

// dkernel[f][c*taps + tap] (+)= sum over splits (in increasing order) of partial[split][tap][c][f]
__global__ void wgrad_reduce_kernel(float *__restrict__ dkernel, const float *__restrict__ partial, int splits, int taps,
                                    int C, int K, int accumulate)
{
    grid_dependency_wait();
    const size_t total = (size_t)K * C * taps;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        // idx enumerates (tap, c, f) with f fastest so that the reads are coalesced
        int f = idx % K;
        size_t t = idx / K;
        int c = t % C;
        int tap = t / C;
        float s = 0.f;
        for (int sp = 0; sp < splits; sp++) s += partial[(((size_t)sp * taps + tap) * C + c) * K + f];
        size_t o = ((size_t)f * C + c) * taps + tap;
        dkernel[o] = accumulate ? dkernel[o] + s : s;
    }
}

// out[i] = sum over the K splits (in increasing order) of partial[split][i] (+ bias of the element's channel)
__global__ void conv_ksplit_reduce_kernel(float *__restrict__ out, const float *__restrict__ partial, int splits, size_t total,
                                          const float *__restrict__ bias, int k_out, size_t plane, int func = -1, double slope = 0.0,
                                          float *__restrict__ pre = nullptr)
{
    grid_dependency_wait();
    const size_t total4 = total / 4;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total4; i += (size_t)gridDim.x * blockDim.x) {
        float4 s = reinterpret_cast<const float4 *>(partial)[i];
        for (int sp = 1; sp < splits; sp++) {
            const float4 v = reinterpret_cast<const float4 *>(partial + (size_t)sp * total)[i];
            s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
        }
        if (bias) {
            const size_t e = i * 4;
            s.x += bias[(e / plane) % k_out]; s.y += bias[((e + 1) / plane) % k_out];
            s.z += bias[((e + 2) / plane) % k_out]; s.w += bias[((e + 3) / plane) % k_out];
        }
        if (pre) reinterpret_cast<float4 *>(pre)[i] = s;
        if (func >= 0) { s.x = act_apply(s.x, func, slope); s.y = act_apply(s.y, func, slope); s.z = act_apply(s.z, func, slope); s.w = act_apply(s.w, func, slope); }
        reinterpret_cast<float4 *>(out)[i] = s;
    }
}

// The same reduction through a shared-memory tile, so that both sides are coalesced: a block owns 32 filters x
// c_run channels x all taps; it reads runs of 32 consecutive filters (128 bytes) per (tap, channel) and writes, per
// filter, the run of c_run*taps consecutive weights.  Splits are added in increasing order as above.
__global__ void wgrad_reduce_tiled_kernel(float *__restrict__ dkernel, const float *__restrict__ partial, int splits, int taps,
                                          int C, int K, int c_run, int accumulate)
{
    grid_dependency_wait();
    extern __shared__ float tile[];                       // [tap][c_run][33]
    const int c_tiles = (C + c_run - 1) / c_run;
    const int f0 = (blockIdx.x / c_tiles) * 32, c0 = (blockIdx.x % c_tiles) * c_run;
    const int cn = min(c_run, C - c0), fn = min(32, K - f0);
    const size_t split_stride = (size_t)taps * C * K;
    if ((K & 3) == 0) {
        // 16-byte loads along the filters (rows of K floats are 16-byte aligned when K is a multiple of 4)
        for (int e = threadIdx.x; e < taps * cn * 8; e += blockDim.x) {
            const int fl = (e & 7) * 4, r = e >> 3, cl = r % cn, tap = r / cn;
            if (fl < fn) {
                const float4 *src = reinterpret_cast<const float4 *>(partial + ((size_t)tap * C + c0 + cl) * K + f0 + fl);
                float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
                for (int sp = 0; sp < splits; sp++) {
                    const float4 v = src[sp * (split_stride >> 2)];
                    sum.x += v.x; sum.y += v.y; sum.z += v.z; sum.w += v.w;
                }
                float *t = &tile[(tap * c_run + cl) * 33 + fl];
                t[0] = sum.x; t[1] = sum.y; t[2] = sum.z; t[3] = sum.w;
            }
        }
    } else {
        for (int e = threadIdx.x; e < taps * cn * 32; e += blockDim.x) {
            const int fl = e & 31, r = e >> 5, cl = r % cn, tap = r / cn;
            if (fl < fn) {
                const float *src = partial + ((size_t)tap * C + c0 + cl) * K + f0 + fl;
                float sum = 0.f;
                for (int sp = 0; sp < splits; sp++) sum += src[sp * split_stride];
                tile[(tap * c_run + cl) * 33 + fl] = sum;
            }
        }
    }
    __syncthreads();
    const int run = cn * taps;
    for (int e = threadIdx.x; e < fn * run; e += blockDim.x) {
        const int j = e % run, fl = e / run, cl = j / taps, tap = j - cl * taps;
        const size_t o = ((size_t)(f0 + fl) * C + c0) * taps + j;
        const float v = tile[(tap * c_run + cl) * 33 + fl];
        dkernel[o] = accumulate ? dkernel[o] + v : v;
    }
}

// ---------------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn()
{
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    }
    return fn;
}

// 5-D fp32 tensor map with 128-byte swizzle (32-byte atoms when the operand is MN-major); dims[0] is the contiguous dimension, pitch[i] is the
// stride of dimension i+1 in ELEMENTS.  Unused trailing dimensions have size 1.
static int make_map(CUtensorMap *m, const float *base, const long long dims[5], const long long pitch[4], const int box[5],
                    bool mn_major = false)
{
    EncodeTiledFn fn = encode_fn();
    if (!fn) return fail(B200_E_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    cuuint64_t gd[5], gs[4];
    cuuint32_t bx[5], es[5];
    for (int i = 0; i < 5; i++) { gd[i] = (cuuint64_t)dims[i]; bx[i] = (cuuint32_t)box[i]; es[i] = 1; }
    for (int i = 0; i < 4; i++) gs[i] = (cuuint64_t)pitch[i] * sizeof(float);
    CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 5, const_cast<float *>(base), gd, gs, bx, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    mn_major ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return fail(B200_E_CUDA, "cuTensorMapEncodeTiled failed (%d) dims %lld %lld %lld %lld %lld box %d %d %d %d %d", (int)r,
                    dims[0], dims[1], dims[2], dims[3], dims[4], box[0], box[1], box[2], box[3], box[4]);
    return B200_OK;
}

// Tensor map of an MN-major operand stored as [rows...][E] (E contiguous elements per row, pitch
// `pitch0`): dimension 0 is a 32-element block of E, dimension 4 the block index (stride 128 bytes), so
// a box {32, b1, b2, b3, nblocks} lands in shared memory as nblocks consecutive [rows][32] blocks.  The
// last block may reach past E (into the next row, by at most 31 elements past the end of the buffer,
// which the caller pads): those elements only ever meet zero-filled or masked partners.
static int make_blocked_map(CUtensorMap *m, const float *base, long long E, const long long dims123[3], const long long pitch[3],
                            const int box123[3], int nblocks_box)
{
    const long long dims[5] = {32, dims123[0], dims123[1], dims123[2], (E + 31) / 32};
    const long long pit[4] = {pitch[0], pitch[1], pitch[2], 32};
    const int box[5] = {32, box123[0], box123[1], box123[2], nblocks_box};
    return make_map(m, base, dims, pit, box, true);
}

static int pow2_ceil(int v) { int p = 1; while (p < v) p <<= 1; return p; }
static int floor_div(int a, int b) { int q = a / b; if ((a % b != 0) && ((a < 0) != (b < 0))) q--; return q; }
static int pos_mod(int a, int b) { int r = a % b; return r < 0 ? r + b : r; }

// Host-visible status word of the current device (pinned, mapped): device-side waits that give up
// write a code here; the library reads it without synchronising.
static unsigned *g_status_host[64];
static unsigned *g_status_dev[64];

int status_word(unsigned **dev)
{
    int d = 0;
    cudaGetDevice(&d);
    if (d < 0 || d >= 64) d = 0;
    if (!g_status_host[d]) {
        void *h = nullptr, *dp = nullptr;
        B200_CUDA(cudaHostAlloc(&h, sizeof(unsigned), cudaHostAllocMapped));
        *(unsigned *)h = 0;
        B200_CUDA(cudaHostGetDevicePointer(&dp, h, 0));
        g_status_host[d] = (unsigned *)h;
        g_status_dev[d] = (unsigned *)dp;
    }
    *dev = g_status_dev[d];
    return B200_OK;
}

unsigned tc_read_status(int clear)
{
    int d = 0;
    cudaGetDevice(&d);
    if (d < 0 || d >= 64 || !g_status_host[d]) return 0;
    unsigned v = *(volatile unsigned *)g_status_host[d];
    if (clear) *(volatile unsigned *)g_status_host[d] = 0;
    return v;
}

void tc_write_status(unsigned code)
{
    int d = 0;
    cudaGetDevice(&d);
    if (d < 0 || d >= 64 || !g_status_host[d]) return;
    *(volatile unsigned *)g_status_host[d] = code;
}

static size_t g_smem_optin_dev[64];

// Optional timing of the tensor-core kernel alone: a pair of events around every launch, read back
// by tc_profile_read().  Used by the benchmark to put a live duration under the roofline figure.
struct EventPair { cudaEvent_t a, b; };
static bool g_profile = false;
static std::vector<EventPair> g_pending, g_pool;

void tc_profile_enable(int on) { g_profile = on != 0; }

int tc_profile_read(double *total_ms, int *launches)
{
    double ms = 0;
    int n = 0;
    for (EventPair &e : g_pending) {
        float t = 0.f;
        B200_CUDA(cudaEventSynchronize(e.b));
        B200_CUDA(cudaEventElapsedTime(&t, e.a, e.b));
        ms += t;
        n++;
        g_pool.push_back(e);
    }
    g_pending.clear();
    if (total_ms) *total_ms = ms;
    if (launches) *launches = n;
    return B200_OK;
}

static int profile_begin(EventPair *e, cudaStream_t s)
{
    if (g_pool.empty()) {
        B200_CUDA(cudaEventCreate(&e->a));
        B200_CUDA(cudaEventCreate(&e->b));
    } else {
        *e = g_pool.back();
        g_pool.pop_back();
    }
    B200_CUDA(cudaEventRecord(e->a, s));
    return B200_OK;
}

// Debug switch: B200CONV_DEEP_STAGES=0 keeps one 32-wide K block per pipeline stage.
static bool deep_stages_enabled()
{
    static int v = -1;
    if (v < 0) {
        const char *e = getenv("B200CONV_DEEP_STAGES");
        v = (e && e[0] == '0') ? 0 : 1;
    }
    return v == 1;
}

template <int MODE, bool X3, int CTAS, bool ACT = false>
static int launch_one(const CUtensorMap maps[4], const TcParams &p, int grid, size_t smem, cudaStream_t s)
{
    if (MODE == MODE_CONV && !ACT && p.ksplit <= 1 && (p.act_func >= 0 || p.pre_out)) return launch_one<MODE, X3, CTAS, MODE == MODE_CONV>(maps, p, grid, smem, s);
    B200_CUDA(cudaFuncSetAttribute(tc_kernel<MODE, X3, CTAS, ACT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    Launch(dim3(grid), dim3(kThreads), smem, s).cluster(CTAS)(tc_kernel<MODE, X3, CTAS, ACT>, maps[0], maps[X3 ? 1 : 0], maps[2], maps[X3 ? 3 : 2], p);
    B200_CUDA(take_launch_error());
    return B200_OK;
}

// p.num_tiles counts work items: tiles (ctas == 1) or tile pairs (ctas == 2, one cluster of two CTAs each).
template <int MODE>
static int launch_tc(const CUtensorMap maps[4], TcParams &p, bool x3, cudaStream_t s, int ctas = 1)
{
    int cur = 0;
    cudaGetDevice(&cur);
    if (cur < 0 || cur >= 64) cur = 0;
    if (!g_smem_optin_dev[cur]) {
        int v = 0;
        B200_CUDA(cudaDeviceGetAttribute(&v, cudaDevAttrMaxSharedMemoryPerBlockOptin, cur));
        g_smem_optin_dev[cur] = (size_t)v;
    }
    const size_t g_smem_optin = g_smem_optin_dev[cur];
    p.b_bytes = (uint32_t)p.b_boxes * p.b_box_bytes;
    p.mini_bytes = (uint32_t)((kABytes + p.b_bytes) * (x3 ? 2 : 1));
    const size_t fixed = 1024 /*alignment slack*/ + 256 /*barriers*/;
    // two K blocks per stage halve the per-stage hand-shakes; taken when at least three such stages fit
    p.ksub = (deep_stages_enabled() && (g_smem_optin - fixed) / (2 * (size_t)p.mini_bytes) >= 3) ? 2 : 1;
    p.stage_bytes = p.mini_bytes * (uint32_t)p.ksub;
    int stages = (int)((g_smem_optin - fixed) / p.stage_bytes);
    if (stages > 8) stages = 8;
    if (stages < 2) return TC_UNSUPPORTED;
    p.stages = stages;
    // tensor memory: two accumulator sets so that the epilogue overlaps the next tile's main loop; a 3xTF32 set holds two
    // accumulators (large term, small terms), so the widest tile (256 columns) leaves room for one set only
    // (the separate accumulator costs the 256-column tile its epilogue overlap: +11 % kernel time on the benchmark layer for a
    // third of the accumulation error, so it is an option: B200CONV_X3_SPLIT_ACC=1)
    static const bool split_acc = getenv("B200CONV_X3_SPLIT_ACC") && getenv("B200CONV_X3_SPLIT_ACC")[0] == '1';
    p.small_off = (x3 && split_acc) ? p.acc_stride : 0;
    p.acc_set_stride = p.small_off ? 2 * p.acc_stride : p.acc_stride;
    p.acc_stages = 2 * p.acc_set_stride <= 512 ? 2 : 1;
    int cols = p.acc_stages * p.acc_set_stride;
    if (cols < 32) cols = 32;
    p.tmem_cols = cols;
    int r = status_word(&p.status);
    if (r) return r;
#ifdef B200_TC_TIMING
    static long long *dbg_dev = nullptr;
    if (!dbg_dev) { cudaMalloc(&dbg_dev, 8 * 256 * sizeof(long long)); }
    cudaMemsetAsync(dbg_dev, 0, 8 * 256 * sizeof(long long), s);
    p.dbg = dbg_dev;
#endif
    const size_t smem = (size_t)stages * p.stage_bytes + fixed;
    const int slots = sm_count() / ctas;
    int grid = (p.num_tiles < slots ? p.num_tiles : slots) * ctas;
    if (grid < 1) return B200_OK;
    EventPair ev;
    if (g_profile && (r = profile_begin(&ev, s))) return r;
    if (ctas == 2) {
        if (MODE == MODE_GEMM) return fail(B200_E_ARG, "no CTA-pair kernel for the plain GEMM");
        constexpr int M2 = MODE == MODE_GEMM ? MODE_CONV : MODE;
        r = x3 ? launch_one<M2, true, 2>(maps, p, grid, smem, s) : launch_one<M2, false, 2>(maps, p, grid, smem, s);
    } else {
        r = x3 ? launch_one<MODE, true, 1>(maps, p, grid, smem, s) : launch_one<MODE, false, 1>(maps, p, grid, smem, s);
    }
    if (r) return r;
    B200_LAUNCH_CHECK();
    if (g_profile) {
        B200_CUDA(cudaEventRecord(ev.b, s));
        g_pending.push_back(ev);
    }
#ifdef B200_TC_TIMING
    if (getenv("B200_TC_TIMING_DUMP")) {
        static long long h[8 * 256];
        cudaStreamSynchronize(s);
        cudaMemcpy(h, dbg_dev, sizeof(h), cudaMemcpyDeviceToHost);
        double sum[6] = {0, 0, 0, 0, 0, 0};
        for (int b = 0; b < grid; b++) for (int i = 0; i < 6; i++) sum[i] += (double)h[b * 8 + i];
        fprintf(stderr, "tc timing mode=%d ctas=%d ksub=%d stages=%d grid=%d tiles=%d: producer wait %.0f | issuer: wait data %.0f, wait tmem %.0f, total %.0f | epilogue: wait %.0f total %.0f (cycles, mean per CTA)\n",
                MODE, ctas, p.ksub, p.stages, grid, p.num_tiles, sum[0] / grid * (ctas == 2 ? 1 : 1), sum[1] / (grid / ctas), sum[2] / (grid / ctas), sum[3] / (grid / ctas), sum[4] / grid, sum[5] / grid);
    }
#endif
    return B200_OK;
}

// Debug switch: B200CONV_CTA_PAIRS=0 in the environment keeps the convolution on single-CTA tiles.
static bool cta_pairs_enabled()
{
    static int v = -1;
    if (v < 0) {
        const char *e = getenv("B200CONV_CTA_PAIRS");
        v = (e && e[0] == '0') ? 0 : 1;
    }
    return v == 1;
}

static void set_kmajor(TcParams &p, bool a_side, int rows)
{
    if (a_side) { p.a_boxes = 1; p.a_box_bytes = kABytes; p.a_lbo = 16; p.a_sbo = 1024; p.a_kadv = 32; p.a_layout = 2; }
    else { p.b_boxes = 1; p.b_box_bytes = (uint32_t)rows * 128; p.b_lbo = 16; p.b_sbo = 1024; p.b_kadv = 32; p.b_layout = 2; }
}
static void set_mnmajor(TcParams &p, bool a_side, int extent)
{
    // MN-major 32-bit operands: 32 elements (128 B) contiguous along M/N per k-row, rows 128 B apart,
    // swizzled in 32-byte atoms over groups of 4 rows (SBO = 512 B between groups); a block of
    // 32 k-rows x 32 elements is 4 KB, blocks follow each other along M/N (LBO); one MMA eats 8 rows.
    // All 32-element blocks of an operand arrive in ONE box: the tensor map carries the block index
    // as an extra dimension with a 128-byte stride (see make_blocked_map), the box is 32 x 32 x blocks.
    if (a_side) { p.a_boxes = 1; p.a_box_bytes = 4 * 4096; p.a_lbo = 4096; p.a_sbo = 512; p.a_kadv = 1024; p.a_layout = 1; }
    else { p.b_boxes = 1; p.b_box_bytes = (uint32_t)(extent / 32) * 4096; p.b_lbo = 4096; p.b_sbo = 512; p.b_kadv = 1024; p.b_layout = 1; }
}

// rowsum (optional, act_pack_rowsum_elems floats): receives per-block partial plane sums when the vector kernel runs;
// *rowsum_runs tells the caller how many partial sums each (image, channel) got (0: not produced).
static int pack_act(const float *src, float *hi, float *lo, int N, int C, int H, int W, int Cp, int sy, int sx, int Hs, int Ws,
                    cudaStream_t s, float *rowsum = nullptr, int *rowsum_runs = nullptr, const PackFunction *pf = nullptr)
{
    const int func = pf ? pf->func : -1;
    const double slope = pf ? pf->slope : 0.0;
    float *act_out = pf ? pf->act_out : nullptr;
    // An unsplit pack is the same re-layout for any way of cutting the H*W pixels of a plane into rows: [n][y][x][c] and
    // [n][c][y][x] are both linear in y*W + x.  Rows of exactly 32 pixels fill the kernel's tile, and the rows a block moves
    // together are then neighbours in memory; failing that, a narrow image becomes a single row (narrow rows would leave most
    // of a tile idle).
    if (sy == 1 && sx == 1 && H > 1) {
        const long long px = (long long)H * W;
        if (px % 32 == 0 && px / 32 <= 65535) { H = (int)(px / 32); W = 32; Hs = H; Ws = W; }
        else if (W < 32 && W % 4 == 0) { W = (int)px; Ws = W; H = 1; Hs = 1; }
    }
    dim3 grid(ceil_div(Ws * sx, 32), Hs * sy, N), block(32, 8);
    if (grid.y > 65535 || grid.z > 65535) return TC_UNSUPPORTED;
    if (rowsum_runs) *rowsum_runs = 0;
    if (W % 4 == 0 && ((uintptr_t)src & 15) == 0 && ((uintptr_t)act_out & 15) == 0) {
        // a block walks 4 rows, one iteration per channel chunk (8 with the bias-gradient sums fused in: one partial sum per 8
        // rows and channel); fewer when that would leave the grid short of a few waves of blocks
        int rows_per_block = rowsum ? 8 : kPackRows;
        while (rows_per_block > 1 && (long long)grid.x * ceil_div((int)grid.y, rows_per_block) * N < 16LL * sm_count()) rows_per_block /= 2;
        dim3 vgrid(grid.x, ceil_div((int)grid.y, rows_per_block), N);
        if (rows_per_block >= 4) Launch(vgrid, 256, 0, s)(pack_act_vec_kernel<4>, src, hi, lo, N, C, H, W, Cp, sy, sx, Hs, Ws, rows_per_block, rowsum, func, slope, act_out);
        else if (rows_per_block == 2) Launch(vgrid, 256, 0, s)(pack_act_vec_kernel<2>, src, hi, lo, N, C, H, W, Cp, sy, sx, Hs, Ws, rows_per_block, rowsum, func, slope, act_out);
        else Launch(vgrid, 256, 0, s)(pack_act_vec_kernel<1>, src, hi, lo, N, C, H, W, Cp, sy, sx, Hs, Ws, rows_per_block, rowsum, func, slope, act_out);
        if (rowsum && rowsum_runs) *rowsum_runs = (int)(vgrid.x * vgrid.y);
    } else
        Launch(grid, block, 0, s)(pack_act_kernel, src, hi, lo, N, C, H, W, Cp, sy, sx, Hs, Ws, func, slope, act_out);
    B200_LAUNCH_CHECK();
    return B200_OK;
}

// dbias[c] (+)= sum over images and partial sums of rowsum[n][c][runs]; one block per channel, its threads stride over the
// (image, partial sum) pairs and combine in a fixed shuffle / shared-memory tree (reproducible run to run)
__global__ void __launch_bounds__(256) dbias_from_rowsums_kernel(float *__restrict__ dbias, const float *__restrict__ rowsum, int N, int C, int runs,
                                                                 int accumulate)
{
    grid_dependency_wait();
    __shared__ float part[8];
    const int c = blockIdx.x;
    const int total = N * runs;
    float s = 0.f;
    for (int j = threadIdx.x; j < total; j += 256) {
        const int n = j / runs, r = j - n * runs;
        s += rowsum[((size_t)n * C + c) * runs + r];
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = s;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = part[0];
        for (int w = 1; w < 8; w++) t += part[w];
        dbias[c] = accumulate ? dbias[c] + t : t;
    }
}

size_t act_pack_rowsum_elems(const ActPack &pk)
{
    return (size_t)pk.n * pk.c * (size_t)(pk.hs * pk.sy) * ceil_div(pk.ws * pk.sx, 32);      // an upper bound: one sum per row
}

int act_pack_fill_with_sums(const ActPack &pk, const float *src, float *rowsum, int *runs, cudaStream_t s)
{
    return pack_act(src, pk.hi, pk.lo, pk.n, pk.c, pk.h, pk.w, pk.cp, pk.sy, pk.sx, pk.hs, pk.ws, s, rowsum, runs);
}

int dbias_from_rowsums(float *dbias, int accumulate, const float *rowsum, int batch, int K, int runs, cudaStream_t s)
{
    Launch(K, 256, 0, s)(dbias_from_rowsums_kernel, dbias, rowsum, batch, K, runs, accumulate);
    B200_LAUNCH_CHECK();
    return B200_OK;
}

// The same re-layout through a shared-memory tile: a block owns one output row r and 32 inner indices i; it reads the
// taps of each (r, i) pair as one contiguous run and writes, per tap, 32 consecutive inner elements (128 bytes).
__device__ __forceinline__ void pack_weight_tile(int block, const float *__restrict__ src, float *__restrict__ hi, float *__restrict__ lo,
                                                                int K, int C, int taps, int ip, int rot, float (*tile)[kMaxTaps + 1])
{
    const int inner = rot ? K : C;
    const int chunks = (ip + 31) / 32;
    const int r = block / chunks, i0 = (block % chunks) * 32;
    for (int e = threadIdx.x; e < 32 * taps; e += blockDim.x) {
        const int il = e / taps, tp = e - il * taps;
        const int i = i0 + il;
        float v = 0.f;
        if (i < inner) v = rot ? src[((size_t)i * C + r) * taps + tp] : src[((size_t)r * C + i) * taps + tp];
        tile[il][tp] = v;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < 32 * taps; e += blockDim.x) {
        const int tp = e >> 5, il = e & 31;
        const int i = i0 + il;
        if (i >= ip) continue;
        const float v = tile[il][rot ? taps - 1 - tp : tp];
        const float vh = ptx::to_tf32(v);
        const size_t o = ((size_t)r * taps + tp) * ip + i;
        hi[o] = vh;
        if (lo) lo[o] = ptx::to_tf32(v - vh);
    }
}

__global__ void __launch_bounds__(256) pack_weight_tiled_kernel(const float *__restrict__ src, float *__restrict__ hi, float *__restrict__ lo,
                                                                int K, int C, int taps, int ip, int rot)
{
    grid_dependency_wait();
    __shared__ float tile[32][kMaxTaps + 1];
    pack_weight_tile(blockIdx.x, src, hi, lo, K, C, taps, ip, rot, tile);
}

// Both orientations in one launch: the first n_forward blocks write the forward pack, the others the rotated one.
__global__ void __launch_bounds__(256) pack_weight_both_kernel(const float *__restrict__ src, float *__restrict__ f_hi, float *__restrict__ f_lo,
                                                               float *__restrict__ b_hi, float *__restrict__ b_lo, int K, int C, int taps, int ip_f,
                                                               int ip_b, int n_forward)
{
    grid_dependency_wait();
    __shared__ float tile[32][kMaxTaps + 1];
    if ((int)blockIdx.x < n_forward) pack_weight_tile(blockIdx.x, src, f_hi, f_lo, K, C, taps, ip_f, 0, tile);
    else pack_weight_tile(blockIdx.x - n_forward, src, b_hi, b_lo, K, C, taps, ip_b, 1, tile);
}

// Both orientations of the weights of up to kMaxPackJobs layers in one launch (the layers of a net packed together at the
// start of a training step instead of one launch per layer).
__global__ void __launch_bounds__(256) pack_weight_many_kernel(const __grid_constant__ WeightPackJobs jobs)
{
    grid_dependency_wait();
    __shared__ float tile[32][kMaxTaps + 1];
    int j = 0;
    while (j + 1 < jobs.count && (int)blockIdx.x >= jobs.job[j + 1].block_begin) j++;
    const WeightPackJob &w = jobs.job[j];
    const int b = (int)blockIdx.x - w.block_begin;
    if (b < w.n_forward) pack_weight_tile(b, w.src, w.f_hi, w.f_lo, w.K, w.C, w.taps, w.ip_f, 0, tile);
    else pack_weight_tile(b - w.n_forward, w.src, w.b_hi, w.b_lo, w.K, w.C, w.taps, w.ip_b, 1, tile);
}

bool weight_pack_job(const b200_conv_geom &g, const float *kernel, float *f_hi, float *f_lo, float *b_hi, float *b_lo, WeightPackJob *job)
{
    const int taps = g.kernel_x * g.kernel_y;
    if (taps < 2 || taps > kMaxTaps) return false;
    job->src = kernel; job->f_hi = f_hi; job->f_lo = f_lo; job->b_hi = b_hi; job->b_lo = b_lo;
    job->K = g.kernel_amount; job->C = g.in_z; job->taps = taps;
    job->ip_f = (int)align_up(g.in_z, 4); job->ip_b = (int)align_up(g.kernel_amount, 4);
    job->n_forward = g.kernel_amount * ((job->ip_f + 31) / 32);
    job->blocks = job->n_forward + g.in_z * ((job->ip_b + 31) / 32);
    job->block_begin = 0;
    return true;
}

int weight_pack_fill_many(WeightPackJobs &jobs, cudaStream_t s)
{
    int total = 0;
    for (int i = 0; i < jobs.count; i++) { jobs.job[i].block_begin = total; total += jobs.job[i].blocks; }
    if (!total) return B200_OK;
    Launch(total, 256, 0, s)(pack_weight_many_kernel, jobs);
    B200_LAUNCH_CHECK();
    return B200_OK;
}

static int pack_weight(const float *src, float *hi, float *lo, int K, int C, int taps, int ip, int rot, cudaStream_t s)
{
    if (taps > 1 && taps <= kMaxTaps) {
        const int rows = rot ? C : K;
        Launch(rows * ((ip + 31) / 32), 256, 0, s)(pack_weight_tiled_kernel, src, hi, lo, K, C, taps, ip, rot);
        B200_LAUNCH_CHECK();
        return B200_OK;
    }
    size_t total = (size_t)(rot ? C : K) * taps * ip;
    int grid = (int)((total + 255) / 256);
    if (grid > sm_count() * 16) grid = sm_count() * 16;
    Launch(grid, 256, 0, s)(pack_weight_kernel, src, hi, lo, K, C, taps, ip, rot);
    B200_LAUNCH_CHECK();
    return B200_OK;
}

static bool geom_supported(const b200_conv_geom &g)
{
    if (g.kernel_x * g.kernel_y > kMaxTaps) return false;
    if (g.stride_x * g.stride_y > kMaxPhases) return false;
    if (g.kernel_x > 100 || g.kernel_y > 100 || g.padding_x > 100 || g.padding_y > 100) return false;   // tap offsets are int8
    return true;
}

// M-tile shape: 128 output positions as a BI x BH x BW box over (image, row, column).
static void tile_shape(int ext_y, int ext_x, int target, int *BW, int *BH, int *BI)
{
    *BW = pow2_ceil(ext_x) < target ? pow2_ceil(ext_x) : target;
    int rest = target / *BW;
    *BH = pow2_ceil(ext_y) < rest ? pow2_ceil(ext_y) : rest;
    *BI = rest / *BH;
}

// ---------------------------------------------------------------------------------------------------
// packed operands
// ---------------------------------------------------------------------------------------------------

// Shape of the phase-split NHWC pack of an n x c x h x w tensor gathered with stride (sy, sx).
ActPack act_pack_shape(int n, int c, int h, int w, int sy, int sx)
{
    ActPack pk;
    pk.n = n; pk.c = c; pk.h = h; pk.w = w; pk.sy = sy; pk.sx = sx;
    pk.cp = (int)align_up(c, 4);
    pk.hs = ceil_div(h, sy); pk.ws = ceil_div(w, sx);
    return pk;
}

int act_pack_fill(const ActPack &pk, const float *src, cudaStream_t s, const PackFunction *pf)
{
    return pack_act(src, pk.hi, pk.lo, pk.n, pk.c, pk.h, pk.w, pk.cp, pk.sy, pk.sx, pk.hs, pk.ws, s, nullptr, nullptr, pf);
}

size_t weight_pack_elems(const b200_conv_geom &g, bool backward)
{
    const int taps = g.kernel_x * g.kernel_y;
    return backward ? (size_t)g.in_z * taps * align_up(g.kernel_amount, 4) : (size_t)g.kernel_amount * taps * align_up(g.in_z, 4);
}

int weight_pack_fill_both(const b200_conv_geom &g, const float *kernel, float *f_hi, float *f_lo, float *b_hi, float *b_lo, cudaStream_t s)
{
    const int taps = g.kernel_x * g.kernel_y;
    const int ip_f = (int)align_up(g.in_z, 4), ip_b = (int)align_up(g.kernel_amount, 4);
    if (taps < 2 || taps > kMaxTaps) {
        int r = pack_weight(kernel, f_hi, f_lo, g.kernel_amount, g.in_z, taps, ip_f, 0, s);
        return r ? r : pack_weight(kernel, b_hi, b_lo, g.kernel_amount, g.in_z, taps, ip_b, 1, s);
    }
    const int n_f = g.kernel_amount * ((ip_f + 31) / 32), n_b = g.in_z * ((ip_b + 31) / 32);
    Launch(n_f + n_b, 256, 0, s)(pack_weight_both_kernel, kernel, f_hi, f_lo, b_hi, b_lo, g.kernel_amount, g.in_z, taps, ip_f, ip_b, n_f);
    B200_LAUNCH_CHECK();
    return B200_OK;
}

int weight_pack_fill(const b200_conv_geom &g, bool backward, const float *kernel, float *hi, float *lo, cudaStream_t s)
{
    const int taps = g.kernel_x * g.kernel_y;
    const int ip = (int)align_up(backward ? g.kernel_amount : g.in_z, 4);
    return pack_weight(kernel, hi, lo, g.kernel_amount, g.in_z, taps, ip, backward ? 1 : 0, s);
}

// Forward convolution, or one backward-data convolution, on packed operands: `act` is the packed
// tensor that is gathered (image, split by the stride, for the forward pass; delta, unsplit, for the
// backward pass), w_hi/w_lo the matching weight pack, `out` the NCHW tensor produced.
// Upper bound of the split-K scratch conv_gemm may use for this problem, in floats (0: the output is large enough that its
// tiles fill the GPU and no split is considered).
size_t conv_gemm_partial_elems(bool backward, const b200_conv_geom &g, int batch)
{
    const int k_out = backward ? g.in_z : g.kernel_amount;
    const size_t pixels = (size_t)batch * (backward ? (size_t)g.in_y * g.in_x : (size_t)g.out_y * g.out_x);
    const size_t out_elems = pixels * k_out;
    // a problem whose widest tiles already give every SM two work items gains nothing from a split: no scratch for it
    if (((pixels + 127) / 128) * (size_t)ceil_div(k_out, 256) >= 2 * (size_t)sm_count()) return 0;
    return out_elems * sizeof(float) <= (16u << 20) ? 8 * out_elems : 0;
}

int conv_gemm(bool backward, const b200_conv_geom &g, float *out, const ActPack &act, const float *w_hi, const float *w_lo,
              const float *bias, bool x3, cudaStream_t s, float *kpartial, size_t kpartial_elems, const EpilogueFunction *ef)
{
    if (!geom_supported(g)) return TC_UNSUPPORTED;
    const int batch = act.n;
    const int taps = g.kernel_x * g.kernel_y;
    const int act_c = act.c;
    const int k_out = backward ? g.in_z : g.kernel_amount;
    const int OH = backward ? g.in_y : g.out_y, OW = backward ? g.in_x : g.out_x;
    const int sy = act.sy, sx = act.sx;                                               // phase split of the gathered tensor
    const int osy = backward ? g.stride_y : 1, osx = backward ? g.stride_x : 1;      // output phases
    const int Cp = act.cp, Hs = act.hs, Ws = act.ws;
    int r;

    TcParams p;
    memset(&p, 0, sizeof(p));
    p.c_chunks = ceil_div(act_c, 32);
    p.n_img = batch; p.k_out = k_out; p.OH = OH; p.OW = OW; p.out_stride_y = osy; p.out_stride_x = osx;
    p.out = out; p.bias = bias;
    p.act_func = ef ? ef->func : -1;
    p.act_slope = ef ? ef->slope : 0.0;
    p.pre_out = ef ? ef->pre_out : nullptr;

    // output phases and their tap lists
    const int pad_y = backward ? g.kernel_y - 1 - g.padding_y : g.padding_y;
    const int pad_x = backward ? g.kernel_x - 1 - g.padding_x : g.padding_x;
    const int ext_y0 = ceil_div(OH, osy), ext_x0 = ceil_div(OW, osx);
    tile_shape(ext_y0, ext_x0, 128, &p.BW, &p.BH, &p.BI);
    int ntaps = 0, mtiles = 0, mpairs = 0, nph = 0, min_taps = 1 << 30, max_taps = 0;
    bool any_empty = false;
    for (int ry = 0; ry < osy; ry++)
        for (int rx = 0; rx < osx; rx++) {
            PhaseInfo pi;
            pi.off_y = ry; pi.off_x = rx;
            pi.ext_y = (OH - ry + osy - 1) / osy; pi.ext_x = (OW - rx + osx - 1) / osx;
            pi.tap_begin = ntaps; pi.tap_count = 0;
            if (pi.ext_y <= 0 || pi.ext_x <= 0) continue;
            for (int ky = 0; ky < g.kernel_y; ky++)
                for (int kx = 0; kx < g.kernel_x; kx++) {
                    TapEntry t;
                    if (!backward) {
                        // input row = sy*oy + ky - pad = sy*(oy + dy) + phase
                        t.dy = (int8_t)floor_div(ky - pad_y, sy); t.dx = (int8_t)floor_div(kx - pad_x, sx);
                        t.in_phase = (uint8_t)(pos_mod(ky - pad_y, sy) * sx + pos_mod(kx - pad_x, sx));
                    } else {
                        // delta row = (osy*yy + ry + ky - pad) / osy, only taps where the division is exact
                        int ny = ry + ky - pad_y, nx = rx + kx - pad_x;
                        if (pos_mod(ny, osy) != 0 || pos_mod(nx, osx) != 0) continue;
                        t.dy = (int8_t)floor_div(ny, osy); t.dx = (int8_t)floor_div(nx, osx);
                        t.in_phase = 0;
                    }
                    t.wtap = (uint8_t)(ky * g.kernel_x + kx);
                    p.taps[ntaps++] = t;
                    pi.tap_count++;
                }
            if (pi.tap_count == 0) { any_empty = true; ntaps = pi.tap_begin; continue; }
            pi.tiles_x = ceil_div(pi.ext_x, p.BW); pi.tiles_y = ceil_div(pi.ext_y, p.BH); pi.tiles_i = ceil_div(batch, p.BI);
            pi.tile_begin = mtiles;
            pi.pair_begin = mpairs;
            if (pi.tap_count < min_taps) min_taps = pi.tap_count;
            if (pi.tap_count > max_taps) max_taps = pi.tap_count;
            mtiles += pi.tiles_x * pi.tiles_y * pi.tiles_i;
            mpairs += (pi.tiles_x * pi.tiles_y * pi.tiles_i + 1) / 2;
            p.phase[nph++] = pi;
        }
    if (any_empty && p.act_func >= 0) return TC_UNSUPPORTED;      // outputs that no tap reaches would miss f(0): the caller applies the function separately
    if (any_empty) B200_CUDA(cudaMemsetAsync(out, 0, sizeof(float) * (size_t)batch * k_out * OH * OW, s));
    if (nph == 0) return B200_OK;
    p.phases = nph;
    // Column tile (BN) and CTA pairing.  The widest tile with CTA pairs (two CTAs share one 256-row MMA, each stages half
    // of the filter rows) moves the fewest operand bytes per flop, but a layer with few output pixels then yields only a
    // handful of work items for 148 SMs.  Model: time ~ waves x K-steps x (A bytes + B bytes per CTA and K-step), with A
    // = 128 rows and B = BN (or BN/2) rows; take the candidate with the least modelled time, the wider one on a tie.
    // Split-K (ks > 1) divides a tile's K steps over ks work items whose partial outputs a second kernel sums in a fixed
    // order: for layers with few output pixels and a long contraction (the 4x4 / 8x8 layers of the DCGAN nets) it fills the
    // SMs with wide tiles instead of many narrow ones that re-read the activations once per column tile.  Cost of the
    // reduction: a launch plus (ks + 1) passes over the output.
    int ctas = 1, ksplit = 1;
    {
        const int bn_max = (int)align_up(k_out < 256 ? k_out : 256, 16);
        const long long out_elems = (long long)batch * k_out * OH * OW;
        const int steps_max = max_taps * p.c_chunks, steps_min = min_taps * p.c_chunks;
        static const bool split_enabled = !(getenv("B200CONV_KSPLIT") && getenv("B200CONV_KSPLIT")[0] == '0');      // debug switch
        long long best = -1;
        for (int bn = bn_max; bn >= 16; bn = (bn > 32 ? (int)align_up(bn / 2, 16) : bn - 16)) {
            for (int c = 2; c >= 1; c--) {
                if (c == 2 && !(cta_pairs_enabled() && bn >= 32)) continue;
                for (int ks = 1; ks <= 8; ks *= 2) {
                    if (ks > 1 && (!split_enabled || !kpartial || any_empty || out_elems % 4 || ((uintptr_t)out & 15) || ((uintptr_t)p.pre_out & 15) || (size_t)ks * out_elems > kpartial_elems ||
                                   steps_min < 4 * ks))
                        break;
                    const long long items = (long long)(c == 2 ? mpairs : mtiles) * ceil_div(k_out, bn) * ks;
                    const long long waves = (items * c + sm_count() - 1) / sm_count();
                    // cycles: bytes staged per CTA and K step at ~32 B/clk; reduction at ~2500 B/clk over the whole GPU
                    const long long cost = waves * ceil_div(steps_max, ks) * (128 + bn / c) * 4 +
                                           (ks > 1 ? 8000 + (long long)(ks + 1) * out_elems * 4 / 2500 : 0);
                    if (best < 0 || cost < best) { best = cost; p.BN = bn; ctas = c; ksplit = ks; }
                }
            }
            if (bn == 16) break;
        }
        // tuning aid: B200CONV_TILE="<BN>,<CTAs>" overrides the choice (read on every call)
        if (const char *e = getenv("B200CONV_TILE")) {
            int bn = 0, c = 0;
            if (sscanf(e, "%d,%d", &bn, &c) == 2 && bn >= 16 && bn <= bn_max && bn % 16 == 0 && (c == 1 || (c == 2 && bn >= 32))) { p.BN = bn; ctas = c; ksplit = 1; }
        }
        p.ksplit = ksplit;
        p.kpartial = kpartial;
        p.out_elems = out_elems;
    }
    p.acc_stride = pow2_ceil(p.BN);
    set_kmajor(p, true, 128);
    set_kmajor(p, false, p.BN / ctas);
    p.idesc = make_idesc_tf32(p.BN, 0, 0, 128 * ctas);
    p.n_tiles_n = ceil_div(k_out, p.BN);
    p.num_tiles = (ctas == 2 ? mpairs : mtiles) * p.n_tiles_n * p.ksplit;

    CUtensorMap maps[4];
    {
        const long long dims[5] = {act_c, Ws, Hs, batch, (long long)sy * sx};
        const long long pitch[4] = {Cp, (long long)Ws * Cp, (long long)Hs * Ws * Cp, (long long)batch * Hs * Ws * Cp};
        const int box[5] = {32, p.BW, p.BH, p.BI, 1};
        if ((r = make_map(&maps[0], act.hi, dims, pitch, box))) return r;
        if (x3 && (r = make_map(&maps[1], act.lo, dims, pitch, box))) return r;
    }
    {
        const long long dims[5] = {act_c, taps, k_out, 1, 1};
        const long long pitch[4] = {Cp, (long long)taps * Cp, (long long)k_out * taps * Cp, (long long)k_out * taps * Cp};
        const int box[5] = {32, 1, p.BN / ctas, 1, 1};
        if ((r = make_map(&maps[2], w_hi, dims, pitch, box))) return r;
        if (x3 && (r = make_map(&maps[3], w_lo, dims, pitch, box))) return r;
    }
    if ((r = launch_tc<MODE_CONV>(maps, p, x3, s, ctas))) return r;
    if (p.ksplit > 1) {
        const size_t total = (size_t)p.out_elems;
        size_t blocks = (total / 4 + 255) / 256;
        if (blocks > (size_t)sm_count() * 16) blocks = (size_t)sm_count() * 16;
        Launch((unsigned)blocks, 256, 0, s)(conv_ksplit_reduce_kernel, out, kpartial, p.ksplit, total, bias, k_out, (size_t)OH * OW, p.act_func, p.act_slope,
                                                                   p.pre_out);
        B200_LAUNCH_CHECK();
    }
    return B200_OK;
}

static int run_conv(bool backward, const b200_conv_geom &g, float *out, const float *act, const float *kernel, const float *bias,
                    int batch, int precision, cudaStream_t s)
{
    if (!geom_supported(g)) return TC_UNSUPPORTED;
    const bool x3 = precision == B200_TF32X3;
    ActPack pk = backward ? act_pack_shape(batch, g.kernel_amount, g.out_y, g.out_x, 1, 1)
                          : act_pack_shape(batch, g.in_z, g.in_y, g.in_x, g.stride_y, g.stride_x);
    const size_t w_elems = weight_pack_elems(g, backward);
    const size_t bytes = (sizeof(float) * (pk.elems() + w_elems) + kPackPad) * (x3 ? 2 : 1) + 8192;
    int r = arena_reserve(bytes, s);
    if (r) return r;
    arena_reset();
    pk.hi = (float *)arena_take(sizeof(float) * pk.elems() + kPackPad);
    pk.lo = x3 ? (float *)arena_take(sizeof(float) * pk.elems() + kPackPad) : nullptr;
    float *w_hi = (float *)arena_take(sizeof(float) * w_elems);
    float *w_lo = x3 ? (float *)arena_take(sizeof(float) * w_elems) : nullptr;
    if (!pk.hi || !w_hi || (x3 && (!pk.lo || !w_lo))) return fail(B200_E_NOMEM, "scratch arena exhausted");
    if ((r = act_pack_fill(pk, act, s))) return r;
    if ((r = weight_pack_fill(g, backward, kernel, w_hi, w_lo, s))) return r;
    return conv_gemm(backward, g, out, pk, w_hi, w_lo, bias, x3, s, nullptr, 0, nullptr);
}

int tc_conv_forward(const b200_conv_geom &g, float *out, const float *image, const float *kernel, const float *bias,
                    int batch, int precision, cudaStream_t s)
{
    return run_conv(false, g, out, image, kernel, bias, batch, precision, s);
}

int tc_conv_backward(const b200_conv_geom &g, float *out_delta, const float *delta, const float *kernel, int batch,
                     int precision, cudaStream_t s)
{
    return run_conv(true, g, out_delta, delta, kernel, nullptr, batch, precision, s);
}

// Debug switch: B200CONV_WGRAD_PACK_TAPS=0 in the environment keeps one tap per work item of the weight gradient.
static bool wgrad_pack_taps_enabled()
{
    static const bool on = !(getenv("B200CONV_WGRAD_PACK_TAPS") && getenv("B200CONV_WGRAD_PACK_TAPS")[0] == '0');
    return on;
}

// Plan of the weight gradient: the pixel chunks that form the K dimension, how many taps share a work item, and the split-K
// factor (number of CTAs along the pixel dimension).
struct WgradPlan {
    int tapm;                  // 0, or filters per member tap (32 or 64) when several taps share the 128 rows of the MMA
    int members;               // taps per work item
    int items;                 // work items per (channel tile, split): taps, or tap groups
    int BW, BH, BI, chunks_x, chunks_y, chunks_i;
    int BN, splits;
    TapGroup groups[kMaxTaps];
};

static WgradPlan wgrad_plan(const b200_conv_geom &g, int batch)
{
    WgradPlan w;
    memset(&w, 0, sizeof(w));
    const int taps = g.kernel_x * g.kernel_y, K = g.kernel_amount;
    const int sy = g.stride_y, sx = g.stride_x;
    w.BN = (int)align_up(g.in_z < 256 ? g.in_z : 256, 32);
    // With at most 64 filters a tap fills a quarter or half of the MMA's 128 rows, and every tap would stage the image chunk
    // again: 4 (2) taps of one stride phase share the rows and one staged image chunk instead.
    if (wgrad_pack_taps_enabled() && K <= 64 && taps >= 2 && taps <= kMaxTaps) {
        w.tapm = K <= 32 ? 32 : 64;
        w.members = 128 / w.tapm;
        const int phases = sy * sx;
        for (int ph = 0; ph < phases; ph++) {
            int open = -1;                                   // group of this phase that still has room
            for (int ky = 0; ky < g.kernel_y; ky++)
                for (int kx = 0; kx < g.kernel_x; kx++) {
                    if (pos_mod(ky - g.padding_y, sy) * sx + pos_mod(kx - g.padding_x, sx) != ph) continue;
                    if (open < 0 || w.groups[open].count == w.members) open = w.items++;
                    TapGroup &grp = w.groups[open];
                    grp.tap[grp.count++] = (uint8_t)(ky * g.kernel_x + kx);
                }
        }
        // the pixel chunks walk a phase plane of the image
        const int hs = ceil_div(g.in_y, sy), ws = ceil_div(g.in_x, sx);
        tile_shape(hs, ws, 32, &w.BW, &w.BH, &w.BI);
        w.chunks_x = ceil_div(ws, w.BW); w.chunks_y = ceil_div(hs, w.BH);
    } else {
        w.items = taps;
        tile_shape(g.out_y, g.out_x, 32, &w.BW, &w.BH, &w.BI);
        w.chunks_x = ceil_div(g.out_x, w.BW); w.chunks_y = ceil_div(g.out_y, w.BH);
    }
    w.chunks_i = ceil_div(batch, w.BI);
    const long long chunks = (long long)w.chunks_x * w.chunks_y * w.chunks_i;
    const int base = (w.tapm ? 1 : ceil_div(K, 128)) * ceil_div(g.in_z, w.BN) * w.items;
    long long splits = sm_count() / base;
    if (splits < 1) splits = 1;
    if (splits > chunks) splits = chunks;
    if (splits > 64) splits = 64;
    w.splits = (int)splits;
    return w;
}

size_t wgrad_partial_elems(const b200_conv_geom &g, int batch)
{
    return (size_t)wgrad_plan(g, batch).splits * g.kernel_x * g.kernel_y * g.in_z * g.kernel_amount;
}

// Batch-summed weight gradient on packed operands: x = image pack (split by the stride), d = delta
// pack (unsplit); `partial` holds wgrad_partial_elems() floats.
int wgrad_gemm(const b200_conv_geom &g, float *dkernel, int accumulate, const ActPack &x, const ActPack &d, float *partial,
               bool x3, cudaStream_t s)
{
    if (!geom_supported(g)) return TC_UNSUPPORTED;
    const int batch = x.n;
    const int taps = g.kernel_x * g.kernel_y;
    const int C = g.in_z, K = g.kernel_amount;
    const int sy = g.stride_y, sx = g.stride_x;
    int r;

    TcParams p;
    memset(&p, 0, sizeof(p));
    const WgradPlan plan = wgrad_plan(g, batch);
    p.BN = plan.BN;
    p.acc_stride = pow2_ceil(p.BN);
    // CTA pairs: two neighbouring filter tiles share one 256-row MMA, each CTA stages half of the channels
    const int ctas = (cta_pairs_enabled() && K > 128 && p.BN % 64 == 0) ? 2 : 1;
    set_mnmajor(p, true, 128);
    set_mnmajor(p, false, p.BN / ctas);
    p.idesc = make_idesc_tf32(p.BN, 1, 1, 128 * ctas);
    p.ft_n = plan.tapm ? 1 : ceil_div(K, 128); p.ct_n = ceil_div(C, p.BN); p.taps_n = taps; p.wg_ctas = ctas;
    p.k_rows = K; p.c_cols = C; p.n_img = batch;
    p.BW = plan.BW; p.BH = plan.BH; p.BI = plan.BI;
    p.chunks_x = plan.chunks_x; p.chunks_y = plan.chunks_y; p.chunks_i = plan.chunks_i;
    p.chunks_total = (long long)p.chunks_x * p.chunks_y * p.chunks_i;
    p.splits = plan.splits;
    p.tapm = plan.tapm; p.members = plan.members; p.items_n = plan.items;
    p.member_bytes = (uint32_t)(plan.tapm / 32) * 4096u;
    memcpy(p.groups, plan.groups, sizeof(p.groups));
    p.num_tiles = ceil_div(p.ft_n, ctas) * p.ct_n * p.items_n * p.splits;   // work items: tiles, or pairs of filter tiles
    p.partial = partial;
    for (int ky = 0; ky < g.kernel_y; ky++)
        for (int kx = 0; kx < g.kernel_x; kx++) {
            TapEntry t;
            t.dy = (int8_t)floor_div(ky - g.padding_y, sy); t.dx = (int8_t)floor_div(kx - g.padding_x, sx);
            t.in_phase = (uint8_t)(pos_mod(ky - g.padding_y, sy) * sx + pos_mod(kx - g.padding_x, sx));
            t.wtap = (uint8_t)(ky * g.kernel_x + kx);
            p.taps[ky * g.kernel_x + kx] = t;
        }

    CUtensorMap maps[4];
    {
        const long long dims[3] = {g.out_x, g.out_y, batch};
        const long long pitch[3] = {d.cp, (long long)g.out_x * d.cp, (long long)g.out_y * g.out_x * d.cp};
        const int box[3] = {p.BW, p.BH, p.BI};
        const int a_blocks = plan.tapm ? plan.tapm / 32 : 4;      // packed taps: a box is one member tap's filters
        if ((r = make_blocked_map(&maps[0], d.hi, K, dims, pitch, box, a_blocks))) return r;
        if (x3 && (r = make_blocked_map(&maps[1], d.lo, K, dims, pitch, box, a_blocks))) return r;
    }
    {
        // phase and image index share one dimension ([phase][n] is contiguous in the pack)
        const long long dims[3] = {x.ws, x.hs, (long long)batch * sy * sx};
        const long long pitch[3] = {x.cp, (long long)x.ws * x.cp, (long long)x.hs * x.ws * x.cp};
        const int box[3] = {p.BW, p.BH, p.BI};
        if ((r = make_blocked_map(&maps[2], x.hi, C, dims, pitch, box, p.BN / 32 / ctas))) return r;
        if (x3 && (r = make_blocked_map(&maps[3], x.lo, C, dims, pitch, box, p.BN / 32 / ctas))) return r;
    }
    if ((r = launch_tc<MODE_WGRAD>(maps, p, x3, s, ctas))) return r;
    // channels per block: runs of about 64 consecutive weights (256 bytes) per filter on the output side
    int c_run = (64 + taps - 1) / taps;
    if (c_run > C) c_run = C;
    // few filters and channels (1x1 products of the few-channel layers): shorter runs so that the splits are summed by more blocks
    while (c_run > 1 && ceil_div(K, 32) * ceil_div(C, c_run) < 2 * sm_count()) c_run = (c_run + 1) / 2;
    const size_t tile_bytes = sizeof(float) * (size_t)taps * c_run * 33;
    if (tile_bytes <= 48 * 1024) {
        const int blocks = ceil_div(K, 32) * ceil_div(C, c_run);
        Launch(blocks, 256, tile_bytes, s)(wgrad_reduce_tiled_kernel, dkernel, p.partial, p.splits, taps, C, K, c_run, accumulate);
        B200_LAUNCH_CHECK();
        return B200_OK;
    }
    size_t total = (size_t)K * C * taps;
    int grid = (int)((total + 255) / 256);
    if (grid > sm_count() * 16) grid = sm_count() * 16;
    Launch(grid, 256, 0, s)(wgrad_reduce_kernel, dkernel, p.partial, p.splits, taps, C, K, accumulate);
    B200_LAUNCH_CHECK();
    return B200_OK;
}

// second stage of the bias gradient: dbias[k] (+)= sum over the batch of the plane sums; one warp per filter, the lanes walk the batch and combine
// in a shuffle tree (a fixed order: reproducible run to run)
__global__ void dbias_reduce_kernel(float *__restrict__ dbias, const float *__restrict__ plane_sums, int batch, int K, int accumulate)
{
    grid_dependency_wait();
    const int lane = threadIdx.x & 31;
    const int k = (int)((blockIdx.x * blockDim.x + threadIdx.x) >> 5);
    if (k >= K) return;
    float s = 0.f;
    for (int w = lane; w < batch; w += 32) s += plane_sums[(size_t)w * K + k];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (lane == 0) dbias[k] = accumulate ? dbias[k] + s : s;
}

// Bias gradient: plane sums of delta per (sample, filter), then the reduction over the batch.
// db_tmp holds batch * K floats.
int dbias_batch(float *dbias, int accumulate, const float *delta, int batch, int K, size_t plane, float *db_tmp, cudaStream_t s)
{
    int r;
    if ((r = b200_summ_xy(db_tmp, batch, delta, batch, K, plane, s))) return r;
    Launch(ceil_div(K * 32, 256), 256, 0, s)(dbias_reduce_kernel, dbias, db_tmp, batch, K, accumulate);
    B200_LAUNCH_CHECK();
    return B200_OK;
}

int tc_conv_wgrad_batch(const b200_conv_geom &g, float *dkernel, float *dbias, int accumulate, const float *image,
                        const float *delta, int batch, int precision, cudaStream_t s)
{
    if (!geom_supported(g)) return TC_UNSUPPORTED;
    const bool x3 = precision == B200_TF32X3;
    ActPack x = act_pack_shape(batch, g.in_z, g.in_y, g.in_x, g.stride_y, g.stride_x);
    ActPack d = act_pack_shape(batch, g.kernel_amount, g.out_y, g.out_x, 1, 1);
    const size_t part_elems = wgrad_partial_elems(g, batch);
    const size_t db_elems = dbias ? (size_t)batch * g.kernel_amount : 0;
    const size_t bytes = (sizeof(float) * (x.elems() + d.elems()) + 2 * kPackPad) * (x3 ? 2 : 1) + sizeof(float) * (part_elems + db_elems) + 32768;
    int r = arena_reserve(bytes, s);
    if (r) return r;
    arena_reset();
    x.hi = (float *)arena_take(sizeof(float) * x.elems() + kPackPad);
    x.lo = x3 ? (float *)arena_take(sizeof(float) * x.elems() + kPackPad) : nullptr;
    d.hi = (float *)arena_take(sizeof(float) * d.elems() + kPackPad);
    d.lo = x3 ? (float *)arena_take(sizeof(float) * d.elems() + kPackPad) : nullptr;
    float *partial = (float *)arena_take(sizeof(float) * part_elems);
    float *db_tmp = dbias ? (float *)arena_take(sizeof(float) * db_elems) : nullptr;
    if (!x.hi || !d.hi || !partial || (x3 && (!x.lo || !d.lo)) || (dbias && !db_tmp)) return fail(B200_E_NOMEM, "scratch arena exhausted");
    if ((r = act_pack_fill(x, image, s))) return r;
    if ((r = act_pack_fill(d, delta, s))) return r;
    if ((r = wgrad_gemm(g, dkernel, accumulate, x, d, partial, x3, s))) return r;
    if (dbias) return dbias_batch(dbias, accumulate, delta, batch, g.kernel_amount, (size_t)g.out_y * g.out_x, db_tmp, s);
    return B200_OK;
}

int tc_gemm(float *out, const float *a, const float *b, int m, int n, int k, int a_mn_major, int b_mn_major,
            int precision, cudaStream_t s)
{
    // TMA needs 16-byte aligned bases and row pitches
    const int a_pitch = a_mn_major ? m : k, b_pitch = b_mn_major ? n : k;
    if ((a_pitch % 4) || (b_pitch % 4)) return TC_UNSUPPORTED;
    if ((size_t)m * n < 4096 || k < 8) return TC_UNSUPPORTED;      // too small to be worth a tensor-core launch
    const bool x3 = precision == B200_TF32X3;
    const size_t a_elems = (size_t)m * k, b_elems = (size_t)n * k;
    // Split-K: a product with few output tiles and a long contraction (the VAE heads: 128 x 256 outputs over 16384 inputs
    // are ONE tile) divides the K steps of a tile over several work items; conv_ksplit_reduce_kernel sums the partial
    // outputs in a fixed order.  Taken when the tiles leave most SMs idle; every split keeps at least 8 K steps.
    int ksplit = 1;
    {
        const int bn = (int)align_up(n < 256 ? n : 256, b_mn_major ? 32 : 16);
        const long long tiles = (long long)ceil_div(m, 128) * ceil_div(n, bn);
        const int steps = ceil_div(k, 32);
        static const bool split_enabled = !(getenv("B200CONV_KSPLIT") && getenv("B200CONV_KSPLIT")[0] == '0');
        if (split_enabled && ((size_t)m * n) % 4 == 0 && ((uintptr_t)out & 15) == 0)
            while (tiles * ksplit * 2 <= sm_count() && steps / (ksplit * 2) >= 8 && ksplit < 64) ksplit *= 2;
    }
    const size_t part_elems = ksplit > 1 ? (size_t)ksplit * m * n : 0;
    const size_t bytes = sizeof(float) * ((a_elems + b_elems) * (x3 ? 2 : 1) + part_elems) + 16384;
    int r = arena_reserve(bytes, s);
    if (r) return r;
    arena_reset();
    float *a_hi = (float *)arena_take(sizeof(float) * a_elems + 256);      // +256: see make_blocked_map
    float *a_lo = x3 ? (float *)arena_take(sizeof(float) * a_elems + 256) : nullptr;
    float *b_hi = (float *)arena_take(sizeof(float) * b_elems + 256);
    float *b_lo = x3 ? (float *)arena_take(sizeof(float) * b_elems + 256) : nullptr;
    float *kpartial = part_elems ? (float *)arena_take(sizeof(float) * part_elems) : nullptr;
    if (!a_hi || !b_hi || (x3 && (!a_lo || !b_lo)) || (part_elems && !kpartial)) return fail(B200_E_NOMEM, "scratch arena exhausted");
    {
        // both operands in one launch: blocks [0, ga) split A, the rest B
        const int ga = (int)((a_elems + 256 * 8 - 1) / (256 * 8)) < sm_count() * 8 ? (int)((a_elems + 256 * 8 - 1) / (256 * 8)) : sm_count() * 8;
        const int gb = (int)((b_elems + 256 * 8 - 1) / (256 * 8)) < sm_count() * 8 ? (int)((b_elems + 256 * 8 - 1) / (256 * 8)) : sm_count() * 8;
        Launch(ga + gb, 256, 0, s)(split_tf32_pair_kernel, a, a_hi, a_lo, a_elems, b, b_hi, b_lo, b_elems, ga);
        B200_LAUNCH_CHECK();
    }

    TcParams p;
    memset(&p, 0, sizeof(p));
    p.BN = (int)align_up(n < 256 ? n : 256, b_mn_major ? 32 : 16);
    p.acc_stride = pow2_ceil(p.BN);
    if (a_mn_major) set_mnmajor(p, true, 128); else set_kmajor(p, true, 128);
    if (b_mn_major) set_mnmajor(p, false, p.BN); else set_kmajor(p, false, p.BN);
    p.idesc = make_idesc_tf32(p.BN, a_mn_major, b_mn_major);
    p.M = m; p.N = n; p.K = k; p.ldc = n; p.a_mn = a_mn_major; p.b_mn = b_mn_major;
    p.n_tiles_n = ceil_div(n, p.BN);
    p.out = out;
    p.ksplit = ksplit;
    p.kpartial = kpartial;
    p.out_elems = (long long)m * n;
    p.num_tiles = ceil_div(m, 128) * p.n_tiles_n * ksplit;

    CUtensorMap maps[4];
    for (int side = 0; side < 2; side++) {
        const bool mn = side == 0 ? a_mn_major != 0 : b_mn_major != 0;
        const long long ext = side == 0 ? m : n;                 // M or N extent of this operand
        float *hi = side == 0 ? a_hi : b_hi, *lo = side == 0 ? a_lo : b_lo;
        const int rows_box = side == 0 ? 128 : p.BN;
        if (mn) {   // stored [k][ext]
            const long long dims[3] = {k, 1, 1};
            const long long pitch[3] = {ext, ext * k, ext * k};
            const int box[3] = {32, 1, 1};
            if ((r = make_blocked_map(&maps[2 * side], hi, ext, dims, pitch, box, rows_box / 32))) return r;
            if (x3 && (r = make_blocked_map(&maps[2 * side + 1], lo, ext, dims, pitch, box, rows_box / 32))) return r;
        } else {    // stored [ext][k]
            const long long dims[5] = {k, ext, 1, 1, 1};
            const long long pitch[4] = {k, (long long)k * ext, (long long)k * ext, (long long)k * ext};
            const int box[5] = {32, rows_box, 1, 1, 1};
            if ((r = make_map(&maps[2 * side], hi, dims, pitch, box))) return r;
            if (x3 && (r = make_map(&maps[2 * side + 1], lo, dims, pitch, box))) return r;
        }
    }
    if ((r = launch_tc<MODE_GEMM>(maps, p, x3, s))) return r;
    if (ksplit > 1) {
        const size_t total = (size_t)m * n;
        size_t blocks = (total / 4 + 255) / 256;
        if (blocks > (size_t)sm_count() * 16) blocks = (size_t)sm_count() * 16;
        Launch((unsigned)blocks, 256, 0, s)(conv_ksplit_reduce_kernel, out, kpartial, ksplit, total, nullptr, 1, total, -1, 0.0, nullptr);
        B200_LAUNCH_CHECK();
    }
    return B200_OK;
}

}  // namespace b200
