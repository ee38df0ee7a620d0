// Layers with very few channels on one side (the RGB end of every network: 3 -> 64 convolutions, 64 -> 3 transposed
// convolutions).  The implicit GEMM stages 32 channels per tap, so with 3 channels nine tenths of every staged tile and of
// every MMA are zeros.  Here the taps are folded into the channel dimension instead (explicit im2col of the small-channel
// tensor: C' = taps x C "channels" per output position) and the three contractions become 1x1 convolutions on the
// tensor-core kernel:
//   forward        y[n,k,oy,ox]      = sum_c' W'[k][c'] col[n,oy,ox,c']                       (conv_gemm, 1x1)
//   backward-data  t[n,c',oy,ox]     = sum_k W''[c'][k] delta[n,k,oy,ox]  then  dx = col2im(t)  (conv_gemm 1x1 + gather)
//   weight grad.   dW'[k][c']        = sum_{n,oy,ox} delta[n,k,oy,ox] col[n,oy,ox,c']          (wgrad_gemm, 1x1) then re-ordered
// with c' = tap * C + c.  col is written once per layer call (high and, in 3xTF32 mode, low TF32 planes) and is
// taps/stride^2 times the size of the small tensor -- a few MB.
#include "common.cuh"
#include "kernels.h"
#include "tc_ptx.cuh"

namespace b200 {

// col[n][oy][ox][tap*C + c] = x[n][c][oy*sy + ky - py][ox*sx + kx - px] (0 outside), pitch cp floats per position (a multiple
// of 4, at most 256).  One block per (n, oy) row of positions.  The C*kh image rows that the row of positions reads are
// staged in shared memory with coalesced loads (STAGED; rows too long for shared memory are gathered from global memory
// instead); a thread then makes four consecutive columns of a position and stores them as one 16-byte vector, the (row, dx)
// of every column coming from a table in shared memory, so that the inner loop has one division per vector.
template <bool STAGED>
__global__ void __launch_bounds__(256) im2col_pack_kernel(float *__restrict__ hi, float *__restrict__ lo, const float *__restrict__ x, int N, int C,
                                                          int H, int W, int OH, int OW, int kh, int kw, int sy, int sx, int py, int px, int cp)
{
    grid_dependency_wait();
    extern __shared__ float staged[];            // STAGED: [C * kh][W]
    __shared__ int4 column[256];                 // x: row offset (staged) or channel-plane offset, y: dy, z: dx, w: 1 for a real column
    const int cc = C * kh * kw;
    for (int j = threadIdx.x; j < cp; j += blockDim.x) {
        int4 e = make_int4(0, 0, 0, 0);
        if (j < cc) {
            const int tap = j / C, c = j - tap * C;
            const int ky = tap / kw, kx = tap - ky * kw;
            e = make_int4(STAGED ? (c * kh + ky) * W : c * H * W, ky - py, kx - px, 1);
        }
        column[j] = e;
    }
    const int qpp = cp / 4;                      // vectors per position
    const int row_quads = OW * qpp;
    for (int row = blockIdx.x; row < N * OH; row += gridDim.x) {
        const int n = row / OH, oy = row - n * OH;
        const float *xn = x + (size_t)n * C * H * W;
        __syncthreads();                         // the table is written; the previous row's readers are done with `staged`
        if (STAGED) {
            for (int r = threadIdx.x >> 5; r < C * kh; r += blockDim.x >> 5) {        // one warp per image row
                const int c = r / kh, ky = r - c * kh;
                const int iy = oy * sy + ky - py;
                const bool inside = iy >= 0 && iy < H;
                const float *src = xn + ((size_t)c * H + (inside ? iy : 0)) * W;
                for (int xx = threadIdx.x & 31; xx < W; xx += 32) staged[r * W + xx] = inside ? src[xx] : 0.f;
            }
            __syncthreads();
        }
        float4 *hrow = reinterpret_cast<float4 *>(hi + (size_t)row * OW * cp);
        float4 *lrow = lo ? reinterpret_cast<float4 *>(lo + (size_t)row * OW * cp) : nullptr;
        for (int q = threadIdx.x; q < row_quads; q += blockDim.x) {
            const int ox = q / qpp, j0 = (q - ox * qpp) * 4;
            float v[4];
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int4 e = column[j0 + i];
                const int ix = ox * sx + e.z;
                if (STAGED) {
                    v[i] = (e.w && ix >= 0 && ix < W) ? staged[e.x + ix] : 0.f;
                } else {
                    const int iy = oy * sy + e.y;
                    v[i] = (e.w && iy >= 0 && iy < H && ix >= 0 && ix < W) ? xn[e.x + iy * W + ix] : 0.f;
                }
            }
            const float4 h = make_float4(ptx::to_tf32(v[0]), ptx::to_tf32(v[1]), ptx::to_tf32(v[2]), ptx::to_tf32(v[3]));
            hrow[q] = h;
            if (lrow) lrow[q] = make_float4(ptx::to_tf32(v[0] - h.x), ptx::to_tf32(v[1] - h.y), ptx::to_tf32(v[2] - h.z), ptx::to_tf32(v[3] - h.w));
        }
    }
}

// forward weights  W'[k][tap*C + c] (pitch cp)  = W[k][c*taps + tap]
// backward weights W''[tap*C + c][k] (pitch kp) = W[k][c*taps + tap]
__global__ void smallc_weight_kernel(float *__restrict__ hi, float *__restrict__ lo, const float *__restrict__ w, int K, int C, int taps,
                                     int pitch, int transposed)
{
    grid_dependency_wait();
    const int cc = C * taps;
    const int rows = transposed ? cc : K, inner = transposed ? K : cc;
    const size_t total = (size_t)rows * pitch;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        const int i = (int)(idx % pitch), r = (int)(idx / pitch);
        float v = 0.f;
        if (i < inner) {
            const int k = transposed ? i : r, j = transposed ? r : i;
            const int tap = j / C, c = j - tap * C;
            v = w[((size_t)k * C + c) * taps + tap];
        }
        const float h = ptx::to_tf32(v);
        hi[idx] = h;
        if (lo) lo[idx] = ptx::to_tf32(v - h);
    }
}

// dx[n][c][y][x] = sum over the taps (ky,kx) with (y + py - ky) % sy == 0 and (x + px - kx) % sx == 0 (and the quotient
// inside the OH x OW plane) of t[n][(ky*kw + kx)*C + c][(y + py - ky)/sy][(x + px - kx)/sx].  One block per (n, c, y) row.
__global__ void col2im_gather_kernel(float *__restrict__ dx, const float *__restrict__ t, int N, int C, int H, int W, int OH, int OW,
                                     int kh, int kw, int sy, int sx, int py, int px)
{
    grid_dependency_wait();
    const int cc = C * kh * kw;
    for (int row = blockIdx.x; row < N * C * H; row += gridDim.x) {
        const int y = row % H;
        const int nc = row / H;
        const int c = nc % C, n = nc / C;
        const float *tn = t + (size_t)n * cc * OH * OW;
        // only the taps congruent to (y + py) mod sy (and likewise in x) divide exactly: start there and step by the stride
        const int ky0 = (y + py) % sy;
        for (int x = threadIdx.x; x < W; x += blockDim.x) {
            float s = 0.f;
            const int kx0 = (x + px) % sx;
            for (int ky = ky0; ky < kh; ky += sy) {
                const int ny = y + py - ky;
                if (ny < 0) break;
                const int oy = ny / sy;
                if (oy >= OH) continue;
                for (int kx = kx0; kx < kw; kx += sx) {
                    const int nx = x + px - kx;
                    if (nx < 0) break;
                    const int ox = nx / sx;
                    if (ox >= OW) continue;
                    s += tn[((size_t)((ky * kw + kx) * C + c) * OH + oy) * OW + ox];
                }
            }
            dx[(size_t)row * W + x] = s;
        }
    }
}

// dkernel[k][c*taps + tap] (+)= dk[k][tap*C + c]
__global__ void smallc_dkernel_kernel(float *__restrict__ dkernel, const float *__restrict__ dk, int K, int C, int taps, int accumulate)
{
    grid_dependency_wait();
    const int cc = C * taps;
    const int total = K * cc;
    for (int idx = blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += gridDim.x * blockDim.x) {
        const int k = idx / cc, j = idx - k * cc;
        const int c = j / taps, tap = j - c * taps;
        const float v = dk[(size_t)k * cc + tap * C + c];
        dkernel[idx] = accumulate ? dkernel[idx] + v : v;
    }
}

// Weights of the mirrored problem of a layer with few filters (see mirror_geom): rows and channels change places and the
// taps run backwards.  dst[c][k*taps + t] = src[k][c*taps + (taps-1-t)]; back = 1 is the inverse for the gradient:
// dst[k][c*taps + t] (+)= src[c][k*taps + (taps-1-t)].
__global__ void mirror_weights_kernel(float *__restrict__ dst, const float *__restrict__ src, int K, int C, int taps, int back, int accumulate)
{
    grid_dependency_wait();
    const int total = K * C * taps;
    for (int idx = blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += gridDim.x * blockDim.x) {
        if (!back) {
            const int c = idx / (K * taps), j = idx - c * (K * taps);
            const int k = j / taps, t = j - k * taps;
            dst[idx] = src[((size_t)k * C + c) * taps + (taps - 1 - t)];
        } else {
            const int k = idx / (C * taps), j = idx - k * (C * taps);
            const int c = j / taps, t = j - c * taps;
            const float v = src[((size_t)c * K + k) * taps + (taps - 1 - t)];
            dst[idx] = accumulate ? dst[idx] + v : v;
        }
    }
}

static inline int grid_for(size_t total)
{
    size_t blocks = (total + 255) / 256, cap = (size_t)sm_count() * 16;
    return (int)(blocks < 1 ? 1 : (blocks < cap ? blocks : cap));
}

bool smallc_applies(const b200_conv_geom &g)
{
    const int cc = g.in_z * g.kernel_x * g.kernel_y;
    return g.in_z <= 8 && cc <= 256 && g.kernel_x * g.kernel_y > 1;
}

b200_conv_geom smallc_geom(const b200_conv_geom &g)
{
    b200_conv_geom q = g;
    q.in_z = g.in_z * g.kernel_x * g.kernel_y;
    q.in_y = g.out_y; q.in_x = g.out_x;
    q.kernel_x = q.kernel_y = 1;
    q.stride_x = q.stride_y = 1;
    q.padding_x = q.padding_y = 0;
    return q;
}

int im2col_pack(const b200_conv_geom &g, const ActPack &col, const float *x, int batch, cudaStream_t s)
{
    const int rows = batch * g.out_y;
    const int grid = rows < sm_count() * 32 ? rows : sm_count() * 32;
    const size_t stage_bytes = sizeof(float) * (size_t)g.in_z * g.kernel_y * g.in_x;
    if (stage_bytes <= 40 * 1024)
        Launch(grid, 256, stage_bytes, s)(im2col_pack_kernel<true>, col.hi, col.lo, x, batch, g.in_z, g.in_y, g.in_x, g.out_y, g.out_x, g.kernel_y,
                                          g.kernel_x, g.stride_y, g.stride_x, g.padding_y, g.padding_x, col.cp);
    else
        Launch(grid, 256, 0, s)(im2col_pack_kernel<false>, col.hi, col.lo, x, batch, g.in_z, g.in_y, g.in_x, g.out_y, g.out_x, g.kernel_y,
                                g.kernel_x, g.stride_y, g.stride_x, g.padding_y, g.padding_x, col.cp);
    B200_LAUNCH_CHECK();
    return B200_OK;
}

int smallc_weights(const b200_conv_geom &g, const float *kernel, float *hi, float *lo, int pitch, bool transposed, cudaStream_t s)
{
    const int taps = g.kernel_x * g.kernel_y;
    const size_t total = (size_t)(transposed ? g.in_z * taps : g.kernel_amount) * pitch;
    Launch(grid_for(total), 256, 0, s)(smallc_weight_kernel, hi, lo, kernel, g.kernel_amount, g.in_z, taps, pitch, transposed ? 1 : 0);
    B200_LAUNCH_CHECK();
    return B200_OK;
}

int col2im_gather(const b200_conv_geom &g, float *dx, const float *t, int batch, cudaStream_t s)
{
    const int rows = batch * g.in_z * g.in_y;
    const int threads = g.in_x >= 128 ? 128 : (g.in_x >= 64 ? 64 : 32);
    Launch(rows < sm_count() * 64 ? rows : sm_count() * 64, threads, 0, s)(col2im_gather_kernel, dx, t, batch, g.in_z, g.in_y, g.in_x, g.out_y, g.out_x, g.kernel_y, g.kernel_x,
                                                        g.stride_y, g.stride_x, g.padding_y, g.padding_x);
    B200_LAUNCH_CHECK();
    return B200_OK;
}

int smallc_dkernel(const b200_conv_geom &g, float *dkernel, const float *dk, int accumulate, cudaStream_t s)
{
    const int taps = g.kernel_x * g.kernel_y;
    Launch(grid_for((size_t)g.kernel_amount * g.in_z * taps), 256, 0, s)(smallc_dkernel_kernel, dkernel, dk, g.kernel_amount, g.in_z, taps, accumulate);
    B200_LAUNCH_CHECK();
    return B200_OK;
}

// A stride-1 convolution C -> K channels with padding p is, read backwards, a convolution K -> C with padding k-1-p and the
// weights of mirror_weights: BackwardConvolution of the one is ForwardConvolution of the other, and the weight gradient of the
// one is the (re-ordered) weight gradient of the other with image and error exchanged.  For a layer with few FILTERS the
// mirrored problem has few input CHANNELS, which is what the folded path above serves.
bool mirror_applies(const b200_conv_geom &g)
{
    if (g.stride_x != 1 || g.stride_y != 1 || g.kernel_amount > 8 || g.in_z <= 8) return false;
    if (g.padding_x > g.kernel_x - 1 || g.padding_y > g.kernel_y - 1) return false;
    return smallc_applies(mirror_geom(g));
}

b200_conv_geom mirror_geom(const b200_conv_geom &g)
{
    b200_conv_geom q = g;
    q.in_z = g.kernel_amount; q.in_y = g.out_y; q.in_x = g.out_x;
    q.kernel_amount = g.in_z; q.out_y = g.in_y; q.out_x = g.in_x;
    q.padding_x = g.kernel_x - 1 - g.padding_x; q.padding_y = g.kernel_y - 1 - g.padding_y;
    return q;
}

int mirror_weights(const b200_conv_geom &g, float *dst, const float *src, int back, int accumulate, cudaStream_t s)
{
    const int taps = g.kernel_x * g.kernel_y;
    Launch(grid_for((size_t)g.kernel_amount * g.in_z * taps), 256, 0, s)(mirror_weights_kernel, dst, src, g.kernel_amount, g.in_z, taps, back, accumulate);
    B200_LAUNCH_CHECK();
    return B200_OK;
}

}  // namespace b200
