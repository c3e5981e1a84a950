// Direct Gaussian sums: the near / small field of the treecode and the exact dense product.
//
// Replaces near_field_run (F3M_src/n_tree.cu:831-902) with skip_conv_1d_shared
// (F3M_src/1_d_conv.cu:255-335) and rbf_call / rbf_call_grad (n_tree.cu:185-241) with
// rbf_1d_reduce_shared_torch(_grad) (1_d_conv.cu:126-214).
//
// The reference gathers every x, y and b through the permutation on every use, runs one target per
// thread over a block-wide tile with two barriers per tile and repeats all exponentials for every
// column of b.  Here the points are already in box order, sources are packed as rows
// [s*y_0 .. s*y_{d-1}, b_0 .. b_{RB-1}] padded to a multiple of four floats with
// s = sqrt(log2(e)/(2 ls^2)), so that a source is one or two 16-byte shared-memory reads broadcast to
// the warp and a pair costs d subtractions, d multiply-adds, one ex2 and RB multiply-adds.  This kernel
// is bound by the SM's FP32 issue rate and its exponential (MUFU) rate, not by HBM: a source row is
// reused by every target of the tile.
#include <math.h>
#include <algorithm>
#include "common.cuh"

namespace f3m {

constexpr int NT = 128;        // threads per CTA
constexpr int ST = 512;        // source rows per shared-memory tile

__host__ __device__ constexpr int row_width(int D, int RB) { return (D + RB + 3) / 4 * 4; }

__device__ __forceinline__ float ex2_approx(float x) {
    float r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}

template <int D, int RB>
__global__ void __launch_bounds__(256) pack_sources(const float *__restrict__ pts, int64_t n, const float *__restrict__ bs,
                                                   int R, int r0, float scale, float *packed) {
    constexpr int W = row_width(D, RB);
    int64_t j = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= n) return;
    float row[W];
#pragma unroll
    for (int k = 0; k < D; k++) row[k] = scale * pts[(size_t)k * n + j];
#pragma unroll
    for (int r = 0; r < RB; r++) row[D + r] = (r0 + r < R) ? bs[(size_t)j * R + r0 + r] : 0.f;
#pragma unroll
    for (int c = D + RB; c < W; c++) row[c] = 0.f;
    float4 *dst = reinterpret_cast<float4 *>(packed + (size_t)j * W);
#pragma unroll
    for (int c = 0; c < W / 4; c++) dst[c] = make_float4(row[4 * c], row[4 * c + 1], row[4 * c + 2], row[4 * c + 3]);
}

// inner product of one target tile with `cnt` packed source rows held in shared memory
template <int D, int RB, int TI, bool GRAD>
__device__ __forceinline__ void tile_accumulate(const float *__restrict__ smem, int cnt, const float (&tx)[TI][D],
                                                float (&acc)[TI][RB]) {
    constexpr int W = row_width(D, RB);
#pragma unroll 4
    for (int j = 0; j < cnt; j++) {
        float row[W];
        const float4 *src = reinterpret_cast<const float4 *>(smem + j * W);
#pragma unroll
        for (int c = 0; c < W / 4; c++) {
            float4 v = src[c];
            row[4 * c] = v.x; row[4 * c + 1] = v.y; row[4 * c + 2] = v.z; row[4 * c + 3] = v.w;
        }
#pragma unroll
        for (int u = 0; u < TI; u++) {
            float d0 = tx[u][0] - row[0];
            float nr2 = -d0 * d0;                       // minus the squared distance, built negated
#pragma unroll
            for (int k = 1; k < D; k++) {
                float dk = tx[u][k] - row[k];
                nr2 = fmaf(-dk, dk, nr2);
            }
            float e = ex2_approx(nr2);
            if (GRAD) e *= -nr2;
#pragma unroll
            for (int r = 0; r < RB; r++) acc[u][r] = fmaf(e, row[D + r], acc[u][r]);
        }
    }
}

// ---------------------------------------------------------------------------------------------
// Direct form: pair = d subtractions, d multiply-adds, ex2, RB multiply-adds.  Used when the boxes
// are wide compared with the lengthscale (see near_kernel_x2 below for the usual case).
// items: (target box, tile) ; tile_off[b] = first item of box b (exclusive scan of tiles per box)
// ---------------------------------------------------------------------------------------------
// (rows outside [row_begin, row_end) belong to another slice of the targets and are not touched)
__device__ __forceinline__ void item_to_tile(int item, const int *__restrict__ tile_off, int nbx,
                                             const int *__restrict__ off_x, int row_begin, int row_end, int &box, int &t0,
                                             int &t1, int full_tile = 0) {
    int lo = 0, hi = nbx;   // largest b with tile_off[b] <= item
    while (hi - lo > 1) {
        int mid = (lo + hi) >> 1;
        if (tile_off[mid] <= item) lo = mid; else hi = mid;
    }
    box = lo;
    const int tile = item - tile_off[box], ntiles = tile_off[box + 1] - tile_off[box];
    const int a = max(off_x[box], row_begin), nb = min(off_x[box + 1], row_end) - a;
    // full_tile > 0 (a kernel whose tiles of at most full_tile / 2 rows cost half): when the rows left over by full tiles
    // are at most half a tile, the box is cut into full tiles and that short one; otherwise its tiles are equally full
    if (full_tile > 0 && nb - (ntiles - 1) * full_tile <= full_tile / 2) {
        t0 = a + tile * full_tile;
        t1 = min(t0 + full_tile, a + nb);
        return;
    }
    t0 = a + (int)(((long long)nb * tile) / ntiles);
    t1 = a + (int)(((long long)nb * (tile + 1)) / ntiles);
}

template <int D, int RB, int TI>
__global__ void __launch_bounds__(NT) near_kernel(const float *__restrict__ xpts, int n_x, const int *__restrict__ off_x,
                                                 int nbx, const int *__restrict__ tile_off,
                                                 const int *__restrict__ ptr, const int *__restrict__ idx,
                                                 const int *__restrict__ off_y, const float *__restrict__ packed,
                                                 float scale, int R, int r0, float *out, int row_begin, int row_end) {
    constexpr int W = row_width(D, RB);
    __shared__ __align__(16) float smem[ST * W];
    int box, t0, t1;
    item_to_tile(blockIdx.x, tile_off, nbx, off_x, row_begin, row_end, box, t0, t1);
    float tx[TI][D], tot[TI][RB];
    int ti[TI];
#pragma unroll
    for (int u = 0; u < TI; u++) {
        ti[u] = t0 + threadIdx.x + u * NT;
        int ii = ti[u] < t1 ? ti[u] : t0;
#pragma unroll
        for (int k = 0; k < D; k++) tx[u][k] = scale * xpts[(size_t)k * n_x + ii];
#pragma unroll
        for (int r = 0; r < RB; r++) tot[u][r] = 0.f;
    }
    const int e0 = ptr[box], e1 = ptr[box + 1];
    for (int e = e0; e < e1; e++) {
        const int by = idx[e];
        const int s0 = off_y[by], s1 = off_y[by + 1];
        float acc[TI][RB];   // per source box, then added to the running total (blocked accumulation)
#pragma unroll
        for (int u = 0; u < TI; u++)
#pragma unroll
            for (int r = 0; r < RB; r++) acc[u][r] = 0.f;
        for (int base = s0; base < s1; base += ST) {
            const int cnt = min(ST, s1 - base);
            __syncthreads();
            const float4 *g = reinterpret_cast<const float4 *>(packed + (size_t)base * W);
            float4 *sdst = reinterpret_cast<float4 *>(smem);
            for (int q = threadIdx.x; q < cnt * (W / 4); q += NT) sdst[q] = __ldg(g + q);
            __syncthreads();
            tile_accumulate<D, RB, TI, false>(smem, cnt, tx, acc);
        }
#pragma unroll
        for (int u = 0; u < TI; u++)
#pragma unroll
            for (int r = 0; r < RB; r++) tot[u][r] += acc[u][r];
    }
#pragma unroll
    for (int u = 0; u < TI; u++)
        if (ti[u] < t1) {
#pragma unroll
            for (int r = 0; r < RB; r++)
                if (r0 + r < R) out[(size_t)ti[u] * R + r0 + r] += tot[u][r];
        }
}

// ---------------------------------------------------------------------------------------------
// Expanded form, the usual case (box edge not much larger than the lengthscale).  With c the centre
// of the SOURCE box and s the scale above,
//     2^(-s^2 |x-y|^2) = 2^(-|xr|^2) * 2^(2 xr.yr) * 2^(-|yr|^2),   xr = s (x-c), yr = s (y-c).
// The last factor is folded into the source's weight when the rows are packed
// (row = [2 yr_0 .. 2 yr_{d-1}, b_0 2^(-|yr|^2) ..]), the first is applied once per (target, source
// box), so that a pair costs d multiply-adds, one ex2 and RB multiply-adds: the exponential unit, not
// the FP32 issue rate, is then the only limit.  |yr| <= sqrt(d)/2 * s * edge and |xr| <= 3.5 sqrt(d) s edge
// for every pair the lists can hold, so nothing overflows while s*edge <= 1, which the host checks.
// ---------------------------------------------------------------------------------------------
constexpr int NT2 = 32;     // threads per CTA: one warp, so a tile holds 64 targets and a box of ~400 points
                            // splits into tiles that are nearly full (measured: 64-thread CTAs lose 7% to padding)
constexpr int TI2 = 2;      // targets per thread


// ---------------------------------------------------------------------------------------------
// Expanded form with packed FP32 pairs (fma.rn.f32x2, sm_100): two SOURCES share every instruction of
// the inner product, the polynomial and the accumulation, which halves the issue slots they take.
// Sources are packed in pairs, column by column: pair block = [c0a c0b c1a c1b ... ] (2 W floats), so a
// 16-byte shared-memory load yields two aligned register pairs.  Box b starts at the even row
// (off[b] + b + 1) & ~1 of the packed array; an odd box gets a zero-weight partner for its last source.
// ---------------------------------------------------------------------------------------------
typedef unsigned long long f32x2;
__device__ __forceinline__ f32x2 pack2(float lo, float hi) {
    f32x2 r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpack2(f32x2 v, float &lo, float &hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
__device__ __forceinline__ f32x2 fma2(f32x2 a, f32x2 b, f32x2 c) {
    f32x2 d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ f32x2 mul2(f32x2 a, f32x2 b) {
    f32x2 d;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__host__ __device__ __forceinline__ int pair_row_start(int off, int box) { return (off + box + 1) & ~1; }

template <int D, int RB>
__global__ void __launch_bounds__(256) pack_pairs_rel(const float *__restrict__ pts, int n, const float *__restrict__ bs,
                                                     int R, int r0, float scale, const int *__restrict__ off_y, int nby,
                                                     const float *__restrict__ ctr_y, const unsigned char *__restrict__ need,
                                                     float *packed) {
    constexpr int W = row_width(D, RB);
    int j = blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= n) return;
    const int by = box_of_row(off_y, nby, j);
    if (need && !need[by]) return;   // a slice of the targets reads only the source boxes its lists name
    const int s0 = off_y[by], s1 = off_y[by + 1];
    float row[W];
    float ny = 0.f;
#pragma unroll
    for (int k = 0; k < D; k++) {
        float yr = scale * (pts[(size_t)k * n + j] - ctr_y[by * D + k]);
        ny = fmaf(-yr, yr, ny);
        row[k] = 2.f * yr;
    }
    const float wy = ex2_approx(ny);
#pragma unroll
    for (int r = 0; r < RB; r++) row[D + r] = (r0 + r < R) ? bs[(size_t)j * R + r0 + r] * wy : 0.f;
#pragma unroll
    for (int c = D + RB; c < W; c++) row[c] = 0.f;
    const int pos = pair_row_start(s0, by) + (j - s0);
    float *dst = packed + (size_t)(pos >> 1) * (2 * W) + (pos & 1);
#pragma unroll
    for (int c = 0; c < W; c++) dst[2 * c] = row[c];
    if (j == s1 - 1 && !(pos & 1)) {   // last source of an odd box: its partner weighs nothing
#pragma unroll
        for (int c = 0; c < W; c++) dst[2 * c + 1] = 0.f;
    }
}

// The same packing with one warp per source box (and per part of a long box): boxes no list of this product names
// are skipped without touching their points, and no point searches for its box.
template <int D, int RB>
__global__ void __launch_bounds__(256) pack_pairs_box(const float *__restrict__ pts, int n, const float *__restrict__ bs, int R,
                                                     int r0, float scale, const int *__restrict__ off_y, int nby,
                                                     const float *__restrict__ ctr_y, const unsigned char *__restrict__ need,
                                                     int nsplit, float *packed) {
    constexpr int W = row_width(D, RB);
    const int lane = threadIdx.x & 31;
    const int by = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    if (by >= nby || (need && !need[by])) return;
    const int s0 = off_y[by], s1 = off_y[by + 1], len = s1 - s0;
    const int c0 = s0 + (int)(((long long)len * blockIdx.y) / nsplit), c1 = s0 + (int)(((long long)len * (blockIdx.y + 1)) / nsplit);
    float ctr[D];
#pragma unroll
    for (int k = 0; k < D; k++) ctr[k] = ctr_y[by * D + k];
    const int prow = pair_row_start(s0, by);
    for (int j = c0 + lane; j < c1; j += 32) {
        float row[W];
        float ny = 0.f;
#pragma unroll
        for (int k = 0; k < D; k++) {
            float yr = scale * (pts[(size_t)k * n + j] - ctr[k]);
            ny = fmaf(-yr, yr, ny);
            row[k] = 2.f * yr;
        }
        const float wy = ex2_approx(ny);
#pragma unroll
        for (int r = 0; r < RB; r++) row[D + r] = (r0 + r < R) ? bs[(size_t)j * R + r0 + r] * wy : 0.f;
#pragma unroll
        for (int c = D + RB; c < W; c++) row[c] = 0.f;
        const int pos = prow + (j - s0);
        float *dst = packed + (size_t)(pos >> 1) * (2 * W) + (pos & 1);
#pragma unroll
        for (int c = 0; c < W; c++) dst[2 * c] = row[c];
        if (j == s1 - 1 && !(pos & 1)) {   // last source of an odd box: its partner weighs nothing
#pragma unroll
            for (int c = 0; c < W; c++) dst[2 * c + 1] = 0.f;
        }
    }
}

// source pairs per shared-memory tile: 6 KB for one column, 12 KB for eight (so that shared memory does not limit the
// CTAs per SM below what the registers allow)
template <int RB> __host__ __device__ constexpr int sp2_of() { return RB >= 4 ? 96 : 192; }

// POLY = 0: every exponential on the MUFU pipe.  POLY = 2 or 3: PNUM of every PDEN source pairs use the
// polynomial of that degree instead (the host enables it only when the exponent is provably small).
template <int D, int RB, int POLY, int PNUM, int PDEN, int TI>
__device__ __forceinline__ void near_tile_x2(const float *__restrict__ xpts, int n_x, const int *__restrict__ ptr,
                                             const int *__restrict__ idx, const int *__restrict__ off_y,
                                             const float *__restrict__ ctr_y, const float *__restrict__ packed, float scale, int R,
                                             int r0, float *out, float pc0, float pc1, float pc2, float pc3, float *smem, int box,
                                             int t0, int t1) {
    constexpr int W = row_width(D, RB);
    float x[TI][D], tot[TI][RB];
    int ti[TI];
    // one target per thread and at most 16 targets: the warp splits into G lane groups that hold the same targets and
    // take every G-th source pair (their sums are added by shuffles at the end), so that no lane idles
    const int nt = t1 - t0;
    const int lg = (TI == 1) ? (nt > 16 ? 5 : (nt > 8 ? 4 : (nt > 4 ? 3 : 2))) : 5;
    const int G = (TI == 1) ? 32 >> lg : 1, grp = (TI == 1) ? (int)threadIdx.x >> lg : 0;
    const int tlane = (TI == 1) ? (int)threadIdx.x & ((1 << lg) - 1) : (int)threadIdx.x;
#pragma unroll
    for (int u = 0; u < TI; u++) {
        ti[u] = t0 + tlane + u * NT2;
        int ii = ti[u] < t1 ? ti[u] : t0;
#pragma unroll
        for (int k = 0; k < D; k++) x[u][k] = xpts[(size_t)k * n_x + ii];
#pragma unroll
        for (int r = 0; r < RB; r++) tot[u][r] = 0.f;
    }
    const f32x2 c1 = pack2(pc1, pc1), c2 = pack2(pc2, pc2), c3 = pack2(pc3, pc3), one = pack2(pc0, pc0);
    const int e0 = ptr[box], e1 = ptr[box + 1];
    for (int e = e0; e < e1; e++) {
        const int by = idx[e];
        const int s0 = off_y[by], cnt = off_y[by + 1] - s0;
        const int npairs = (cnt + 1) >> 1;
        const float *rows = packed + (size_t)pair_row_start(s0, by) * W;
        f32x2 xr[TI][D], acc[TI][RB];
        float fx[TI];
#pragma unroll
        for (int u = 0; u < TI; u++) {
            float nx = 0.f;
#pragma unroll
            for (int k = 0; k < D; k++) {
                const float v = scale * (x[u][k] - __ldg(ctr_y + by * D + k));
                nx = fmaf(-v, v, nx);
                xr[u][k] = pack2(v, v);
            }
            fx[u] = ex2_approx(nx);
#pragma unroll
            for (int r = 0; r < RB; r++) acc[u][r] = pack2(0.f, 0.f);
        }
        constexpr int SP2 = sp2_of<RB>();
        for (int base = 0; base < npairs; base += SP2) {
            const int np = min(SP2, npairs - base);
            __syncthreads();
            const float4 *g = reinterpret_cast<const float4 *>(rows + (size_t)base * 2 * W);
            float4 *sdst = reinterpret_cast<float4 *>(smem);
            for (int q = threadIdx.x; q < np * (2 * W / 4); q += NT2) sdst[q] = __ldg(g + q);
            __syncthreads();
            auto body = [&](int jl, bool poly) {   // jl: the lane group's jl-th pair of the tile
                f32x2 col[W];
                const int j = (TI == 1) ? jl * G + grp : jl;
                const ulonglong2 *src = reinterpret_cast<const ulonglong2 *>(smem + j * 2 * W);
#pragma unroll
                for (int q = 0; q < W / 2; q++) {
                    const ulonglong2 v = src[q];
                    col[2 * q] = v.x;
                    col[2 * q + 1] = v.y;
                }
#pragma unroll
                for (int u = 0; u < TI; u++) {
                    f32x2 t = mul2(xr[u][0], col[0]);
#pragma unroll
                    for (int k = 1; k < D; k++) t = fma2(xr[u][k], col[k], t);
                    f32x2 ev;
                    if (POLY && poly) {
                        ev = (POLY == 2) ? fma2(fma2(c2, t, c1), t, one) : fma2(fma2(fma2(c3, t, c2), t, c1), t, one);
                    } else {
                        float ta, tb;
                        unpack2(t, ta, tb);
                        ev = pack2(ex2_approx(ta), ex2_approx(tb));
                    }
#pragma unroll
                    for (int r = 0; r < RB; r++) acc[u][r] = fma2(ev, col[D + r], acc[u][r]);
                }
            };
            int j = 0;
            const int npl = (TI == 1) ? (np - grp + G - 1) / G : np;   // pairs of this lane group
            if (POLY) {
#pragma unroll 1
                for (; j + PDEN <= npl; j += PDEN) {
#pragma unroll
                    for (int q = 0; q < PDEN; q++) body(j + q, ((q + 1) * PNUM) / PDEN != (q * PNUM) / PDEN);
                }
            } else {
#pragma unroll 4
                for (; j + 1 <= npl; j++) body(j, false);
            }
            for (; j < npl; j++) body(j, false);
        }
#pragma unroll
        for (int u = 0; u < TI; u++)
#pragma unroll
            for (int r = 0; r < RB; r++) {
                float lo, hi;
                unpack2(acc[u][r], lo, hi);
                tot[u][r] = fmaf(fx[u], lo + hi, tot[u][r]);
            }
    }
    if (TI == 1) {
        for (int o = 1 << lg; o < 32; o <<= 1)
#pragma unroll
            for (int r = 0; r < RB; r++) tot[0][r] += __shfl_xor_sync(0xffffffffu, tot[0][r], o);
    }
#pragma unroll
    for (int u = 0; u < TI; u++)
        if (ti[u] < t1 && grp == 0) {
#pragma unroll
            for (int r = 0; r < RB; r++)
                if (r0 + r < R) out[(size_t)ti[u] * R + r0 + r] += tot[u][r];
        }
}


// 16-byte asynchronous copy global -> shared (completion tracked per thread in commit groups)
__device__ __forceinline__ void cp_async16(float *smem_dst, const float *gsrc) {
    const unsigned sa = (unsigned)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(sa), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// A tile of at most 32 targets (small boxes: clustered data, four and five dimensions), one warp.  Two things differ
// from near_tile_x2.  (1) With TS <= 16 targets (TS a power of two) the warp splits into 32 / TS lane groups that hold
// the same targets and take every (32 / TS)-th source pair; the groups' sums are added by shuffles at the end, so no
// lane idles.  (2) Source boxes of a dozen points give a handful of pair iterations each, too few to hide the chain
// list entry -> box offsets -> packed rows behind: the shared-memory tile is two half tiles, the rows of the next chunk
// arrive by asynchronous copies while the current one is consumed, and the offsets and centres of the two boxes after
// it are already in registers.
template <int D, int RB, int POLY, int PNUM, int PDEN>
__device__ __forceinline__ void near_tile_x2_small(const float *__restrict__ xpts, int n_x, const int *__restrict__ ptr,
                                                   const int *__restrict__ idx, const int *__restrict__ off_y,
                                                   const float *__restrict__ ctr_y, const float *__restrict__ packed,
                                                   float scale, int R, int r0, float *out, float pc0, float pc1, float pc2,
                                                   float pc3, float *smem, int box, int t0, int t1) {
    constexpr int W = row_width(D, RB);
    constexpr int SPH = sp2_of<RB>() / 2;   // source pairs per half tile
    constexpr int V4 = 2 * W / 4;           // 16-byte pieces of a pair block
    const int lane = threadIdx.x;
    const int nt = t1 - t0;
    const int lg = nt > 16 ? 5 : (nt > 8 ? 4 : (nt > 4 ? 3 : 2));
    const int TS = 1 << lg, G = 32 >> lg;
    const int g = lane >> lg;
    const int ti = t0 + (lane & (TS - 1));
    float x[D], tot[RB];
    {
        const int ii = ti < t1 ? ti : t0;
#pragma unroll
        for (int k = 0; k < D; k++) x[k] = xpts[(size_t)k * n_x + ii];
#pragma unroll
        for (int r = 0; r < RB; r++) tot[r] = 0.f;
    }
    const f32x2 c1 = pack2(pc1, pc1), c2 = pack2(pc2, pc2), c3 = pack2(pc3, pc3), one = pack2(pc0, pc0);
    const int e0 = ptr[box], e1 = ptr[box + 1];
    if (e0 == e1) return;
    struct Src {
        int npairs;
        const float *rows;
        float ctr[D];
    };
    auto load_src = [&](int by, Src &sb) {
        const int s0 = off_y[by];
        sb.npairs = (off_y[by + 1] - s0 + 1) >> 1;
        sb.rows = packed + (size_t)pair_row_start(s0, by) * W;
#pragma unroll
        for (int k = 0; k < D; k++) sb.ctr[k] = __ldg(ctr_y + by * D + k);
    };
    auto issue_copy = [&](float *dst, const Src &sb, int base) {
        const int pieces = min(SPH, sb.npairs - base) * V4;
        const float *src = sb.rows + (size_t)base * 2 * W;
        for (int q = lane; q < pieces; q += NT2) cp_async16(dst + 4 * q, src + 4 * q);
    };
    Src cur, n1, n2;
    load_src(idx[e0], cur);
    n1 = cur; n2 = cur;
    if (e0 + 1 < e1) load_src(idx[e0 + 1], n1);
    if (e0 + 2 < e1) load_src(idx[e0 + 2], n2);
    int by3 = e0 + 3 < e1 ? idx[e0 + 3] : 0;
    issue_copy(smem, cur, 0);
    cp_async_commit();
    int e = e0, base = 0, pb = 0;
    f32x2 xr[D], acc[RB];
    float fx = 0.f;
    while (true) {
        const bool more_in_box = base + SPH < cur.npairs;
        const bool have_next = more_in_box || e + 1 < e1;
        float *bufc = smem + pb * (SPH * 2 * W), *bufn = smem + (pb ^ 1) * (SPH * 2 * W);
        if (have_next) {
            if (more_in_box) issue_copy(bufn, cur, base + SPH);
            else issue_copy(bufn, n1, 0);
        }
        cp_async_commit();
        cp_async_wait<1>();   // everything but the group just committed has landed
        __syncthreads();
        if (base == 0) {
            float nx = 0.f;
#pragma unroll
            for (int k = 0; k < D; k++) {
                const float v = scale * (x[k] - cur.ctr[k]);
                nx = fmaf(-v, v, nx);
                xr[k] = pack2(v, v);
            }
            fx = ex2_approx(nx);
#pragma unroll
            for (int r = 0; r < RB; r++) acc[r] = pack2(0.f, 0.f);
        }
        const int np = min(SPH, cur.npairs - base);
        int q = 0;
#pragma unroll 2
        for (int j = g; j < np; j += G) {
            f32x2 col[W];
            const ulonglong2 *src = reinterpret_cast<const ulonglong2 *>(bufc + j * 2 * W);
#pragma unroll
            for (int c = 0; c < W / 2; c++) {
                const ulonglong2 v = src[c];
                col[2 * c] = v.x;
                col[2 * c + 1] = v.y;
            }
            f32x2 t = mul2(xr[0], col[0]);
#pragma unroll
            for (int k = 1; k < D; k++) t = fma2(xr[k], col[k], t);
            f32x2 ev;
            if (POLY && ((q + 1) * PNUM) / PDEN != (q * PNUM) / PDEN) {
                ev = (POLY == 2) ? fma2(fma2(c2, t, c1), t, one) : fma2(fma2(fma2(c3, t, c2), t, c1), t, one);
            } else {
                float ta, tb;
                unpack2(t, ta, tb);
                ev = pack2(ex2_approx(ta), ex2_approx(tb));
            }
#pragma unroll
            for (int r = 0; r < RB; r++) acc[r] = fma2(ev, col[D + r], acc[r]);
            if (POLY && ++q == PDEN) q = 0;
        }
        if (!more_in_box) {
#pragma unroll
            for (int r = 0; r < RB; r++) {
                float lo, hi;
                unpack2(acc[r], lo, hi);
                tot[r] = fmaf(fx, lo + hi, tot[r]);
            }
        }
        __syncthreads();   // the copy issued in the next round overwrites the half tile read here
        if (more_in_box) base += SPH;
        else {
            if (++e >= e1) break;
            base = 0;
            cur = n1;
            n1 = n2;
            if (e + 2 < e1) load_src(by3, n2);
            by3 = e + 3 < e1 ? idx[e + 3] : 0;
        }
        pb ^= 1;
    }
    cp_async_wait<0>();
    for (int o = TS; o < 32; o <<= 1)
#pragma unroll
        for (int r = 0; r < RB; r++) tot[r] += __shfl_xor_sync(0xffffffffu, tot[r], o);
    if (g == 0 && ti < t1) {
#pragma unroll
        for (int r = 0; r < RB; r++)
            if (r0 + r < R) out[(size_t)ti * R + r0 + r] += tot[r];
    }
}

// TI = targets per thread.  MIXED: a tile of at most 32 targets runs a one-target form, which does half the work (the
// pipelined one for small boxes); the host picks this variant only when such tiles exist.
template <int D, int RB, int POLY, int PNUM, int PDEN, bool MIXED>
__global__ void __launch_bounds__(NT2, RB == 1 ? 32 : (RB <= 4 ? 20 : 12)) near_kernel_x2(const float *__restrict__ xpts, int n_x, const int *__restrict__ off_x,
                                                     int nbx, const int *__restrict__ tile_off,
                                                     const int *__restrict__ ptr, const int *__restrict__ idx,
                                                     const int *__restrict__ off_y, const float *__restrict__ ctr_y,
                                                     const float *__restrict__ packed, float scale, int R, int r0,
                                                     float *out, float pc0, float pc1, float pc2, float pc3, int row_begin,
                                                     int row_end) {
    constexpr int W = row_width(D, RB);
    __shared__ __align__(16) float smem[sp2_of<RB>() * 2 * W];
    int box, t0, t1;
    item_to_tile(blockIdx.x, tile_off, nbx, off_x, row_begin, row_end, box, t0, t1, MIXED ? NT2 * TI2 : 0);
    if (MIXED && t1 - t0 <= NT2) {
        // a box of at most 32 points has neighbours of its own kind (same level, same local density): short source boxes,
        // where the pipelined form pays; the last tile of a large box meets large source boxes and keeps the plain loop
        if (RB >= 4 && off_x[box + 1] - off_x[box] <= NT2)   // one column: measured slower than the plain loop on clustered data
            near_tile_x2_small<D, RB, POLY, PNUM, PDEN>(xpts, n_x, ptr, idx, off_y, ctr_y, packed, scale, R, r0, out, pc0, pc1, pc2,
                                                        pc3, smem, box, t0, t1);
        else
            near_tile_x2<D, RB, POLY, PNUM, PDEN, 1>(xpts, n_x, ptr, idx, off_y, ctr_y, packed, scale, R, r0, out, pc0, pc1, pc2, pc3,
                                                     smem, box, t0, t1);
    } else
        near_tile_x2<D, RB, POLY, PNUM, PDEN, TI2>(xpts, n_x, ptr, idx, off_y, ctr_y, packed, scale, R, r0, out, pc0, pc1, pc2, pc3, smem,
                                                   box, t0, t1);
}

#include "near_mma.cuh"

// tiles[b] = tiles of the rows of target box b inside [row_begin, row_end) (0 when the box has no pairs or no row
// there); *n_small counts the boxes whose last tile holds at most 32 targets
__global__ void __launch_bounds__(256) near_tiles_per_box(int nbx, const int *__restrict__ off_x, const int *__restrict__ ptr,
                                                         int row_begin, int row_end, int tile_pts, int *tiles, int *n_small) {
    int b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b > nbx) return;
    int t = 0;
    if (b < nbx && ptr[b + 1] > ptr[b]) {
        const int len = min(off_x[b + 1], row_end) - max(off_x[b], row_begin);
        if (len > 0) {
            t = (len + tile_pts - 1) / tile_pts;
            if (n_small && (len - 1) % tile_pts < 32) atomicAdd(n_small, 1);   // its last tile holds at most 32 targets
        }
    }
    tiles[b] = t;
}

// ---------------------------------------------------------------------------------------------
// Moment form of the near field (optional, F3M_FLAG_NEAR_MOMENTS).  In the expanded form the pair term
// is fx_i * 2^(t_ij) * w_j with t_ij = xr_i . Y_j.  When |t| is provably small for every pair of a list
// (boxes much smaller than the lengthscale), 2^t = 1 + c1 t + c2 t^2 (+ c3 t^3) to within 5e-7 / 1e-6
// relative, and the sum over the sources of a box collapses into moments of that box that do not depend on
// the target:   sum_j w_j 2^(t_ij) = M0 + c1 xr.M1 + c2 xr^T M2 xr (+ c3 M3[xr,xr,xr]).
// The near sum of a target then costs ~20 multiply-adds per source BOX instead of ~6 issue slots per source
// POINT.  The pair lists are untouched; only the way their sums are evaluated changes, with a truncation error
// of the size of the ex2.approx error.  Lists whose exponent bound is larger keep the direct kernels.
// ---------------------------------------------------------------------------------------------
template <int D, int ORD>
struct MomLayout {
    static constexpr int N2 = D * (D + 1) / 2;
    static constexpr int N3 = ORD >= 3 ? D * (D + 1) * (D + 2) / 6 : 0;
    static constexpr int NM = 1 + D + N2 + N3;
};

// one warp per (source box, column)
template <int D, int ORD>
__global__ void __launch_bounds__(256) near_moments_kernel(const float *__restrict__ pts, int n, const float *__restrict__ bs,
                                                          int R, float scale, const int *__restrict__ off_y, int nby,
                                                          const float *__restrict__ ctr_y, float *mom) {
    using ML = MomLayout<D, ORD>;
    constexpr float C1 = 0.69314718056f, C2 = 0.24022650696f, C3 = 0.05550410866f;
    const int lane = threadIdx.x & 31;
    const int wid = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    if (wid >= nby * R) return;
    const int by = wid / R, r = wid - by * R;
    float c[D];
#pragma unroll
    for (int k = 0; k < D; k++) c[k] = ctr_y[by * D + k];
    float acc[ML::NM];
#pragma unroll
    for (int q = 0; q < ML::NM; q++) acc[q] = 0.f;
    for (int j = off_y[by] + lane; j < off_y[by + 1]; j += 32) {
        float Y[D], ny = 0.f;
#pragma unroll
        for (int k = 0; k < D; k++) {
            const float yr = scale * (pts[(size_t)k * n + j] - c[k]);
            ny = fmaf(-yr, yr, ny);
            Y[k] = 2.f * yr;
        }
        const float w = bs[(size_t)j * R + r] * ex2_approx(ny);
        acc[0] += w;
        int q2 = 1 + D, q3 = 1 + D + ML::N2;
#pragma unroll
        for (int a = 0; a < D; a++) {
            const float wa = w * Y[a];
            acc[1 + a] += wa;
#pragma unroll
            for (int b = a; b < D; b++) {
                const float wab = wa * Y[b];
                acc[q2++] += wab;
                if (ORD >= 3) {
#pragma unroll
                    for (int cc = b; cc < D; cc++) { acc[q3] = fmaf(wab, Y[cc], acc[q3]); q3++; }
                }
            }
        }
    }
#pragma unroll
    for (int q = 0; q < ML::NM; q++) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) acc[q] += __shfl_xor_sync(0xffffffffu, acc[q], o);
    }
    if (lane == 0) {
        // fold the Taylor coefficients and the multiplicities of the symmetric tensors into the stored moments
        float *m = mom + (size_t)wid * ML::NM;
        m[0] = acc[0];
        int q2 = 1 + D, q3 = 1 + D + ML::N2;
#pragma unroll
        for (int a = 0; a < D; a++) {
            m[1 + a] = C1 * acc[1 + a];
#pragma unroll
            for (int b = a; b < D; b++) {
                m[q2] = C2 * (a == b ? 1.f : 2.f) * acc[q2];
                q2++;
                if (ORD >= 3) {
#pragma unroll
                    for (int cc = b; cc < D; cc++) {
                        const float mult = (a == b && b == cc) ? 1.f : ((a == b || b == cc) ? 3.f : 6.f);
                        m[q3] = C3 * mult * acc[q3];
                        q3++;
                    }
                }
            }
        }
    }
}

// one thread per target; items = (target box, tile of 128 targets)
template <int D, int ORD>
__global__ void __launch_bounds__(128) near_taylor_kernel(const float *__restrict__ xpts, int n_x, const int *__restrict__ off_x,
                                                         int nbx, const int *__restrict__ tile_off,
                                                         const int *__restrict__ ptr, const int *__restrict__ idx,
                                                         const float *__restrict__ ctr_y, const float *__restrict__ mom,
                                                         float scale, int R, float *out, int row_begin, int row_end) {
    using ML = MomLayout<D, ORD>;
    int box, t0, t1;
    item_to_tile(blockIdx.x, tile_off, nbx, off_x, row_begin, row_end, box, t0, t1);
    const int i = t0 + threadIdx.x;
    if (i >= t1) return;
    float x[D];
#pragma unroll
    for (int k = 0; k < D; k++) x[k] = xpts[(size_t)k * n_x + i];
    const int e0 = ptr[box], e1 = ptr[box + 1];
    for (int r = 0; r < R; r++) {
        float tot = 0.f;
        for (int e = e0; e < e1; e++) {
            const int by = idx[e];
            float xr[D], nx = 0.f;
#pragma unroll
            for (int k = 0; k < D; k++) {
                xr[k] = scale * (x[k] - __ldg(ctr_y + by * D + k));
                nx = fmaf(-xr[k], xr[k], nx);
            }
            const float *m = mom + ((size_t)by * R + r) * ML::NM;
            float poly = __ldg(m);
            int q2 = 1 + D, q3 = 1 + D + ML::N2;
#pragma unroll
            for (int a = 0; a < D; a++) {
                float s1 = __ldg(m + 1 + a);
#pragma unroll
                for (int b = a; b < D; b++) {
                    float s2 = __ldg(m + q2);
                    q2++;
                    if (ORD >= 3) {
#pragma unroll
                        for (int cc = b; cc < D; cc++) { s2 = fmaf(xr[cc], __ldg(m + q3), s2); q3++; }
                    }
                    s1 = fmaf(xr[b], s2, s1);
                }
                poly = fmaf(xr[a], s1, poly);
            }
            tot = fmaf(ex2_approx(nx), poly, tot);
        }
        out[(size_t)i * R + r] += tot;
    }
}

// Polynomial of degree deg (<= 3) through the Chebyshev points of [tlo, thi] for 2^t, as monomial coefficients.
// Its error is at most h^(deg+1) / (2^deg (deg+1)!) with h = ln2 (thi - tlo) / 2.
static void exp2_poly_fit(double tlo, double thi, int deg, double (&cf)[4]) {
    for (int i = 0; i < 4; i++) cf[i] = 0.0;
    cf[0] = 1.0;
    if (deg <= 0) return;
    const int m = deg + 1;
    double tn[4], dd[4];
    for (int i = 0; i < m; i++) {
        tn[i] = 0.5 * (thi + tlo) + 0.5 * (thi - tlo) * cos((2 * i + 1) * 3.14159265358979323846 / (2.0 * m));
        dd[i] = exp2(tn[i]);
    }
    for (int j = 1; j < m; j++)   // Newton divided differences
        for (int i = m - 1; i >= j; i--) dd[i] = (dd[i] - dd[i - 1]) / (tn[i] - tn[i - j]);
    cf[0] = 0.0;
    for (int i = m - 1; i >= 0; i--) {   // Horner on the Newton form: cf(t) = cf(t) (t - tn[i]) + dd[i]
        for (int q = m - 1; q >= 1; q--) cf[q] = cf[q - 1] - tn[i] * cf[q];
        cf[0] = -tn[i] * cf[0] + dd[i];
    }
}
// degree that keeps the interpolation error of 2^t on an interval of half width hw below 3e-7 (0: none does)
static int exp2_poly_degree(double hw) {
    const double h = hw * 0.6931471805599453;
    if (h * h * h / 24.0 <= 3e-7) return 2;
    if (h * h * h * h / 192.0 <= 3e-7) return 3;
    return 0;
}

static inline float near_scale(float lcs) { return sqrtf(lcs * 1.4426950408889634f); }

// Largest |x_k - c_k| / edge over the pairs a list can hold, x a target and c the centre of the source box:
// 2.5 for pairs kept for refinement (centres closer than two edges), 5.5 for "small" pairs, which are children of
// kept parents.  Level-1 pairs of two different point sets are children of the root pair, which is kept without
// any distance test, and the two cubes have separate origins (n_tree.cu:1096-1098): "small" pairs there are
// classified by size before distance (1_d_conv.cu:916-920), so their distance is bounded only by the offset
// between the two cubes.
static double list_reach(const f3m_plan *pl, int level, const PairCSR &csr) {
    const bool final_near = (&csr == &pl->lists[level].keep);
    if (final_near) return 2.5;
    if (level == 1 && !pl->same) {
        double off = 0.0;
        for (int k = 0; k < pl->d; k++) off = std::max(off, fabs((double)pl->tx.origin[k] - (double)pl->ty->origin[k]));
        return off / (double)pl->ty->levels[1].edge + 1.5;
    }
    return 5.5;
}
// the expanded form multiplies 2^(-|xr|^2) by 2^(2 xr.yr): beyond this bound on the cross term the second factor
// could overflow while the first underflows, so such lists use the direct form
constexpr double TMAX_EXPANDED = 64.0;

// one list, one block of RB columns starting at r0
template <int D, int RB>
static void direct_impl(f3m_plan *pl, int level, const PairCSR &csr, const float *bs, int R, int r0, float *out,
                        int row_begin, int row_end, cudaStream_t s) {
    Tree &tx = pl->tx, &ty = *pl->ty;
    Level &lx = tx.levels[level], &ly = ty.levels[level];
    const float scale = near_scale(pl->lcs);
    // bound of the cross term |2 xr.yr| over the pairs of the list: |xr_k| <= reach * se, |yr_k| <= se / 2
    const double reach = level > 0 ? list_reach(pl, level, csr) : 0.0;
    const double tmax = D * reach * ((double)scale * ly.edge) * ((double)scale * ly.edge);
    const bool expanded = scale * ly.edge <= 1.0f && level > 0 && tmax <= TMAX_EXPANDED;
    // tensor-core form (on request): one column, boxes at most half a scaled unit wide, so that the split
    // operands keep the exponent at FP32 accuracy
    const bool use_mma = RB == 1 && expanded && scale * ly.edge <= 0.5f && (pl->prm.flags & F3M_FLAG_NEAR_TENSOR_CORES);
    const int tile_pts = use_mma ? MM_M : (expanded ? NT2 * TI2 : NT);
    DevBuf<int> tiles;
    tiles.alloc((size_t)lx.nb + 1, s);
    int *n_small = pl->d_flags + FL_NSMALL;
    F3M_CUDA(cudaMemsetAsync(n_small, 0, sizeof(int), s));
    near_tiles_per_box<<<(unsigned)((lx.nb + 1 + 255) / 256), 256, 0, s>>>(lx.nb, lx.off.p, csr.ptr.p, row_begin, row_end,
                                                                           tile_pts, tiles.p, n_small);
    F3M_LAUNCH_CHECK();
    exclusive_scan_i32(tiles.p, tiles.p, (int64_t)lx.nb + 1, s);
    F3M_CUDA(cudaMemcpyAsync(pl->h_pinned, tiles.p + lx.nb, sizeof(int), cudaMemcpyDeviceToHost, s));
    F3M_CUDA(cudaMemcpyAsync(pl->h_pinned + 1, n_small, sizeof(int), cudaMemcpyDeviceToHost, s));
    F3M_CUDA(cudaStreamSynchronize(s));
    const int items = pl->h_pinned[0];
    const bool small_tiles = pl->h_pinned[1] > 0;   // some tiles hold at most 32 targets: use the kernel that halves their work
    if (items <= 0) return;
    // Packed sources are kept for the lists of one level that share (column block, form): the "small" list of the last
    // level and the final near list read the same boxes' rows.
    f3m_plan::PackCache &pc = pl->pack_cache;
    const bool cached = !use_mma && pc.level == level && pc.r0 == r0 && pc.rb == RB && pc.expanded == expanded;
    if (!use_mma && !cached) {
        // the pair layout of the expanded form starts every box on an even row
        pc.buf.alloc((size_t)(ty.n + (expanded ? ly.nb + 2 : 0)) * row_width(D, RB), s);
        pc.level = level; pc.r0 = r0; pc.rb = RB; pc.expanded = expanded;
    }
    DevBuf<float> &packed = pc.buf;
    const unsigned g = (unsigned)((ty.n + 255) / 256);
    if (use_mma) {
        using S = MmaShape<D>;
        const size_t rows = mm_rows_total(ty.n, ly.nb);
        DevBuf<float4> Bc;
        DevBuf<float> Gb;
        Bc.alloc(rows * S::KC, s);
        Gb.alloc(rows, s);
        pl->last.begin(ST_PERMUTE, s);
        pack_split_rows<D><<<g, 256, 0, s>>>(ty.pts.p, (int)ty.n, bs, R, r0, scale, ly.off.p, ly.nb, ly.ctr.p, Bc.p, rows, Gb.p);
        pl->last.end(s);
        F3M_LAUNCH_CHECK();
        int *counter = pl->d_flags + FL_MMA_COUNTER;
        F3M_CUDA(cudaMemsetAsync(counter, 0, sizeof(int), s));
        // range of t = 2 u.v - |v|^2 over the pairs of the list: |u| <= reach * se, |v| <= se / 2 per dimension
        const double se = (double)scale * ly.edge;
        const double thi = D * se * se * reach, tlo = -D * se * se * (reach + 0.25);
        const int deg = exp2_poly_degree(0.5 * (thi - tlo));
        double cf[4];
        exp2_poly_fit(tlo, thi, deg, cf);
        int dev = 0, nsm = 0;
        F3M_CUDA(cudaGetDevice(&dev));
        F3M_CUDA(cudaDeviceGetAttribute(&nsm, cudaDevAttrMultiProcessorCount, dev));
        const int grid = std::min(items, 2 * nsm);
        pl->last.begin(ST_DIRECT, s);
#define F3M_NEAR_MMA(DEG_, NP_)                                                                                               \
    {                                                                                                                         \
        F3M_CUDA(cudaFuncSetAttribute(near_mma_kernel<D, DEG_, NP_>, cudaFuncAttributeMaxDynamicSharedMemorySize,             \
                                      mm_smem_bytes<D>()));                                                                   \
        near_mma_kernel<D, DEG_, NP_><<<grid, MM_THREADS, mm_smem_bytes<D>(), s>>>(                                                 \
            tx.pts.p, (int)tx.n, lx.off.p, lx.nb, tiles.p, items, csr.ptr.p, csr.idx.p, ly.off.p, ly.ctr.p, Bc.p, rows, Gb.p, \
            scale, R, r0, out, counter, pl->d_flags, (float)cf[0], (float)cf[1], (float)cf[2], (float)cf[3], row_begin,       \
            row_end);                                                                                                         \
    }
        if (deg == 2) F3M_NEAR_MMA(2, 6)
        else if (deg == 3) F3M_NEAR_MMA(3, 5)
        else F3M_NEAR_MMA(0, 0)
#undef F3M_NEAR_MMA
        pl->last.end(s);
        pl->last.direct_launches++;
        pl->last.direct_variants[DV_TENSOR]++;
        F3M_LAUNCH_CHECK();
        return;
    }
    if (!cached) {
        pl->last.begin(ST_PERMUTE, s);
        if (expanded) {
            // only the boxes that a direct list of this level names (for this slice of the targets, when the product is
            // shared by several GPUs) are packed
            const unsigned char *need = level_source_flags(pl, level, s);
            const int nsplit = std::max(1, std::min(65535, (ly.max_count + 2047) / 2048));
            pack_pairs_box<D, RB><<<dim3((unsigned)(((int64_t)ly.nb * 32 + 255) / 256), nsplit), 256, 0, s>>>(
                ty.pts.p, (int)ty.n, bs, R, r0, scale, ly.off.p, ly.nb, ly.ctr.p, need, nsplit, packed.p);
        } else
            pack_sources<D, RB><<<g, 256, 0, s>>>(ty.pts.p, ty.n, bs, R, r0, scale, packed.p);
        pl->last.end(s);
        F3M_LAUNCH_CHECK();
    }
    pl->last.begin(ST_DIRECT, s);
    if (expanded) {
        const int poly = exp2_poly_degree(tmax);
        pl->last.direct_variants[poly == 2 ? DV_POLY2 : (poly == 3 ? DV_POLY3 : DV_MUFU)]++;
        double cf[4];
        exp2_poly_fit(-tmax, tmax, poly, cf);
#define F3M_NEAR_EXP2(POLY_, PNUM_, PDEN_, MIXED_)                                                                                       \
    near_kernel_x2<D, RB, POLY_, PNUM_, PDEN_, MIXED_><<<items, NT2, 0, s>>>(tx.pts.p, (int)tx.n, lx.off.p, lx.nb, tiles.p, csr.ptr.p, \
                                                                            csr.idx.p, ly.off.p, ly.ctr.p, packed.p, scale, R, r0, out, \
                                                                            (float)cf[0], (float)cf[1], (float)cf[2], (float)cf[3], row_begin, row_end)
#define F3M_NEAR_EXP(POLY_, PNUM_, PDEN_)                         \
    {                                                             \
        if (small_tiles) F3M_NEAR_EXP2(POLY_, PNUM_, PDEN_, true); \
        else F3M_NEAR_EXP2(POLY_, PNUM_, PDEN_, false);            \
    }
        if (poly == 2) F3M_NEAR_EXP(2, 2, 5)
        else if (poly == 3) F3M_NEAR_EXP(3, 1, 3)
        else F3M_NEAR_EXP(0, 0, 1)
#undef F3M_NEAR_EXP2
#undef F3M_NEAR_EXP
    }
    else {
        pl->last.direct_variants[DV_DIRECT]++;
        near_kernel<D, RB, 1><<<items, NT, 0, s>>>(tx.pts.p, (int)tx.n, lx.off.p, lx.nb, tiles.p, csr.ptr.p, csr.idx.p, ly.off.p,
                                                   packed.p, scale, R, r0, out, row_begin, row_end);
    }
    pl->last.end(s);
    pl->last.direct_launches++;
    F3M_LAUNCH_CHECK();
}

template <int D, int ORD>
static void taylor_impl(f3m_plan *pl, int level, const PairCSR &csr, const float *bs, int R, float *out, int row_begin,
                        int row_end, cudaStream_t s) {
    using ML = MomLayout<D, ORD>;
    Tree &tx = pl->tx, &ty = *pl->ty;
    Level &lx = tx.levels[level], &ly = ty.levels[level];
    const float scale = near_scale(pl->lcs);
    DevBuf<int> tiles;
    tiles.alloc((size_t)lx.nb + 1, s);
    near_tiles_per_box<<<(unsigned)((lx.nb + 1 + 255) / 256), 256, 0, s>>>(lx.nb, lx.off.p, csr.ptr.p, row_begin, row_end, 128,
                                                                           tiles.p, nullptr);
    F3M_LAUNCH_CHECK();
    exclusive_scan_i32(tiles.p, tiles.p, (int64_t)lx.nb + 1, s);
    F3M_CUDA(cudaMemcpyAsync(pl->h_pinned, tiles.p + lx.nb, sizeof(int), cudaMemcpyDeviceToHost, s));
    F3M_CUDA(cudaStreamSynchronize(s));
    const int items = pl->h_pinned[0];
    if (items <= 0) return;
    DevBuf<float> mom;
    mom.alloc((size_t)ly.nb * R * ML::NM, s);
    pl->last.begin(ST_DIRECT, s);
    near_moments_kernel<D, ORD><<<(unsigned)(((size_t)ly.nb * R * 32 + 255) / 256), 256, 0, s>>>(ty.pts.p, (int)ty.n, bs, R, scale,
                                                                                             ly.off.p, ly.nb, ly.ctr.p, mom.p);
    F3M_LAUNCH_CHECK();
    near_taylor_kernel<D, ORD><<<items, 128, 0, s>>>(tx.pts.p, (int)tx.n, lx.off.p, lx.nb, tiles.p, csr.ptr.p, csr.idx.p, ly.ctr.p,
                                                    mom.p, scale, R, out, row_begin, row_end);
    pl->last.end(s);
    pl->last.direct_launches++;
    pl->last.direct_variants[DV_MOMENTS]++;
    F3M_LAUNCH_CHECK();
}

template <int D>
static void direct_d(f3m_plan *pl, int level, const PairCSR &csr, const float *bs, int R, float *out, int rb, int re,
                     cudaStream_t s) {
    if ((pl->prm.flags & F3M_FLAG_NEAR_MOMENTS) && level > 0) {
        // exponent bound of the cross term over the pairs of the list (see direct_impl)
        const float se = near_scale(pl->lcs) * pl->ty->levels[level].edge;
        const float tmax = (float)(D * list_reach(pl, level, csr)) * se * se;
        if (se <= 1.0f && tmax <= 0.02f) { taylor_impl<D, 2>(pl, level, csr, bs, R, out, rb, re, s); return; }
        if (se <= 1.0f && tmax <= 0.1f) { taylor_impl<D, 3>(pl, level, csr, bs, R, out, rb, re, s); return; }
    }
    for (int r0 = 0; r0 < R;) {
        const int left = R - r0;
        if (left >= 5) { direct_impl<D, 8>(pl, level, csr, bs, R, r0, out, rb, re, s); r0 += 8; }
        else if (left >= 2) { direct_impl<D, 4>(pl, level, csr, bs, R, r0, out, rb, re, s); r0 += 4; }
        else { direct_impl<D, 1>(pl, level, csr, bs, R, r0, out, rb, re, s); r0 += 1; }
    }
}

void direct_sums(f3m_plan *pl, int level, const PairCSR &csr, const float *bs, int R, float *out_sorted, int64_t row_begin,
                 int64_t row_end, cudaStream_t s) {
    if (csr.count == 0) return;
    const int rb = (int)row_begin, re = (int)row_end;
    switch (pl->d) {
        case 1: direct_d<1>(pl, level, csr, bs, R, out_sorted, rb, re, s); break;
        case 2: direct_d<2>(pl, level, csr, bs, R, out_sorted, rb, re, s); break;
        case 3: direct_d<3>(pl, level, csr, bs, R, out_sorted, rb, re, s); break;
        case 4: direct_d<4>(pl, level, csr, bs, R, out_sorted, rb, re, s); break;
        default: direct_d<5>(pl, level, csr, bs, R, out_sorted, rb, re, s); break;
    }
}

// ---------------------------------------------------------------------------------------------
// exact dense products
// ---------------------------------------------------------------------------------------------
template <int D, int RB>
__global__ void __launch_bounds__(256) pack_rows_dense(const float *__restrict__ Y, int64_t n, const float *__restrict__ b, int R,
                                                      int r0, float scale, float *packed) {
    constexpr int W = row_width(D, RB);
    int64_t j = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= n) return;
    float *dst = packed + (size_t)j * W;
#pragma unroll
    for (int k = 0; k < D; k++) dst[k] = scale * Y[j * D + k];
#pragma unroll
    for (int r = 0; r < RB; r++) dst[D + r] = (r0 + r < R) ? b[(size_t)j * R + r0 + r] : 0.f;
#pragma unroll
    for (int c = D + RB; c < W; c++) dst[c] = 0.f;
}

template <int D, int RB, bool GRAD>
__global__ void __launch_bounds__(NT) dense_kernel(const float *__restrict__ X, int64_t n, const float *__restrict__ packed,
                                                  int64_t m, float scale, float post, int R, int r0, float *out) {
    constexpr int W = row_width(D, RB);
    __shared__ __align__(16) float smem[ST * W];
    const int64_t i = (int64_t)blockIdx.x * NT + threadIdx.x;
    const int64_t ii = i < n ? i : n - 1;
    float tx[1][D], tot[1][RB];
#pragma unroll
    for (int k = 0; k < D; k++) tx[0][k] = scale * X[ii * D + k];
#pragma unroll
    for (int r = 0; r < RB; r++) tot[0][r] = 0.f;
    for (int64_t base = 0; base < m; base += ST) {
        const int cnt = (int)min((int64_t)ST, m - base);
        __syncthreads();
        const float4 *g = reinterpret_cast<const float4 *>(packed + (size_t)base * W);
        float4 *sdst = reinterpret_cast<float4 *>(smem);
        for (int q = threadIdx.x; q < cnt * (W / 4); q += NT) sdst[q] = __ldg(g + q);
        __syncthreads();
        float acc[1][RB];
#pragma unroll
        for (int r = 0; r < RB; r++) acc[0][r] = 0.f;
        tile_accumulate<D, RB, 1, GRAD>(smem, cnt, tx, acc);
#pragma unroll
        for (int r = 0; r < RB; r++) tot[0][r] += acc[0][r];
    }
    if (i < n)
#pragma unroll
        for (int r = 0; r < RB; r++)
            if (r0 + r < R) out[(size_t)i * R + r0 + r] = tot[0][r] * post;
}

template <int D, bool GRAD>
static void dense_d(const float *X, int64_t N, const float *Y, int64_t M, const float *b, int R, float ls, float *out,
                    cudaStream_t s) {
    const float lcs = 1.f / (2.f * ls * ls);
    const float scale = near_scale(lcs);
    // GRAD: sum r^2 exp(..) b / ls^3 with r^2 = (scaled r^2) / scale^2   (n_tree.cu:222-239)
    const float post = GRAD ? 1.f / (scale * scale) / (ls * ls * ls) : 1.f;
    const unsigned gy = (unsigned)((M + 255) / 256), gx = (unsigned)((N + NT - 1) / NT);
    for (int r0 = 0; r0 < R;) {
        DevBuf<float> packed;
        if (R - r0 >= 2) {
            packed.alloc((size_t)M * row_width(D, 4), s);
            pack_rows_dense<D, 4><<<gy, 256, 0, s>>>(Y, M, b, R, r0, scale, packed.p);
            F3M_LAUNCH_CHECK();
            dense_kernel<D, 4, GRAD><<<gx, NT, 0, s>>>(X, N, packed.p, M, scale, post, R, r0, out);
            r0 += 4;
        } else {
            packed.alloc((size_t)M * row_width(D, 1), s);
            pack_rows_dense<D, 1><<<gy, 256, 0, s>>>(Y, M, b, R, r0, scale, packed.p);
            F3M_LAUNCH_CHECK();
            dense_kernel<D, 1, GRAD><<<gx, NT, 0, s>>>(X, N, packed.p, M, scale, post, R, r0, out);
            r0 += 1;
        }
        F3M_LAUNCH_CHECK();
    }
}

template <bool GRAD>
void dense_f32(const float *X, int64_t N, const float *Y, int64_t M, const float *b, int R, int d, float ls, float *out,
               cudaStream_t s) {
    switch (d) {
        case 1: dense_d<1, GRAD>(X, N, Y, M, b, R, ls, out, s); break;
        case 2: dense_d<2, GRAD>(X, N, Y, M, b, R, ls, out, s); break;
        case 3: dense_d<3, GRAD>(X, N, Y, M, b, R, ls, out, s); break;
        case 4: dense_d<4, GRAD>(X, N, Y, M, b, R, ls, out, s); break;
        default: dense_d<5, GRAD>(X, N, Y, M, b, R, ls, out, s); break;
    }
}
template void dense_f32<false>(const float *, int64_t, const float *, int64_t, const float *, int, int, float, float *, cudaStream_t);
template void dense_f32<true>(const float *, int64_t, const float *, int64_t, const float *, int, int, float, float *, cudaStream_t);

// float64 dense product with a double-precision exponential (accuracy reference on the device).
// grid.y slices the sources so that a few thousand target rows still fill the GPU; slices are combined
// with double atomics into a zeroed output.
__global__ void __launch_bounds__(128) dense_f64_kernel(const double *__restrict__ X, int64_t n, const double *__restrict__ Y,
                                                       int64_t m, const double *__restrict__ b, int R, int d, double lcs,
                                                       double *out) {
    __shared__ double sy[128 * F3M_MAX_DIM];
    const int64_t i = (int64_t)blockIdx.x * 128 + threadIdx.x;
    const int64_t per = (m + gridDim.y - 1) / gridDim.y;
    const int64_t m0 = (int64_t)blockIdx.y * per, m1 = min(m, m0 + per);
    double xi[F3M_MAX_DIM];
    for (int k = 0; k < d; k++) xi[k] = X[(i < n ? i : n - 1) * d + k];
    for (int r = 0; r < R; r++) {
        double acc = 0.;
        for (int64_t base = m0; base < m1; base += 128) {
            int cnt = (int)min((int64_t)128, m1 - base);
            __syncthreads();
            for (int q = threadIdx.x; q < cnt * d; q += 128) sy[q] = Y[base * d + q];
            __syncthreads();
            for (int j = 0; j < cnt; j++) {
                double r2 = 0.;
                for (int k = 0; k < d; k++) { double dk = xi[k] - sy[j * d + k]; r2 += dk * dk; }
                acc += exp(-r2 * lcs) * b[(base + j) * R + r];
            }
        }
        if (i < n) atomicAdd(&out[i * R + r], acc);
    }
}

void dense_f64(const double *X, int64_t N, const double *Y, int64_t M, const double *b, int R, int d, double ls, double *out,
               cudaStream_t s) {
    F3M_CUDA(cudaMemsetAsync(out, 0, (size_t)N * R * sizeof(double), s));
    const unsigned gx = (unsigned)((N + 127) / 128);
    int64_t want = (int64_t)NUM_SMS_HINT * 16 / gx;
    unsigned gy = (unsigned)std::max<int64_t>(1, std::min<int64_t>(std::min<int64_t>(want, (M + 4095) / 4096), 4096));
    dense_f64_kernel<<<dim3(gx, gy), 128, 0, s>>>(X, N, Y, M, b, R, d, 1.0 / (2.0 * ls * ls), out);
    F3M_LAUNCH_CHECK();
}

// ---------------------------------------------------------------------------------------------
// Exact dense product without any allocation.
//
// Some hosts may not touch the CUDA allocator once they are running: a service that handed all device
// memory to its own pool at start-up, or a control loop with a "no allocation after initialisation"
// rule, because an allocation can stall the whole device.  For them f3m_rbf_dense_f32_static computes
// the same product as f3m_rbf_dense_f32 with its only scratch buffer -- the packed source rows -- in a
// fixed array that is part of the library image.  Every GPU that loads libf3m.so holds this array
// (F3M_STATIC_SCRATCH_FLOATS floats = 16 MiB) until the process exits.
//
// In host code the array's name is only a stand-in, not a device address; the address a kernel can use
// is obtained once per device, with that device current, through cudaGetSymbolAddress.  The first call
// on a device performs this look-up, so make that first call before any stream capture starts.
// All calls share the one array: it keeps whatever the previous call packed (every row a call reads is
// rewritten by that call first, so nothing has to be cleared), and two calls that overlap on the GPU
// -- different streams, or different host threads -- race on it.
// ---------------------------------------------------------------------------------------------
static __device__ __align__(256) float g_static_scratch[F3M_STATIC_SCRATCH_FLOATS];

static float *static_scratch_for_current_device() {
    static std::atomic<float *> ptr_of_device[64];   // zero-initialised; two threads may both look the address up, both get the same
    int dev = 0;
    F3M_CUDA(cudaGetDevice(&dev));
    F3M_REQUIRE(dev >= 0 && dev < 64, F3M_ERR_UNSUPPORTED, "device ordinal %d not supported by the static entry point", dev);
    float *p = ptr_of_device[dev].load(std::memory_order_acquire);
    if (!p) {
        F3M_CUDA(cudaGetSymbolAddress((void **)&p, g_static_scratch));
        ptr_of_device[dev].store(p, std::memory_order_release);
    }
    return p;
}

template <int D>
static void dense_static_d(const float *X, int64_t N, const float *Y, int64_t M, const float *b, int R, float ls, float *out,
                           float *scratch, cudaStream_t s) {
    const float lcs = 1.f / (2.f * ls * ls);
    const float scale = near_scale(lcs);
    const unsigned gy = (unsigned)((M + 255) / 256), gx = (unsigned)((N + NT - 1) / NT);
    for (int r0 = 0; r0 < R;) {   // column blocks reuse the scratch one after the other on the same stream
        if (R - r0 >= 2) {
            pack_rows_dense<D, 4><<<gy, 256, 0, s>>>(Y, M, b, R, r0, scale, scratch);
            F3M_LAUNCH_CHECK();
            dense_kernel<D, 4, false><<<gx, NT, 0, s>>>(X, N, scratch, M, scale, 1.f, R, r0, out);
            r0 += 4;
        } else {
            pack_rows_dense<D, 1><<<gy, 256, 0, s>>>(Y, M, b, R, r0, scale, scratch);
            F3M_LAUNCH_CHECK();
            dense_kernel<D, 1, false><<<gx, NT, 0, s>>>(X, N, scratch, M, scale, 1.f, R, r0, out);
            r0 += 1;
        }
        F3M_LAUNCH_CHECK();
    }
}

void dense_f32_static(const float *X, int64_t N, const float *Y, int64_t M, const float *b, int R, int d, float ls, float *out,
                      cudaStream_t s) {
    const int64_t width = row_width(d, R >= 2 ? 4 : 1);
    F3M_REQUIRE(M * width <= (int64_t)F3M_STATIC_SCRATCH_FLOATS, F3M_ERR_TOO_LARGE,
                "f3m_rbf_dense_f32_static holds %lld packed floats; M=%lld sources of %lld floats each need %lld "
                "(use f3m_rbf_dense_f32, which allocates)",
                (long long)F3M_STATIC_SCRATCH_FLOATS, (long long)M, (long long)width, (long long)(M * width));
    float *scratch = static_scratch_for_current_device();
    switch (d) {
        case 1: dense_static_d<1>(X, N, Y, M, b, R, ls, out, scratch, s); break;
        case 2: dense_static_d<2>(X, N, Y, M, b, R, ls, out, scratch, s); break;
        case 3: dense_static_d<3>(X, N, Y, M, b, R, ls, out, scratch, s); break;
        case 4: dense_static_d<4>(X, N, Y, M, b, R, ls, out, scratch, s); break;
        default: dense_static_d<5>(X, N, Y, M, b, R, ls, out, scratch, s); break;
    }
}

// ---------------------------------------------------------------------------------------------
// issue-rate probes: register-only loops of ex2 and of fma
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) probe_ex2(float *out, int iters) {
    float a = threadIdx.x * 1e-3f, b = a + 0.1f, c = a + 0.2f, d = a + 0.3f;
#pragma unroll 8
    for (int i = 0; i < iters; i++) {
        a = ex2_approx(-a); b = ex2_approx(-b); c = ex2_approx(-c); d = ex2_approx(-d);
    }
    if (a + b + c + d == 12345.f) out[0] = a;
}
__global__ void __launch_bounds__(256) probe_fma(float *out, int iters) {
    float a = threadIdx.x * 1e-3f, b = a + 0.1f, c = a + 0.2f, d = a + 0.3f, e = a + 0.4f, f = a + 0.5f, g = a + 0.6f, h = a + 0.7f;
    const float m = -1e-6f;   // x <- x*m + x: two distinct source registers per instruction (no register-bank conflicts)
#pragma unroll 8
    for (int i = 0; i < iters; i++) {
        a = fmaf(a, m, a); b = fmaf(b, m, b); c = fmaf(c, m, c); d = fmaf(d, m, d);
        e = fmaf(e, m, e); f = fmaf(f, m, f); g = fmaf(g, m, g); h = fmaf(h, m, h);
    }
    if (a + b + c + d + e + f + g + h == 12345.f) out[0] = a;
}

void measure_peaks(double *gexp, double *gfma, cudaStream_t s) {
    DevBuf<float> o;
    o.alloc(4, s);
    cudaEvent_t e0, e1;
    F3M_CUDA(cudaEventCreate(&e0));
    F3M_CUDA(cudaEventCreate(&e1));
    int dev, sms;
    F3M_CUDA(cudaGetDevice(&dev));
    F3M_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    const int grid = sms * 8, iters = 1 << 14;
    float ms;
    for (int rep = 0; rep < 2; rep++) {   // first repetition warms up
        F3M_CUDA(cudaEventRecord(e0, s));
        probe_ex2<<<grid, 256, 0, s>>>(o.p, iters);
        F3M_CUDA(cudaEventRecord(e1, s));
        F3M_CUDA(cudaEventSynchronize(e1));
        F3M_CUDA(cudaEventElapsedTime(&ms, e0, e1));
        *gexp = (double)grid * 256 * iters * 4 / (ms * 1e-3) * 1e-9;
        F3M_CUDA(cudaEventRecord(e0, s));
        probe_fma<<<grid, 256, 0, s>>>(o.p, iters);
        F3M_CUDA(cudaEventRecord(e1, s));
        F3M_CUDA(cudaEventSynchronize(e1));
        F3M_CUDA(cudaEventElapsedTime(&ms, e0, e1));
        *gfma = (double)grid * 256 * iters * 8 / (ms * 1e-3) * 1e-9;
    }
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
}

}  // namespace f3m
