// Box division, first half: bounding cube, Morton keys, LSD radix sort, physical permutation.
//
// The reference assigns points to boxes level by level with a hash lookup and two global atomics
// per point per level and never moves the points (n_tree_cuda::divide, F3M_src/n_tree.cu:105-179;
// box_division_cum_hash / box_division_assign_hash, F3M_src/1_d_conv.cu:1127-1191).  Here every
// point gets ONE key -- its cell at the deepest level a 30-bit index can hold, bits interleaved so
// that every level's box is a key prefix -- the keys are sorted once, and the points are gathered
// into sorted planes.  All levels are then read off the sorted keys (tree.cu).  All kernels in this
// file are HBM-bound streaming passes.
#include "common.cuh"

namespace f3m {

// ---------------------------------------------------------------------------------------------
// device-wide exclusive scan (three launches, no inter-block waiting)
// ---------------------------------------------------------------------------------------------
constexpr int SCAN_THREADS = 512;
constexpr int SCAN_ITEMS = 8;
constexpr int SCAN_TILE = SCAN_THREADS * SCAN_ITEMS;

__device__ __forceinline__ int block_exclusive_scan(int v, int *total_out, int *smem /* >= 33 ints */) {
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
    int inc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        int t = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += t;
    }
    if (lane == 31) smem[wid] = inc;
    __syncthreads();
    if (wid == 0) {
        int w = lane < nw ? smem[lane] : 0;
        int winc = w;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            int t = __shfl_up_sync(0xffffffffu, winc, o);
            if (lane >= o) winc += t;
        }
        smem[lane] = winc - w;
        if (lane == 31) smem[32] = winc;
    }
    __syncthreads();
    int res = smem[wid] + inc - v;
    if (total_out) *total_out = smem[32];
    __syncthreads();
    return res;
}

__global__ void __launch_bounds__(SCAN_THREADS) scan_tile_sums(const int *__restrict__ in, int64_t n, int *part) {
    __shared__ int sm[33];
    int64_t base = (int64_t)blockIdx.x * SCAN_TILE + (int64_t)threadIdx.x * SCAN_ITEMS;
    int s = 0;
#pragma unroll
    for (int k = 0; k < SCAN_ITEMS; k++)
        if (base + k < n) s += in[base + k];
    int total;
    block_exclusive_scan(s, &total, sm);
    if (threadIdx.x == 0) part[blockIdx.x] = total;
}

__global__ void __launch_bounds__(1024) scan_partials(int *part, int nparts) {
    __shared__ int sm[33];
    int carry = 0;
    for (int base = 0; base < nparts; base += 1024) {
        int i = base + threadIdx.x;
        int v = i < nparts ? part[i] : 0;
        int total;
        int ex = block_exclusive_scan(v, &total, sm);
        if (i < nparts) part[i] = ex + carry;
        carry += total;
    }
}

__global__ void __launch_bounds__(SCAN_THREADS) scan_tile_write(const int *in, int *out, int64_t n,
                                                               const int *__restrict__ part) {
    __shared__ int sm[33];
    int64_t base = (int64_t)blockIdx.x * SCAN_TILE + (int64_t)threadIdx.x * SCAN_ITEMS;
    int v[SCAN_ITEMS];
    int s = 0;
#pragma unroll
    for (int k = 0; k < SCAN_ITEMS; k++) {
        v[k] = (base + k < n) ? in[base + k] : 0;
        s += v[k];
    }
    int ex = block_exclusive_scan(s, nullptr, sm) + part[blockIdx.x];
#pragma unroll
    for (int k = 0; k < SCAN_ITEMS; k++) {
        if (base + k < n) out[base + k] = ex;
        ex += v[k];
    }
}

void exclusive_scan_i32(const int *in, int *out, int64_t n, cudaStream_t s) {
    if (n <= 0) return;
    int nt = (int)((n + SCAN_TILE - 1) / SCAN_TILE);
    DevBuf<int> part;
    part.alloc(nt, s);
    scan_tile_sums<<<nt, SCAN_THREADS, 0, s>>>(in, n, part.p);
    F3M_LAUNCH_CHECK();
    scan_partials<<<1, 1024, 0, s>>>(part.p, nt);
    F3M_LAUNCH_CHECK();
    scan_tile_write<<<nt, SCAN_THREADS, 0, s>>>(in, out, n, part.p);
    F3M_LAUNCH_CHECK();
}

// ---------------------------------------------------------------------------------------------
// bounding cube (calculate_edge_X / calculate_edge, F3M_src/n_tree.cu:25-46)
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ unsigned enc_f32(float f) {
    unsigned u = __float_as_uint(f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
static inline float dec_f32(unsigned u) {
    unsigned v = (u & 0x80000000u) ? (u & 0x7fffffffu) : ~u;
    float f;
    memcpy(&f, &v, 4);
    return f;
}

template <int D>
__global__ void __launch_bounds__(256) bbox_kernel(const float *__restrict__ X, int64_t n, unsigned *mm) {
    float lo[D], hi[D];
    bool nan_seen = false;   // fminf / fmaxf skip NaN: a NaN coordinate is reported through the maximum instead
#pragma unroll
    for (int k = 0; k < D; k++) { lo[k] = INFINITY; hi[k] = -INFINITY; }
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
#pragma unroll
        for (int k = 0; k < D; k++) {
            float v = X[i * D + k];
            nan_seen |= (v != v);
            lo[k] = fminf(lo[k], v);
            hi[k] = fmaxf(hi[k], v);
        }
    }
    if (__any_sync(0xffffffffu, nan_seen) && (threadIdx.x & 31) == 0) atomicMax(&mm[MAXD], 0xffffffffu);   // decodes to NaN
#pragma unroll
    for (int k = 0; k < D; k++) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            lo[k] = fminf(lo[k], __shfl_xor_sync(0xffffffffu, lo[k], o));
            hi[k] = fmaxf(hi[k], __shfl_xor_sync(0xffffffffu, hi[k], o));
        }
    }
    if ((threadIdx.x & 31) == 0) {
#pragma unroll
        for (int k = 0; k < D; k++) {
            atomicMin(&mm[k], enc_f32(lo[k]));
            atomicMax(&mm[MAXD + k], enc_f32(hi[k]));
        }
    }
}

void bounding_box(const float *X, int64_t n, int d, float *h_min, float *h_max, f3m_plan *pl, cudaStream_t s) {
    unsigned *mm = reinterpret_cast<unsigned *>(pl->d_flags) + 16;   // 2*MAXD words
    unsigned init[2 * MAXD];
    for (int k = 0; k < MAXD; k++) { init[k] = 0xffffffffu; init[MAXD + k] = 0u; }
    F3M_CUDA(cudaMemcpyAsync(mm, init, sizeof(init), cudaMemcpyHostToDevice, s));
    int grid = (int)std::min<int64_t>((n + 255) / 256, NUM_SMS_HINT * 8);
    switch (d) {
        case 1: bbox_kernel<1><<<grid, 256, 0, s>>>(X, n, mm); break;
        case 2: bbox_kernel<2><<<grid, 256, 0, s>>>(X, n, mm); break;
        case 3: bbox_kernel<3><<<grid, 256, 0, s>>>(X, n, mm); break;
        case 4: bbox_kernel<4><<<grid, 256, 0, s>>>(X, n, mm); break;
        default: bbox_kernel<5><<<grid, 256, 0, s>>>(X, n, mm); break;
    }
    F3M_LAUNCH_CHECK();
    unsigned *h = reinterpret_cast<unsigned *>(pl->h_pinned);
    F3M_CUDA(cudaMemcpyAsync(h, mm, sizeof(init), cudaMemcpyDeviceToHost, s));
    F3M_CUDA(cudaStreamSynchronize(s));
    for (int k = 0; k < d; k++) {
        h_min[k] = dec_f32(h[k]);
        h_max[k] = dec_f32(h[MAXD + k]);
    }
}

// ---------------------------------------------------------------------------------------------
// Morton keys.  Cell of a point at depth L:  q_k = floor( (2^L (x_k - min_k)) / edge )  in float32,
// the expression of box_division_cum_hash (1_d_conv.cu:1143).  Multiplying by 2^L is exact, so
// the cell at a coarser level l is q_k >> (L-l): one key serves every level.  Bit j of q_k goes
// to key bit d*j+k: within each d-bit group dimension 0 is the least significant bit, which is
// the child code of get_centers (1_d_conv.cu:887-899), and coarser levels are more significant,
// which is the reference's "children of compacted parents" numbering.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float div_mode(float a, float b, int ieee) {
    if (ieee) return __fdiv_rn(a, b);
    float r;
    asm("div.approx.ftz.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
    return r;
}

template <int D>
__global__ void __launch_bounds__(256) morton_kernel(const float *__restrict__ X, int64_t n, float side, float edge0,
                                                    float o0, float o1, float o2, float o3, float o4, int L, int ieee,
                                                    uint32_t *keys, int *vals) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float org[5] = {o0, o1, o2, o3, o4};
    uint32_t key = 0;
    const int qmax = (1 << L) - 1;
#pragma unroll
    for (int k = 0; k < D; k++) {
        float t = __fsub_rn(X[i * D + k], org[k]);
        float v = floorf(div_mode(__fmul_rn(side, t), edge0, ieee));
        int q = (int)v;
        q = max(0, min(qmax, q));
        for (int j = 0; j < L; j++) key |= (uint32_t)((q >> j) & 1) << (D * j + k);
    }
    keys[i] = key;
    vals[i] = (int)i;
}

// ---------------------------------------------------------------------------------------------
// LSD radix sort, 8 bits per pass.  A fixed grid of blocks (a multiple of the SM count) each owns
// a contiguous chunk of the input; per pass: per-block digit histogram, one scan over the
// (digit, block) matrix, stable scatter with warp-level multi-split ranking.
// ---------------------------------------------------------------------------------------------
constexpr int RS_THREADS = 256;
constexpr int RS_ITEMS = 8;
constexpr int RS_WARPS = RS_THREADS / 32;
constexpr int RS_TILE = RS_THREADS * RS_ITEMS;

__global__ void __launch_bounds__(RS_THREADS) rs_hist(const uint32_t *__restrict__ keys, int64_t n, int shift,
                                                     int64_t chunk, int *counts, int G) {
    __shared__ int h[256];
    h[threadIdx.x] = 0;
    __syncthreads();
    int64_t beg = (int64_t)blockIdx.x * chunk, end = min(n, beg + chunk);
    for (int64_t i = beg + threadIdx.x; i < end; i += RS_THREADS) atomicAdd(&h[(keys[i] >> shift) & 255], 1);
    __syncthreads();
    counts[threadIdx.x * G + blockIdx.x] = h[threadIdx.x];
}

// Stable scatter of one pass.  Keys of a tile are first ranked (warp-level multi-split), then staged in
// shared memory in digit order, so that the global writes of a tile are runs of consecutive addresses
// per digit instead of 4-byte scatters.
__global__ void __launch_bounds__(RS_THREADS) rs_scatter(const uint32_t *__restrict__ keys, const int *__restrict__ vals,
                                                        int64_t n, int shift, int64_t chunk,
                                                        const int *__restrict__ scanned, int G, uint32_t *okeys,
                                                        int *ovals) {
    __shared__ int base[256];              // next global position per digit for this block
    __shared__ int dstart[256];            // start of the digit inside the staged tile
    __shared__ int wcnt[RS_WARPS][256];    // per-warp digit counts, then per-warp bases
    __shared__ uint32_t skeys[RS_TILE];
    __shared__ int svals[RS_TILE];
    __shared__ int scan_sm[33];
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    base[threadIdx.x] = scanned[threadIdx.x * G + blockIdx.x];
    for (int q = 0; q < RS_WARPS; q++) wcnt[q][threadIdx.x] = 0;
    __syncthreads();
    int64_t beg = (int64_t)blockIdx.x * chunk, end = min(n, beg + chunk);
    for (int64_t tile = beg; tile < end; tile += RS_TILE) {
        const int tile_cnt = (int)min((int64_t)RS_TILE, end - tile);
        uint32_t k[RS_ITEMS];
        int v[RS_ITEMS], off[RS_ITEMS];
#pragma unroll
        for (int r = 0; r < RS_ITEMS; r++) {
            int64_t i = tile + (int64_t)w * (32 * RS_ITEMS) + r * 32 + lane;
            bool valid = i < end;
            k[r] = valid ? keys[i] : 0u;
            v[r] = valid ? vals[i] : 0;
            int dg = valid ? (int)((k[r] >> shift) & 255) : 256;
            unsigned m = __match_any_sync(0xffffffffu, dg);
            int leader = __ffs(m) - 1;
            int rank = __popc(m & ((1u << lane) - 1));
            int old = 0;
            if (lane == leader && valid) {
                old = wcnt[w][dg];
                wcnt[w][dg] = old + __popc(m);
            }
            old = __shfl_sync(m, old, leader);
            off[r] = valid ? old + rank : -1;
            __syncwarp();
        }
        __syncthreads();
        int tile_total;
        {
            int run = 0;
#pragma unroll
            for (int q = 0; q < RS_WARPS; q++) {
                int c = wcnt[q][threadIdx.x];
                wcnt[q][threadIdx.x] = run;
                run += c;
            }
            tile_total = run;
        }
        dstart[threadIdx.x] = block_exclusive_scan(tile_total, nullptr, scan_sm);   // ends with a barrier
        __syncthreads();
#pragma unroll
        for (int r = 0; r < RS_ITEMS; r++) {
            if (off[r] >= 0) {
                int dg = (k[r] >> shift) & 255;
                int sp = dstart[dg] + wcnt[w][dg] + off[r];
                skeys[sp] = k[r];
                svals[sp] = v[r];
            }
        }
        __syncthreads();
        for (int q = threadIdx.x; q < tile_cnt; q += RS_THREADS) {
            uint32_t kk = skeys[q];
            int dg = (kk >> shift) & 255;
            int64_t pos = (int64_t)base[dg] + (q - dstart[dg]);
            okeys[pos] = kk;
            ovals[pos] = svals[q];
        }
        __syncthreads();
        base[threadIdx.x] += tile_total;
        for (int q = 0; q < RS_WARPS; q++) wcnt[q][threadIdx.x] = 0;
        __syncthreads();
    }
}

template <int D>
__global__ void __launch_bounds__(256) gather_points(const float *__restrict__ X, const int *__restrict__ perm, int64_t n,
                                                    float *pts) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    int64_t src = perm[i];
#pragma unroll
    for (int k = 0; k < D; k++) pts[(int64_t)k * n + i] = X[src * D + k];
}

__global__ void __launch_bounds__(256) gather_rows_kernel(const float *__restrict__ src, const int *__restrict__ perm,
                                                         float *dst, int64_t n, int cols) {
    int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= n * cols) return;
    int64_t i = e / cols;
    int c = (int)(e - i * cols);
    dst[e] = src[(int64_t)perm[i] * cols + c];
}
__global__ void __launch_bounds__(256) scatter_rows_kernel(const float *__restrict__ src, const int *__restrict__ perm,
                                                          float *dst, int64_t n, int cols) {
    int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= n * cols) return;
    int64_t i = e / cols;
    int c = (int)(e - i * cols);
    dst[(int64_t)perm[i] * cols + c] = src[e];
}
// rows that are entirely zero are skipped (dst must be zero-filled): used when only a slice of the sorted
// rows was computed, so that the random writes are paid for that slice only
__global__ void __launch_bounds__(256) scatter_rows_nonzero_kernel(const float *__restrict__ src, const int *__restrict__ perm,
                                                                  float *dst, int64_t n, int cols) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    bool any = false;
    for (int c = 0; c < cols; c++) any |= (src[i * cols + c] != 0.f);
    if (!any) return;
    const int64_t r = perm[i];
    for (int c = 0; c < cols; c++) dst[r * cols + c] = src[i * cols + c];
}
void scatter_rows_nonzero(const float *src, const int *perm, float *dst, int64_t n, int cols, cudaStream_t s) {
    if (n == 0) return;
    F3M_CUDA(cudaMemsetAsync(dst, 0, (size_t)n * cols * sizeof(float), s));
    scatter_rows_nonzero_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(src, perm, dst, n, cols);
    F3M_LAUNCH_CHECK();
}
void gather_rows(const float *src, const int *perm, float *dst, int64_t n, int cols, cudaStream_t s) {
    int64_t tot = n * cols;
    if (tot == 0) return;
    gather_rows_kernel<<<(unsigned)((tot + 255) / 256), 256, 0, s>>>(src, perm, dst, n, cols);
    F3M_LAUNCH_CHECK();
}
void scatter_rows(const float *src, const int *perm, float *dst, int64_t n, int cols, cudaStream_t s) {
    int64_t tot = n * cols;
    if (tot == 0) return;
    scatter_rows_kernel<<<(unsigned)((tot + 255) / 256), 256, 0, s>>>(src, perm, dst, n, cols);
    F3M_LAUNCH_CHECK();
}

void build_sorted_tree(Tree &t, const float *X, int64_t n, int d, const float *origin, float edge0, int math_mode,
                       f3m_plan *pl, cudaStream_t s) {
    (void)pl;
    F3M_REQUIRE(n < (int64_t)0x7fffffff, F3M_ERR_OVERFLOW, "point count %lld does not fit a 31-bit index", (long long)n);
    t.n = n;
    t.d = d;
    t.data = X;
    t.edge0 = edge0;
    for (int k = 0; k < d; k++) t.origin[k] = origin[k];
    // deepest level a 30-bit cell index holds (the reference's int cell index overflows beyond that)
    t.lmax = std::min(30 / d, 20);
    const int L = t.lmax;
    const int bits = d * L;
    DevBuf<uint32_t> k0, k1;
    DevBuf<int> v0, v1;
    k0.alloc(n, s); k1.alloc(n, s); v0.alloc(n, s); v1.alloc(n, s);
    const float side = (float)(1u << L);
    unsigned grid = (unsigned)((n + 255) / 256);
    const float *o = t.origin;
    const int ieee = math_mode == F3M_MATH_IEEE;
    switch (d) {
        case 1: morton_kernel<1><<<grid, 256, 0, s>>>(X, n, side, edge0, o[0], o[1], o[2], o[3], o[4], L, ieee, k0.p, v0.p); break;
        case 2: morton_kernel<2><<<grid, 256, 0, s>>>(X, n, side, edge0, o[0], o[1], o[2], o[3], o[4], L, ieee, k0.p, v0.p); break;
        case 3: morton_kernel<3><<<grid, 256, 0, s>>>(X, n, side, edge0, o[0], o[1], o[2], o[3], o[4], L, ieee, k0.p, v0.p); break;
        case 4: morton_kernel<4><<<grid, 256, 0, s>>>(X, n, side, edge0, o[0], o[1], o[2], o[3], o[4], L, ieee, k0.p, v0.p); break;
        default: morton_kernel<5><<<grid, 256, 0, s>>>(X, n, side, edge0, o[0], o[1], o[2], o[3], o[4], L, ieee, k0.p, v0.p); break;
    }
    F3M_LAUNCH_CHECK();

    int G = (int)std::min<int64_t>((n + RS_TILE - 1) / RS_TILE, NUM_SMS_HINT * 10);
    if (G < 1) G = 1;
    int64_t chunk = (n + G - 1) / G;
    chunk = (chunk + RS_TILE - 1) / RS_TILE * RS_TILE;
    DevBuf<int> counts;
    counts.alloc((size_t)256 * G + 1, s);
    uint32_t *ka = k0.p, *kb = k1.p;
    int *va = v0.p, *vb = v1.p;
    bool in_first = true;
    for (int shift = 0; shift < bits; shift += 8) {
        rs_hist<<<G, RS_THREADS, 0, s>>>(ka, n, shift, chunk, counts.p, G);
        F3M_LAUNCH_CHECK();
        exclusive_scan_i32(counts.p, counts.p, (int64_t)256 * G, s);
        rs_scatter<<<G, RS_THREADS, 0, s>>>(ka, va, n, shift, chunk, counts.p, G, kb, vb);
        F3M_LAUNCH_CHECK();
        std::swap(ka, kb);
        std::swap(va, vb);
        in_first = !in_first;
    }
    if (in_first) { t.keys = std::move(k0); t.perm = std::move(v0); }
    else { t.keys = std::move(k1); t.perm = std::move(v1); }
    t.pts.alloc((size_t)n * d, s);
    switch (d) {
        case 1: gather_points<1><<<grid, 256, 0, s>>>(X, t.perm.p, n, t.pts.p); break;
        case 2: gather_points<2><<<grid, 256, 0, s>>>(X, t.perm.p, n, t.pts.p); break;
        case 3: gather_points<3><<<grid, 256, 0, s>>>(X, t.perm.p, n, t.pts.p); break;
        case 4: gather_points<4><<<grid, 256, 0, s>>>(X, t.perm.p, n, t.pts.p); break;
        default: gather_points<5><<<grid, 256, 0, s>>>(X, t.perm.p, n, t.pts.p); break;
    }
    F3M_LAUNCH_CHECK();
}

}  // namespace f3m
