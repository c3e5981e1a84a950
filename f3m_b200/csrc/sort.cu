// Box division, first half: bounding cube, Morton keys, LSD radix sort, physical permutation.
//
// The reference assigns points to boxes level by level with a hash lookup and two global atomics
// per point per level and never moves the points (n_tree_cuda::divide, F3M_src/n_tree.cu:105-179;
// box_division_cum_hash / box_division_assign_hash, F3M_src/1_d_conv.cu:1127-1191).  Here every
// point gets ONE key -- its cell at the deepest level a 30-bit index can hold, bits interleaved so
// that every level's box is a key prefix -- the keys are sorted once, and the points are gathered
// into sorted planes by the sort itself (the coordinates travel with the keys).  All levels are then read
// off the sorted keys (tree.cu).  All kernels in this file are HBM-bound streaming passes.
#include <algorithm>
#include "common.cuh"

namespace f3m {

// ---------------------------------------------------------------------------------------------
// device-wide exclusive scan of up to four arrays of one length at once (three launches, no inter-block waiting)
// ---------------------------------------------------------------------------------------------
constexpr int SCAN_THREADS = 512;
constexpr int SCAN_ITEMS = 8;
constexpr int SCAN_TILE = SCAN_THREADS * SCAN_ITEMS;
struct ScanArrays {
    const int *in[4];
    int *out[4];
};

__global__ void __launch_bounds__(SCAN_THREADS) scan_tile_sums(ScanArrays a, int64_t n, int nt, int *part) {
    __shared__ int sm[33];
    const int *__restrict__ in = a.in[blockIdx.y];
    int64_t base = (int64_t)blockIdx.x * SCAN_TILE + (int64_t)threadIdx.x * SCAN_ITEMS;
    int s = 0;
#pragma unroll
    for (int k = 0; k < SCAN_ITEMS; k++)
        if (base + k < n) s += in[base + k];
    int total;
    block_exclusive_scan(s, &total, sm);
    if (threadIdx.x == 0) part[(size_t)blockIdx.y * nt + blockIdx.x] = total;
}

// one block per array; the array's sum goes to totals64 as a 64-bit number (an int32 sum can wrap unnoticed)
__global__ void __launch_bounds__(1024) scan_partials(int *part, int nparts, long long *totals64) {
    __shared__ int sm[33];
    int *row = part + (size_t)blockIdx.x * nparts;
    long long carry = 0;
    for (int base = 0; base < nparts; base += 1024) {
        int i = base + threadIdx.x;
        int v = i < nparts ? row[i] : 0;
        int total;
        int ex = block_exclusive_scan(v, &total, sm);
        if (i < nparts) row[i] = ex + (int)carry;
        carry += total;
    }
    if (threadIdx.x == 0 && totals64) totals64[blockIdx.x] = carry;
}

__global__ void __launch_bounds__(SCAN_THREADS) scan_tile_write(ScanArrays a, int64_t n, int nt, const int *__restrict__ part) {
    __shared__ int sm[33];
    const int *in = a.in[blockIdx.y];
    int *out = a.out[blockIdx.y];
    int64_t base = (int64_t)blockIdx.x * SCAN_TILE + (int64_t)threadIdx.x * SCAN_ITEMS;
    int v[SCAN_ITEMS];
    int s = 0;
#pragma unroll
    for (int k = 0; k < SCAN_ITEMS; k++) {
        v[k] = (base + k < n) ? in[base + k] : 0;
        s += v[k];
    }
    int ex = block_exclusive_scan(s, nullptr, sm) + part[(size_t)blockIdx.y * nt + blockIdx.x];
#pragma unroll
    for (int k = 0; k < SCAN_ITEMS; k++) {
        if (base + k < n) out[base + k] = ex;
        ex += v[k];
    }
}

// arrays[k] is scanned in place, k < narr <= 4; totals64 (device, narr entries, may be null) receives the sums
void exclusive_scan_multi(int *const *arrays, int narr, int64_t n, long long *totals64, cudaStream_t s) {
    if (n <= 0 || narr <= 0) return;
    F3M_REQUIRE(narr <= 4, F3M_ERR_INTERNAL, "exclusive_scan_multi takes at most four arrays");
    const int nt = (int)((n + SCAN_TILE - 1) / SCAN_TILE);
    ScanArrays a{};
    for (int k = 0; k < narr; k++) { a.in[k] = arrays[k]; a.out[k] = arrays[k]; }
    DevBuf<int> part;
    part.alloc((size_t)nt * narr, s);
    scan_tile_sums<<<dim3(nt, narr), SCAN_THREADS, 0, s>>>(a, n, nt, part.p);
    F3M_LAUNCH_CHECK();
    scan_partials<<<narr, 1024, 0, s>>>(part.p, nt, totals64);
    F3M_LAUNCH_CHECK();
    scan_tile_write<<<dim3(nt, narr), SCAN_THREADS, 0, s>>>(a, n, nt, part.p);
    F3M_LAUNCH_CHECK();
}

void exclusive_scan_i32(const int *in, int *out, int64_t n, cudaStream_t s) {
    if (n <= 0) return;
    const int nt = (int)((n + SCAN_TILE - 1) / SCAN_TILE);
    ScanArrays a{};
    a.in[0] = in; a.out[0] = out;
    DevBuf<int> part;
    part.alloc(nt, s);
    scan_tile_sums<<<dim3(nt, 1), SCAN_THREADS, 0, s>>>(a, n, nt, part.p);
    F3M_LAUNCH_CHECK();
    scan_partials<<<1, 1024, 0, s>>>(part.p, nt, nullptr);
    F3M_LAUNCH_CHECK();
    scan_tile_write<<<dim3(nt, 1), SCAN_THREADS, 0, s>>>(a, n, nt, part.p);
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
    unsigned *mm = reinterpret_cast<unsigned *>(pl->d_flags) + FL_BBOX;   // 2*MAXD words
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

// ---------------------------------------------------------------------------------------------
// LSD radix sort of (key, input row, coordinates), least significant digit first, digits of up to 10 bits.
// Only the key bits the tree will use are sorted (d bits per level).  The coordinates travel with the keys, so the
// last pass leaves the points in sorted planes and no gather through the permutation is needed; every pass reads
// and writes its arrays once, in streams (HBM-bound: 8 + 4 d bytes per point read and written).
//
// A fixed grid of blocks (one wave: SM count x resident blocks) each owns a contiguous run of tiles.  Per pass:
// digit histogram per block (the first one is taken while the keys are computed), one scan per digit over the
// blocks, stable scatter.  The scatter ranks a tile's keys with warp-level match (warp-private counters), stages
// every array of the tile in shared memory in digit order and writes runs of consecutive addresses.
// No block waits for another block.
// ---------------------------------------------------------------------------------------------
constexpr int RS_T = 256;                 // threads per block
constexpr int RS_I = 8;                   // keys per thread and tile
constexpr int RS_W = RS_T / 32;
constexpr int RS_TILE = RS_T * RS_I;      // 2048 keys
constexpr int RS_MAXBITS = 10;
constexpr int RS_MAXBINS = 1 << RS_MAXBITS;
constexpr int RS_DPT = RS_MAXBINS / RS_T; // digits owned by a thread

struct MortonCfg {
    float org[MAXD];
    float side, edge0;
    int L, ieee;
};

// Morton key of one point; spread[v] moves bit j of the 5-bit value v to bit D*j (a 32-entry table in shared memory)
template <int D>
__device__ __forceinline__ uint32_t morton_key(const float (&x)[D], const MortonCfg &cfg, const uint32_t *spread) {
    const int qmax = (1 << cfg.L) - 1;
    uint32_t key = 0;
#pragma unroll
    for (int k = 0; k < D; k++) {
        float t = __fsub_rn(x[k], cfg.org[k]);
        int q = (int)floorf(div_mode(__fmul_rn(cfg.side, t), cfg.edge0, cfg.ieee));
        q = max(0, min(qmax, q));
        uint32_t sk = 0;
#pragma unroll
        for (int c = 0; c < 4; c++)   // 5 bits at a time; 20 bits hold the deepest key (d = 1)
            if (5 * c < cfg.L) sk |= spread[(q >> (5 * c)) & 31] << (5 * D * c);
        key |= sk << k;
    }
    return key;
}
template <int D>
__device__ __forceinline__ void fill_spread_table(uint32_t *spread) {
    if (threadIdx.x < 32) {
        uint32_t v = 0;
        for (int j = 0; j < 5; j++) v |= ((threadIdx.x >> j) & 1u) << (D * j);
        spread[threadIdx.x] = v;
    }
}

// keys of a block's chunk and the histogram of their first digit
template <int D>
__global__ void __launch_bounds__(512) morton_hist_kernel(const float *__restrict__ X, int64_t n, MortonCfg cfg, int shift,
                                                         int dbits, int64_t chunk, uint32_t *keys, int *counts, int G) {
    __shared__ int hist[RS_MAXBINS];
    __shared__ uint32_t spread[32];   // bit j of a 5-bit value -> bit D*j
    for (int q = threadIdx.x; q < RS_MAXBINS; q += blockDim.x) hist[q] = 0;
    fill_spread_table<D>(spread);
    __syncthreads();
    const uint32_t mask = (1u << dbits) - 1u;
    const int64_t beg = (int64_t)blockIdx.x * chunk, end = min(n, beg + chunk);
    constexpr int U = 4;   // points per thread and round: all their loads are issued before the first is used
    for (int64_t i0 = beg + threadIdx.x; i0 < end; i0 += (int64_t)U * blockDim.x) {
        float x[U][D];
#pragma unroll
        for (int u = 0; u < U; u++) {
            const int64_t i = i0 + (int64_t)u * blockDim.x;
#pragma unroll
            for (int k = 0; k < D; k++) x[u][k] = i < end ? X[i * D + k] : 0.f;
        }
#pragma unroll
        for (int u = 0; u < U; u++) {
            const int64_t i = i0 + (int64_t)u * blockDim.x;
            if (i >= end) break;
            const uint32_t key = morton_key<D>(x[u], cfg, spread);
            keys[i] = key;
            atomicAdd(&hist[(key >> shift) & mask], 1);
        }
    }
    __syncthreads();
    const int nbins = 1 << dbits;
    for (int q = threadIdx.x; q < nbins; q += blockDim.x) counts[(size_t)q * G + blockIdx.x] = hist[q];
}

__global__ void __launch_bounds__(512) rs_hist(const uint32_t *__restrict__ keys, int64_t n, int shift, int dbits, int64_t chunk,
                                              int *counts, int G) {
    __shared__ int hist[RS_MAXBINS];
    for (int q = threadIdx.x; q < RS_MAXBINS; q += blockDim.x) hist[q] = 0;
    __syncthreads();
    const uint32_t mask = (1u << dbits) - 1u;
    const int64_t beg = (int64_t)blockIdx.x * chunk, end = min(n, beg + chunk);
    for (int64_t i = beg + threadIdx.x; i < end; i += blockDim.x) atomicAdd(&hist[(keys[i] >> shift) & mask], 1);
    __syncthreads();
    const int nbins = 1 << dbits;
    for (int q = threadIdx.x; q < nbins; q += blockDim.x) counts[(size_t)q * G + blockIdx.x] = hist[q];
}

// one block per digit: exclusive scan of the digit's counts over the blocks, and the digit's total
__global__ void __launch_bounds__(256) rs_scan_rows(int *counts, int G, int *tot) {
    __shared__ int sm[33];
    int *row = counts + (size_t)blockIdx.x * G;
    int carry = 0;
    for (int base = 0; base < G; base += 256) {
        const int i = base + threadIdx.x;
        const int v = i < G ? row[i] : 0;
        int total;
        const int ex = block_exclusive_scan(v, &total, sm);
        if (i < G) row[i] = ex + carry;
        carry += total;
    }
    if (threadIdx.x == 0) tot[blockIdx.x] = carry;
}

// Words of the record that travels with a key: [input row, x_0 .. x_{D-1}], padded so that it moves as 8- or
// 16-byte vectors.
template <int D> struct Rec { static constexpr int VW = 2, RV = (D + 2) / 2; };   // D = 1: 1 x 8 B; D = 4, 5: 3 x 8 B
template <> struct Rec<2> { static constexpr int VW = 4, RV = 1; };                // 16 B
template <> struct Rec<3> { static constexpr int VW = 4, RV = 1; };                // 16 B
template <int VW> struct VecOf;
template <> struct VecOf<2> { typedef uint2 type; };
template <> struct VecOf<4> { typedef uint4 type; };

struct SortIO {
    const uint32_t *kin;       // keys of this pass's input order
    const float *X;            // first pass: the caller's row-major points (the record is built from them)
    int row0;                  // first pass: the record's row is row0 + position
    const void *rin;           // later passes: records of the input order
    uint32_t *kout;
    void *rout;                // records of the output order
    int first;
};

__host__ __device__ constexpr size_t rs_smem_bytes(int nbins, int rec_words) {
    // per-warp counters (u16), gofs + bbase (int), staged keys, staged records
    return (size_t)RS_W * nbins * 2 + (size_t)2 * nbins * 4 + (size_t)RS_TILE * 4 + (size_t)RS_TILE * rec_words * 4;
}

// STABLE = false ranks a key among the tile's keys of its digit in whatever order the shared-memory atomics grant.
// That would do for a first pass on one GPU (points that agree in every sorted bit lie in one finest-level box), but
// the order then differs from run to run, so the host uses the stable form for every pass.
template <int D, bool STABLE>
__global__ void __launch_bounds__(RS_T, 3) rs_scatter(SortIO io, int64_t n, int shift, int dbits, int64_t chunk,
                                                  const int *__restrict__ rowex, const int *__restrict__ tot, int G) {
    constexpr int VW = Rec<D>::VW, RV = Rec<D>::RV, RW = VW * RV;
    typedef typename VecOf<VW>::type vec_t;
    extern __shared__ __align__(16) unsigned char rs_smem[];
    __shared__ int scan_sm[33];
    const int nbins = 1 << dbits;
    vec_t *stage_rec = reinterpret_cast<vec_t *>(rs_smem);                                  // [RS_TILE][RV]
    uint32_t *stage_key = reinterpret_cast<uint32_t *>(rs_smem + (size_t)RS_TILE * RW * 4);   // [RS_TILE]
    int *gofs = reinterpret_cast<int *>(stage_key + RS_TILE);   // global position of staged slot q of digit g: gofs[g] + q
    int *bbase = gofs + nbins;                                  // next global position per digit for this block
    unsigned short *wcnt = reinterpret_cast<unsigned short *>(bbase + nbins);   // [RS_W][nbins] counts, then start slots
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const uint32_t mask = (uint32_t)nbins - 1u;
    unsigned short *wrow = wcnt + (size_t)w * nbins;
    // digits [d0, d0 + dpt) belong to this thread (none when the block has more threads than digits)
    const int dpt = (nbins + RS_T - 1) / RS_T;
    const int d0 = threadIdx.x * dpt;
    const bool owner = d0 < nbins;
    {
        int t[RS_DPT], sum = 0;
#pragma unroll
        for (int q = 0; q < RS_DPT; q++) {
            t[q] = (q < dpt && owner) ? tot[d0 + q] : 0;
            sum += t[q];
        }
        int ex = block_exclusive_scan(sum, nullptr, scan_sm);
#pragma unroll
        for (int q = 0; q < RS_DPT; q++) {
            if (q < dpt && owner) {
                bbase[d0 + q] = ex + rowex[(size_t)(d0 + q) * G + blockIdx.x];
                ex += t[q];
                for (int ww = 0; ww < RS_W; ww++) wcnt[(size_t)ww * nbins + d0 + q] = 0;
                gofs[d0 + q] = 0;
            }
        }
    }
    __syncthreads();
    const int64_t beg = (int64_t)blockIdx.x * chunk, end = min(n, beg + chunk);
    for (int64_t tile = beg; tile < end; tile += RS_TILE) {
        const int tile_cnt = (int)min((int64_t)RS_TILE, end - tile);
        const int j0 = w * (32 * RS_I) + lane;   // item r of this lane: point tile + j0 + 32 r
        const uint32_t *__restrict__ kin = io.kin + tile;
        uint32_t key[RS_I];
        vec_t rec[RS_I][RV];
        int sp[RS_I];
#pragma unroll
        for (int r = 0; r < RS_I; r++) key[r] = (j0 + 32 * r < tile_cnt) ? kin[j0 + 32 * r] : 0u;
        if (io.first) {
            const float *__restrict__ xin = io.X + tile * D;
#pragma unroll
            for (int r = 0; r < RS_I; r++) {
                const int j = j0 + 32 * r;
                uint32_t wds[RW];
#pragma unroll
                for (int q = 0; q < RW; q++) wds[q] = 0u;
                if (j < tile_cnt) {
                    wds[0] = (uint32_t)(io.row0 + tile + j);
#pragma unroll
                    for (int k = 0; k < D; k++) wds[1 + k] = __float_as_uint(xin[j * D + k]);
                }
#pragma unroll
                for (int v = 0; v < RV; v++) {
                    if (VW == 4) rec[r][v] = *reinterpret_cast<vec_t *>(&wds[4 * v]);
                    else { uint2 t2 = make_uint2(wds[2 * v], wds[2 * v + 1]); rec[r][v] = *reinterpret_cast<vec_t *>(&t2); }
                }
            }
        } else {
            const vec_t *__restrict__ rin = reinterpret_cast<const vec_t *>(io.rin) + tile * RV;
#pragma unroll
            for (int r = 0; r < RS_I; r++) {
                const int j = j0 + 32 * r;
#pragma unroll
                for (int v = 0; v < RV; v++)
                    if (j < tile_cnt) rec[r][v] = rin[j * RV + v];
            }
        }
        if (STABLE) {
            // rank inside the warp: items in (r, lane) order = input order.  The lanes that hold the same digit are
            // found with one ballot per digit bit (the match instruction costs a step per distinct value, and nearly
            // all 32 digits of a warp are distinct).
#pragma unroll
            for (int r = 0; r < RS_I; r++) {
                const bool valid = j0 + 32 * r < tile_cnt;
                const int dg = (int)((key[r] >> shift) & mask);
                unsigned m = __ballot_sync(0xffffffffu, valid);
#pragma unroll
                for (int bit = 0; bit < RS_MAXBITS; bit++) {
                    if (bit < dbits) {
                        const unsigned bal = __ballot_sync(0xffffffffu, (dg >> bit) & 1);
                        m &= ((dg >> bit) & 1) ? bal : ~bal;
                    }
                }
                // m: valid lanes with this lane's digit (meaningless on invalid lanes, which take no part)
                const int leader = __ffs(m) - 1;
                int old = 0;
                if (valid && lane == leader) {
                    old = wrow[dg];
                    wrow[dg] = (unsigned short)(old + __popc(m));
                }
                old = __shfl_sync(0xffffffffu, old, valid ? leader : lane);
                sp[r] = valid ? old + __popc(m & ((1u << lane) - 1u)) : -1;
                __syncwarp();
            }
        } else {
            // one counter per digit for the whole tile (kept in gofs until the scan below replaces it)
#pragma unroll
            for (int r = 0; r < RS_I; r++)
                sp[r] = (j0 + 32 * r < tile_cnt) ? atomicAdd(&gofs[(key[r] >> shift) & mask], 1) : -1;
        }
        __syncthreads();
        // per digit: start slot in the staged tile (per warp in the stable form), global position of slot 0
        int tsum[RS_DPT];
        {
            int sum = 0;
#pragma unroll
            for (int q = 0; q < RS_DPT; q++) {
                int run = 0;
                if (q < dpt && owner) {
                    if (STABLE) for (int ww = 0; ww < RS_W; ww++) run += wcnt[(size_t)ww * nbins + d0 + q];
                    else run = gofs[d0 + q];
                }
                tsum[q] = run;
                sum += run;
            }
            int ex = block_exclusive_scan(sum, nullptr, scan_sm);
#pragma unroll
            for (int q = 0; q < RS_DPT; q++) {
                if (q < dpt && owner) {
                    gofs[d0 + q] = bbase[d0 + q] - ex;
                    if (STABLE) {
                        int run = ex;
                        for (int ww = 0; ww < RS_W; ww++) {
                            const int c = wcnt[(size_t)ww * nbins + d0 + q];
                            wcnt[(size_t)ww * nbins + d0 + q] = (unsigned short)run;
                            run += c;
                        }
                    } else
                        wcnt[d0 + q] = (unsigned short)ex;   // row 0 holds the start slots
                    ex += tsum[q];
                }
            }
        }
        __syncthreads();
#pragma unroll
        for (int r = 0; r < RS_I; r++) {
            if (sp[r] >= 0) {
                const int slot = sp[r] + (STABLE ? wrow : wcnt)[(key[r] >> shift) & mask];
                stage_key[slot] = key[r];
#pragma unroll
                for (int v = 0; v < RV; v++) stage_rec[slot * RV + v] = rec[r][v];
            }
        }
        __syncthreads();
        // positions of the staged slots (runs of consecutive global positions per digit); then the counters are
        // cleared for the next tile and the block's positions advance
        int pos[RS_I];
#pragma unroll
        for (int k = 0; k < RS_I; k++) {
            const int q = threadIdx.x + k * RS_T;
            pos[k] = q < tile_cnt ? gofs[(stage_key[q] >> shift) & mask] + q : -1;
        }
        if (!STABLE) __syncthreads();   // gofs is cleared below: every thread must have read it
#pragma unroll
        for (int q = 0; q < RS_DPT; q++) {
            if (q < dpt && owner) {
                bbase[d0 + q] += tsum[q];
                if (STABLE) for (int ww = 0; ww < RS_W; ww++) wcnt[(size_t)ww * nbins + d0 + q] = 0;
                else gofs[d0 + q] = 0;
            }
        }
#pragma unroll
        for (int k = 0; k < RS_I; k++) {
            if (pos[k] >= 0) {
                const int q = threadIdx.x + k * RS_T;
                io.kout[pos[k]] = stage_key[q];
                vec_t *rout = reinterpret_cast<vec_t *>(io.rout) + (size_t)pos[k] * RV;
#pragma unroll
                for (int v = 0; v < RV; v++) rout[v] = stage_rec[q * RV + v];
            }
        }
        __syncthreads();
    }
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

// records [input row, x_0 .. x_{D-1}] of the sorted order -> permutation and coordinate planes
template <int D>
__global__ void __launch_bounds__(256) unpack_records(const void *__restrict__ recs, int64_t n, int *perm, float *pts) {
    constexpr int VW = Rec<D>::VW, RV = Rec<D>::RV, RW = VW * RV;
    typedef typename VecOf<VW>::type vec_t;
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    uint32_t wds[RW];
#pragma unroll
    for (int v = 0; v < RV; v++) {
        const vec_t t = reinterpret_cast<const vec_t *>(recs)[i * RV + v];
        const uint32_t *tw = reinterpret_cast<const uint32_t *>(&t);
#pragma unroll
        for (int c = 0; c < VW; c++) wds[VW * v + c] = tw[c];
    }
    perm[i] = (int)wds[0];
#pragma unroll
    for (int c = 0; c < D; c++) pts[(size_t)c * n + i] = __uint_as_float(wds[1 + c]);
}

// keys and records [row0 + position, coordinates] of n points, sorted by the key bits [shift0, shift0 + bits)
template <int D>
static void sort_records(const float *X, int64_t n, int row0, const MortonCfg &cfg, int shift0, int bits, DevBuf<uint32_t> &keys_out,
                         DevBuf<uint32_t> &recs_out, cudaStream_t s) {
    constexpr int RW = Rec<D>::VW * Rec<D>::RV;
    const int passes = (bits + RS_MAXBITS - 1) / RS_MAXBITS;
    const int dbits_all = (bits + passes - 1) / passes;
    const size_t smem = rs_smem_bytes(1 << dbits_all, RW);
    // one wave of blocks, each with a contiguous run of whole tiles
    int dev = 0, sms = NUM_SMS_HINT, occ = 1;
    F3M_CUDA(cudaGetDevice(&dev));
    F3M_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    F3M_CUDA(cudaFuncSetAttribute(rs_scatter<D, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    F3M_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, rs_scatter<D, true>, RS_T, smem));
    const int64_t ntiles = (n + RS_TILE - 1) / RS_TILE;
    const int64_t wave = (int64_t)sms * std::max(1, occ);
    const int64_t tpb = (ntiles + wave - 1) / wave;
    const int G = (int)((ntiles + tpb - 1) / tpb);
    const int64_t chunk = tpb * RS_TILE;

    DevBuf<uint32_t> kA, kB, rA, rB;   // keys and records, ping-pong
    DevBuf<int> counts, tot;
    kA.alloc(n, s); kB.alloc(n, s);
    rB.alloc((size_t)n * RW, s);
    if (passes > 1) rA.alloc((size_t)n * RW, s);
    counts.alloc((size_t)RS_MAXBINS * G, s);
    tot.alloc(RS_MAXBINS, s);

    for (int pass = 0; pass < passes; pass++) {
        const int shift = shift0 + pass * dbits_all;
        const int dbits = std::min(dbits_all, shift0 + bits - shift);
        const bool to_b = (pass % 2) == 0;
        if (pass == 0) morton_hist_kernel<D><<<G, 512, 0, s>>>(X, n, cfg, shift, dbits, chunk, kA.p, counts.p, G);
        else rs_hist<<<G, 512, 0, s>>>(to_b ? kA.p : kB.p, n, shift, dbits, chunk, counts.p, G);
        F3M_LAUNCH_CHECK();
        rs_scan_rows<<<1 << dbits, 256, 0, s>>>(counts.p, G, tot.p);
        F3M_LAUNCH_CHECK();
        SortIO io{};
        io.first = pass == 0;
        io.row0 = row0;
        io.kin = to_b ? kA.p : kB.p;
        io.kout = to_b ? kB.p : kA.p;
        io.X = X;
        io.rin = to_b ? rA.p : rB.p;
        io.rout = to_b ? rB.p : rA.p;
        // every pass stable, the first one too: ranks that build the same plan on different GPUs must end with the same
        // permutation (their sorted slices are exchanged), and the form ranked by atomics measured no faster
        rs_scatter<D, true><<<G, RS_T, rs_smem_bytes(1 << dbits, RW), s>>>(io, n, shift, dbits, chunk, counts.p, tot.p, G);
        F3M_LAUNCH_CHECK();
    }
    keys_out = std::move(passes % 2 == 1 ? kB : kA);
    recs_out = std::move(passes % 2 == 1 ? rB : rA);
}

template <int D>
static void sort_passes(Tree &t, const float *X, const MortonCfg &cfg, int shift0, int bits, cudaStream_t s) {
    const int64_t n = t.n;
    DevBuf<uint32_t> recs;
    sort_records<D>(X, n, 0, cfg, shift0, bits, t.keys, recs, s);
    t.perm.alloc(n, s);
    t.pts.alloc((size_t)n * D, s);
    unpack_records<D><<<(unsigned)((n + 255) / 256), 256, 0, s>>>(recs.p, n, t.perm.p, t.pts.p);
    F3M_LAUNCH_CHECK();
}

static MortonCfg morton_cfg(int d, const float *origin, float edge0, int math_mode) {
    MortonCfg cfg{};
    for (int k = 0; k < d; k++) cfg.org[k] = origin[k];
    cfg.L = std::min(30 / d, 20);
    cfg.side = (float)(1u << cfg.L);
    cfg.edge0 = edge0;
    cfg.ieee = math_mode == F3M_MATH_IEEE;
    return cfg;
}

int record_words(int d) {
    switch (d) {
        case 1: return Rec<1>::VW * Rec<1>::RV;
        case 2: return Rec<2>::VW * Rec<2>::RV;
        case 3: return Rec<3>::VW * Rec<3>::RV;
        case 4: return Rec<4>::VW * Rec<4>::RV;
        default: return Rec<5>::VW * Rec<5>::RV;
    }
}

// points of one finest sorted cell in a sorted run: first and one-past-last position (0, 0 for cells the run misses)
__global__ void __launch_bounds__(256) cell_bounds_kernel(const uint32_t *__restrict__ keys, int64_t n, int shift0, int *seg_start,
                                                         int *seg_end) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        const uint32_t c = keys[i] >> shift0;
        if (i == 0 || (keys[i - 1] >> shift0) != c) seg_start[c] = (int)i;
        if (i == n - 1 || (keys[i + 1] >> shift0) != c) seg_end[c] = (int)i + 1;
    }
}
__global__ void __launch_bounds__(256) cell_counts_kernel(int ncells, const int *__restrict__ seg_start, const int *__restrict__ seg_end,
                                                         int *counts) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c < ncells) counts[c] = seg_end[c] - seg_start[c];
}

// One rank's share of a sort that several GPUs do together: the records [input row, coordinates] of the n points of
// X (rows row0 ... of the whole set), sorted by the first `depth` levels of their keys, and the number of points in
// every cell of that depth (2^(d depth) counts), into the caller's arrays.
void sort_shard(const float *X, int64_t n, int64_t row0, int d, const float *origin, float edge0, int math_mode, int depth,
                uint32_t *recs_out, int *cell_counts_out, cudaStream_t s) {
    F3M_REQUIRE(row0 + n < (int64_t)0x7fffffff, F3M_ERR_OVERFLOW, "row %lld does not fit a 31-bit index", (long long)(row0 + n));
    const MortonCfg cfg = morton_cfg(d, origin, edge0, math_mode);
    depth = std::max(1, std::min(depth, cfg.L));
    F3M_REQUIRE(d * depth <= 22, F3M_ERR_UNSUPPORTED, "shards sorted by %d key bits: the cell table holds at most 22", d * depth);
    const int shift0 = d * (cfg.L - depth), bits = d * depth, ncells = 1 << bits;
    DevBuf<uint32_t> keys, recs;
    switch (d) {
        case 1: sort_records<1>(X, n, (int)row0, cfg, shift0, bits, keys, recs, s); break;
        case 2: sort_records<2>(X, n, (int)row0, cfg, shift0, bits, keys, recs, s); break;
        case 3: sort_records<3>(X, n, (int)row0, cfg, shift0, bits, keys, recs, s); break;
        case 4: sort_records<4>(X, n, (int)row0, cfg, shift0, bits, keys, recs, s); break;
        default: sort_records<5>(X, n, (int)row0, cfg, shift0, bits, keys, recs, s); break;
    }
    F3M_CUDA(cudaMemcpyAsync(recs_out, recs.p, (size_t)n * record_words(d) * 4, cudaMemcpyDeviceToDevice, s));
    DevBuf<int> a, b;
    a.alloc(ncells, s); b.alloc(ncells, s);
    a.zero(); b.zero();
    const unsigned g = (unsigned)std::max<int64_t>(1, std::min<int64_t>((n + 255) / 256, NUM_SMS_HINT * 16));
    cell_bounds_kernel<<<g, 256, 0, s>>>(keys.p, n, shift0, a.p, b.p);
    F3M_LAUNCH_CHECK();
    cell_counts_kernel<<<(unsigned)((ncells + 255) / 256), 256, 0, s>>>(ncells, a.p, b.p, cell_counts_out);
    F3M_LAUNCH_CHECK();
}

// ---------------------------------------------------------------------------------------------
// A tree from sorted runs (one per rank).  Every run is sorted by the same key bits, so the points of one finest
// sorted cell form one segment per run and the merged order is cell by cell, run by run -- the same on every rank.
// The levels of the tree follow from the cell counts alone (tree.cu builds them from one pseudo key per occupied
// cell), so they -- and the interaction lists -- can be built while the records are still on the wire; the records
// are merged in afterwards, one warp per cell (taken apart into permutation and coordinate planes on the way).
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) cell_totals_kernel(int ncells, int nruns, const int *__restrict__ counts, int *total,
                                                         int *occupied) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c > ncells) return;
    int t = 0;
    if (c < ncells)
        for (int r = 0; r < nruns; r++) t += counts[(size_t)r * ncells + c];
    total[c] = t;   // entry ncells = 0: the scans turn it into the grand totals
    occupied[c] = t > 0;
}

// occupied cell number rank[c]: its pseudo key (cell id at the key's position) and the merged offset of its points
__global__ void __launch_bounds__(256) occupied_cells_kernel(int ncells, const int *__restrict__ total_before,
                                                            const int *__restrict__ rank, int shift0, uint32_t *pkeys, int *fine_off) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c > ncells) return;
    if (c == ncells) { fine_off[rank[c]] = total_before[c]; return; }
    if (rank[c + 1] != rank[c]) {
        pkeys[rank[c]] = (uint32_t)c << shift0;
        fine_off[rank[c]] = total_before[c];
    }
}

template <int D>
__global__ void __launch_bounds__(256) merge_runs_kernel(const void *__restrict__ recs, int64_t stride, int nruns, int ncells,
                                                        const int *__restrict__ counts, const int *__restrict__ seg_start,
                                                        const int *__restrict__ cell_off, int64_t n, int *perm, float *pts) {
    constexpr int VW = Rec<D>::VW, RV = Rec<D>::RV, RW = VW * RV;
    typedef typename VecOf<VW>::type vec_t;
    const int lane = threadIdx.x & 31;
    const int c = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    if (c >= ncells) return;
    int dst = cell_off[c];
    if (cell_off[c + 1] == dst) return;
    for (int r = 0; r < nruns; r++) {
        const int a = seg_start[(size_t)r * (ncells + 1) + c], len = counts[(size_t)r * ncells + c];
        const vec_t *rc = reinterpret_cast<const vec_t *>(recs) + (size_t)r * stride * RV;
        for (int i = a + lane; i < a + len; i += 32) {
            const int o = dst + (i - a);
            uint32_t wds[RW];
#pragma unroll
            for (int v = 0; v < RV; v++) {
                const vec_t t = rc[(size_t)i * RV + v];
                const uint32_t *tw = reinterpret_cast<const uint32_t *>(&t);
#pragma unroll
                for (int q = 0; q < VW; q++) wds[VW * v + q] = tw[q];
            }
            perm[o] = (int)wds[0];
#pragma unroll
            for (int q = 0; q < D; q++) pts[(size_t)q * n + o] = __uint_as_float(wds[1 + q]);
        }
        dst += len;
    }
}

// counts: (nruns, ncells) device array, the cell counts of every run.  Prepares the tree's size, the tables the
// merge needs and the pseudo keys the levels are built from; the points themselves come with attach_runs.
void tree_from_cell_counts(Tree &t, const int *counts, int nruns, int d, const float *origin, float edge0, int depth, f3m_plan *pl,
                           cudaStream_t s) {
    t.d = d;
    t.data = nullptr;   // the points exist as runs only: this tree cannot be sorted again to a greater depth
    t.edge0 = edge0;
    for (int k = 0; k < d; k++) t.origin[k] = origin[k];
    t.lmax = std::min(30 / d, 20);
    depth = std::max(1, std::min(depth, t.lmax));
    F3M_REQUIRE(d * depth <= 22, F3M_ERR_UNSUPPORTED, "runs sorted by %d key bits: the cell table holds at most 22", d * depth);
    t.sorted_depth = depth;
    const int shift0 = d * (t.lmax - depth), ncells = 1 << (d * depth);
    Tree::Runs &ru = t.runs;
    ru.nruns = nruns; ru.ncells = ncells;
    ru.counts.alloc((size_t)nruns * ncells, s);
    F3M_CUDA(cudaMemcpyAsync(ru.counts.p, counts, (size_t)nruns * ncells * sizeof(int), cudaMemcpyDeviceToDevice, s));
    ru.cell_off.alloc((size_t)ncells + 1, s);
    DevBuf<int> rank;
    rank.alloc((size_t)ncells + 1, s);
    cell_totals_kernel<<<(unsigned)((ncells + 1 + 255) / 256), 256, 0, s>>>(ncells, nruns, ru.counts.p, ru.cell_off.p, rank.p);
    F3M_LAUNCH_CHECK();
    int *both[2] = {ru.cell_off.p, rank.p};
    long long *d_tot = reinterpret_cast<long long *>(pl->d_flags + FL_LISTTOT);
    exclusive_scan_multi(both, 2, (int64_t)ncells + 1, d_tot, s);
    // position of every cell inside its run: one scan per run (rows of ncells + 1, the last entry closes the row)
    ru.seg_start.alloc((size_t)nruns * (ncells + 1), s);
    for (int r = 0; r < nruns; r++) {
        int *row = ru.seg_start.p + (size_t)r * (ncells + 1);
        F3M_CUDA(cudaMemcpyAsync(row, ru.counts.p + (size_t)r * ncells, (size_t)ncells * sizeof(int), cudaMemcpyDeviceToDevice, s));
        F3M_CUDA(cudaMemsetAsync(row + ncells, 0, sizeof(int), s));
    }
    for (int r0 = 0; r0 < nruns; r0 += 4) {
        int *rows[4];
        const int nr = std::min(4, nruns - r0);
        for (int q = 0; q < nr; q++) rows[q] = ru.seg_start.p + (size_t)(r0 + q) * (ncells + 1);
        exclusive_scan_multi(rows, nr, (int64_t)ncells + 1, nullptr, s);
    }
    long long *h = reinterpret_cast<long long *>(pl->h_pinned + FL_LISTTOT);
    F3M_CUDA(cudaMemcpyAsync(h, d_tot, 2 * sizeof(long long), cudaMemcpyDeviceToHost, s));
    F3M_CUDA(cudaStreamSynchronize(s));
    const long long n = h[0], nocc = h[1];
    F3M_REQUIRE(n > 0 && n < 0x7fffffffLL, F3M_ERR_OVERFLOW, "point count %lld does not fit a 31-bit index", n);
    t.n = n;
    ru.pkeys.alloc((size_t)nocc, s);
    ru.fine_off.alloc((size_t)nocc + 1, s);
    occupied_cells_kernel<<<(unsigned)((ncells + 1 + 255) / 256), 256, 0, s>>>(ncells, ru.cell_off.p, rank.p, shift0, ru.pkeys.p,
                                                                               ru.fine_off.p);
    F3M_LAUNCH_CHECK();
    ru.nocc = (int)nocc;
    ru.pending = true;
}

// records: the all-gathered sorted runs, run r at record r * stride
void tree_attach_runs(Tree &t, const uint32_t *recs, int64_t stride, cudaStream_t s) {
    Tree::Runs &ru = t.runs;
    F3M_REQUIRE(ru.pending, F3M_ERR_ARG, "this plan does not wait for sorted runs");
    const int64_t n = t.n;
    const int d = t.d, nruns = ru.nruns, ncells = ru.ncells;
    t.perm.alloc(n, s); t.pts.alloc((size_t)n * d, s);
    const unsigned gm = (unsigned)(((int64_t)ncells * 32 + 255) / 256);
    switch (d) {
        case 1: merge_runs_kernel<1><<<gm, 256, 0, s>>>(recs, stride, nruns, ncells, ru.counts.p, ru.seg_start.p, ru.cell_off.p, n, t.perm.p, t.pts.p); break;
        case 2: merge_runs_kernel<2><<<gm, 256, 0, s>>>(recs, stride, nruns, ncells, ru.counts.p, ru.seg_start.p, ru.cell_off.p, n, t.perm.p, t.pts.p); break;
        case 3: merge_runs_kernel<3><<<gm, 256, 0, s>>>(recs, stride, nruns, ncells, ru.counts.p, ru.seg_start.p, ru.cell_off.p, n, t.perm.p, t.pts.p); break;
        case 4: merge_runs_kernel<4><<<gm, 256, 0, s>>>(recs, stride, nruns, ncells, ru.counts.p, ru.seg_start.p, ru.cell_off.p, n, t.perm.p, t.pts.p); break;
        default: merge_runs_kernel<5><<<gm, 256, 0, s>>>(recs, stride, nruns, ncells, ru.counts.p, ru.seg_start.p, ru.cell_off.p, n, t.perm.p, t.pts.p); break;
    }
    F3M_LAUNCH_CHECK();
    F3M_CUDA(cudaStreamSynchronize(s));
    ru = Tree::Runs{};   // the tables are no longer needed
}

// Sorts the points of one tree by the first `depth` levels of their Morton key (all later levels are read off the
// sorted keys, tree.cu) and leaves keys, permutation and coordinate planes in the tree.
void build_sorted_tree(Tree &t, const float *X, int64_t n, int d, const float *origin, float edge0, int math_mode, int depth,
                       cudaStream_t s) {
    F3M_REQUIRE(n < (int64_t)0x7fffffff, F3M_ERR_OVERFLOW, "point count %lld does not fit a 31-bit index", (long long)n);
    t.n = n;
    t.d = d;
    t.data = X;
    t.edge0 = edge0;
    for (int k = 0; k < d; k++) t.origin[k] = origin[k];
    // deepest level a 30-bit cell index holds (the reference's int cell index overflows beyond that)
    t.lmax = std::min(30 / d, 20);
    depth = std::max(1, std::min(depth, t.lmax));
    t.sorted_depth = depth;
    t.keys.release(); t.perm.release(); t.pts.release();   // a second sort (deeper) replaces the first
    const MortonCfg cfg = morton_cfg(d, origin, edge0, math_mode);
    const int shift0 = d * (t.lmax - depth), bits = d * depth;
    switch (d) {
        case 1: sort_passes<1>(t, X, cfg, shift0, bits, s); break;
        case 2: sort_passes<2>(t, X, cfg, shift0, bits, s); break;
        case 3: sort_passes<3>(t, X, cfg, shift0, bits, s); break;
        case 4: sort_passes<4>(t, X, cfg, shift0, bits, s); break;
        default: sort_passes<5>(t, X, cfg, shift0, bits, s); break;
    }
}

}  // namespace f3m
