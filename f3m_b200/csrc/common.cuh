// Internal declarations shared by the translation units of libf3m.so.
#pragma once
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>
#include <atomic>
#include <vector>
#include "f3m.h"

namespace f3m {

constexpr int MAXD = F3M_MAX_DIM;
constexpr int MAXP = 64;   // interpolation nodes per dimension the kernels hold
constexpr int NUM_SMS_HINT = 148;

// ---- error handling: every CUDA call is checked, the message is kept per thread --------------
void set_error(const char *fmt, ...);
struct Fail {
    int code;
};
#define F3M_CUDA(call)                                                                           \
    do {                                                                                         \
        cudaError_t e__ = (call);                                                                \
        if (e__ != cudaSuccess) {                                                                \
            f3m::set_error("%s failed at %s:%d: %s", #call, __FILE__, __LINE__,                  \
                           cudaGetErrorString(e__));                                             \
            throw f3m::Fail{F3M_ERR_CUDA};                                                       \
        }                                                                                        \
    } while (0)
extern std::atomic<long long> g_launches;   // kernels launched by this library (all threads; informational)
#define F3M_LAUNCH_CHECK()                                                                       \
    do {                                                                                         \
        f3m::g_launches.fetch_add(1, std::memory_order_relaxed);                                                                   \
        F3M_CUDA(cudaGetLastError());                                                            \
    } while (0)
#define F3M_REQUIRE(cond, code, ...)                                                             \
    do {                                                                                         \
        if (!(cond)) {                                                                           \
            f3m::set_error(__VA_ARGS__);                                                         \
            throw f3m::Fail{code};                                                               \
        }                                                                                        \
    } while (0)

// ---- device buffers --------------------------------------------------------------------------
// Device memory comes from a small caching allocator inside the library (api.cu): blocks are obtained
// with cudaMalloc once, kept on a free list when released and handed out again to requests of a similar
// size, so that a repeated product makes no driver call at all.  (The driver's stream-ordered pool
// was tried first; with multi-GB buffers freed and re-requested every call it re-mapped memory at
// unpredictable times, 200 ms at a time.)  A released block may be reused immediately by work that is
// enqueued later on the same stream; every entry point synchronises its stream before it returns, so
// blocks never cross streams while in use.  f3m_release_cached_memory() returns the free list to the driver.
void *dev_alloc(size_t bytes, size_t *granted);
void dev_free(void *p, size_t granted);

template <typename T>
struct DevBuf {
    T *p = nullptr;
    size_t n = 0;
    size_t granted = 0;
    cudaStream_t s = nullptr;
    DevBuf() = default;
    DevBuf(const DevBuf &) = delete;
    DevBuf &operator=(const DevBuf &) = delete;
    DevBuf(DevBuf &&o) noexcept : p(o.p), n(o.n), granted(o.granted), s(o.s) { o.p = nullptr; o.n = 0; }
    DevBuf &operator=(DevBuf &&o) noexcept {
        if (this != &o) {
            release();
            p = o.p; n = o.n; granted = o.granted; s = o.s;
            o.p = nullptr; o.n = 0;
        }
        return *this;
    }
    void alloc(size_t count, cudaStream_t stream) {
        release();
        s = stream;
        n = count;
        if (count == 0) count = 1;
        p = static_cast<T *>(dev_alloc(count * sizeof(T), &granted));
    }
    void zero() { F3M_CUDA(cudaMemsetAsync(p, 0, (n ? n : 1) * sizeof(T), s)); }
    void release() {
        if (p) dev_free(p, granted);
        p = nullptr;
        n = 0;
    }
    ~DevBuf() { release(); }
};

// ---- block-wide exclusive scan (all threads of the block call it; blockDim.x a multiple of 32, at most 1024) ----
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

// largest b with off[b] <= i: the box of sorted row i (off = box offsets of a level, nb boxes)
__device__ __forceinline__ int box_of_row(const int *__restrict__ off, int nb, int i) {
    int lo = 0, hi = nb;
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (off[mid] <= i) lo = mid; else hi = mid;
    }
    return lo;
}

// chebyshev_nodes_1D / get_w_j_first_kind (F3M_src/n_tree.cu:265-285): first-kind Chebyshev nodes and barycentric
// weights with the reference's float32 expression (PI as a float, arguments rounded to float before cos / sin).
inline void cheb_nodes_weights(int p, float *node, float *w) {
    const float PI = (float)(atan(1.) * 4.);
    for (int i = 0; i < p; i++) {
        const float arg = ((float)i * 2.f + 1.f) * PI / (float)(2 * (p - 1) + 2);
        node[i] = (float)cos((double)arg);
        w[i] = (float)(pow(-1.0, i) * sin(((2. * (float)i + 1.) * PI) / (2. * (float)(p - 1.0) + 2.)));
    }
}

// ---- small per-plan device words (f3m_plan::d_flags) and their pinned host mirror ------------------
constexpr int FLAG_WORDS = 256;
enum FlagSlot {
    FL_ERR = 0,          // device-side consistency check failed
    FL_LISTTOT = 8,      // 6 words: 64-bit far / small / keep pair counts of the level being built
    FL_BBOX = 16,        // 2 * MAXD words
    FL_MMA_COUNTER = 32, // tile cursor of the tensor-core near kernel
    FL_LEAF = 40,        // 2 words: small / big finest-level boxes
    FL_NSMALL = 42,      // target tiles of at most 32 points
    FL_LVTOT = 64,       // boxes per level of the batch being built (F3M_MAX_LEVELS words)
    FL_LVMAX = 96,       // largest box per level (F3M_MAX_LEVELS words)
    FL_PAIRWORK = 128    // 2 words per level: 64-bit sum of n_x * n_y over the level's direct lists
};

// ---- tree ------------------------------------------------------------------------------------
struct Level {
    int nb = 0;             // occupied boxes
    float edge = 0.f;       // box edge at this level
    int max_count = 0;
    DevBuf<int> off;        // (nb+1) offsets into the sorted point order
    DevBuf<uint32_t> code;  // (nb) Morton prefix
    DevBuf<int> parent;     // (nb) compact id of the parent box one level up
    DevBuf<int> child_start;// (nb+1) first child (compact id one level down); filled when that level exists
    DevBuf<float> ctr;      // (nb,d) centres
};

struct Tree {
    int64_t n = 0;
    int d = 0;
    const float *data = nullptr;   // caller's rows
    float origin[MAXD] = {0};      // per-dimension minimum
    float edge0 = 0.f;             // cube edge
    int lmax = 0;                  // depth of the Morton key
    int sorted_depth = 0;          // the keys are sorted by their first sorted_depth levels (d bits each)
    DevBuf<uint32_t> keys;         // (n) Morton keys at depth lmax, sorted by their first sorted_depth levels
    DevBuf<int> perm;              // (n) sorted position -> input row
    DevBuf<float> pts;             // (d,n) sorted coordinates, one plane per dimension
    std::vector<Level> levels;     // levels[0] is the root
    // A tree whose points arrive as sorted runs (one per rank): the levels are built from one pseudo key per occupied
    // finest sorted cell (pkeys) and offsets into the merged order (fine_off) before the points are attached.
    struct Runs {
        bool pending = false;      // levels may be built, points not merged in yet
        int nruns = 0, ncells = 0, nocc = 0;
        DevBuf<int> counts;        // (nruns, ncells) points per cell and run
        DevBuf<int> seg_start;     // (nruns, ncells + 1) position of the cell inside its run
        DevBuf<int> cell_off;      // (ncells + 1) merged offset of the cell
        DevBuf<uint32_t> pkeys;    // (nocc) pseudo key of every occupied cell
        DevBuf<int> fine_off;      // (nocc + 1) merged offset of every occupied cell
    } runs;
};

struct PairCSR {
    DevBuf<int> ptr;  // (boxes_x+1)
    DevBuf<int> idx;  // source box per pair
    int64_t count = 0;
};

struct LevelLists {
    PairCSR far, small, keep;
    int p = 0;        // nodes per dimension used for the far field of this level
    // far rows re-ordered by box offset (last axis most significant) with the packed offsets, built on first use
    DevBuf<uint32_t> far_okey;
    DevBuf<int> far_oidx;
    bool far_ordered = false;
};

// Device time per stage, from CUDA events recorded on the product's stream and read after its
// final synchronisation (no extra synchronisation inside the product).
enum Stage { ST_PERMUTE = 0, ST_DIRECT = 1, ST_P2M = 2, ST_M2L = 3, ST_L2P = 4, ST_UNPERMUTE = 5, ST_TOTAL = 6, ST_BUILD = 7 };
// forms of the direct-sum kernels (counted per launch, see f3m_plan_last_direct_variants)
enum DirectVariant { DV_MUFU = 0, DV_POLY2 = 1, DV_POLY3 = 2, DV_DIRECT = 3, DV_MOMENTS = 4, DV_TENSOR = 5, DV_COUNT = 6 };
struct Timings {
    float ms[8] = {0};
    int direct_launches = 0;
    int direct_variants[DV_COUNT] = {0};
    struct Span { int stage; cudaEvent_t a, b; bool closed; };
    std::vector<Span> spans;
    void begin(int stage, cudaStream_t s) {
        Span sp{stage, nullptr, nullptr, false};
        F3M_CUDA(cudaEventCreate(&sp.a));
        F3M_CUDA(cudaEventCreate(&sp.b));
        F3M_CUDA(cudaEventRecord(sp.a, s));
        spans.push_back(sp);
    }
    void end(cudaStream_t s) {
        F3M_CUDA(cudaEventRecord(spans.back().b, s));
        spans.back().closed = true;
    }
    // Call after the stream has been synchronised.  A span that was never closed (the product failed in between)
    // is dropped; a failed query must not stay behind as the runtime's last error, or the next launch check of an
    // unrelated call would report it.
    void resolve() {
        for (auto &sp : spans) {
            float t = 0.f;
            if (sp.closed) {
                if (cudaEventElapsedTime(&t, sp.a, sp.b) == cudaSuccess) ms[sp.stage] += t;
                else (void)cudaGetLastError();
            }
            cudaEventDestroy(sp.a);
            cudaEventDestroy(sp.b);
        }
        spans.clear();
    }
};

}  // namespace f3m

struct f3m_plan {
    int device = 0;
    int d = 0;
    bool same = false;
    f3m_params prm{};
    float lcs = 0.f;
    f3m::Tree tx, ty_store;
    f3m::Tree *ty = nullptr;
    std::vector<f3m::LevelLists> lists;   // lists[l] for level l (index 0 unused)
    int levels = 0;
    f3m_plan_stats stats{};
    f3m::Timings last;
    // sharded moments (multi-GPU): either write the finest-level moments of a slice of the source boxes
    // into moments_out and stop, or take the complete finest-level moments from ext_mom instead of computing them
    // finest-level boxes split by size for P2M / L2P (index 0: target tree, 1: source tree): boxes of at most
    // LEAF_SMALL points are handled one per warp, the others one per CTA; built on first use
    f3m::DevBuf<int> leaf_small[2], leaf_big[2];
    int n_leaf_small[2] = {0, 0}, n_leaf_big[2] = {0, 0};
    bool leaf_split[2] = {false, false};
    float *moments_out = nullptr;
    int64_t mom_begin = 0, mom_end = 0;
    int64_t mom_box_begin = -1, mom_box_end = -1;   // >= 0: moments_out covers these source boxes only
    const float *ext_mom = nullptr;
    // source boxes named by the direct lists of a level over ALL targets (a constant of the plan, built on first use)
    std::vector<f3m::DevBuf<unsigned char>> src_need;
    // packed sources of the last direct list (valid inside one product)
    struct PackCache {
        int level = -1, r0 = 0, rb = 0;
        bool expanded = false;
        f3m::DevBuf<float> buf;
        void reset() { level = -1; buf.release(); }
    } pack_cache;
    // a product shared by several GPUs, in phases (f3m_plan_shard_begin / _near / _far): state kept between the calls
    struct Shard {
        bool active = false;
        bool all_sources = false;                          // no halo bookkeeping: bs holds every row
        int R = 0;
        int64_t row_begin = 0, row_end = 0;
        f3m::DevBuf<float> bs;                             // b in sorted order, filled for the boxes this rank reads
        std::vector<f3m::DevBuf<unsigned char>> need;      // per level: source boxes named by the rank's direct lists
    } shard;
    int *h_pinned = nullptr;              // pinned host words for count read-back (FLAG_WORDS ints)
    int *d_flags = nullptr;               // device status / counters (FLAG_WORDS ints, see FlagSlot)
    ~f3m_plan();
};

namespace f3m {

// ---- sort.cu ---------------------------------------------------------------------------------
void bounding_box(const float *X, int64_t n, int d, float *h_min, float *h_max, f3m_plan *pl, cudaStream_t s);
void build_sorted_tree(Tree &t, const float *X, int64_t n, int d, const float *origin, float edge0,
                       int math_mode, int depth, cudaStream_t s);
int record_words(int d);   // 32-bit words of the record [input row, coordinates] that travels with a key in the sort
void sort_shard(const float *X, int64_t n, int64_t row0, int d, const float *origin, float edge0, int math_mode, int depth,
                uint32_t *recs_out, int *cell_counts_out, cudaStream_t s);
void tree_from_cell_counts(Tree &t, const int *counts, int nruns, int d, const float *origin, float edge0, int depth, f3m_plan *pl,
                           cudaStream_t s);
void tree_attach_runs(Tree &t, const uint32_t *recs, int64_t stride, cudaStream_t s);
void exclusive_scan_i32(const int *in, int *out, int64_t n, cudaStream_t s);  // n values; out may alias in
// up to four arrays of n values scanned in place by one set of launches; their sums as 64-bit numbers -> totals64 (device)
void exclusive_scan_multi(int *const *arrays, int narr, int64_t n, long long *totals64, cudaStream_t s);
void gather_rows(const float *src, const int *perm, float *dst, int64_t n, int cols, cudaStream_t s);
void scatter_rows(const float *src, const int *perm, float *dst, int64_t n, int cols, cudaStream_t s);
void scatter_rows_nonzero(const float *src, const int *perm, float *dst, int64_t n, int cols, cudaStream_t s);

// ---- tree.cu ---------------------------------------------------------------------------------
void build_root(Tree &t, cudaStream_t s);
void build_levels(Tree &t, int l_last, f3m_plan *pl, cudaStream_t s);   // appends levels up to l_last (<= sorted_depth)
void build_level_lists(f3m_plan *pl, int level, cudaStream_t s);     // uses lists[level-1].keep
void accumulate_pair_work(f3m_plan *pl, int level, const PairCSR &csr, cudaStream_t s);   // adds into FL_PAIRWORK (device)

// ---- far.cu ----------------------------------------------------------------------------------
int nodes_per_dim(int d, int nr_interpolation);   // get_node_list for perfect powers, floor otherwise
void far_field_level(f3m_plan *pl, int level, const float *b_sorted, int R, float *out_sorted,
                     int64_t row_begin, int64_t row_end, cudaStream_t s);   // per-level path (far.cu)
void far_field(f3m_plan *pl, const float *b_sorted, int R, float *out_sorted, int64_t row_begin, int64_t row_end,
               cudaStream_t s);                                               // whole product (far_fast.cu)
int64_t far_moments_size(const f3m_plan *pl, int R);

// ---- shard.cu --------------------------------------------------------------------------------
const unsigned char *level_source_flags(f3m_plan *pl, int level, cudaStream_t s);   // per source box of the level: named by a direct list?
void shard_partition(f3m_plan *pl, int R, int nparts, int64_t *h_bounds, cudaStream_t s);
void shard_mark_and_gather(f3m_plan *pl, const float *b, int R, int row_begin, int row_end, int box_begin, int box_end,
                           bool everything, cudaStream_t s);
void shard_count_rows_by_owner(const f3m_plan *pl, int64_t row_begin, int64_t row_end, const int64_t *h_bounds, int nranks,
                               int64_t *h_counts, cudaStream_t s);
void shard_pack_rows_by_owner(const f3m_plan *pl, const float *acc_sorted, int R, int64_t row_begin, int64_t row_end,
                              const int64_t *h_bounds, int nranks, const int64_t *h_counts, float *send, cudaStream_t s);
void shard_gathered_rows_to_input_order(const f3m_plan *pl, const float *gathered, int R, const int64_t *h_slice_bounds, int nslices,
                                        int64_t stride, int64_t in_lo, int64_t in_hi, float *out, cudaStream_t s);
void shard_place_rows(const float *recs, int64_t n, int R, int64_t in_lo, int64_t in_hi, float *out, int *d_err, cudaStream_t s);
void shard_rows_to_input_order(const f3m_plan *pl, const float *acc_sorted, int R, int64_t in_lo, int64_t in_hi, float *out,
                               cudaStream_t s);

// ---- near.cu ---------------------------------------------------------------------------------
void direct_sums(f3m_plan *pl, int level, const PairCSR &csr, const float *b_sorted, int R, float *out_sorted,
                 int64_t row_begin, int64_t row_end, cudaStream_t s);
template <bool GRAD>
void dense_f32(const float *X, int64_t N, const float *Y, int64_t M, const float *b, int R, int d, float ls, float *out,
               cudaStream_t s);
void dense_f64(const double *X, int64_t N, const double *Y, int64_t M, const double *b, int R, int d, double ls, double *out,
               cudaStream_t s);
void measure_peaks(double *gexp, double *gfma, cudaStream_t s);
void dense_f32_static(const float *X, int64_t N, const float *Y, int64_t M, const float *b, int R, int d, float ls, float *out,
                      cudaStream_t s);

}  // namespace f3m
