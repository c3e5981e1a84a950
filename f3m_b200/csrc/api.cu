// extern "C" entry points of libf3m.so and the level loop of the treecode.
//
// The loop below is the control flow of FFM_XY<float,d> (F3M_src/n_tree.cu:1056-1125) and
// far_field_run (n_tree.cu:982-1053), split into a part that does not depend on b (plan) and a part
// that does (apply).
#include <stdarg.h>
#include <math.h>
#include <algorithm>
#include <mutex>
#include <utility>
#include <vector>
#include "common.cuh"

namespace f3m {

std::atomic<long long> g_launches{0};
static thread_local char g_err[512] = "";

void set_error(const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}

// ---- caching device allocator ------------------------------------------------------------------
namespace {
struct FreeBlock { void *p; size_t bytes; int device; };
std::mutex g_mem_mu;
std::vector<FreeBlock> g_free_blocks;

size_t round_request(size_t bytes) {
    if (bytes < 512) bytes = 512;
    const size_t q = bytes >= (1u << 20) ? (1u << 20) : 512;   // 1 MiB granularity for large blocks
    return (bytes + q - 1) / q * q;
}
}  // namespace

// ---- caller-owned workspace ---------------------------------------------------------------------
// While a thread runs an entry point that was given a workspace, every device buffer of the library comes out of
// that memory: a first-fit list of free ranges, 256-byte granularity, neighbours merged on release.  Nothing is
// taken from or returned to the driver.
namespace {
struct Arena {
    char *base = nullptr;
    size_t size = 0, used = 0, peak = 0;
    std::vector<std::pair<size_t, size_t>> free_ranges;   // (offset, length), sorted by offset
    void reset(void *p, size_t n) {
        base = static_cast<char *>(p);
        const size_t mis = (256 - (reinterpret_cast<uintptr_t>(p) & 255)) & 255;   // first 256-byte boundary inside
        size = n > mis ? n - mis : 0;
        base += mis;
        used = peak = 0;
        free_ranges.assign(1, {0, size / 256 * 256});
    }
    void *take(size_t bytes, size_t *granted) {
        const size_t need = (bytes + 255) / 256 * 256;
        for (size_t i = 0; i < free_ranges.size(); i++) {
            if (free_ranges[i].second < need) continue;
            const size_t off = free_ranges[i].first;
            if (free_ranges[i].second == need) free_ranges.erase(free_ranges.begin() + i);
            else { free_ranges[i].first += need; free_ranges[i].second -= need; }
            used += need;
            peak = std::max(peak, used);
            *granted = need;
            return base + off;
        }
        return nullptr;
    }
    bool owns(const void *p) const { return p >= base && p < base + size; }
    void give(void *p, size_t len) {
        const size_t off = static_cast<char *>(p) - base;
        used -= len;
        size_t i = 0;
        while (i < free_ranges.size() && free_ranges[i].first < off) i++;
        free_ranges.insert(free_ranges.begin() + i, {off, len});
        if (i + 1 < free_ranges.size() && free_ranges[i].first + free_ranges[i].second == free_ranges[i + 1].first) {
            free_ranges[i].second += free_ranges[i + 1].second;
            free_ranges.erase(free_ranges.begin() + i + 1);
        }
        if (i > 0 && free_ranges[i - 1].first + free_ranges[i - 1].second == free_ranges[i].first) {
            free_ranges[i - 1].second += free_ranges[i].second;
            free_ranges.erase(free_ranges.begin() + i);
        }
    }
};
thread_local Arena *g_arena = nullptr;
thread_local size_t g_last_ws_peak = 0;
}  // namespace

void *dev_alloc(size_t bytes, size_t *granted) {
    if (g_arena) {
        void *p = g_arena->take(bytes ? bytes : 1, granted);
        if (!p) {
            set_error("the workspace of %zu bytes is too small: %zu bytes are in use and %zu more were requested "
                      "(f3m_workspace_bytes gives an estimate; clustered point sets need more)", g_arena->size, g_arena->used, bytes);
            throw Fail{F3M_ERR_TOO_LARGE};
        }
        return p;
    }
    const size_t need = round_request(bytes);
    int dev = 0;
    F3M_CUDA(cudaGetDevice(&dev));
    {
        std::lock_guard<std::mutex> lk(g_mem_mu);
        int best = -1;
        for (size_t i = 0; i < g_free_blocks.size(); i++) {
            const FreeBlock &b = g_free_blocks[i];
            if (b.device != dev || b.bytes < need || b.bytes > need + need / 4 + (1u << 20)) continue;
            if (best < 0 || b.bytes < g_free_blocks[best].bytes) best = (int)i;
        }
        if (best >= 0) {
            FreeBlock b = g_free_blocks[best];
            g_free_blocks.erase(g_free_blocks.begin() + best);
            *granted = b.bytes;
            return b.p;
        }
    }
    void *p = nullptr;
    cudaError_t e = cudaMalloc(&p, need);
    if (e == cudaErrorMemoryAllocation) {   // give the cached blocks back and try once more
        cudaGetLastError();
        {
            std::lock_guard<std::mutex> lk(g_mem_mu);
            for (size_t i = 0; i < g_free_blocks.size();) {
                if (g_free_blocks[i].device == dev) { cudaFree(g_free_blocks[i].p); g_free_blocks.erase(g_free_blocks.begin() + i); }
                else i++;
            }
        }
        e = cudaMalloc(&p, need);
    }
    if (e != cudaSuccess) {
        set_error("cudaMalloc of %zu bytes failed: %s", need, cudaGetErrorString(e));
        throw Fail{F3M_ERR_CUDA};
    }
    *granted = need;
    return p;
}

void dev_free(void *p, size_t granted) {
    if (g_arena && g_arena->owns(p)) { g_arena->give(p, granted); return; }
    int dev = 0;
    cudaGetDevice(&dev);
    cudaPointerAttributes attr;
    if (cudaPointerGetAttributes(&attr, p) == cudaSuccess) dev = attr.device;
    std::lock_guard<std::mutex> lk(g_mem_mu);
    g_free_blocks.push_back(FreeBlock{p, granted, dev});
}

}  // namespace f3m

using namespace f3m;

// Small per-plan scratch (FLAG_WORDS pinned host words for read-backs, as many device words for flags and counters).
// cudaHostAlloc / cudaMalloc / cudaFree serialise the device, so slots are created once and recycled:
// a plan takes a slot of its device from a free list and gives it back when it is destroyed.
namespace {
struct ScratchSlot { int device; int *h_pinned; int *d_flags; };
std::mutex g_slot_mu;
std::vector<ScratchSlot> g_free_slots;

ScratchSlot take_slot(int device) {
    {
        std::lock_guard<std::mutex> lk(g_slot_mu);
        for (size_t i = 0; i < g_free_slots.size(); i++)
            if (g_free_slots[i].device == device) {
                ScratchSlot sl = g_free_slots[i];
                g_free_slots.erase(g_free_slots.begin() + i);
                return sl;
            }
    }
    ScratchSlot sl{device, nullptr, nullptr};
    F3M_CUDA(cudaHostAlloc((void **)&sl.h_pinned, FLAG_WORDS * sizeof(int), cudaHostAllocDefault));
    F3M_CUDA(cudaMalloc((void **)&sl.d_flags, FLAG_WORDS * sizeof(int)));
    return sl;
}
void give_slot(const ScratchSlot &sl) {
    std::lock_guard<std::mutex> lk(g_slot_mu);
    g_free_slots.push_back(sl);
}
}  // namespace

f3m_plan::~f3m_plan() {
    last.resolve();
    if (h_pinned && d_flags) give_slot(ScratchSlot{device, h_pinned, d_flags});
}

template <typename F>
static int guarded(F &&f) {
    try {
        g_err[0] = 0;
        f();
        return F3M_OK;
    } catch (const Fail &e) {
        return e.code;
    } catch (const std::exception &e) {
        set_error("%s", e.what());
        return F3M_ERR_INTERNAL;
    }
}

static void check_common(const void *X, int64_t N, const void *Y, int64_t M, int d, const f3m_params *prm) {
    F3M_REQUIRE(X && Y && prm, F3M_ERR_ARG, "null pointer argument");
    F3M_REQUIRE(N > 0 && M > 0, F3M_ERR_ARG, "empty point set (N=%lld, M=%lld)", (long long)N, (long long)M);
    F3M_REQUIRE(d >= 1 && d <= F3M_MAX_DIM, F3M_ERR_ARG, "dimension %d outside 1..%d", d, F3M_MAX_DIM);
    F3M_REQUIRE(prm->ls > 0.f, F3M_ERR_ARG, "lengthscale must be positive");
    F3M_REQUIRE(prm->nr_interpolation >= 1, F3M_ERR_ARG, "nr_interpolation must be >= 1");
}

static void plan_build_levels(f3m_plan *pl, const float *X, int64_t N, const float *Y, int64_t M, const float *xmin, const float *ymin,
                              float edge0, cudaStream_t s);

// levels the sort covers: the level loop stops at the first level whose largest box holds at most min_points points;
// for evenly spread points that is the level where the mean occupancy falls below min_points (one more when the mean
// is within a factor two of it)
static int estimate_depth(int64_t n, int d, float min_points) {
    const int lmax = std::min(30 / d, 20);
    int L = 1;
    auto mean = [&](int l) { return (double)n / pow(2.0, (double)d * l); };
    while (L < lmax && mean(L) > (double)min_points) L++;
    if (L < lmax && mean(L) > 0.5 * (double)min_points) L++;
    return L;
}

static void plan_begin(f3m_plan *pl, int d, const f3m_params *prm, bool same, cudaStream_t s) {
    F3M_CUDA(cudaGetDevice(&pl->device));
    pl->d = d;
    pl->prm = *prm;
    pl->same = same;
    pl->lcs = 1 / (2 * prm->ls * prm->ls);                // n_tree.cu:1060
    {
        ScratchSlot sl = take_slot(pl->device);
        pl->h_pinned = sl.h_pinned;
        pl->d_flags = sl.d_flags;
    }
    F3M_CUDA(cudaMemsetAsync(pl->d_flags, 0, FLAG_WORDS * sizeof(int), s));
    pl->last.begin(ST_BUILD, s);
}

static void plan_build(f3m_plan *pl, const float *X, int64_t N, const float *Y, int64_t M, int d, const f3m_params *prm,
                       cudaStream_t s) {
    // n_tree.cu:1072 tests the address only; a leading slice of X starts at the same address but is another
    // (smaller) point set, so the sizes must agree too
    plan_begin(pl, d, prm, X == Y && N == M, s);

    // bounding cube: calculate_edge_X / calculate_edge (n_tree.cu:25-46), float32 throughout
    float xmin[MAXD], xmax[MAXD], ymin[MAXD], ymax[MAXD];
    bounding_box(X, N, d, xmin, xmax, pl, s);
    float range = 0.f;
    bool finite = true;   // std::max drops a NaN operand, so non-finite extents are checked one by one
    for (int k = 0; k < d; k++) {
        finite = finite && std::isfinite(xmin[k]) && std::isfinite(xmax[k]);
        range = std::max(range, xmax[k] - xmin[k]);
    }
    if (!pl->same) {
        bounding_box(Y, M, d, ymin, ymax, pl, s);
        float ry = 0.f;
        for (int k = 0; k < d; k++) {
            finite = finite && std::isfinite(ymin[k]) && std::isfinite(ymax[k]);
            ry = std::max(ry, ymax[k] - ymin[k]);
        }
        range = std::max(range, ry);
    }
    F3M_REQUIRE(finite, F3M_ERR_ARG, "degenerate or non-finite bounding cube (a coordinate is NaN or infinite)");
    float edge0 = range * 1.01f;
    F3M_REQUIRE(edge0 > 0.f && std::isfinite(edge0), F3M_ERR_ARG, "degenerate or non-finite bounding cube (edge %g)", edge0);

    // Only the key bits of the levels the loop below will visit are sorted.  If the loop does go deeper than estimated
    // (clustered points), the trees are sorted again to the full key depth.
    int depth = estimate_depth(N, d, prm->min_points);
    if (!pl->same) depth = std::min(depth, estimate_depth(M, d, prm->min_points));
    build_sorted_tree(pl->tx, X, N, d, xmin, edge0, prm->math_mode, depth, s);
    build_root(pl->tx, s);
    if (pl->same) pl->ty = &pl->tx;
    else {
        build_sorted_tree(pl->ty_store, Y, M, d, ymin, edge0, prm->math_mode, depth, s);
        build_root(pl->ty_store, s);
        pl->ty = &pl->ty_store;
    }
    plan_build_levels(pl, X, N, Y, M, xmin, ymin, edge0, s);
}

// second half of the plan: levels, interaction lists, work accounting (the trees hold sorted points)
static void plan_build_levels(f3m_plan *pl, const float *X, int64_t N, const float *Y, int64_t M, const float *xmin, const float *ymin,
                              float edge0, cudaStream_t s) {
    const f3m_params *prm = &pl->prm;
    const int d = pl->d;
    Tree &tx = pl->tx, &ty = *pl->ty;

    // root pair list (n_tree.cu:1071)
    pl->lists.clear();
    pl->lists.emplace_back();
    {
        PairCSR &k = pl->lists[0].keep;
        k.ptr.alloc(2, s); k.idx.alloc(1, s);
        int h[2] = {0, 1};
        F3M_CUDA(cudaMemcpyAsync(k.ptr.p, h, sizeof(h), cudaMemcpyHostToDevice, s));
        F3M_CUDA(cudaMemsetAsync(k.idx.p, 0, 4, s));
        F3M_CUDA(cudaStreamSynchronize(s));
        k.count = 1;
    }
    pl->stats = f3m_plan_stats{};
    int level = 0;
    auto go_on = [&]() {
        if (pl->lists[level].keep.count == 0) return false;
        bool gx = (float)tx.levels[level].max_count > prm->min_points;     // n_tree.cu:1075
        if (pl->same) return gx;
        return gx && (float)ty.levels[level].max_count > prm->min_points;  // n_tree.cu:1099
    };
    const int p_full = nodes_per_dim(d, prm->nr_interpolation);
    int p_small = nodes_per_dim(d, std::min((int)lround(pow(3.0, d)), prm->nr_interpolation));
    while (go_on()) {
        const int need = level + 1;
        F3M_REQUIRE(need <= tx.lmax, F3M_ERR_DEPTH,
                    "tree needs level %d but a 30-bit cell index holds %d levels in %d dimensions", need, tx.lmax, d);
        if (need > tx.sorted_depth) {
            F3M_REQUIRE(X != nullptr, F3M_ERR_UNSUPPORTED,
                        "the tree needs level %d but the runs it was merged from are sorted to level %d: build the plan from the points",
                        need, tx.sorted_depth);
            // deeper than estimated: sort to the full key depth (levels already built keep their boxes)
            build_sorted_tree(tx, X, N, d, xmin, edge0, prm->math_mode, tx.lmax, s);
            if (!pl->same) build_sorted_tree(ty, Y, M, d, ymin, edge0, prm->math_mode, ty.lmax, s);
        }
        if ((int)tx.levels.size() <= need) {
            // a first batch up to the estimated depth, later batches three levels at a time
            const int last = tx.sorted_depth < tx.lmax ? tx.sorted_depth : std::min(tx.sorted_depth, need + 2);
            build_levels(tx, last, pl, s);
            if (!pl->same) build_levels(ty, last, pl, s);
        }
        level++;
        pl->lists.emplace_back();
        build_level_lists(pl, level, s);
        LevelLists &ll = pl->lists[level];
        // nodes for this level: get_interpolation_rule (n_tree.cu:971-978, 1022-1028)
        ll.p = p_full;
        if (prm->var_compression) {
            float e = tx.levels[level].edge;
            float eff = e * e * pl->lcs;
            if (eff < 0.01f) ll.p = p_small;
        }
        int P = 1;
        for (int k = 0; k < d; k++) P *= ll.p;
        pl->stats.far_box_pairs += ll.far.count;
        pl->stats.node_pairs += ll.far.count * (int64_t)P * P;
        pl->stats.near_box_pairs += ll.small.count;
        accumulate_pair_work(pl, level, ll.small, s);
    }
    pl->levels = level;
    if (level > 0) {
        pl->stats.near_box_pairs += pl->lists[level].keep.count;
        accumulate_pair_work(pl, level, pl->lists[level].keep, s);
    } else {
        // no level was built: the root pair is summed directly
        pl->stats.near_box_pairs = 1;
        pl->stats.direct_pairs = N * M;
    }
    pl->stats.levels = level;
    pl->stats.shared_tree = pl->same;
    pl->stats.edge0 = edge0;
    pl->last.end(s);
    F3M_CUDA(cudaMemcpyAsync(pl->h_pinned + FL_PAIRWORK, pl->d_flags + FL_PAIRWORK, sizeof(long long), cudaMemcpyDeviceToHost, s));
    F3M_CUDA(cudaStreamSynchronize(s));
    if (level > 0) pl->stats.direct_pairs = *reinterpret_cast<long long *>(pl->h_pinned + FL_PAIRWORK);
    pl->last.ms[ST_BUILD] = 0.f;
    pl->last.resolve();
    pl->stats.build_ms = pl->last.ms[ST_BUILD];
}

static void plan_apply(f3m_plan *pl, const float *b, int R, float *out, int64_t row_begin, int64_t row_end,
                       cudaStream_t s) {
    F3M_REQUIRE(b && out && R >= 1, F3M_ERR_ARG, "bad right-hand side (R=%d)", R);
    F3M_REQUIRE(!pl->tx.runs.pending, F3M_ERR_ARG, "the plan still waits for its sorted runs (f3m_plan_attach_runs)");
    int dev;
    F3M_CUDA(cudaGetDevice(&dev));
    F3M_REQUIRE(dev == pl->device, F3M_ERR_ARG, "plan was built on device %d, current device is %d", pl->device, dev);
    Tree &tx = pl->tx, &ty = *pl->ty;
    const int64_t N = tx.n, M = ty.n;
    row_begin = std::max<int64_t>(0, row_begin);
    row_end = std::min<int64_t>(N, row_end);
    for (float &m : pl->last.ms) m = 0.f;
    pl->last.ms[ST_BUILD] = pl->stats.build_ms;
    pl->last.direct_launches = 0;
    for (int &v : pl->last.direct_variants) v = 0;
    pl->last.begin(ST_TOTAL, s);
    pl->pack_cache.reset();
    struct DropPacked { f3m_plan *p; ~DropPacked() { p->pack_cache.reset(); } } drop_packed{pl};

    pl->last.begin(ST_PERMUTE, s);
    DevBuf<float> bs, outs;
    bs.alloc((size_t)M * R, s);
    gather_rows(b, ty.perm.p, bs.p, M, R, s);
    outs.alloc((size_t)N * R, s);
    outs.zero();
    pl->last.end(s);

    const int L = pl->levels;
    if (L == 0) {
        // largest box already small enough: one direct product over the root pair
        direct_sums(pl, 0, pl->lists[0].keep, bs.p, R, outs.p, row_begin, row_end, s);
    }
    for (int level = 1; level <= L; level++) {
        LevelLists &ll = pl->lists[level];
        direct_sums(pl, level, ll.small, bs.p, R, outs.p, row_begin, row_end, s);   // n_tree.cu:1018-1020
    }
    far_field(pl, bs.p, R, outs.p, row_begin, row_end, s);                          // n_tree.cu:1021-1051, all levels
    if (L > 0) direct_sums(pl, L, pl->lists[L].keep, bs.p, R, outs.p, row_begin, row_end, s);   // n_tree.cu:1092-1094

    pl->last.begin(ST_UNPERMUTE, s);
    if (row_begin <= 0 && row_end >= N) scatter_rows(outs.p, tx.perm.p, out, N, R, s);
    else scatter_rows_nonzero(outs.p, tx.perm.p, out, N, R, s);   // a slice: most rows are zero
    pl->last.end(s);
    F3M_CUDA(cudaEventRecord(pl->last.spans[0].b, s));   // closes the ST_TOTAL span opened first
    pl->last.spans[0].closed = true;
    F3M_CUDA(cudaMemcpyAsync(pl->h_pinned, pl->d_flags, sizeof(int), cudaMemcpyDeviceToHost, s));
    F3M_CUDA(cudaStreamSynchronize(s));
    pl->last.resolve();
    F3M_REQUIRE(pl->h_pinned[0] == 0, F3M_ERR_INTERNAL, "device-side consistency check failed (code %d)", pl->h_pinned[0]);
}

extern "C" {

int f3m_version(void) { return 100; }

const char *f3m_status_string(int st) {
    switch (st) {
        case F3M_OK: return "ok";
        case F3M_ERR_ARG: return "invalid argument";
        case F3M_ERR_CUDA: return "CUDA error";
        case F3M_ERR_DEPTH: return "tree deeper than a 30-bit cell index";
        case F3M_ERR_OVERFLOW: return "list or offset exceeds 31 bits";
        case F3M_ERR_UNSUPPORTED: return "unsupported configuration";
        case F3M_ERR_INTERNAL: return "internal consistency check failed";
        case F3M_ERR_TOO_LARGE: return "problem exceeds the fixed capacity of this entry point";
        default: return "unknown status";
    }
}

const char *f3m_last_error(void) { return g_err; }
long long f3m_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

int f3m_plan_create(f3m_plan **plan, const float *X, int64_t N, const float *Y, int64_t M, int32_t d,
                    const f3m_params *prm, void *stream) {
    if (!plan) return F3M_ERR_ARG;
    *plan = nullptr;
    f3m_plan *pl = nullptr;
    int st = guarded([&] {
        check_common(X, N, Y, M, d, prm);
        pl = new f3m_plan();
        plan_build(pl, X, N, Y, M, d, prm, (cudaStream_t)stream);
    });
    if (st != F3M_OK) {
        if (pl) { cudaStreamSynchronize((cudaStream_t)stream); delete pl; }
        return st;
    }
    *plan = pl;
    return F3M_OK;
}

int f3m_plan_apply_range(f3m_plan *plan, const float *b, int32_t R, float *out, int64_t row_begin, int64_t row_end,
                         void *stream) {
    if (!plan) return F3M_ERR_ARG;
    int st = guarded([&] { plan_apply(plan, b, R, out, row_begin, row_end, (cudaStream_t)stream); });
    if (st != F3M_OK) { cudaStreamSynchronize((cudaStream_t)stream); plan->last.resolve(); }
    return st;
}

int f3m_plan_moments_size(const f3m_plan *plan, int32_t R, int64_t *nfloats) {
    if (!plan || !nfloats || R < 1) return F3M_ERR_ARG;
    *nfloats = far_moments_size(plan, R);
    return F3M_OK;
}

int f3m_plan_moments_range(f3m_plan *plan, const float *b, int32_t R, int64_t src_begin, int64_t src_end, float *mom_out,
                           void *stream) {
    if (!plan || !b || !mom_out) return F3M_ERR_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    int st = guarded([&] {
        F3M_REQUIRE(R >= 1, F3M_ERR_ARG, "bad right-hand side (R=%d)", R);
        int dev;
        F3M_CUDA(cudaGetDevice(&dev));
        F3M_REQUIRE(dev == plan->device, F3M_ERR_ARG, "plan was built on device %d, current device is %d", plan->device, dev);
        F3M_REQUIRE(far_moments_size(plan, R) > 0, F3M_ERR_UNSUPPORTED, "this plan does not exchange moments (see f3m_plan_moments_size)");
        Tree &ty = *plan->ty;
        DevBuf<float> bs;
        bs.alloc((size_t)ty.n * R, s);
        gather_rows(b, ty.perm.p, bs.p, ty.n, R, s);
        plan->moments_out = mom_out;
        plan->mom_begin = src_begin;
        plan->mom_end = src_end;
        far_field(plan, bs.p, R, nullptr, 0, 0, s);
        F3M_CUDA(cudaStreamSynchronize(s));
    });
    plan->moments_out = nullptr;
    if (st != F3M_OK) cudaStreamSynchronize(s);
    plan->last.resolve();
    return st;
}

int f3m_plan_apply_range_moments(f3m_plan *plan, const float *b, int32_t R, float *out, int64_t row_begin, int64_t row_end,
                                 const float *mom, void *stream) {
    if (!plan || !mom) return F3M_ERR_ARG;
    if (far_moments_size(plan, R) <= 0) return F3M_ERR_UNSUPPORTED;
    plan->ext_mom = mom;
    int st = f3m_plan_apply_range(plan, b, R, out, row_begin, row_end, stream);
    plan->ext_mom = nullptr;
    return st;
}

/* ---- a plan from runs sorted on several GPUs ----------------------------------------------------------------- */

int f3m_sort_depth(int64_t n, int32_t d, float min_points) {
    if (n < 1 || d < 1 || d > F3M_MAX_DIM) return 0;
    return estimate_depth(n, d, min_points);
}

int f3m_record_words(int32_t d) { return (d < 1 || d > F3M_MAX_DIM) ? 0 : record_words(d); }

int f3m_bounding_box_f32(const float *X, int64_t n, int32_t d, float *min_out, float *max_out, void *stream) {
    if (!X || !min_out || !max_out || n < 1 || d < 1 || d > F3M_MAX_DIM) return F3M_ERR_ARG;
    return guarded([&] {
        f3m_plan tmp;   // only its scratch words are used
        F3M_CUDA(cudaGetDevice(&tmp.device));
        ScratchSlot sl = take_slot(tmp.device);
        tmp.h_pinned = sl.h_pinned;
        tmp.d_flags = sl.d_flags;
        bounding_box(X, n, d, min_out, max_out, &tmp, (cudaStream_t)stream);
    });
}

int f3m_sort_shard_f32(const float *X, int64_t n, int64_t row_offset, int32_t d, const float *origin, float edge0, int32_t math_mode,
                       int32_t depth, void *records_out, int32_t *cell_counts_out, void *stream) {
    if (!X || !origin || !records_out || !cell_counts_out || n < 1 || row_offset < 0 || d < 1 || d > F3M_MAX_DIM) return F3M_ERR_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    return guarded([&] {
        F3M_REQUIRE(edge0 > 0.f && std::isfinite(edge0), F3M_ERR_ARG, "degenerate or non-finite bounding cube (edge %g)", edge0);
        sort_shard(X, n, row_offset, d, origin, edge0, math_mode, depth, static_cast<uint32_t *>(records_out), cell_counts_out, s);
        F3M_CUDA(cudaStreamSynchronize(s));
    });
}

int f3m_plan_create_from_cell_counts(f3m_plan **plan, const int32_t *cell_counts, int32_t nruns, int32_t d, const float *origin,
                                     float edge0, int32_t depth, const f3m_params *prm, void *stream) {
    if (!plan) return F3M_ERR_ARG;
    *plan = nullptr;
    f3m_plan *pl = nullptr;
    cudaStream_t s = (cudaStream_t)stream;
    int st = guarded([&] {
        F3M_REQUIRE(cell_counts && origin && prm && nruns >= 1, F3M_ERR_ARG, "null pointer argument");
        F3M_REQUIRE(d >= 1 && d <= F3M_MAX_DIM, F3M_ERR_ARG, "dimension %d outside 1..%d", d, F3M_MAX_DIM);
        F3M_REQUIRE(prm->ls > 0.f && prm->nr_interpolation >= 1, F3M_ERR_ARG, "bad parameters");
        F3M_REQUIRE(edge0 > 0.f && std::isfinite(edge0), F3M_ERR_ARG, "degenerate or non-finite bounding cube (edge %g)", edge0);
        pl = new f3m_plan();
        plan_begin(pl, d, prm, true, s);
        tree_from_cell_counts(pl->tx, cell_counts, nruns, d, origin, edge0, depth, pl, s);
        build_root(pl->tx, s);
        pl->ty = &pl->tx;
        plan_build_levels(pl, nullptr, pl->tx.n, nullptr, pl->tx.n, origin, origin, edge0, s);
    });
    if (st != F3M_OK) {
        if (pl) { cudaStreamSynchronize(s); delete pl; }
        return st;
    }
    *plan = pl;
    return F3M_OK;
}

int f3m_plan_attach_runs(f3m_plan *plan, const void *records, int64_t run_stride, void *stream) {
    if (!plan || !records || run_stride < 1) return F3M_ERR_ARG;
    return guarded([&] {
        int dev;
        F3M_CUDA(cudaGetDevice(&dev));
        F3M_REQUIRE(dev == plan->device, F3M_ERR_ARG, "plan was built on device %d, current device is %d", plan->device, dev);
        tree_attach_runs(plan->tx, static_cast<const uint32_t *>(records), run_stride, (cudaStream_t)stream);
    });
}

/* ---- one product shared by several GPUs, in phases ------------------------------------------------------------ */

int f3m_plan_partition_rows(f3m_plan *plan, int32_t R, int32_t nparts, int64_t *bounds, void *stream) {
    if (!plan || !bounds || nparts < 1 || R < 1) return F3M_ERR_ARG;
    return guarded([&] {
        int dev;
        F3M_CUDA(cudaGetDevice(&dev));
        F3M_REQUIRE(dev == plan->device, F3M_ERR_ARG, "plan was built on device %d, current device is %d", plan->device, dev);
        shard_partition(plan, R, nparts, bounds, (cudaStream_t)stream);
    });
}

int f3m_plan_shard_begin(f3m_plan *plan, const float *b, int32_t R, int64_t row_begin, int64_t row_end, int64_t box_begin,
                         int64_t box_end, float *mom_slice, void *stream) {
    if (!plan || !b) return F3M_ERR_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    int st = guarded([&] {
        F3M_REQUIRE(R >= 1, F3M_ERR_ARG, "bad right-hand side (R=%d)", R);
        F3M_REQUIRE(!plan->tx.runs.pending, F3M_ERR_ARG, "the plan still waits for its sorted runs (f3m_plan_attach_runs)");
        int dev;
        F3M_CUDA(cudaGetDevice(&dev));
        F3M_REQUIRE(dev == plan->device, F3M_ERR_ARG, "plan was built on device %d, current device is %d", plan->device, dev);
        Tree &tx = plan->tx, &ty = *plan->ty;
        const int L = plan->levels;
        f3m_plan::Shard &sh = plan->shard;
        sh.active = false;
        sh.R = R;
        sh.row_begin = std::max<int64_t>(0, row_begin);
        sh.row_end = std::min<int64_t>(tx.n, row_end);
        for (float &m : plan->last.ms) m = 0.f;
        plan->last.ms[ST_BUILD] = plan->stats.build_ms;
        plan->last.direct_launches = 0;
        for (int &v : plan->last.direct_variants) v = 0;
        const int64_t msize = far_moments_size(plan, R);
        const bool exchange = msize > 0 && mom_slice != nullptr;
        const int nby = ty.levels[L].nb;
        box_begin = std::max<int64_t>(0, std::min<int64_t>(box_begin, nby));
        box_end = std::max<int64_t>(box_begin, std::min<int64_t>(box_end, nby));
        plan->last.begin(ST_PERMUTE, s);
        shard_mark_and_gather(plan, b, R, (int)sh.row_begin, (int)sh.row_end, exchange ? (int)box_begin : 0, exchange ? (int)box_end : 0,
                              !exchange, s);
        plan->last.end(s);
        if (exchange && box_end > box_begin) {
            // sorted-row range of the source boxes [box_begin, box_end)
            const int *off = ty.levels[L].off.p;
            F3M_CUDA(cudaMemcpyAsync(plan->h_pinned + 0, off + box_begin, sizeof(int), cudaMemcpyDeviceToHost, s));
            F3M_CUDA(cudaMemcpyAsync(plan->h_pinned + 1, off + box_end, sizeof(int), cudaMemcpyDeviceToHost, s));
            F3M_CUDA(cudaStreamSynchronize(s));
            const int64_t per_box = msize / nby;
            plan->moments_out = mom_slice - box_begin * per_box;   // the kernels address moments by box number
            plan->mom_begin = plan->h_pinned[0];
            plan->mom_end = plan->h_pinned[1];
            plan->mom_box_begin = box_begin;
            plan->mom_box_end = box_end;
            far_field(plan, sh.bs.p, R, nullptr, 0, 0, s);
        }
        F3M_CUDA(cudaStreamSynchronize(s));
        sh.active = true;
    });
    plan->moments_out = nullptr;
    plan->mom_box_begin = plan->mom_box_end = -1;
    if (st != F3M_OK) cudaStreamSynchronize(s);
    plan->last.resolve();
    return st;
}

int f3m_plan_shard_near(f3m_plan *plan, float *acc_sorted, void *stream) {
    if (!plan || !acc_sorted) return F3M_ERR_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    int st = guarded([&] {
        f3m_plan::Shard &sh = plan->shard;
        F3M_REQUIRE(sh.active, F3M_ERR_ARG, "f3m_plan_shard_near without f3m_plan_shard_begin");
        const int L = plan->levels, R = sh.R;
        const int64_t rb = sh.row_begin, re = sh.row_end;
        plan->pack_cache.reset();
        struct DropPacked { f3m_plan *p; ~DropPacked() { p->pack_cache.reset(); } } drop_packed{plan};
        if (re > rb) F3M_CUDA(cudaMemsetAsync(acc_sorted + rb * R, 0, (size_t)(re - rb) * R * sizeof(float), s));
        if (L == 0) direct_sums(plan, 0, plan->lists[0].keep, sh.bs.p, R, acc_sorted, rb, re, s);
        for (int level = 1; level <= L; level++) direct_sums(plan, level, plan->lists[level].small, sh.bs.p, R, acc_sorted, rb, re, s);
        if (L > 0) direct_sums(plan, L, plan->lists[L].keep, sh.bs.p, R, acc_sorted, rb, re, s);
        F3M_CUDA(cudaStreamSynchronize(s));
    });
    if (st != F3M_OK) cudaStreamSynchronize(s);
    plan->last.resolve();
    return st;
}

int f3m_plan_shard_far(f3m_plan *plan, const float *mom, float *acc_sorted, void *stream) {
    if (!plan || !acc_sorted) return F3M_ERR_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    int st = guarded([&] {
        f3m_plan::Shard &sh = plan->shard;
        F3M_REQUIRE(sh.active, F3M_ERR_ARG, "f3m_plan_shard_far without f3m_plan_shard_begin");
        F3M_REQUIRE(mom || sh.all_sources, F3M_ERR_ARG, "this product exchanges moments: pass the gathered moment array");
        plan->ext_mom = sh.all_sources ? nullptr : mom;
        far_field(plan, sh.bs.p, sh.R, acc_sorted, sh.row_begin, sh.row_end, s);
        F3M_CUDA(cudaMemcpyAsync(plan->h_pinned, plan->d_flags + FL_ERR, sizeof(int), cudaMemcpyDeviceToHost, s));
        F3M_CUDA(cudaStreamSynchronize(s));
        F3M_REQUIRE(plan->h_pinned[0] == 0, F3M_ERR_INTERNAL, "device-side consistency check failed (code %d)", plan->h_pinned[0]);
    });
    plan->ext_mom = nullptr;
    if (st != F3M_OK) cudaStreamSynchronize(s);
    plan->last.resolve();
    return st;
}

int f3m_plan_shard_end(f3m_plan *plan) {
    if (!plan) return F3M_ERR_ARG;
    plan->shard.active = false;
    plan->shard.bs.release();
    plan->shard.need.clear();
    return F3M_OK;
}

int f3m_plan_gathered_rows_to_input_order(const f3m_plan *plan, const float *gathered, int32_t R, const int64_t *slice_bounds,
                                          int32_t nslices, int64_t stride, int64_t in_lo, int64_t in_hi, float *out, void *stream) {
    if (!plan || !gathered || !slice_bounds || !out || R < 1 || in_lo < 0 || in_hi < in_lo || in_hi > plan->tx.n) return F3M_ERR_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    return guarded([&] {
        shard_gathered_rows_to_input_order(plan, gathered, R, slice_bounds, nslices, stride, in_lo, in_hi, out, s);
        F3M_CUDA(cudaStreamSynchronize(s));
    });
}

int f3m_plan_count_rows_by_owner(const f3m_plan *plan, int64_t row_begin, int64_t row_end, const int64_t *in_bounds, int32_t nranks,
                                 int64_t *counts, void *stream) {
    if (!plan || !in_bounds || !counts || row_begin < 0 || row_end < row_begin || row_end > plan->tx.n) return F3M_ERR_ARG;
    return guarded([&] { shard_count_rows_by_owner(plan, row_begin, row_end, in_bounds, nranks, counts, (cudaStream_t)stream); });
}

int f3m_plan_pack_rows_by_owner(const f3m_plan *plan, const float *acc_sorted, int32_t R, int64_t row_begin, int64_t row_end,
                                const int64_t *in_bounds, int32_t nranks, const int64_t *counts, float *send, void *stream) {
    if (!plan || !acc_sorted || !in_bounds || !counts || !send || R < 1 || row_begin < 0 || row_end < row_begin || row_end > plan->tx.n)
        return F3M_ERR_ARG;
    return guarded([&] {
        shard_pack_rows_by_owner(plan, acc_sorted, R, row_begin, row_end, in_bounds, nranks, counts, send, (cudaStream_t)stream);
    });
}

int f3m_plan_place_rows(f3m_plan *plan, const float *records, int64_t n, int32_t R, int64_t in_lo, int64_t in_hi, float *out,
                        void *stream) {
    if (!plan || !records || !out || n < 0 || R < 1 || in_hi < in_lo) return F3M_ERR_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    return guarded([&] {
        shard_place_rows(records, n, R, in_lo, in_hi, out, plan->d_flags + FL_ERR, s);
        F3M_CUDA(cudaMemcpyAsync(plan->h_pinned, plan->d_flags + FL_ERR, sizeof(int), cudaMemcpyDeviceToHost, s));
        F3M_CUDA(cudaStreamSynchronize(s));
        F3M_REQUIRE(plan->h_pinned[0] == 0, F3M_ERR_INTERNAL, "a received row lies outside this rank's input rows (code %d)", plan->h_pinned[0]);
    });
}

int f3m_plan_rows_to_input_order(const f3m_plan *plan, const float *acc_sorted, int32_t R, int64_t in_lo, int64_t in_hi, float *out,
                                 void *stream) {
    if (!plan || !acc_sorted || !out || R < 1 || in_lo < 0 || in_hi < in_lo || in_hi > plan->tx.n) return F3M_ERR_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    return guarded([&] {
        int dev;
        F3M_CUDA(cudaGetDevice(&dev));
        F3M_REQUIRE(dev == plan->device, F3M_ERR_ARG, "plan was built on device %d, current device is %d", plan->device, dev);
        shard_rows_to_input_order(plan, acc_sorted, R, in_lo, in_hi, out, s);
        F3M_CUDA(cudaStreamSynchronize(s));
    });
}

int f3m_plan_apply(f3m_plan *plan, const float *b, int32_t R, float *out, void *stream) {
    if (!plan) return F3M_ERR_ARG;
    return f3m_plan_apply_range(plan, b, R, out, 0, plan->tx.n, stream);
}

int f3m_plan_destroy(f3m_plan *plan) {
    if (!plan) return F3M_OK;
    // every entry point that enqueues work on the plan's buffers synchronises its stream before it
    // returns, so the buffers can go back to the stream-ordered pool without a device-wide wait
    delete plan;
    return F3M_OK;
}

int f3m_kmvm_f32(const float *X, int64_t N, const float *Y, int64_t M, const float *b, int32_t R, int32_t d,
                 const f3m_params *prm, float *out, void *stream) {
    f3m_plan *pl = nullptr;
    int st = f3m_plan_create(&pl, X, N, Y, M, d, prm, stream);
    if (st != F3M_OK) return st;
    st = f3m_plan_apply(pl, b, R, out, stream);
    f3m_plan_destroy(pl);
    return st;
}

size_t f3m_workspace_bytes(int64_t N, int64_t M, int32_t R, int32_t d, const f3m_params *prm) {
    if (N < 1 || M < 1 || R < 1 || d < 1 || d > F3M_MAX_DIM || !prm) return 0;
    const double n = (double)N, m = (double)M, pts = n + m;
    const int RB = R == 1 ? 1 : 8, W = (d + RB + 3) / 4 * 4, RW = record_words(d);
    const int p = nodes_per_dim(d, prm->nr_interpolation);
    double P = 1;
    for (int k = 0; k < d; k++) P *= p;
    // boxes of the last level when the level loop stops at boxes of at most min_points points (evenly spread points)
    const double boxes = std::max(1.0, pts * pow(2.0, d) / std::max(1.0f, prm->min_points));
    const double sort_peak = pts * (12.0 + 4.0 * d + 8.0 + 8.0 * RW);                       // keys, records (twice), planes
    const double tree = pts * (8.0 + 4.0 * d) + boxes * (pow(6.0, d) + 2.0 * pow(3.0, d)) * 12.0 + 64.0 * boxes;
    const double product = 4.0 * R * (n + m) + 4.0 * W * (m + boxes) + 2.3 * boxes * P * RB * 4.0 + 8.0 * boxes;
    return (size_t)(1.15 * std::max(sort_peak + pts * (8.0 + 4.0 * d), tree + product)) + ((size_t)64 << 20);
}

size_t f3m_last_workspace_peak(void) { return g_last_ws_peak; }

int f3m_kmvm_ws_f32(const float *X, int64_t N, const float *Y, int64_t M, const float *b, int32_t R, int32_t d,
                    const f3m_params *prm, float *out, void *workspace, size_t workspace_bytes, void *stream) {
    if (!workspace || workspace_bytes < 4096) return F3M_ERR_ARG;
    Arena arena;
    arena.reset(workspace, workspace_bytes);
    struct Scope {   // every buffer of the call is gone before the arena is
        Arena *prev;
        explicit Scope(Arena *a) : prev(g_arena) { g_arena = a; }
        ~Scope() { g_last_ws_peak = g_arena->peak; g_arena = prev; }
    } scope(&arena);
    return f3m_kmvm_f32(X, N, Y, M, b, R, d, prm, out, stream);
}

int f3m_kmvm_host_f32(const float *X, int64_t N, const float *Y, int64_t M, const float *b, int32_t R, int32_t d,
                      const f3m_params *prm, float *out) {
    int st = guarded([&] {
        check_common(X, N, Y, M, d, prm);
        F3M_REQUIRE(b && out && R >= 1, F3M_ERR_ARG, "bad right-hand side");
        const bool same = (X == Y && N == M);
        // two streams: the coordinates go first and the tree is built from them while b is still on the link
        cudaStream_t s = nullptr, sb = nullptr;
        cudaEvent_t ev_x = nullptr, ev_b = nullptr;
        f3m_plan *pl = nullptr;
        DevBuf<float> dX, dY, db, dout;   // declared before the guard below: released after the streams are drained
        struct Cleanup {
            cudaStream_t &s, &sb; cudaEvent_t &ex, &eb; f3m_plan *&pl;
            ~Cleanup() {
                if (s) cudaStreamSynchronize(s);
                if (sb) cudaStreamSynchronize(sb);
                if (pl) f3m_plan_destroy(pl);
                if (ex) cudaEventDestroy(ex);
                if (eb) cudaEventDestroy(eb);
                if (s) cudaStreamDestroy(s);
                if (sb) cudaStreamDestroy(sb);
            }
        } cleanup{s, sb, ev_x, ev_b, pl};
        F3M_CUDA(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
        F3M_CUDA(cudaStreamCreateWithFlags(&sb, cudaStreamNonBlocking));
        F3M_CUDA(cudaEventCreateWithFlags(&ev_x, cudaEventDisableTiming));
        F3M_CUDA(cudaEventCreateWithFlags(&ev_b, cudaEventDisableTiming));
        dX.alloc((size_t)N * d, s);
        F3M_CUDA(cudaMemcpyAsync(dX.p, X, (size_t)N * d * sizeof(float), cudaMemcpyHostToDevice, s));
        if (!same) {
            dY.alloc((size_t)M * d, s);
            F3M_CUDA(cudaMemcpyAsync(dY.p, Y, (size_t)M * d * sizeof(float), cudaMemcpyHostToDevice, s));
        }
        F3M_CUDA(cudaEventRecord(ev_x, s));
        db.alloc((size_t)M * R, s);
        F3M_CUDA(cudaStreamWaitEvent(sb, ev_x, 0));
        F3M_CUDA(cudaMemcpyAsync(db.p, b, (size_t)M * R * sizeof(float), cudaMemcpyHostToDevice, sb));
        F3M_CUDA(cudaEventRecord(ev_b, sb));
        dout.alloc((size_t)N * R, s);
        int st2 = f3m_plan_create(&pl, dX.p, N, same ? dX.p : dY.p, M, d, prm, s);
        if (st2 != F3M_OK) throw Fail{st2};
        F3M_CUDA(cudaStreamWaitEvent(s, ev_b, 0));
        st2 = f3m_plan_apply(pl, db.p, R, dout.p, s);
        if (st2 != F3M_OK) throw Fail{st2};
        F3M_CUDA(cudaMemcpyAsync(out, dout.p, (size_t)N * R * sizeof(float), cudaMemcpyDeviceToHost, s));
        F3M_CUDA(cudaStreamSynchronize(s));
    });
    return st;
}

int f3m_plan_get_stats(const f3m_plan *plan, f3m_plan_stats *stats) {
    if (!plan || !stats) return F3M_ERR_ARG;
    *stats = plan->stats;
    return F3M_OK;
}

int f3m_plan_get_level(const f3m_plan *plan, int32_t level, f3m_level_info *info) {
    if (!plan || !info || level < 1 || level > plan->levels) return F3M_ERR_ARG;
    const Level &lx = plan->tx.levels[level], &ly = plan->ty->levels[level];
    const LevelLists &ll = plan->lists[level];
    info->level = level;
    info->boxes_x = lx.nb; info->boxes_y = ly.nb;
    info->max_count_x = lx.max_count; info->max_count_y = ly.max_count;
    info->n_far = ll.far.count; info->n_small = ll.small.count; info->n_keep = ll.keep.count;
    info->edge = lx.edge;
    info->nodes_per_dim = ll.p;
    return F3M_OK;
}

int f3m_plan_copy_array(const f3m_plan *plan, int32_t level, int32_t tree, int32_t what, void *host_dst, size_t dst_bytes) {
    if (!plan || !host_dst) return F3M_ERR_ARG;
    return guarded([&] {
        const Tree &t = tree == 0 ? plan->tx : *plan->ty;
        const void *src = nullptr;
        size_t bytes = 0;
        if (what == F3M_ARR_SORTED_INDEX) { src = t.perm.p; bytes = (size_t)t.n * 4; }
        else {
            F3M_REQUIRE(level >= 0 && level <= plan->levels, F3M_ERR_ARG, "level %d outside 0..%d", level, plan->levels);
            const Level &L = t.levels[level];
            const LevelLists &ll = plan->lists[level];
            const int nbx = plan->tx.levels[level].nb;
            switch (what) {
                case F3M_ARR_BOX_OFFSETS: src = L.off.p; bytes = ((size_t)L.nb + 1) * 4; break;
                case F3M_ARR_BOX_CENTERS: src = L.ctr.p; bytes = (size_t)L.nb * plan->d * 4; break;
                case F3M_ARR_BOX_CODES: src = L.code.p; bytes = (size_t)L.nb * 4; break;
                case F3M_ARR_FAR_PTR: src = ll.far.ptr.p; bytes = ((size_t)nbx + 1) * 4; break;
                case F3M_ARR_FAR_IDX: src = ll.far.idx.p; bytes = (size_t)ll.far.count * 4; break;
                case F3M_ARR_SMALL_PTR: src = ll.small.ptr.p; bytes = ((size_t)nbx + 1) * 4; break;
                case F3M_ARR_SMALL_IDX: src = ll.small.idx.p; bytes = (size_t)ll.small.count * 4; break;
                case F3M_ARR_KEEP_PTR: src = ll.keep.ptr.p; bytes = ((size_t)nbx + 1) * 4; break;
                case F3M_ARR_KEEP_IDX: src = ll.keep.idx.p; bytes = (size_t)ll.keep.count * 4; break;
                default: F3M_REQUIRE(false, F3M_ERR_ARG, "unknown array id %d", what);
            }
            F3M_REQUIRE(level >= 1 || what == F3M_ARR_BOX_OFFSETS || what == F3M_ARR_BOX_CENTERS || what == F3M_ARR_BOX_CODES ||
                            what == F3M_ARR_KEEP_PTR || what == F3M_ARR_KEEP_IDX,
                        F3M_ERR_ARG, "level 0 has no far/small lists");
        }
        F3M_REQUIRE(dst_bytes >= bytes, F3M_ERR_ARG, "destination holds %zu bytes, array needs %zu", dst_bytes, bytes);
        if (bytes) F3M_CUDA(cudaMemcpy(host_dst, src, bytes, cudaMemcpyDeviceToHost));
    });
}

int f3m_rbf_dense_f32(const float *X, int64_t N, const float *Y, int64_t M, const float *b, int32_t R, int32_t d, float ls,
                      float *out, void *stream) {
    return guarded([&] {
        F3M_REQUIRE(X && Y && b && out && N > 0 && M > 0 && R >= 1 && d >= 1 && d <= F3M_MAX_DIM && ls > 0, F3M_ERR_ARG,
                    "bad argument to f3m_rbf_dense_f32");
            dense_f32<false>(X, N, Y, M, b, R, d, ls, out, (cudaStream_t)stream);
        F3M_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
    });
}

int f3m_rbf_dense_grad_f32(const float *X, int64_t N, const float *Y, int64_t M, const float *b, int32_t R, int32_t d,
                           float ls, float *out, void *stream) {
    return guarded([&] {
        F3M_REQUIRE(X && Y && b && out && N > 0 && M > 0 && R >= 1 && d >= 1 && d <= F3M_MAX_DIM && ls > 0, F3M_ERR_ARG,
                    "bad argument to f3m_rbf_dense_grad_f32");
            dense_f32<true>(X, N, Y, M, b, R, d, ls, out, (cudaStream_t)stream);
        F3M_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
    });
}

int f3m_rbf_dense_f64(const double *X, int64_t N, const double *Y, int64_t M, const double *b, int32_t R, int32_t d,
                      double ls, double *out, void *stream) {
    return guarded([&] {
        F3M_REQUIRE(X && Y && b && out && N > 0 && M > 0 && R >= 1 && d >= 1 && d <= F3M_MAX_DIM && ls > 0, F3M_ERR_ARG,
                    "bad argument to f3m_rbf_dense_f64");
        dense_f64(X, N, Y, M, b, R, d, ls, out, (cudaStream_t)stream);
        F3M_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
    });
}

int f3m_rbf_dense_f32_static(const float *X, int64_t N, const float *Y, int64_t M, const float *b, int32_t R, int32_t d,
                             float ls, float *out, void *stream) {
    return guarded([&] {
        F3M_REQUIRE(X && Y && b && out && N > 0 && M > 0 && R >= 1 && d >= 1 && d <= F3M_MAX_DIM && ls > 0, F3M_ERR_ARG,
                    "bad argument to f3m_rbf_dense_f32_static");
        dense_f32_static(X, N, Y, M, b, R, d, ls, out, (cudaStream_t)stream);   // no allocation anywhere on this path
        F3M_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
    });
}

int f3m_measure_peaks(double *gexp_per_s, double *gfma_per_s, void *stream) {
    if (!gexp_per_s || !gfma_per_s) return F3M_ERR_ARG;
    return guarded([&] {
            measure_peaks(gexp_per_s, gfma_per_s, (cudaStream_t)stream);
    });
}

int f3m_release_cached_memory(void) {
    std::lock_guard<std::mutex> lk(g_mem_mu);
    for (auto &b : g_free_blocks) cudaFree(b.p);
    g_free_blocks.clear();
    return F3M_OK;
}

int f3m_plan_last_timings(const f3m_plan *plan, float ms[8]) {
    if (!plan || !ms) return F3M_ERR_ARG;
    for (int i = 0; i < 8; i++) ms[i] = plan->last.ms[i];
    return F3M_OK;
}

int f3m_plan_last_direct_launches(const f3m_plan *plan) { return plan ? plan->last.direct_launches : 0; }

int f3m_plan_last_direct_variants(const f3m_plan *plan, int32_t counts[6]) {
    if (!plan || !counts) return F3M_ERR_ARG;
    for (int i = 0; i < 6; i++) counts[i] = plan->last.direct_variants[i];
    return F3M_OK;
}

}  // extern "C"
