// One product shared by several GPUs: helpers of the phase entry points (f3m_plan_partition_rows,
// f3m_plan_shard_begin / _near / _far, f3m_plan_rows_to_input_order).
//
// The reference has no counterpart: its multi-GPU mode runs independent block products in separate processes
// (par_FFM_block, experiments/FFM_classes.py:128-211).  Here every rank holds the same plan and owns a contiguous
// slice of the sorted target rows, cut at finest-level box starts.  What a rank reads from the sources is limited
// to the boxes its own direct lists name (its slice plus a halo) and to the boxes whose moments it computes.
#include <algorithm>
#include "common.cuh"

namespace f3m {

__device__ __forceinline__ int lower_bound_i32(const int *__restrict__ a, int n, int v) {
    int lo = 0, hi = n;
    while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        if (a[mid] < v) lo = mid + 1; else hi = mid;
    }
    return lo;
}

// ---------------------------------------------------------------------------------------------
// which source boxes does a slice of the targets read?
// ---------------------------------------------------------------------------------------------
// one warp per target box of the level: boxes with a row inside [row_begin, row_end) mark the sources of their row
__global__ void __launch_bounds__(256) mark_list_sources(int nbx, const int *__restrict__ off_x, const int *__restrict__ ptr,
                                                   const int *__restrict__ idx, int row_begin, int row_end, unsigned char *need) {
    const int lane = threadIdx.x & 31;
    const int box = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    if (box >= nbx) return;
    if (off_x[box + 1] <= row_begin || off_x[box] >= row_end) return;
    for (int e = ptr[box] + lane; e < ptr[box + 1]; e += 32) need[idx[e]] = 1;
}

// one block per source box of a coarser level: a marked box marks the finest-level boxes it contains
__global__ void __launch_bounds__(128) need_to_finest(int nb, const int *__restrict__ off, const unsigned char *__restrict__ need,
                                                     int nb_fine, const int *__restrict__ off_fine, unsigned char *need_fine) {
    const int b = blockIdx.x;
    if (b >= nb || !need[b]) return;
    const int j0 = lower_bound_i32(off_fine, nb_fine, off[b]), j1 = lower_bound_i32(off_fine, nb_fine, off[b + 1]);
    for (int j = j0 + threadIdx.x; j < j1; j += blockDim.x) need_fine[j] = 1;
}

__global__ void __launch_bounds__(256) mark_box_range(int box_begin, int box_end, unsigned char *need) {
    const int j = box_begin + blockIdx.x * blockDim.x + threadIdx.x;
    if (j < box_end) need[j] = 1;
}

// one warp per finest-level source box: rows of b of the marked boxes, in sorted order
__global__ void __launch_bounds__(256) gather_rows_of_boxes(int nb, const int *__restrict__ off, const unsigned char *__restrict__ need,
                                                           const float *__restrict__ b, const int *__restrict__ perm, int cols,
                                                           float *bs) {
    const int lane = threadIdx.x & 31;
    const int box = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    if (box >= nb || !need[box]) return;
    const int64_t e0 = (int64_t)off[box] * cols, e1 = (int64_t)off[box + 1] * cols;
    for (int64_t e = e0 + lane; e < e1; e += 32) {
        const int64_t i = e / cols;
        const int c = (int)(e - i * cols);
        bs[e] = b[(int64_t)perm[i] * cols + c];
    }
}

// Source boxes of `level` that a direct list of the level names: for the slice of the running sharded product, else for
// all targets (kept in the plan: the lists do not change).
const unsigned char *level_source_flags(f3m_plan *pl, int level, cudaStream_t s) {
    if (pl->shard.active) return pl->shard.all_sources ? nullptr : pl->shard.need[level].p;
    if (level < 1) return nullptr;
    if ((int)pl->src_need.size() <= pl->levels) pl->src_need.resize(pl->levels + 1);
    DevBuf<unsigned char> &f = pl->src_need[level];
    if (!f.p) {
        Level &lx = pl->tx.levels[level];
        f.alloc((size_t)pl->ty->levels[level].nb, s);
        f.zero();
        auto mark = [&](const PairCSR &csr) {
            if (csr.count == 0) return;
            mark_list_sources<<<(unsigned)(((int64_t)lx.nb * 32 + 255) / 256), 256, 0, s>>>(lx.nb, lx.off.p, csr.ptr.p, csr.idx.p, 0,
                                                                                            (int)pl->tx.n, f.p);
            F3M_LAUNCH_CHECK();
        };
        mark(pl->lists[level].small);
        if (level == pl->levels) mark(pl->lists[level].keep);
    }
    return f.p;
}

void shard_mark_and_gather(f3m_plan *pl, const float *b, int R, int row_begin, int row_end, int box_begin, int box_end,
                           bool everything, cudaStream_t s) {
    Tree &tx = pl->tx, &ty = *pl->ty;
    const int L = pl->levels;
    f3m_plan::Shard &sh = pl->shard;
    sh.need.resize(L + 1);
    sh.bs.alloc((size_t)ty.n * R, s);
    if (everything || L == 0) {
        // no halo bookkeeping: all sources (plans without far pairs, or whose moments cannot be exchanged)
        for (int l = 0; l <= L; l++) sh.need[l].release();
        gather_rows(b, ty.perm.p, sh.bs.p, ty.n, R, s);
        sh.all_sources = true;
        return;
    }
    sh.all_sources = false;
    for (int l = 1; l <= L; l++) {
        sh.need[l].alloc((size_t)ty.levels[l].nb, s);
        sh.need[l].zero();
    }
    auto mark = [&](int level, const PairCSR &csr) {
        if (csr.count == 0) return;
        Level &lx = tx.levels[level];
        mark_list_sources<<<(unsigned)(((int64_t)lx.nb * 32 + 255) / 256), 256, 0, s>>>(lx.nb, lx.off.p, csr.ptr.p, csr.idx.p, row_begin,
                                                                                   row_end, sh.need[level].p);
        F3M_LAUNCH_CHECK();
    };
    for (int l = 1; l <= L; l++) mark(l, pl->lists[l].small);
    mark(L, pl->lists[L].keep);
    Level &lf = ty.levels[L];
    for (int l = 1; l < L; l++) {
        if (pl->lists[l].small.count == 0) continue;
        Level &ly = ty.levels[l];
        need_to_finest<<<ly.nb, 128, 0, s>>>(ly.nb, ly.off.p, sh.need[l].p, lf.nb, lf.off.p, sh.need[L].p);
        F3M_LAUNCH_CHECK();
    }
    // rows of b for the direct sums (marked boxes) and for this rank's share of the moments
    DevBuf<unsigned char> rows_need;
    rows_need.alloc((size_t)lf.nb, s);
    F3M_CUDA(cudaMemcpyAsync(rows_need.p, sh.need[L].p, (size_t)lf.nb, cudaMemcpyDeviceToDevice, s));
    if (box_end > box_begin) {
        mark_box_range<<<(unsigned)((box_end - box_begin + 255) / 256), 256, 0, s>>>(box_begin, box_end, rows_need.p);
        F3M_LAUNCH_CHECK();
    }
    gather_rows_of_boxes<<<(unsigned)(((int64_t)lf.nb * 32 + 255) / 256), 256, 0, s>>>(lf.nb, lf.off.p, rows_need.p, b, ty.perm.p, R,
                                                                                      sh.bs.p);
    F3M_LAUNCH_CHECK();
    // rows_need is released here; the kernel above is already queued on the stream the next user of the block is on
}

// ---------------------------------------------------------------------------------------------
// rows of the sorted result that belong to one range of INPUT rows, written in input order
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) rows_to_input_order(const float *__restrict__ acc, const int *__restrict__ perm, int64_t n,
                                                          int cols, int64_t in_lo, int64_t in_hi, float *out) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int64_t r = perm[i];
    if (r < in_lo || r >= in_hi) return;
    for (int c = 0; c < cols; c++) out[(r - in_lo) * cols + c] = acc[i * cols + c];
}

void shard_rows_to_input_order(const f3m_plan *pl, const float *acc_sorted, int R, int64_t in_lo, int64_t in_hi, float *out,
                               cudaStream_t s) {
    const Tree &tx = pl->tx;
    rows_to_input_order<<<(unsigned)((tx.n + 255) / 256), 256, 0, s>>>(acc_sorted, tx.perm.p, tx.n, R, in_lo, in_hi, out);
    F3M_LAUNCH_CHECK();
}

// ---------------------------------------------------------------------------------------------
// rows of a slice of the sorted result, grouped by the rank that owns the INPUT row (for an all-to-all)
// ---------------------------------------------------------------------------------------------
constexpr int OWN_T = 256, OWN_I = 8, OWN_MAXR = 64;   // at most 64 ranks

struct OwnerBounds { long long lo[OWN_MAXR + 1]; };   // rank g owns the input rows [lo[g], lo[g+1])

__device__ __forceinline__ int owner_of(const OwnerBounds &ob, int nranks, long long row) {
    int a = 0, b = nranks;   // largest g with lo[g] <= row
    while (b - a > 1) {
        const int mid = (a + b) >> 1;
        if (ob.lo[mid] <= row) a = mid; else b = mid;
    }
    return a;
}

// pass 0: counts[g] += rows of the slice owned by rank g.  pass 1: cursor[g] holds the start of g's group in the
// send buffer; every block reserves its share and writes [values of the row, input row] records (cols + 1 words)
__global__ void __launch_bounds__(OWN_T) rows_by_owner_kernel(int pass, const float *__restrict__ acc, const int *__restrict__ perm,
                                                             int64_t row_begin, int64_t row_end, int cols, OwnerBounds ob, int nranks,
                                                             unsigned long long *cursor, float *send) {
    __shared__ int cnt[OWN_MAXR];
    __shared__ unsigned long long base[OWN_MAXR];
    if (threadIdx.x < OWN_MAXR) cnt[threadIdx.x] = 0;
    __syncthreads();
    const int64_t i0 = row_begin + (int64_t)blockIdx.x * (OWN_T * OWN_I) + threadIdx.x;
    int own[OWN_I], slot[OWN_I];
#pragma unroll
    for (int k = 0; k < OWN_I; k++) {
        const int64_t i = i0 + (int64_t)k * OWN_T;
        own[k] = -1;
        if (i < row_end) {
            own[k] = owner_of(ob, nranks, perm[i]);
            slot[k] = atomicAdd(&cnt[own[k]], 1);
        }
    }
    __syncthreads();
    if (threadIdx.x < nranks && cnt[threadIdx.x] > 0)
        base[threadIdx.x] = atomicAdd(&cursor[threadIdx.x], (unsigned long long)cnt[threadIdx.x]);
    if (pass == 0) return;
    __syncthreads();
#pragma unroll
    for (int k = 0; k < OWN_I; k++) {
        if (own[k] < 0) continue;
        const int64_t i = i0 + (int64_t)k * OWN_T;
        float *dst = send + (base[own[k]] + (unsigned long long)slot[k]) * (unsigned long long)(cols + 1);
        for (int c = 0; c < cols; c++) dst[c] = acc[i * cols + c];
        dst[cols] = __int_as_float(perm[i]);
    }
}

// h_counts[g] = rows of [row_begin, row_end) whose input row belongs to rank g (h_bounds: nranks + 1 input-row cuts)
void shard_count_rows_by_owner(const f3m_plan *pl, int64_t row_begin, int64_t row_end, const int64_t *h_bounds, int nranks,
                               int64_t *h_counts, cudaStream_t s) {
    F3M_REQUIRE(nranks >= 1 && nranks <= OWN_MAXR, F3M_ERR_ARG, "1..%d ranks", OWN_MAXR);
    OwnerBounds ob{};
    for (int g = 0; g <= nranks; g++) ob.lo[g] = h_bounds[g];
    DevBuf<unsigned long long> cur;
    cur.alloc(OWN_MAXR, s);
    cur.zero();
    const int64_t rows = row_end - row_begin;
    if (rows > 0) {
        rows_by_owner_kernel<<<(unsigned)((rows + OWN_T * OWN_I - 1) / (OWN_T * OWN_I)), OWN_T, 0, s>>>(
            0, nullptr, pl->tx.perm.p, row_begin, row_end, 1, ob, nranks, cur.p, nullptr);
        F3M_LAUNCH_CHECK();
    }
    unsigned long long h[OWN_MAXR];
    F3M_CUDA(cudaMemcpyAsync(h, cur.p, sizeof(h), cudaMemcpyDeviceToHost, s));
    F3M_CUDA(cudaStreamSynchronize(s));
    for (int g = 0; g < nranks; g++) h_counts[g] = (int64_t)h[g];
}

// send: (rows, cols + 1) floats, the rows of rank 0 first, then rank 1, ...; h_counts from the call above
void shard_pack_rows_by_owner(const f3m_plan *pl, const float *acc_sorted, int R, int64_t row_begin, int64_t row_end,
                              const int64_t *h_bounds, int nranks, const int64_t *h_counts, float *send, cudaStream_t s) {
    F3M_REQUIRE(nranks >= 1 && nranks <= OWN_MAXR, F3M_ERR_ARG, "1..%d ranks", OWN_MAXR);
    OwnerBounds ob{};
    for (int g = 0; g <= nranks; g++) ob.lo[g] = h_bounds[g];
    unsigned long long h[OWN_MAXR] = {0};
    unsigned long long run = 0;
    for (int g = 0; g < nranks; g++) { h[g] = run; run += (unsigned long long)h_counts[g]; }
    DevBuf<unsigned long long> cur;
    cur.alloc(OWN_MAXR, s);
    F3M_CUDA(cudaMemcpyAsync(cur.p, h, sizeof(h), cudaMemcpyHostToDevice, s));
    const int64_t rows = row_end - row_begin;
    if (rows > 0) {
        rows_by_owner_kernel<<<(unsigned)((rows + OWN_T * OWN_I - 1) / (OWN_T * OWN_I)), OWN_T, 0, s>>>(
            1, acc_sorted, pl->tx.perm.p, row_begin, row_end, R, ob, nranks, cur.p, send);
        F3M_LAUNCH_CHECK();
    }
    F3M_CUDA(cudaStreamSynchronize(s));   // h lives on this frame
}

// The sorted result as an all-gather of the ranks' slices leaves it: slice g (sorted rows [lo[g], lo[g+1])) starts at row
// g * stride of `gathered`.  Rows of the input range [in_lo, in_hi) go to out in input order.
__global__ void __launch_bounds__(256) gathered_rows_to_input_order(const float *__restrict__ gathered, const int *__restrict__ perm,
                                                                   int64_t n, int cols, OwnerBounds slices, int nslices, int64_t stride,
                                                                   int64_t in_lo, int64_t in_hi, float *out) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int64_t r = perm[i];
    if (r < in_lo || r >= in_hi) return;
    const int g = owner_of(slices, nslices, i);
    const float *src = gathered + ((int64_t)g * stride + (i - slices.lo[g])) * cols;
    for (int c = 0; c < cols; c++) out[(r - in_lo) * cols + c] = src[c];
}

void shard_gathered_rows_to_input_order(const f3m_plan *pl, const float *gathered, int R, const int64_t *h_slice_bounds, int nslices,
                                        int64_t stride, int64_t in_lo, int64_t in_hi, float *out, cudaStream_t s) {
    F3M_REQUIRE(nslices >= 1 && nslices <= OWN_MAXR, F3M_ERR_ARG, "1..%d slices", OWN_MAXR);
    OwnerBounds ob{};
    for (int g = 0; g <= nslices; g++) ob.lo[g] = h_slice_bounds[g];
    const Tree &tx = pl->tx;
    gathered_rows_to_input_order<<<(unsigned)((tx.n + 255) / 256), 256, 0, s>>>(gathered, tx.perm.p, tx.n, R, ob, nslices, stride, in_lo,
                                                                                in_hi, out);
    F3M_LAUNCH_CHECK();
}

// records [values, input row] -> out[(input row - in_lo)] (the receiving side of the all-to-all)
__global__ void __launch_bounds__(256) place_rows_kernel(const float *__restrict__ recs, int64_t n, int cols, int64_t in_lo,
                                                        int64_t in_hi, float *out, int *err) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float *src = recs + i * (cols + 1);
    const int64_t r = __float_as_int(src[cols]);
    if (r < in_lo || r >= in_hi) { atomicExch(err, 3); return; }
    for (int c = 0; c < cols; c++) out[(r - in_lo) * cols + c] = src[c];
}

void shard_place_rows(const float *recs, int64_t n, int R, int64_t in_lo, int64_t in_hi, float *out, int *d_err, cudaStream_t s) {
    if (n <= 0) return;
    place_rows_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(recs, n, R, in_lo, in_hi, out, d_err);
    F3M_LAUNCH_CHECK();
}

// ---------------------------------------------------------------------------------------------
// slices of equal estimated work
// ---------------------------------------------------------------------------------------------
// one warp per target box of a level: estimated cost of its direct lists and of its far row, added to the
// finest-level box that holds the box's first row (the slice of that row computes the whole box, apart from the
// clipping of coarse direct tiles, which only matters for boxes that straddle a cut)
__global__ void __launch_bounds__(256) box_work_kernel(int nbx, const int *__restrict__ off_x, const int *__restrict__ off_y,
                                                      const int *__restrict__ ptr_a, const int *__restrict__ idx_a,
                                                      const int *__restrict__ ptr_b, const int *__restrict__ idx_b,
                                                      const int *__restrict__ far_ptr, double w_pair, double w_far, double w_point,
                                                      int nb_fine, const int *__restrict__ off_fine, unsigned long long *work) {
    const int lane = threadIdx.x & 31;
    const int box = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    if (box >= nbx) return;
    long long ny = 0;
    if (ptr_a)
        for (int e = ptr_a[box] + lane; e < ptr_a[box + 1]; e += 32) { const int by = idx_a[e]; ny += off_y[by + 1] - off_y[by]; }
    if (ptr_b)
        for (int e = ptr_b[box] + lane; e < ptr_b[box + 1]; e += 32) { const int by = idx_b[e]; ny += off_y[by + 1] - off_y[by]; }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ny += __shfl_xor_sync(0xffffffffu, ny, o);
    if (lane) return;
    const double nx = (double)(off_x[box + 1] - off_x[box]);
    double w = w_pair * nx * (double)ny + w_point * nx;
    if (far_ptr) w += w_far * (double)(far_ptr[box + 1] - far_ptr[box]);
    // integer units: the sums must come out identical on every rank, whatever order the atomics run in
    if (w > 0.0) atomicAdd(&work[lower_bound_i32(off_fine, nb_fine, off_x[box])], (unsigned long long)llrint(w) + 1ull);
}

// sums of the work over tiles of PART_TILE consecutive finest-level boxes
constexpr int PART_TILE = 4096;
__global__ void __launch_bounds__(256) work_tile_sums(int nb, const unsigned long long *__restrict__ work, unsigned long long *tile_sum) {
    __shared__ unsigned long long part[8];
    const int j0 = blockIdx.x * PART_TILE;
    unsigned long long s = 0;
    for (int j = j0 + threadIdx.x; j < min(nb, j0 + PART_TILE); j += blockDim.x) s += work[j];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = s;
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned long long t = 0;
        for (int w = 0; w < 8; w++) t += part[w];
        tile_sum[blockIdx.x] = t;
    }
}

// one block: running sum over the tiles, then inside the few tiles where it passes k / nparts of the total.  All sums
// are integers, so every rank computes the same cuts from the same plan.
__global__ void __launch_bounds__(1024) partition_kernel(int nb, int ntiles, const unsigned long long *__restrict__ work,
                                                        unsigned long long *tile_sum, const int *__restrict__ off, int nparts,
                                                        long long *bounds) {
    __shared__ unsigned long long total_s;
    if (threadIdx.x == 0) {
        unsigned long long run = 0;
        for (int t = 0; t < ntiles; t++) { const unsigned long long v = tile_sum[t]; tile_sum[t] = run; run += v; }   // exclusive, in place
        total_s = run;
        bounds[0] = 0;
        bounds[nparts] = off[nb];
        for (int k = 1; k < nparts; k++) bounds[k] = -1;
    }
    __syncthreads();
    const unsigned long long total = total_s;
    if (total == 0) {   // no work estimate (no lists): even row counts
        if (threadIdx.x == 0)
            for (int k = 1; k < nparts; k++) {
                const int target = (int)(((long long)off[nb] * k) / nparts);
                bounds[k] = off[lower_bound_i32(off, nb, target)];
            }
        return;
    }
    for (int t = threadIdx.x; t < ntiles; t += blockDim.x) {
        const unsigned long long before_tile = tile_sum[t], after_tile = t + 1 < ntiles ? tile_sum[t + 1] : total;
        if ((int)((double)before_tile * nparts / (double)total) == (int)((double)after_tile * nparts / (double)total)) continue;
        unsigned long long run = before_tile;
        for (int j = t * PART_TILE; j < min(nb, (t + 1) * PART_TILE); j++) {
            const unsigned long long before = run;
            run += work[j];
            // cut k lies after box j when the running sum passes k * total / nparts inside this box
            const int k0 = (int)((double)before * nparts / (double)total), k1 = (int)((double)run * nparts / (double)total);
            for (int k = k0 + 1; k <= k1 && k < nparts; k++) bounds[k] = off[j + 1];
        }
    }
}

void shard_partition(f3m_plan *pl, int R, int nparts, int64_t *h_bounds, cudaStream_t s) {
    Tree &tx = pl->tx, &ty = *pl->ty;
    const int L = pl->levels, d = pl->d;
    if (L == 0) {   // one box: nothing to cut
        for (int k = 0; k <= nparts; k++) h_bounds[k] = k == 0 ? 0 : tx.n;
        return;
    }
    Level &lf = tx.levels[L];
    DevBuf<unsigned long long> work;
    work.alloc((size_t)lf.nb, s);
    work.zero();
    // cost per unit, relative to one direct pair of one column in three dimensions (measured on the N = 1e8 uniform
    // workload: direct sums 2.0e-13 s per pair, node-to-node step 7.8e-14 s per multiply-add, finest-level
    // interpolation 1.8e-13 s per point and node)
    for (int l = 1; l <= L; l++) {
        LevelLists &ll = pl->lists[l];
        Level &lx = tx.levels[l], &ly = ty.levels[l];
        int P = 1;
        for (int k = 0; k < d; k++) P *= std::max(1, ll.p);
        const double w_pair = (double)(d + R + 1) / 5.0;
        const double w_far = 0.39 * (double)d * ll.p * P * R;
        const double w_point = (l == L) ? 0.9 * (double)P * R : 0.0;
        const bool has_keep = (l == L) && ll.keep.count > 0;
        if (ll.small.count == 0 && ll.far.count == 0 && !has_keep && w_point == 0.0) continue;
        box_work_kernel<<<(unsigned)(((int64_t)lx.nb * 32 + 255) / 256), 256, 0, s>>>(
            lx.nb, lx.off.p, ly.off.p, ll.small.count ? ll.small.ptr.p : nullptr, ll.small.idx.p, has_keep ? ll.keep.ptr.p : nullptr,
            ll.keep.idx.p, ll.far.count ? ll.far.ptr.p : nullptr, w_pair, w_far, w_point, lf.nb, lf.off.p, work.p);
        F3M_LAUNCH_CHECK();
    }
    DevBuf<long long> bounds;
    bounds.alloc((size_t)nparts + 1, s);
    const int ntiles = (lf.nb + PART_TILE - 1) / PART_TILE;
    DevBuf<unsigned long long> tile_sum;
    tile_sum.alloc((size_t)ntiles, s);
    work_tile_sums<<<ntiles, 256, 0, s>>>(lf.nb, work.p, tile_sum.p);
    F3M_LAUNCH_CHECK();
    partition_kernel<<<1, 1024, 0, s>>>(lf.nb, ntiles, work.p, tile_sum.p, lf.off.p, nparts, bounds.p);
    F3M_LAUNCH_CHECK();
    std::vector<long long> h((size_t)nparts + 1);
    F3M_CUDA(cudaMemcpyAsync(h.data(), bounds.p, ((size_t)nparts + 1) * sizeof(long long), cudaMemcpyDeviceToHost, s));
    F3M_CUDA(cudaStreamSynchronize(s));
    // a cut that no box produced (more parts than boxes with work) repeats the previous one: that part is empty
    h_bounds[0] = 0;
    for (int k = 1; k <= nparts; k++) h_bounds[k] = h[k] < 0 ? h_bounds[k - 1] : std::max<int64_t>(h[k], h_bounds[k - 1]);
    h_bounds[nparts] = tx.n;
}

}  // namespace f3m
