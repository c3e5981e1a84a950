/*
 * f3m.h -- C ABI of libf3m.so, a B200 (sm_100a) engine for Gaussian kernel matrix-vector
 * products  out = K(X,Y) b,  K_ij = exp(-|x_i - y_j|^2 / (2 ls^2)),  computed with the F3M
 * treecode (2^d-tree, near/far interaction lists, Chebyshev/Lagrange interpolation).
 *
 * Every entry point is plain C: raw pointers, sizes, an opaque handle and an int status
 * (0 = ok).  No exceptions cross the boundary, nothing is printed, and there is no CPU fallback:
 * a call on a machine without a usable CUDA device returns F3M_ERR_CUDA.
 *
 * Unless stated otherwise, pointers are DEVICE pointers on the current CUDA device, arrays are
 * dense row-major float32, and `stream` is a cudaStream_t passed as void* (NULL = legacy default
 * stream).  Work is enqueued on that stream; the call returns after the stream has been
 * synchronised, because list sizes are read back on the host while the tree is built.
 *
 * Threading: calls that use one device must be serialised by the caller (one host thread at a time per
 * device, or an external lock).  The library reuses device blocks it has released as soon as later work is
 * enqueued on the same stream; a second host thread on another stream of the same device could be handed a
 * block that queued kernels still read.  A plan must not be used from two host threads at once.
 *
 * Each declaration names the interface of the reference implementation (MrHuff/F3M) that it
 * replaces, as path:line inside that repository.
 */
#ifndef F3M_H
#define F3M_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define F3M_MAX_DIM 5           /* dimensions 1..5 are built (reference table: 1..10, F3M_src/pybinder_setup.cu:17-36) */
#define F3M_MAX_LEVELS 24

enum f3m_status {
    F3M_OK = 0,
    F3M_ERR_ARG = 1,        /* bad pointer / size / dimension */
    F3M_ERR_CUDA = 2,       /* a CUDA runtime call or kernel launch failed; see f3m_last_error() */
    F3M_ERR_DEPTH = 3,      /* the tree would need more levels than a 30-bit cell index holds */
    F3M_ERR_OVERFLOW = 4,   /* a list or offset does not fit in 31 bits */
    F3M_ERR_UNSUPPORTED = 5,/* e.g. more interpolation nodes per dimension than the kernels hold */
    F3M_ERR_INTERNAL = 6,   /* a device-side consistency check failed */
    F3M_ERR_TOO_LARGE = 7   /* problem larger than a fixed-capacity entry point allows */
};

/* numeric flavour of the box index and of the far test */
#define F3M_MATH_FASTMATH 0 /* div.approx / sqrt.approx / fused multiply-add: the instructions the reference's
                               --use_fast_math build executes (F3M_src/setup.py:16) -- default */
#define F3M_MATH_IEEE 1     /* IEEE divide, sqrt, no contraction: what a CPU restatement computes */

/* Optional evaluation of the near field by box moments: when every pair of a near / small list has a provably
 * tiny exponent (boxes much smaller than the lengthscale), the sum over a source box is replaced by its 2nd/3rd
 * order Taylor moments (truncation error <= 1e-6 relative, the size of the ex2.approx error).  The pair lists do
 * not change.  Off by default: the default near field is the direct sum of the reference
 * (near_field_run, F3M_src/n_tree.cu:831-902). */
#define F3M_FLAG_NEAR_MOMENTS 1

/* Optional evaluation of the direct near sums on the tensor cores (one column, boxes at most half a scaled
 * lengthscale wide): the exponent matrix -|x_i - y_j|^2 / (2 l^2) of a 128-target x 256-source tile is a TF32
 * tcgen05 product of split (head + tail) operands, exact to FP32 rounding; the exponentials and the sum stay on
 * the CUDA cores.  Same sums as the default near field; no counterpart in the reference. */
#define F3M_FLAG_NEAR_TENSOR_CORES 2

/* Parameters of FFM_XY<float,d> (F3M_src/n_tree.cu:1056-1059) / FFM.__init__ (experiments/FFM_classes.py:9-19). */
typedef struct f3m_params {
    float ls;                 /* lengthscale l;  K = exp(-r^2/(2 l^2)) */
    float min_points;         /* refine while the largest box holds more points than this (n_tree.cu:1075,1099) */
    int32_t nr_interpolation; /* interpolation nodes per box, p^d */
    int32_t var_compression;  /* 0/1: extra far rules of boolean_separate_interactions_small_var_comp (1_d_conv.cu:955-1029) */
    float eff_var_limit;
    int32_t small_field_points;
    int32_t math_mode;        /* F3M_MATH_FASTMATH or F3M_MATH_IEEE */
    int32_t flags;            /* F3M_FLAG_* bits, 0 by default */
} f3m_params;

typedef struct f3m_plan f3m_plan;   /* tree + interaction lists of one (X, Y) pair; reusable for many b */

/* -------- library ------------------------------------------------------------------------- */
int f3m_version(void);
/* The library keeps the device blocks it has used on a free list and reuses them; this returns the
 * unused ones to the driver (call it between phases of very different sizes, or before another
 * framework needs the memory).  Must not run concurrently with other calls into the library. */
int f3m_release_cached_memory(void);
const char *f3m_status_string(int status);
/* Message of the last failing call made by this thread ("" if none). */
const char *f3m_last_error(void);

/* -------- the hot path ------------------------------------------------------------------- */

/* One complete product: replaces FFM_XY<float,d> (F3M_src/n_tree.cu:1056-1125), which
 * ffm_3d_float.FFM_XY_FLOAT_d binds (F3M_src/pybinder_setup.cu:17-36).
 * X (N,d), Y (M,d), b (M,R), out (N,R).  Pass Y == X (same pointer, and M == N) for the shared-tree
 * case; the reference detects it by the pointer alone (n_tree.cu:1072), here a Y that starts at X's address
 * with another row count (a leading slice of X) is an ordinary second point set.  out is overwritten. */
int f3m_kmvm_f32(const float *X, int64_t N, const float *Y, int64_t M, const float *b, int32_t R,
                 int32_t d, const f3m_params *prm, float *out, void *stream);

/* The same product with every temporary taken from memory the CALLER owns (the reference's FFM_XY allocates
 * through torch, n_tree.cu:1061 and throughout; a host that hands out memory from its own
 * allocator passes a slice of it here).  workspace: device memory of workspace_bytes bytes, free for the duration
 * of the call; nothing is requested from or returned to the driver inside the call, apart from a per-device slot of
 * 1 KB of flags and pinned read-back words that the library creates the first time a device is used.
 * f3m_workspace_bytes estimates the need for evenly spread points (sort buffers, tree, lists, packed sources,
 * moments); strongly clustered sets build deeper trees and need more.  A workspace that runs out ends the call
 * with F3M_ERR_TOO_LARGE and a message that names the request; f3m_last_workspace_peak returns the high-water
 * mark of this thread's last f3m_kmvm_ws_f32 call (bytes), for sizing after a trial run. */
size_t f3m_workspace_bytes(int64_t N, int64_t M, int32_t R, int32_t d, const f3m_params *prm);
int f3m_kmvm_ws_f32(const float *X, int64_t N, const float *Y, int64_t M, const float *b, int32_t R, int32_t d,
                    const f3m_params *prm, float *out, void *workspace, size_t workspace_bytes, void *stream);
size_t f3m_last_workspace_peak(void);

/* Same product with HOST buffers: copies X, Y, b to the device, runs f3m_kmvm_f32 and copies the
 * result back, all inside the call.  This is what a caller holding CPU tensors pays end to end
 * (FFM.__init__/__matmul__ move X, Y, b to the device, experiments/FFM_classes.py:23-50). */
int f3m_kmvm_host_f32(const float *X, int64_t N, const float *Y, int64_t M, const float *b, int32_t R,
                      int32_t d, const f3m_params *prm, float *out);

/* Split form: everything that does not depend on b (bounding cube, sort, box division,
 * interaction lists -- n_tree.cu:25-180, 594-811, 903-969) is done once ...                  */
int f3m_plan_create(f3m_plan **plan, const float *X, int64_t N, const float *Y, int64_t M, int32_t d,
                    const f3m_params *prm, void *stream);
/* ... and applied to any number of right-hand sides (far_field_compute_v2 n_tree.cu:489-593,
 * near_field_run n_tree.cu:831-902).  b (M,R), out (N,R) overwritten.
 * row_begin/row_end restrict the product to the target boxes whose sorted point range starts
 * inside [row_begin,row_end) (a slice of the sorted target order, used to shard target boxes
 * over GPUs); rows outside the slice are written as 0.  Use 0, N for the whole product. */
int f3m_plan_apply(f3m_plan *plan, const float *b, int32_t R, float *out, void *stream);
int f3m_plan_apply_range(f3m_plan *plan, const float *b, int32_t R, float *out, int64_t row_begin,
                         int64_t row_end, void *stream);
/* Sharing box moments between GPUs (no counterpart in the reference, whose multi-GPU mode is independent
 * processes: experiments/FFM_classes.py:128-211).  Every rank holds the same plan.  f3m_plan_moments_range
 * computes the finest-level moments of the source boxes that start inside [src_begin, src_end) of the sorted
 * order into mom_out (nfloats floats from f3m_plan_moments_size, zero for all other boxes); the caller sums the
 * arrays of all ranks (an all-reduce over NVLink) and passes the result to f3m_plan_apply_range_moments, which
 * then skips its own pass over the sources.  nfloats == 0 means this plan cannot exchange moments (node counts
 * change between levels, more than 8 nodes per dimension, or more than 8 columns): use f3m_plan_apply_range. */
int f3m_plan_moments_size(const f3m_plan *plan, int32_t R, int64_t *nfloats);
int f3m_plan_moments_range(f3m_plan *plan, const float *b, int32_t R, int64_t src_begin, int64_t src_end,
                           float *mom_out, void *stream);
int f3m_plan_apply_range_moments(f3m_plan *plan, const float *b, int32_t R, float *out, int64_t row_begin,
                                 int64_t row_end, const float *mom, void *stream);

/* A plan whose sort is shared by several GPUs (no counterpart in the reference).  Each rank sorts its own shard of
 * the points inside the GLOBAL bounding cube (origin = per-dimension minimum over all ranks, edge0 = 1.01f * largest
 * extent, both float32 as in calculate_edge_X, n_tree.cu:39-46) to the depth f3m_sort_depth gives for the TOTAL
 * point count.  The levels and interaction lists follow from the number of points per finest sorted cell alone, so
 * every rank builds them from the gathered cell counts (a few megabytes) while the sorted runs themselves (records of
 * f3m_record_words(d) 32-bit words per point: [input row, coordinates]) are still being all-gathered, and merges
 * the runs in afterwards.
 *   f3m_bounding_box_f32              per-dimension minimum and maximum of a shard (HOST arrays of d floats).
 *   f3m_sort_shard_f32                records_out (n records): the shard sorted; row_offset = input row of the
 *                                     shard's first point in the whole set; cell_counts_out: 2^(d depth) counts.
 *   f3m_plan_create_from_cell_counts  cell_counts: (nruns, 2^(d depth)) device array, row r = counts of run r.  The plan
 *                                     is that of f3m_plan_create on the whole set with Y = X, except for the order of
 *                                     the points inside a finest sorted cell (run by run).  If the level loop needs
 *                                     more levels than `depth` (strongly clustered points): F3M_ERR_UNSUPPORTED --
 *                                     build the plan from the gathered points instead.
 *   f3m_plan_attach_runs              records: the gathered runs, run r at record r * run_stride.  Products can be
 *                                     computed after this call. */
int f3m_sort_depth(int64_t n_total, int32_t d, float min_points);
int f3m_record_words(int32_t d);
int f3m_bounding_box_f32(const float *X, int64_t n, int32_t d, float *min_out, float *max_out, void *stream);
int f3m_sort_shard_f32(const float *X, int64_t n, int64_t row_offset, int32_t d, const float *origin, float edge0,
                       int32_t math_mode, int32_t depth, void *records_out, int32_t *cell_counts_out, void *stream);
int f3m_plan_create_from_cell_counts(f3m_plan **plan, const int32_t *cell_counts, int32_t nruns, int32_t d, const float *origin,
                                     float edge0, int32_t depth, const f3m_params *prm, void *stream);
int f3m_plan_attach_runs(f3m_plan *plan, const void *records, int64_t run_stride, void *stream);

/* One product shared by several GPUs in phases, so that the exchange of the moments over NVLink runs while the
 * direct sums are computed (no counterpart in the reference: par_FFM_block runs independent block products,
 * experiments/FFM_classes.py:128-211).  Every rank holds the same plan (built from all points) and owns one slice
 * [row_begin, row_end) of the SORTED target rows; slices are cut at finest-level box starts.
 *
 *   f3m_plan_partition_rows  cuts the sorted rows into nparts slices of equal estimated work (direct pairs, far
 *                            pairs, finest-level interpolation); bounds is a HOST array of nparts + 1 entries.
 *   f3m_plan_shard_begin     marks the source boxes the slice's direct lists name, brings the rows of b of those
 *                            boxes and of the source boxes [box_begin, box_end) into sorted order, and writes the
 *                            finest-level moments of the boxes [box_begin, box_end) to mom_slice
 *                            ((box_end - box_begin) * nfloats / boxes floats, nfloats from f3m_plan_moments_size).
 *                            mom_slice == NULL or nfloats == 0: no exchange, the rank reads all sources itself.
 *   (the caller gathers the moment slices of all ranks into one array, boxes in order)
 *   f3m_plan_shard_near      direct sums of the slice into acc_sorted (N x R, sorted row order; only the rows of
 *                            the slice are written, and they are overwritten).
 *   f3m_plan_shard_far       adds the far field of the slice, taking the finest-level moments from mom (all boxes).
 *   f3m_plan_shard_end       releases what the phases kept in the plan.
 *   f3m_plan_rows_to_input_order  out[(r - in_lo)] = acc_sorted[position of input row r] for in_lo <= r < in_hi:
 *                            the rows of the (gathered) sorted result that belong to one range of input rows.
 *   f3m_plan_gathered_rows_to_input_order  the same from the buffer an all-gather of the ranks' slices leaves: slice g
 *                            (sorted rows slice_bounds[g] .. slice_bounds[g+1], HOST array) starts at row g * stride.
 *   f3m_plan_count_rows_by_owner / f3m_plan_pack_rows_by_owner / f3m_plan_place_rows   the same without gathering
 *                            the whole result: rank g owns the input rows [in_bounds[g], in_bounds[g+1]) (HOST array of
 *                            nranks + 1 cuts).  count: how many rows of the slice [row_begin, row_end) belong to each
 *                            rank (HOST array counts).  pack: those rows as records of R + 1 floats [values, input row
 *                            as an integer's bits], grouped by owner in rank order -- the send buffer of an
 *                            all-to-all.  place: received records into out[(input row - in_lo)].
 * A plan runs one sharded product at a time and must not be used from two host threads at once. */
int f3m_plan_partition_rows(f3m_plan *plan, int32_t R, int32_t nparts, int64_t *bounds, void *stream);
int f3m_plan_shard_begin(f3m_plan *plan, const float *b, int32_t R, int64_t row_begin, int64_t row_end, int64_t box_begin,
                         int64_t box_end, float *mom_slice, void *stream);
int f3m_plan_shard_near(f3m_plan *plan, float *acc_sorted, void *stream);
int f3m_plan_shard_far(f3m_plan *plan, const float *mom, float *acc_sorted, void *stream);
int f3m_plan_shard_end(f3m_plan *plan);
int f3m_plan_rows_to_input_order(const f3m_plan *plan, const float *acc_sorted, int32_t R, int64_t in_lo, int64_t in_hi,
                                 float *out, void *stream);
int f3m_plan_gathered_rows_to_input_order(const f3m_plan *plan, const float *gathered, int32_t R, const int64_t *slice_bounds,
                                          int32_t nslices, int64_t stride, int64_t in_lo, int64_t in_hi, float *out, void *stream);
int f3m_plan_count_rows_by_owner(const f3m_plan *plan, int64_t row_begin, int64_t row_end, const int64_t *in_bounds,
                                 int32_t nranks, int64_t *counts, void *stream);
int f3m_plan_pack_rows_by_owner(const f3m_plan *plan, const float *acc_sorted, int32_t R, int64_t row_begin, int64_t row_end,
                                const int64_t *in_bounds, int32_t nranks, const int64_t *counts, float *send, void *stream);
int f3m_plan_place_rows(f3m_plan *plan, const float *records, int64_t n, int32_t R, int64_t in_lo, int64_t in_hi, float *out,
                        void *stream);
int f3m_plan_destroy(f3m_plan *plan);

/* -------- introspection (parity checks and work accounting) ------------------------------ */

typedef struct f3m_level_info {
    int32_t level;        /* 1-based depth */
    int32_t boxes_x;      /* occupied target boxes */
    int32_t boxes_y;      /* occupied source boxes */
    int32_t max_count_x, max_count_y;
    int64_t n_far, n_small, n_keep; /* pairs per class at this level (separate_interactions n_tree.cu:701-787) */
    float edge;           /* box edge at this level */
    int32_t nodes_per_dim;/* p used at this level */
} f3m_level_info;

typedef struct f3m_plan_stats {
    int32_t levels;            /* levels built */
    int32_t shared_tree;       /* 1 if X is Y */
    int64_t direct_pairs;      /* sum over small + final-near box pairs of n_x*n_y */
    int64_t node_pairs;        /* sum over far box pairs of P^2 (the reference's M2L work) */
    int64_t far_box_pairs;
    int64_t near_box_pairs;    /* small + final near */
    float edge0;               /* cube edge */
    float build_ms;            /* device time of f3m_plan_create */
} f3m_plan_stats;

int f3m_plan_get_stats(const f3m_plan *plan, f3m_plan_stats *stats);
int f3m_plan_get_level(const f3m_plan *plan, int32_t level, f3m_level_info *info);

/* Copy one array of the plan into a HOST buffer the caller sized from f3m_plan_get_level.
 * tree: 0 = target (X) tree, 1 = source (Y) tree.  `what`:                                  */
#define F3M_ARR_SORTED_INDEX 0  /* int32 (n)        sorted position -> input row    (n_tree.cu:59 sorted_index) */
#define F3M_ARR_BOX_OFFSETS 1   /* int32 (boxes+1)  per level                       (n_tree.cu:70 unique_counts_cum_reindexed) */
#define F3M_ARR_BOX_CENTERS 2   /* float (boxes,d)  per level                       (n_tree.cu:65 centers) */
#define F3M_ARR_FAR_PTR 3       /* int32 (boxes_x+1) CSR row pointers of the far list of the level */
#define F3M_ARR_FAR_IDX 4       /* int32 (n_far)     source box of every far pair, grouped by target box */
#define F3M_ARR_SMALL_PTR 5
#define F3M_ARR_SMALL_IDX 6
#define F3M_ARR_KEEP_PTR 7      /* pairs handed to the next level; at the last level: the final near list */
#define F3M_ARR_KEEP_IDX 8
#define F3M_ARR_BOX_CODES 9     /* uint32 (boxes) Morton prefix of every box */
int f3m_plan_copy_array(const f3m_plan *plan, int32_t level, int32_t tree, int32_t what, void *host_dst,
                        size_t dst_bytes);

/* -------- exact dense op ------------------------------------------------------------------ */

/* out[i] = sum_j exp(-|x_i-y_j|^2/(2 ls^2)) b_j : replaces rbf_call<float,d> / rbf_call<double,d>
 * (F3M_src/n_tree.cu:185-211; rbf_float_d / rbf_double_d, pybinder_setup.cu:40-62).  The f64 entry
 * uses a double-precision exponential (the reference evaluates expf even for double, 1_d_conv.cu:72). */
int f3m_rbf_dense_f32(const float *X, int64_t N, const float *Y, int64_t M, const float *b, int32_t R,
                      int32_t d, float ls, float *out, void *stream);
int f3m_rbf_dense_f64(const double *X, int64_t N, const double *Y, int64_t M, const double *b, int32_t R,
                      int32_t d, double ls, double *out, void *stream);
/* out[i] = ls^-3 sum_j r_ij^2 exp(-r_ij^2/(2 ls^2)) b_j : replaces rbf_call_grad<float,d>
 * (n_tree.cu:213-241; rbf_float_d_grad, pybinder_setup.cu:64-73). */
int f3m_rbf_dense_grad_f32(const float *X, int64_t N, const float *Y, int64_t M, const float *b, int32_t R,
                           int32_t d, float ls, float *out, void *stream);

/* The same product as f3m_rbf_dense_f32 for hosts that must not allocate device memory while they run
 * (all memory pre-reserved by the host's own pool, or a no-allocation-after-start-up rule because an
 * allocation can stall the device).  It has no counterpart in the reference.  Its scratch -- the packed
 * source rows -- lives in a fixed 16 MiB array inside the library image (F3M_STATIC_SCRATCH_FLOATS floats,
 * held by every GPU that loads the library), so it calls no cudaMalloc, cudaFree or pool routine.
 * Limit: M * w <= F3M_STATIC_SCRATCH_FLOATS with w = 4 floats per source for d <= 3 and one column
 * (in general d + min(R,4) rounded up to a multiple of 4); larger inputs return F3M_ERR_TOO_LARGE.
 * The first call on a device looks up the array's device address; make it before any stream capture.
 * Calls share the array: calls that overlap on the GPU (other streams or host threads) race. */
#define F3M_STATIC_SCRATCH_FLOATS (4 * 1024 * 1024)
int f3m_rbf_dense_f32_static(const float *X, int64_t N, const float *Y, int64_t M, const float *b, int32_t R,
                             int32_t d, float ls, float *out, void *stream);

/* -------- measurement helpers -------------------------------------------------------------- */

/* Measures the SM's exponential (MUFU.EX2) and FP32 FMA issue peaks with two register-only
 * kernels: results in giga-operations per second for the whole device. */
int f3m_measure_peaks(double *gexp_per_s, double *gfma_per_s, void *stream);
/* Device time (ms) of the stages of the last f3m_plan_apply: [0]=sort/permute of b, [1]=small+near
 * direct sums, [2]=P2M, [3]=M2L, [4]=L2P, [5]=output un-permute, [6]=total, [7]=f3m_plan_create of this plan. */
int f3m_plan_last_timings(const f3m_plan *plan, float ms[8]);
/* Number of direct-sum kernel launches inside the last f3m_plan_apply, and kernels launched by the
 * library since it was loaded (all entry points). */
int f3m_plan_last_direct_launches(const f3m_plan *plan);
/* Which form of the direct-sum kernel those launches took (the host picks it per list from a bound on the
 * exponent, see near_field_run n_tree.cu:831-902 for the sums themselves): counts[0] expanded form with every
 * exponential on the special-function unit, [1] expanded form with 2/5 of the pairs on a degree-2 polynomial,
 * [2] with 1/3 on a degree-3 polynomial, [3] direct form (differences, wide boxes), [4] moment form
 * (F3M_FLAG_NEAR_MOMENTS), [5] tensor-core form (F3M_FLAG_NEAR_TENSOR_CORES). */
int f3m_plan_last_direct_variants(const f3m_plan *plan, int32_t counts[6]);
long long f3m_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* F3M_H */
