/*
 * C ABI of libpointelligence_b200.so -- the sm_100a implementation of the
 * point-convolution hot path (sparse engines + geometry stage).
 *
 * Conventions
 *   - every pointer argument named d_* is a DEVICE pointer on the current
 *     CUDA device; h_* is a HOST pointer.  Nothing is retained after a call.
 *   - the library allocates no device memory: outputs and scratch ("workspace")
 *     are owned by the caller; each *_workspace_bytes() function returns the
 *     scratch size the matching call needs.  Workspaces must be 256-byte
 *     aligned.
 *   - all work is enqueued on `stream` (a cudaStream_t passed as void*).
 *     Calls that have to return a data-dependent count to the host
 *     (pcx_radius_count, pcx_radius_taps_fill, pcx_grid_sample_count) synchronise
 *     that stream once.
 *   - every function returns PCX_OK (0) or a negative pcx_status; it never
 *     throws and never terminates the process.  pcx_last_error_string() gives
 *     the message of the last failure on the calling thread.
 *   - feature rows are dense row-major; indices are int32; tap segment
 *     offsets are int64 (K+1 entries, seg[K] == T).
 *
 * Each entry point cites the reference interface it stands in for (paths are
 * relative to the reference project's root).
 */
#ifndef POINTELLIGENCE_B200_H
#define POINTELLIGENCE_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
    PCX_OK = 0,
    PCX_E_ARG = -1,         /* null pointer, negative size, bad enum          */
    PCX_E_DTYPE = -2,       /* unsupported element type                        */
    PCX_E_ALIGN = -3,       /* pointer / leading dimension not aligned         */
    PCX_E_CAPACITY = -4,    /* workspace or output buffer too small            */
    PCX_E_LAUNCH = -5,      /* CUDA runtime reported an error                  */
    PCX_E_UNSUPPORTED = -6, /* shape outside what this build implements        */
    PCX_E_DEVICE = -7       /* a kernel reported a bounded wait that ran out   */
} pcx_status;

typedef enum { PCX_F32 = 0, PCX_F16 = 1, PCX_BF16 = 2 } pcx_dtype;

/* engine selector for the sparse primitives */
typedef enum {
    PCX_ENGINE_AUTO = 0,    /* tcgen05 tensor-core path when the shape allows  */
    PCX_ENGINE_CUDA_CORE = 1, /* fp32 FMA path (any shape, IEEE fp32)          */
    PCX_ENGINE_TENSOR = 2   /* tcgen05 path or PCX_E_UNSUPPORTED               */
} pcx_engine;

/* May be OR-ed into the `engine` argument of pcx_mvmr: the caller guarantees that
 * every output row occurs in exactly one triplet (T == n_out; the fan-in-1
 * contract of a subdivision rulebook in the forward direction, or of a grid
 * partition in the input-gradient direction: layers/contract.py:27-64
 * exact_cover_out / exact_cover_in, engines of sparse_engines/tig.py:227-291).
 * The tensor engine then stores each rounded row itself: no accumulator is
 * cleared, nothing is reduced, no rounding pass follows.  Other engines ignore
 * the flag.  A rulebook that breaks the guarantee gives an unspecified result
 * in the rows concerned (no fault). */
#define PCX_ENGINE_FLAG_FAN_IN_ONE 0x100

int pcx_version(void);
const char *pcx_last_error_string(void);

/* Device-side status word: kernels that give up on a bounded wait set a bit
 * (1 = MVMR tensor kernel, 2 = VVOR tensor kernel, 4 = output-stationary MVMR
 * kernel, 8 = pcx_debug_wait_runs_out).  Synchronises `stream`,
 * copies the word to *h_status and clears it when `clear` is non-zero.
 * No counterpart in the reference (its kernels have no device-side waits). */
int pcx_device_status(unsigned int *h_status, int clear, void *stream);

/* Measurement hooks (no counterpart in the reference, whose benchmarks time
 * from Python).  pcx_launch_count: kernels this library has launched (reset
 * when `reset` is non-zero).  pcx_profile_enable(1) makes every sparse entry
 * point bracket its dominant kernel with CUDA events on the launch stream;
 * pcx_profile_get returns the kernel's label and duration of record `index`
 * (it waits for that record's stop event); pcx_profile_enable(0) stops. */
long long pcx_launch_count(int reset);
int pcx_profile_enable(int on);
int pcx_profile_count(void);
int pcx_profile_get(int index, const char **name, float *milliseconds);

/* ------------------------------------------------------------------------
 * MVMR:  out[scatter[t], g, :] += feat[gather[t], g, :] @ W[tap(t), g]
 *
 * Replaces sparse_engines/tig.py:1090-1206 (tig_forward), :1220-1309
 * (tig_grad_input) and the public operator sparse_engines/mvmr_triton.py:148-254
 * (extensions/sparse_engines_cuda/csrc/definitions.cpp:24 on the native side).
 *
 *   d_weight   (K, G, C, M) elements of `dtype`
 *   transpose  0: feat rows have C channels, out rows M   (forward)
 *              1: feat rows have M channels, out rows C, W used transposed
 *                 (input gradient; same triplets with gather/scatter swapped)
 *   d_feat     (n_feat, G*in_width)   d_out (n_out, G*out_width), `dtype`
 *   d_gather / d_scatter  (T) int32 row indices into feat / out
 *   d_seg_offs (K+1) int64 tap segment offsets of tap-sorted triplets, or NULL
 *   d_tap_idx  (T) int32 tap per triplet; required when d_seg_offs is NULL
 *              (then any order is accepted), ignored otherwise
 *   d_ws       workspace of pcx_mvmr_workspace_bytes(); holds the fp32
 *              accumulator that is rounded once into d_out
 * Rows of out that no triplet touches are written as zero.
 */
size_t pcx_mvmr_workspace_bytes(int64_t n_out, int K, int G, int C, int M,
                                int transpose, int dtype);
int pcx_mvmr(const void *d_weight, const void *d_feat, const int32_t *d_gather,
             const int32_t *d_scatter, const int64_t *d_seg_offs,
             const int32_t *d_tap_idx, void *d_out, int64_t T, int64_t n_feat,
             int64_t n_out, int K, int G, int C, int M, int transpose,
             int dtype, int engine, void *d_ws, size_t ws_bytes, void *stream);

/* ------------------------------------------------------------------------
 * Output-stationary MVMR: same result as pcx_mvmr (fp16 / bf16, one group,
 * tap-sorted triplets), computed from a "plan" of the rulebook.
 *
 * Replaces the same reference code as pcx_mvmr and, for the regrouping of the
 * rulebook by output row with its (row, tap) buckets summed before the
 * contraction, sparse_engines/fused_point_conv.py:344-423 (kernel) and
 * :785-870 (rulebook preparation).
 *
 * pcx_mvmr_plan_build regroups the triplets (scatter, gather, tap) by blocks
 * of 128 output rows, the rows ordered by the set of taps that touch them.  A
 * plan depends on the index arrays only: build it once per rulebook and
 * direction (forward: scatter = output index, gather = input index; input
 * gradient: the two swapped) and use it for every layer and step that shares
 * the rulebook.  pcx_mvmr_planned then keeps the fp32 sums of every block in
 * tensor memory across all taps and writes each output row once: no
 * workspace, no zero-fill, no atomics, bit-reproducible.  Rows that no
 * triplet touches are written as zero.
 *
 *   group_blocks  blocks that share the weight tiles they stream;
 *                 pcx_mvmr_plan_group_blocks(out_width) gives the value to use
 *                 for an output row of out_width channels.  The same value
 *                 must be passed to both calls (a plan built for one value is
 *                 not valid for another).
 *   d_plan        caller-owned, 256-byte aligned, pcx_mvmr_plan_bytes();
 *                 pcx_mvmr_planned updates a work counter inside it, so two
 *                 launches that use the same plan must not overlap on the GPU
 *   limits        K <= 512, channel counts multiples of 16, out_width <= 256,
 *                 T < 2^31, ceil(n_out / 128) * K * 128 <= 2^32
 * The feature rows of a (row, tap) bucket with several triplets are summed
 * first (fp32 sum, one rounding to the feature type) into the workspace, by a
 * small kernel in front of the main one: pcx_mvmr_plan_multi_buckets reads the
 * number of such buckets back from a built plan (it synchronises `stream`),
 * pcx_mvmr_planned_workspace_bytes gives the workspace size for it.
 */
int pcx_mvmr_plan_group_blocks(int out_width);
size_t pcx_mvmr_plan_bytes(int64_t T, int64_t n_out, int K, int group_blocks);
size_t pcx_mvmr_plan_workspace_bytes(int64_t T, int64_t n_out, int K,
                                     int group_blocks);
int pcx_mvmr_plan_build(const int32_t *d_scatter, const int32_t *d_gather,
                        const int64_t *d_seg_offs, int64_t T, int K,
                        int64_t n_out, int group_blocks, void *d_plan,
                        size_t plan_bytes, void *d_ws, size_t ws_bytes,
                        void *stream);
int pcx_mvmr_plan_multi_buckets(const void *d_plan, int64_t *h_count,
                                void *stream);
size_t pcx_mvmr_planned_workspace_bytes(int64_t multi_buckets, int in_width);
int pcx_mvmr_planned(const void *d_weight, const void *d_feat, void *d_plan,
                     size_t plan_bytes, void *d_out, int64_t T, int64_t n_feat,
                     int64_t n_out, int K, int C, int M, int transpose,
                     int dtype, int group_blocks, int64_t multi_buckets,
                     void *d_ws, size_t ws_bytes, void *stream);

/* Launches one thread that waits on a barrier nothing arrives at: the bounded
 * wait gives up after limit_ns (at most 100 ms), sets bit 8 of the device
 * status word and the kernel returns.  For tests of the status path; no
 * counterpart in the reference. */
int pcx_debug_wait_runs_out(unsigned long long limit_ns, void *stream);

/* ------------------------------------------------------------------------
 * VVOR:  out[o[t], g, m, c] += a[ai[t], g, m] * b[bi[t], g, c]
 *
 * Replaces sparse_engines/tig.py:1390-1465 (tig_grad_weight, with a = input
 * features, b = output gradient, o = tap -> dW (K,G,C_in,C_out)) and the
 * public operator sparse_engines/vvor_triton.py:116-223
 * (definitions.cpp:25 on the native side).
 *
 *   d_a (n_a, G*Ma)  d_b (n_b, G*Cb)  d_out (n_o, G, Ma, Cb), all `dtype`
 *   d_seg_offs (n_o+1) int64 when the triplets are sorted by o, else NULL and
 *   d_o_idx (T) int32 gives o per triplet.
 */
size_t pcx_vvor_workspace_bytes(int64_t n_o, int G, int Ma, int Cb, int dtype);
int pcx_vvor(const void *d_a, const int32_t *d_a_idx, const void *d_b,
             const int32_t *d_b_idx, const int64_t *d_seg_offs,
             const int32_t *d_o_idx, void *d_out, int64_t T, int64_t n_a,
             int64_t n_b, int64_t n_o, int G, int Ma, int Cb, int dtype,
             int engine, void *d_ws, size_t ws_bytes, void *stream);

/* ------------------------------------------------------------------------
 * VVOR without a workspace.  No counterpart in the reference.
 *
 * Same result as pcx_vvor for triplets sorted by output row (d_seg_offs is
 * required), but the scratch lives in a fixed __device__ array inside the
 * library (about 8 MiB per GPU that loads it), so the call allocates nothing
 * and needs no caller-owned workspace.  For hosts that cannot allocate device
 * memory where the gradient is needed (allocator callbacks, no-cudaMalloc
 * regions, plugins that only own the tensors they were handed).
 * Limits: n_o <= 4095 and n_o*G*Ma*Cb <= pcx_vvor_static_scratch_max_elements()
 * (2^21); larger shapes return PCX_E_CAPACITY.  The first call with a given
 * device current looks the array's address up (do it before any stream
 * capture).  All calls share the array: calls that overlap on the GPU race.
 */
size_t pcx_vvor_static_scratch_max_elements(void);
int pcx_vvor_static_scratch(const void *d_a, const int32_t *d_a_idx, const void *d_b,
                            const int32_t *d_b_idx, const int64_t *d_seg_offs,
                            void *d_out, int64_t T, int64_t n_a, int64_t n_b,
                            int64_t n_o, int G, int Ma, int Cb, int dtype,
                            void *stream);

/* ------------------------------------------------------------------------
 * Residual R-net selector of the full-cover strided rulebook.
 *
 * Replaces layers/triplets.py:156-232 (_select_residual_full_cover_centers
 * with its _rank_priorities): among the n points that no initial centre
 * covers, choose centres in rounds -- a point whose priority (most active
 * neighbours, then farthest from its stride cell's initial centre, then lowest
 * source index) is the best of its active neighbourhood becomes a centre and
 * retires that neighbourhood -- until no point is active.
 *
 *   pcx_rnet_far     d_far[v] = |points[v] - centres[centre_of[v]]|^2, one
 *                    rounding per operation ((dx^2 + dy^2) + dz^2)
 *   pcx_rnet_rounds  runs `rounds` (1..64) rounds on the lists d_neighbors /
 *                    d_offsets (query-major neighbours within R, self
 *                    included; offsets n+1), updating d_active (1 = still to be
 *                    covered; all ones before the first call) and setting
 *                    d_chosen[v] = 1 for new centres (zeroed by the caller).
 *                    h_remaining[r] = active points after round r; the call
 *                    synchronises the stream once to hand these back.  Rounds
 *                    on an exhausted set change nothing.
 */
size_t pcx_rnet_workspace_bytes(int64_t n, int rounds);
int pcx_rnet_far(const float *d_points, const float *d_centres,
                 const int64_t *d_centre_of, int64_t n, float *d_far,
                 void *stream);
int pcx_rnet_rounds(const int64_t *d_neighbors, const int64_t *d_offsets,
                    const float *d_far, const int64_t *d_source, int64_t n,
                    int rounds, uint8_t *d_active, uint8_t *d_chosen,
                    int32_t *h_remaining, void *d_ws, size_t ws_bytes,
                    void *stream);

/* ------------------------------------------------------------------------
 * Segment reductions (op: 0 sum, 1 mean, 2 max, 3 min; fp32 accumulation,
 * inputs, outputs and gradients all in `dtype`).
 *
 * pcx_segment_reduce: out[s] = reduce of the rows of segment s, segments being
 * consecutive runs of d_lengths[s] rows of x (N, C).  Replaces
 * large_segment_reduce (sparse_engines/large_segment_reduce_triton.py:25-77,
 * :180-188): empty segments give 0 (sum, mean) or -inf / +inf (max / min),
 * fp16 results are clamped to +-65504.  _backward replaces :94-166: the
 * gradient is broadcast (divided by max(len,1) for mean) or, for max / min,
 * given to every element equal to the reduced value; d_x and d_out are only
 * read for max / min.
 *
 * pcx_indexed_segment_reduce: y[k] = reduce over the d_lengths[k] consecutive
 * entries e of list k of x[d_indices[e]].  Replaces indexed_segment_reduce
 * (sparse_engines/indexed_segment_reduce_triton.py:25-63, :147-173): an empty
 * list gives 0 (sum), NaN (mean) or -inf / +inf.  _backward replaces :84-140
 * (scatter-add of the gradient; value match for max / min).
 */
size_t pcx_segment_reduce_workspace_bytes(int64_t S, int C);
int pcx_segment_reduce(const void *d_x, const int64_t *d_lengths, void *d_out,
                       int64_t N, int64_t S, int C, int op, int dtype,
                       void *d_ws, size_t ws_bytes, void *stream);
int pcx_segment_reduce_backward(const void *d_grad_out, const void *d_x,
                                const void *d_out, const int64_t *d_lengths,
                                void *d_grad_x, int64_t N, int64_t S, int C,
                                int op, int dtype, void *d_ws, size_t ws_bytes,
                                void *stream);
size_t pcx_indexed_segment_reduce_workspace_bytes(int64_t K, int64_t n_x, int C,
                                                  int dtype, int backward);
int pcx_indexed_segment_reduce(const void *d_x, const int32_t *d_indices,
                               const int64_t *d_lengths, void *d_y, int64_t n_x,
                               int64_t E, int64_t K, int C, int op, int dtype,
                               void *d_ws, size_t ws_bytes, void *stream);
int pcx_indexed_segment_reduce_backward(const void *d_grad_y, const void *d_x,
                                        const void *d_y, const int32_t *d_indices,
                                        const int64_t *d_lengths, void *d_grad_x,
                                        int64_t n_x, int64_t E, int64_t K, int C,
                                        int op, int dtype, void *d_ws,
                                        size_t ws_bytes, void *stream);

/* ------------------------------------------------------------------------
 * Fused layer normalisation over a ragged batch (samples = consecutive runs of
 * d_lengths[s] rows), with the residual add and the ReLU of a residual block:
 *   y = relu?((x - mean_s) * rstd_s * weight + bias (+ residual))
 * mean_s / rstd_s over all rows x channels of sample s, two-pass, as
 * RaggedLayerNorm composes them (layers/norm.py:59-83, :118-130 of the
 * reference, which runs it as a chain of torch reductions and elementwise
 * launches).  d_weight / d_bias (fp32, C) may both be null (no affine);
 * d_residual may be null.  d_mean / d_rstd (fp32, S) are outputs kept for the
 * backward.  _backward: d_y is read only when relu != 0; d_grad_weight /
 * d_grad_bias (fp32, C) and d_grad_residual may be null.
 */
size_t pcx_ragged_layer_norm_workspace_bytes(int64_t N, int64_t S);
int pcx_ragged_layer_norm(const void *d_x, const int64_t *d_lengths,
                          const float *d_weight, const float *d_bias,
                          const void *d_residual, void *d_y, float *d_mean,
                          float *d_rstd, int64_t N, int64_t S, int C, double eps,
                          int relu, int dtype, void *d_ws, size_t ws_bytes,
                          void *stream);
int pcx_ragged_layer_norm_backward(const void *d_grad_y, const void *d_x,
                                   const void *d_y, const int64_t *d_lengths,
                                   const float *d_weight, const float *d_mean,
                                   const float *d_rstd, void *d_grad_x,
                                   float *d_grad_weight, float *d_grad_bias,
                                   void *d_grad_residual, int64_t N, int64_t S,
                                   int C, int relu, int dtype, void *d_ws,
                                   size_t ws_bytes, void *stream);

/* Group and instance normalisation over a ragged batch:
 *   y = (x - mean_{s,g}) * rstd_{s,g} * weight + bias
 * with the statistics over the rows of sample s and the W = C / G consecutive
 * channels of group g (instance norm: G = C), two-pass, as RaggedGroupNorm /
 * RaggedInstanceNorm compose them (layers/norm.py:86-116 of the reference).
 * d_mean / d_rstd (fp32, S * G, index s * G + g) are outputs kept for the
 * backward; d_weight / d_bias (fp32, C) may both be null; workspace of
 * pcx_ragged_group_norm_workspace_bytes(S, G).  G <= 8192 (4096 backward). */
size_t pcx_ragged_group_norm_workspace_bytes(int64_t S, int G);
int pcx_ragged_group_norm(const void *d_x, const int64_t *d_lengths,
                          const float *d_weight, const float *d_bias, void *d_y,
                          float *d_mean, float *d_rstd, int64_t N, int64_t S, int C,
                          int G, double eps, int dtype, void *d_ws, size_t ws_bytes,
                          void *stream);
int pcx_ragged_group_norm_backward(const void *d_grad_y, const void *d_x,
                                   const int64_t *d_lengths, const float *d_weight,
                                   const float *d_mean, const float *d_rstd,
                                   void *d_grad_x, float *d_grad_weight,
                                   float *d_grad_bias, int64_t N, int64_t S, int C,
                                   int G, int dtype, void *d_ws, size_t ws_bytes,
                                   void *stream);

/* ------------------------------------------------------------------------
 * Tap bookkeeping.
 * pcx_seg_offs: seg[k] = first position with value >= k in a sorted int32
 *   array (sparse_engines/_seg_offs.py:21-44, kernel_offset_segments).
 * pcx_expand_taps: k[t] = tap of position t, from segment offsets
 *   (layers/triplets.py:673-676, the repeat_interleave that materialises k).
 */
int pcx_seg_offs(const int32_t *d_sorted, int64_t T, int K, int64_t *d_seg_offs,
                 void *stream);
int pcx_expand_taps(const int64_t *d_seg_offs, int K, int64_t T, int32_t *d_k,
                    void *stream);

/* ------------------------------------------------------------------------
 * Exact fixed-radius search on a sorted grid of cell side 2R, optionally
 * emitting the accepted pairs grouped by kernel tap.
 *
 * Replaces internals/neighbors.py:469-838 (radius_search_strided_grid in
 * "exact8" mode; entry points radius_search_sorted_grid8 :886-916 and
 * radius_search_sorted_grid8_segments :919-955) together with the kernels of
 * sparse_engines/strided_grid_radius_triton_kernel.py:35-248.
 *
 * Two calls bracket the one device-to-host hand-over of the edge count:
 *
 *   pcx_radius_count  builds the sorted grid, evaluates the predicate for
 *       every (query, candidate) pair and returns the number of accepted
 *       pairs in *h_total.  d_num_neighbors (Q) int64 is final after this.
 *       With kernel_size > 0 it also writes d_seg_offs (kernel_size^3+1).
 *   pcx_radius_fill   writes the pairs.  kernel_size == 0: d_neighbors (E)
 *       int64 query-major (+ d_distances (E) fp32 when not NULL).
 *       kernel_size > 0: d_out_i / d_out_j (E) int32 grouped by tap, inside a
 *       tap ordered by query; d_out_k (E) int32 optional.
 *
 *   d_points (P,3) / d_queries (Q,3) fp32; d_point_sample / d_query_sample
 *   int32 sample id per row or both NULL; distance_type 0 = ball, 1 = Chebyshev.
 *   d_ws must stay untouched between the two calls (workspace of
 *   pcx_radius_workspace_bytes); d_ws2 is the fill-only scratch of
 *   pcx_radius_fill_workspace_bytes(total).
 */
/* fp32 arithmetic of the radius predicate: 0 = every operation rounded (the
 * expression of sparse_engines/strided_grid_radius_triton_kernel.py:25-31 as
 * written), 1 = sum of squares contracted into FMAs (what that expression
 * compiles to on a B200; the default), 2 = 1 with the approximate square root.
 * Process-wide; only pairs within an ulp or two of the radius are affected. */
int pcx_set_radius_predicate(int variant);
int pcx_get_radius_predicate(void);
size_t pcx_radius_workspace_bytes(int64_t P, int64_t Q, int kernel_size);
size_t pcx_radius_fill_workspace_bytes(int64_t total, int kernel_size);
int pcx_radius_count(const float *d_points, const float *d_queries,
                     const int32_t *d_point_sample, const int32_t *d_query_sample,
                     int64_t P, int64_t Q, double radius, int distance_type,
                     int kernel_size, double kernel_grid_size,
                     int64_t *d_num_neighbors, int64_t *d_seg_offs,
                     int64_t *h_total, void *d_ws, size_t ws_bytes, void *stream);
int pcx_radius_fill(const float *d_points, const float *d_queries, int64_t P,
                    int64_t Q, double radius, int distance_type, int kernel_size,
                    double kernel_grid_size, int64_t total, int64_t *d_neighbors,
                    float *d_distances, int32_t *d_out_i, int32_t *d_out_j,
                    int32_t *d_out_k, void *d_ws, size_t ws_bytes, void *d_ws2,
                    size_t ws2_bytes, void *stream);

/* The tap-segmented search (kernel_size 3 or 5) in one enqueue and ONE host
 * hand-over; same outputs, bit for bit, as pcx_radius_count + pcx_radius_fill
 * with kernel_size > 0 (same reference interface: internals/neighbors.py:919-955
 * followed by the stable sort by tap of layers/triplets.py:431-520).
 *
 *   pcx_radius_taps_count  enqueues the binning, the count pass and the tap
 *       segment offsets (d_num_neighbors (Q) int64, d_seg_offs (k^3+1) int64)
 *       and returns without synchronising.
 *   pcx_radius_taps_total  (optional) hands the number of pairs to the host
 *       (one synchronisation) for a caller that has no capacity estimate.
 *   pcx_radius_taps_fill   writes d_out_i / d_out_j (/ d_out_k when not NULL),
 *       buffers of `capacity` int32 each, synchronises once and returns the
 *       number of pairs in *h_total.  When the pairs do not fit it writes
 *       nothing and returns PCX_E_CAPACITY with *h_total set: call it again
 *       with buffers of that size (the state is kept in d_ws, which must stay
 *       untouched between the calls).
 *   h_total points at THREE int64: [0] the number of pairs, [1] the number of
 *   queries that have no neighbour (the reference asserts there is none,
 *   layers/triplets.py:431-520; the count saves the caller a pass and a
 *   hand-over of its own), [2] the device status word of pcx_device_status as
 *   it stood at this hand-over (not cleared).
 *   pcx_radius_taps_supported  1 when kernel_size is served by this path. */
int pcx_radius_taps_supported(int kernel_size);
size_t pcx_radius_taps_workspace_bytes(int64_t P, int64_t Q, int kernel_size);
int pcx_radius_taps_count(const float *d_points, const float *d_queries,
                          const int32_t *d_point_sample, const int32_t *d_query_sample,
                          int64_t P, int64_t Q, double radius, int distance_type,
                          int kernel_size, double kernel_grid_size,
                          int64_t *d_num_neighbors, int64_t *d_seg_offs, void *d_ws,
                          size_t ws_bytes, void *stream);
int pcx_radius_taps_total(int64_t P, int64_t Q, int kernel_size, int64_t *h_total,
                          void *d_ws, size_t ws_bytes, void *stream);
int pcx_radius_taps_fill(const float *d_queries, const int32_t *d_point_sample,
                         const int32_t *d_query_sample, int64_t P, int64_t Q,
                         double radius, int distance_type, int kernel_size,
                         double kernel_grid_size, int64_t capacity, int32_t *d_out_i,
                         int32_t *d_out_j, int32_t *d_out_k, int64_t *h_total,
                         void *d_ws, size_t ws_bytes, void *stream);

/* ------------------------------------------------------------------------
 * Centre-nearest grid down-sampling: one observed point per occupied cell of
 * side `cell`, the one nearest the cell centre (ties: lowest index), cells in
 * ascending (sample, z, y, x) order.
 *
 * Replaces internals/grid_sample.py:42-121 (grid_sample_filter,
 * reduction="center_nearest"), internals/grid_indexing.py:20-111 and
 * internals/grid_sample_triton_kernel.py:55-151.
 *
 *   pcx_grid_sample_count   bins and sorts the points, returns the number of
 *       occupied cells in *h_num_cells.
 *   pcx_grid_sample_select  writes d_indices (S) int64, d_out_points (S,3),
 *       d_out_sample (S) int32 (may be NULL) and, when not NULL, d_mapping (N)
 *       int64 = cell ordinal of every input point.
 */
size_t pcx_grid_sample_workspace_bytes(int64_t N);
int pcx_grid_sample_count(const float *d_points, const int32_t *d_sample,
                          int64_t N, double cell, int64_t *h_num_cells,
                          void *d_ws, size_t ws_bytes, void *stream);
int pcx_grid_sample_select(const float *d_points, const int32_t *d_sample,
                           int64_t N, double cell, int64_t num_cells,
                           int64_t *d_indices, float *d_out_points,
                           int32_t *d_out_sample, int64_t *d_mapping,
                           void *d_ws, size_t ws_bytes, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* POINTELLIGENCE_B200_H */
