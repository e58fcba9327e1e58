/*
 * tiga_b200.h -- C ABI of libtiga_b200.so: hand-written sm_100a CUDA kernels
 * for Tiga's fused CSR message-passing path (forward and autograd backward).
 *
 * This boundary replaces, for that one path, the reference's native C ABI
 * `gfrt_*` (include/tiga/Runtime/CAPI.h:50-114 of walkerchi/TIGA-lang: module
 * load + kernel launch of Triton-compiled images) together with the launch
 * ABI of those images (python/tiga/codegen/ttir.py:103-121: positional device
 * pointers `(row_ptr, col_idx, *fields, out)`, scalars, then scratch
 * pointers).  The same discipline is kept:
 *
 *   - every function returns an int32 status with the reference's codes
 *     (CAPI.h:21-27) and never throws or aborts; tgb_last_error() gives the
 *     thread-local message of the last non-zero status;
 *   - the caller passes raw device addresses, element counts and the CUDA
 *     stream handle to launch on (CAPI.h:78-80 wraps an external stream the
 *     same way); nothing here allocates or frees device memory, and no call
 *     synchronises the device except tgb_csr_plan_create (documented there);
 *   - a plan is an opaque host handle over caller-owned device memory.
 *
 * Functions are re-entrant; the only mutable global state is the thread-local
 * error string.  One process drives one GPU at a time (the current device of
 * the calling thread must be the one that owns the pointers).
 */
#ifndef TIGA_B200_H
#define TIGA_B200_H

#include <stdint.h>

#if defined(_WIN32)
#define TGB_API __declspec(dllexport)
#else
#define TGB_API __attribute__((visibility("default")))
#endif

#ifdef __cplusplus
extern "C" {
#endif

/* Status codes: identical to GFRTStatus (include/tiga/Runtime/CAPI.h:21-27). */
enum {
  TGB_STATUS_OK = 0,
  TGB_STATUS_INVALID_ARGUMENT = 1,
  TGB_STATUS_UNSUPPORTED = 2,
  TGB_STATUS_OUT_OF_MEMORY = 3,
  TGB_STATUS_INTERNAL = 4
};

/* Element types of feature buffers. */
enum { TGB_DTYPE_F32 = 0, TGB_DTYPE_BF16 = 1 };

/* Reducers.  SUM/MEAN: python/tiga/reducer/core.py:85-143.  MAX: a user
 * Reducer whose combine is tg.math.maximum (the variadic-reduce algebra
 * branch, lib/Target/Triton/Translate.cpp:3353-3402). */
enum { TGB_REDUCER_SUM = 0, TGB_REDUCER_MEAN = 1, TGB_REDUCER_MAX = 2,
       TGB_REDUCER_PROD = 3 /* edge programs only */ };

/* Flags of tgb_csr_reduce_fwd. */
enum {
  TGB_REDUCE_ACCUMULATE = 1 /* SUM only: out[i,:] += row sum; rows without edges
                               are left untouched (second pass of a relation
                               whose edges were split in two parts, e.g. owned
                               and ghost sources of a halo partition) */
};

/* Plan flags. */
enum {
  TGB_PLAN_FORWARD = 1,   /* degree-bucket work lists over the CSR rows        */
  TGB_PLAN_TRANSPOSE = 2  /* + transposed relation (stable), needed by *_bwd_dx */
};

/* replaces gfrt_status_string (CAPI.h:50) */
TGB_API const char *tgb_status_string(int32_t status);
/* replaces the message the reference raises after a non-zero status
 * (python/tiga/runtime/__init__.py:279-284) */
TGB_API const char *tgb_last_error(void);
/* replaces gfrt_runtime_version (CAPI.h:51) */
TGB_API const char *tgb_version(void);
/* number of kernels this library has launched from the calling process */
TGB_API int64_t tgb_launch_count(void);
/* Copies one int32 (an error word of the tensor-core entry points) from device
 * memory to pinned host memory with a one-thread kernel on `stream`: no copy
 * engine is involved, so the mirror never waits behind a bulk transfer that
 * another stream has in flight.  The host word must be page-locked memory that
 * the device can address (cudaHostAlloc / a pinned Torch tensor). */
TGB_API int32_t tgb_mirror_word(const void *device_word, void *pinned_host_word,
                                uint64_t stream);

/* ------------------------------------------------------------------------
 * Plans: the per-graph schedule.  Replaces the reference's schedule passes
 * (lib/Transforms/SelectKernelSchedule.cpp:136-254, PlanDegreeBuckets.cpp:
 * 32-143, PlanSplitRows.cpp:34-117) and its device work-list kernels
 * gf_degree_reset/histogram/prefix/scatter (lib/Target/Triton/Translate.cpp:
 * 4048-4210), and the transposed-relation build of the generated source VJP
 * (python/tiga/interop/torch/relation_vjp.py:61-87).
 *
 * Rows are ordered by degree bucket (0, 1, 2, 3-4, 5-8, ... powers of two),
 * heaviest bucket first, stable by row id inside a bucket.  Rows longer than
 * the split threshold are cut into fixed-size edge segments that are reduced
 * by separate thread groups and summed by a finalize kernel in segment order.
 * ------------------------------------------------------------------------ */
typedef struct tgb_csr_plan tgb_csr_plan;

/* Bytes of device memory a plan needs: `persistent_bytes` lives as long as the
 * plan, `temp_bytes` only during tgb_csr_plan_create.  index_bits is 32 or 64
 * (row_ptr and col_idx share it, python/tiga/interop/torch/graph.py:594-601).
 * Limits: num_dst, num_src < 2^31; num_edges < 2^32. */
TGB_API int32_t tgb_csr_plan_sizes(int64_t num_dst, int64_t num_src,
                                   int64_t num_edges, int32_t index_bits,
                                   int32_t flags, uint64_t *persistent_bytes,
                                   uint64_t *temp_bytes);

/* Builds the plan into `persistent` (256-byte aligned device memory the caller
 * keeps alive until tgb_csr_plan_destroy).  row_ptr/col_idx are device
 * pointers that must stay valid and unchanged while the plan is used.
 * This is the one call that synchronises `stream` (it reads three counters
 * back to size the grids). */
TGB_API int32_t tgb_csr_plan_create(const void *row_ptr, const void *col_idx,
                                    int64_t num_dst, int64_t num_src,
                                    int64_t num_edges, int32_t index_bits,
                                    int32_t flags, void *persistent,
                                    uint64_t persistent_bytes, void *temp,
                                    uint64_t temp_bytes, uint64_t stream,
                                    tgb_csr_plan **out_plan);

/* Frees the host handle only (device memory belongs to the caller). */
TGB_API int32_t tgb_csr_plan_destroy(tgb_csr_plan *plan);

/* info[0]=num_dst [1]=num_src [2]=num_edges [3]=min_degree [4]=max_degree
 * [5]=long rows (forward) [6]=segments (forward) [7]=long rows (transposed)
 * [8]=segments (transposed) [9]=split threshold (edges) [10]=segment edges
 * [11]=min in-degree of sources [12]=max in-degree of sources.
 * Mirrors Graph.degree_bounds (python/tiga/interop/torch/graph.py:1224-1245)
 * and the bucket summary of PlanDegreeBuckets.cpp:145-170. */
TGB_API int32_t tgb_csr_plan_info(const tgb_csr_plan *plan, int64_t *info16);

/* Edge map: this CSR is a sub-relation of a larger edge list (the owned-source
 * or ghost-source part of a halo partition, python/tiga/distributed/
 * transport.py:790-895 splits rows the same way), and edge e of the CSR is
 * entry edge_map[e] (uint32, device memory kept alive by the caller) of the
 * weight array passed to *_fwd / *_bwd_dx and of the dw array written by
 * *_bwd_dw.  Saves the gather/scatter passes that would otherwise permute the
 * weights and their gradients on every call.  Set once, right after create. */
TGB_API int32_t tgb_csr_plan_set_edge_map(tgb_csr_plan *plan,
                                          const void *edge_map, uint64_t stream);

/* Device pointers of the plan's arrays, for tests and Graph.transpose():
 * which = 0 forward row order (int32[num_dst]), 1 transposed row_ptr
 * (int64[num_src+1]), 2 transposed destinations (int32[E]), 3 transposed edge
 * ids (uint32[E], the stable argsort of col_idx), 4 transposed row order. */
TGB_API int32_t tgb_csr_plan_array(const tgb_csr_plan *plan, int32_t which,
                                   uint64_t *device_ptr, int64_t *count);

/* Scratch bytes one reduce call needs for split rows (partial sums), for a
 * feature row of `feature_elems` elements; direction 0 = forward/dw over the
 * CSR rows, 1 = dx over the transposed rows (includes 4 bytes per edge for the
 * weights in transposed order), 2 = dx when the caller passes those weights. */
TGB_API int32_t tgb_csr_plan_scratch_bytes(const tgb_csr_plan *plan,
                                           int32_t direction, int32_t reducer,
                                           int64_t feature_elems, int32_t dtype,
                                           uint64_t *bytes);

/* ------------------------------------------------------------------------
 * Fused gather + reduce over CSR rows.
 * ------------------------------------------------------------------------ */

/* out[i,:] = reduce_{e in row i} (w ? w[e] : 1) * x[col[e],:]
 * Replaces the generated gf_csr_weighted_sum / gf_csr_additive_tile /
 * gf_csr_algebra_tile kernels and the row-split pair gf_row_split_partial /
 * gf_row_split_finalize (lib/Target/Triton/Translate.cpp:776-1601,
 * 2630-3450, 4212-4390) and the torch.sparse.mm fallback
 * (python/tiga/interop/torch/message_passing.py:3287-3292).
 *   x   [num_src, F] row-major contiguous, out [num_dst, F] (fully written)
 *   w   [E] or NULL;  identity = start value of SUM / MAX rows
 *   aux MAX only: int32 [num_dst, F] winning edge id per element (-1 = none)
 * MEAN divides by the row length (empty row -> NaN). */
TGB_API int32_t tgb_csr_reduce_fwd(const tgb_csr_plan *plan, int32_t reducer,
                                   const void *x, const void *w, void *out,
                                   void *aux, int64_t F, int32_t dtype,
                                   float identity, int32_t flags, void *scratch,
                                   uint64_t scratch_bytes, uint64_t stream);

/* dx[j,:] = sum_{e: col[e]=j} w[e] * dy[dst(e),:]  as a gather over the stable
 * transposed relation (no atomics).  Replaces _CSRWeightedSumFunction.backward
 * (python/tiga/interop/torch/message_passing.py:386-409) and
 * compile_source_vjp (python/tiga/interop/torch/relation_vjp.py:45-105).
 * MEAN: dy rows are divided by the destination's row length first (done into
 * scratch).  MAX: only the winning edge of each (row, element) contributes.
 * SUM / MEAN with weights: a first pass writes the weights in transposed order
 * into scratch (4 bytes per edge, included in tgb_csr_plan_scratch_bytes for
 * direction 1) so that the gather reads them in order; a caller that has them
 * already (tgb_csr_transposed_weights, e.g. kept across the layers that share
 * one weight array) passes them as `aux` and that pass is skipped. */
TGB_API int32_t tgb_csr_reduce_bwd_dx(const tgb_csr_plan *plan, int32_t reducer,
                                      const void *dy, const void *w,
                                      const void *aux, void *dx, int64_t F,
                                      int32_t dtype, void *scratch,
                                      uint64_t scratch_bytes, uint64_t stream);

/* w_t[k] = w[eid[k]]: the weights in the order of the plan's stable transposed
 * relation (`jacobian = w[order]` of python/tiga/interop/torch/relation_vjp.py:
 * 61-87).  float32 [E]; honours an edge map.  The plan needs TGB_PLAN_TRANSPOSE. */
TGB_API int32_t tgb_csr_transposed_weights(const tgb_csr_plan *plan, const void *w,
                                           void *w_t, uint64_t stream);

/* dw[e] = <dy[dst(e),:], x[col[e],:]>  (per-edge dot product; the contract of
 * benchmarks/autograd/message_passing_backward.py:346-353). */
TGB_API int32_t tgb_csr_reduce_bwd_dw(const tgb_csr_plan *plan, int32_t reducer,
                                      const void *dy, const void *x,
                                      const void *aux, void *dw, int64_t F,
                                      int32_t dtype, void *scratch,
                                      uint64_t scratch_bytes, uint64_t stream);

/* Forward sum that needs no scratch buffer from the caller and performs no
 * allocation of any kind (no counterpart in the reference: its runtime always
 * allocates outputs and scratch itself).  Meant for callers that cannot call
 * cudaMalloc where they need the result -- code inside a region that must not
 * synchronise or take the allocator lock, or a host that gives a plug-in no
 * allocator.  Computes exactly what tgb_csr_reduce_fwd(TGB_REDUCER_SUM) does.
 *
 * The partial rows of split rows live in an 8 MiB array inside the library
 * image (held by every GPU that loads the library until exit), so the graph
 * must satisfy  split-row segments x F <= 2 097 152  (tgb_csr_plan_info
 * info[6] gives the segments); larger calls fail with TGB_STATUS_UNSUPPORTED
 * and a message naming both numbers.  The first call on each device looks up
 * the array's device address (cudaGetSymbolAddress); make that first call
 * outside any stream capture.  All calls share the one array: nothing in it
 * has to be cleared between calls (every segment rewrites its row before it is
 * read), but two calls that overlap on the GPU, e.g. on different streams,
 * race on it -- serialise them. */
TGB_API int32_t tgb_csr_wsum_fwd_noalloc(const tgb_csr_plan *plan, const void *x,
                                         const void *w, void *out, int64_t F,
                                         float identity, uint64_t stream);

/* ------------------------------------------------------------------------
 * Edge attention over CSR rows (online-softmax reducer), bf16 features.
 *
 * Program: s = (src.x*a_src).sum(-1) + (dst.x*a_dst).sum(-1) per head,
 * score = maximum(s, slope*s), out = online_softmax(score, src.x).
 * Replaces, for this program, the reference's gf_edge_nn_attention /
 * gf_edge_nn_attention_vjp kernels (python/tiga/compiler/edge_nn_attention.py:
 * 127-338, 344-611) and the eager evaluator it falls back to for bf16
 * multi-head scores (python/tiga/interop/torch/message_passing.py:2848-2894,
 * reducer_oracle.py:60-137).  x [rows, H, D] bf16 contiguous, 16-byte aligned;
 * H*D/8 a power of two <= 32 and D/8 a power of two.
 * ------------------------------------------------------------------------ */

/* scores[n,h] = bf16(sum_d bf16(x[n,h,d]*a[h,d])) as float32 [n, H]. */
TGB_API int32_t tgb_gat_node_scores(const void *x, const void *a, int64_t n,
                                    int32_t H, int32_t D, void *scores,
                                    uint64_t stream);

/* Scratch bytes of tgb_gat_fwd (backward = 0) or tgb_gat_bwd (backward = 1). */
TGB_API int32_t tgb_gat_scratch_bytes(const tgb_csr_plan *plan, int32_t H,
                                      int32_t D, int32_t backward,
                                      uint64_t *bytes);

/* out [num_dst,H,D] bf16 (0 for an empty row, reducer_oracle.py:132-136);
 * m, l [num_dst,H] float32 = row maximum and denominator, saved for the
 * backward like the reference does (edge_nn_attention.py:330-334). */
TGB_API int32_t tgb_gat_fwd(const tgb_csr_plan *plan, const void *x_src,
                            const void *s_src, const void *s_dst, void *out,
                            void *m, void *l, int32_t H, int32_t D, float slope,
                            void *scratch, uint64_t scratch_bytes,
                            uint64_t stream);

/* Gradients of the program: dx_src [num_src,H,D] and dx_dst [num_dst,H,D] in
 * bf16 (add them when one tensor plays both roles), da_src/da_dst [H,D] in
 * float32.  No atomics: a destination-major pass writes the per-edge softmax
 * weight and pre-activation cotangent, a source-major pass over the plan's
 * transposed relation gathers them. */
TGB_API int32_t tgb_gat_bwd(const tgb_csr_plan *plan, const void *x_src,
                            const void *x_dst, const void *a_src,
                            const void *a_dst, const void *s_src,
                            const void *s_dst, const void *out,
                            const void *dout, const void *m, const void *l,
                            int32_t H, int32_t D, float slope, void *dx_src,
                            void *dx_dst, void *da_src, void *da_dst,
                            void *scratch, uint64_t scratch_bytes,
                            uint64_t stream);

/* ------------------------------------------------------------------------
 * Row movers of the halo exchange (float32 rows of F elements, int64 ids that
 * are unique within one call).  Replace the pack / unpack / reverse-halo
 * segment-sum of the reference's device halo path
 * (python/tiga/distributed/transport.py:1060-1133, 446-574).
 * ------------------------------------------------------------------------ */
/* packed[i, :] = rows[ids[i], :] */
TGB_API int32_t tgb_rows_gather(const void *rows, const void *ids, void *packed,
                                int64_t n, int64_t F, uint64_t stream);
/* rows[ids[i], :] += packed[i, :]   (no atomics: ids are unique) */
TGB_API int32_t tgb_rows_scatter_add(void *rows, const void *ids,
                                     const void *packed, int64_t n, int64_t F,
                                     uint64_t stream);

/* ------------------------------------------------------------------------
 * Dense-relation attention (online-softmax reducer over an implicit dense or
 * lower-triangular relation), packed variable-length sequences, bf16, on the
 * tensor cores (tcgen05 + tensor memory, TMA loads).
 * Replaces gf_dense_streaming_reduce (lib/Target/Triton/Translate.cpp:
 * 1603-1912) and _execute_structured_dense (python/tiga/interop/torch/
 * message_passing.py:1910-2020); the packed relation is Graph.cu_seqlens /
 * Graph.cat of triangular blocks (python/tiga/graph/core.py:314-351,650-709),
 * which the reference materialises edge by edge and evaluates eagerly.
 *   q, out        [tokens, H, D] bf16 contiguous, D in {64, 128}
 *   k, v          [tokens, H_kv, D]; H a multiple of H_kv: query head h reads
 *                 key/value head h / (H / H_kv) (grouped queries, the query-lane
 *                 to source-lane map of Translate.cpp:1654-1680)
 *   lse           [tokens, H] float32: log-sum-exp of the scaled scores
 *   tiles         int32 [n_tiles, 4] = {first query, sequence begin, sequence
 *                 end, head}: one entry per (128-query tile, head); one CTA
 *                 each, launched in table order (keep the entries of one
 *                 (sequence, head) adjacent so they share K/V in L2)
 *   causal        1: query i attends keys seq_begin..i; 0: its whole sequence
 * error_flag: one zero-initialised int32 in device memory (bounded waits).
 * ------------------------------------------------------------------------ */
TGB_API int32_t tgb_varlen_attn_fwd(const void *q, const void *k, const void *v,
                                    void *out, void *lse, const void *tiles,
                                    int64_t n_tiles, int64_t tokens, int32_t H,
                                    int32_t H_kv, int32_t D, float scale,
                                    int32_t causal, void *error_flag,
                                    uint64_t stream);

/* Gradients of tgb_varlen_attn_fwd (no counterpart in the reference, whose
 * dense path is forward only: python/tiga/interop/torch/message_passing.py:
 * 1910-2020 returns without an autograd Function).  dq [tokens, H, D], dk, dv
 * [tokens, H_kv, D] bf16; delta is scratch, float32 [tokens, H]; query_tiles
 * (n_tiles entries, one per 128-query tile and query head) as in the forward,
 * key_tiles (n_key_tiles entries, one per 128-key tile and key/value head; field
 * 0 = first key of the tile) for the key-major kernel.  No atomics: dK/dV are
 * accumulated per key tile over the query blocks of every query head of its
 * group, dQ per query tile over its key blocks. */
TGB_API int32_t tgb_varlen_attn_bwd(const void *q, const void *k, const void *v,
                                    const void *out, const void *dout,
                                    const void *lse, void *dq, void *dk,
                                    void *dv, void *delta,
                                    const void *query_tiles,
                                    const void *key_tiles, int64_t n_tiles,
                                    int64_t n_key_tiles, int64_t tokens,
                                    int32_t H, int32_t H_kv, int32_t D,
                                    float scale, int32_t causal,
                                    void *error_flag, uint64_t stream);

/* ------------------------------------------------------------------------
 * Online-softmax reducer with per-edge scores and per-source values:
 *   edge(): return self.reducer(edge.score, src.value)
 *   out[i,h,:] = sum_e p[e,h] * value[col[e],h,:],  p = softmax of score over row i
 * Replaces the reference's stable-weighted reduction tile
 * (lib/Target/Triton/Translate.cpp:3296-3352) and the eager evaluator
 * (python/tiga/interop/torch/reducer_oracle.py:60-137) for this program:
 * float32 state, an empty row yields exactly 0.
 *   score [E, H] float32; value [num_src, H, D] float32 or bf16 (value_dtype);
 *   out [num_dst, H, D] float32; m, l [num_dst, H] float32 (kept for the backward).
 * Backward (no atomics): d_score [E, H] float32, d_value [num_src, H, D] float32;
 * dout, out float32; p_scratch = E*H floats; the plan needs TGB_PLAN_TRANSPOSE.
 * ------------------------------------------------------------------------ */
TGB_API int32_t tgb_softmax_field_fwd(const tgb_csr_plan *plan, const void *score,
                                      const void *value, int32_t value_dtype,
                                      void *out, void *m, void *l, int32_t H,
                                      int32_t D, uint64_t stream);
TGB_API int32_t tgb_softmax_field_bwd(const tgb_csr_plan *plan, const void *score,
                                      const void *value, int32_t value_dtype,
                                      const void *out, const void *dout,
                                      const void *m, const void *l, int32_t H,
                                      int32_t D, void *d_score, void *d_value,
                                      void *p_scratch, uint64_t stream);

/* Self-test of the bounded waits of the tensor-core kernels (no reference
 * counterpart): one warp waits at most `polls` (<= 2^20) polls on a barrier that
 * nothing signals, gives up, stores code 99 in `error_flag` (int32, zero before
 * the call) and 1 in `fell_through` (int32), and the kernel returns. */
TGB_API int32_t tgb_selftest_bounded_wait(void *error_flag, uint32_t polls,
                                          void *fell_through, uint64_t stream);

/* ------------------------------------------------------------------------
 * Dense float32 linear on the tensor cores (tcgen05, 3xTF32 split):
 *   out[M, N] = a[M, K] @ b_t[N, K]^T
 * The GCN layer's `aggregate @ W`, which the reference leaves to Torch user
 * code after its kernel (examples/gcn.py:20-30 of the reference; the reference's
 * own GEMM is f16-only, lib/Target/Triton/Translate.cpp:6306-6322).  b_t is
 * the weight stored [N, K] (pass W^T for a @ W, W itself for dout @ W^T).
 * N in {64, 128}, K in {32, 64, 96, 128}; 16-byte aligned row-major inputs.
 * `error_flag` is one int32 in device memory (zero-initialised by the caller):
 * every wait in the kernel is bounded, and a wait that gives up stores a
 * non-zero code there instead of hanging.
 * ------------------------------------------------------------------------ */
TGB_API int32_t tgb_linear_f32(const void *a, const void *b_t, void *out,
                               int64_t M, int32_t K, int32_t N,
                               void *error_flag, uint64_t stream);

/* Weight gradient of the linear: dw[K, N] = a[M, K]^T @ dout[M, N], tensor
 * cores (tcgen05, 3xTF32), deterministic split over the M rows: every
 * persistent CTA accumulates its row tiles in tensor memory and writes one
 * partial [128, N] matrix into `partial`, a second kernel adds the first K rows
 * of them in CTA order; more than 8192 rows per CTA are processed in several
 * such rounds whose results are added in order (bounds the rounding of the
 * round-toward-zero accumulators).  `partial` must hold
 * tgb_linear_dw_partials(M) matrices of 128*N floats.
 * K in {32, 64, 96, 128}, N in {64, 128}. */
TGB_API int32_t tgb_linear_dw_f32(const void *a, const void *dout, void *dw,
                                  void *partial, uint64_t partial_bytes,
                                  int64_t M, int32_t K, int32_t N,
                                  void *error_flag, uint64_t stream);
TGB_API int32_t tgb_linear_dw_partials(int64_t M, int32_t *count);

/* ------------------------------------------------------------------------
 * Peer windows (one node): device memory of another process mapped into this
 * one, so that tgb_rows_gather / tgb_peer_copy store straight into a peer's halo
 * buffer over NVLink instead of packing, sending and receiving
 * (python/tiga/distributed/nccl.py:256-284 of the reference moves the same rows
 * through ncclSend / ncclRecv).  Legacy CUDA IPC; no multicast object is made.
 * Completion is signalled by the caller's own stream-ordered collective.
 * ------------------------------------------------------------------------ */

/* 64-byte handle of the allocation that holds `ptr`, and ptr's byte offset in it. */
TGB_API int32_t tgb_peer_export(const void *ptr, void *handle64, uint64_t *offset);
/* Maps a peer's allocation (a handle from tgb_peer_export in another process)
 * into this process; open a handle once per process and close it at the end. */
TGB_API int32_t tgb_peer_open(const void *handle64, uint64_t *mapped_base);
TGB_API int32_t tgb_peer_close(uint64_t mapped_base);
/* Asynchronous device-to-device copy to any mapped address (peer or local). */
TGB_API int32_t tgb_peer_copy(uint64_t dst, const void *src, uint64_t bytes, uint64_t stream);

/* ------------------------------------------------------------------------
 * Dynamic relations: radius and k-nearest-neighbour builders, and the fused
 * radius consumer that never materialises the relation.
 *
 * Replace, for contiguous float32 positions on the device, the Torch tensor
 * programs of Graph.radius / Graph.knn (python/tiga/interop/torch/graph.py:
 * 391-534 constructors, :851-1003 resolve_csr, :1023-1125 cell-list
 * candidates, :1127-1176 pair selection, :1203-1210 minimum image,
 * :1403-1444 implicit edge fields), the hash-grid directory of
 * python/tiga/interop/torch/radius_grid.py and the generated
 * radius-distance-sum kernel (`gf-kernel-to-ttir-generated-radius-distance-sum`,
 * tests/python/test_reference.py:533-560).
 *
 * Results are bit-identical to the reference's CPU evaluation: same edge order
 * (destination ascending; inside a row the 3^D neighbour cells in meshgrid
 * order, first axis slowest, and the points of a cell in ascending index),
 * same float32 operation order (displacement = source - destination,
 * distance = sqrt(fma(z, z, fma(y, y, x * x))), lattice products as fused
 * multiply-add chains in increasing k).
 * ------------------------------------------------------------------------ */

/* Geometry of the broad phase.  Open boundary: cell = floor(p / cell_size).
 * Periodic: fractional = p @ inverse, wrapped to [0, 1), cell = min(floor(
 * fractional * extents), extents - 1); `lattice`, `inverse` row-major
 * [dims, dims]; `extents` = cells per axis, computed by the caller as
 * floor(1 / (cell_size * column norms of inverse)), at least 1
 * (graph.py:1044-1054). */
typedef struct tgb_cell_space {
  int32_t dims;      /* 1, 2 or 3 */
  int32_t periodic;  /* 0 open boundary, 1 lattice */
  float cell_size;   /* edge of a cell = the scalar cutoff */
  float lattice[9];
  float inverse[9];
  int32_t extents[3];
} tgb_cell_space;

/* Bytes of the cell directory of `n` points (`persistent_bytes`, alive while
 * the directory is used) and of the scratch of its construction. */
TGB_API int32_t tgb_cell_directory_sizes(int64_t n, int32_t dims,
                                         uint64_t *persistent_bytes,
                                         uint64_t *temp_bytes);

/* Sorts the points into modular hash buckets of their cells (stable: ascending
 * index inside a bucket) and writes the directory into `persistent`.
 * positions: float32 [n, dims], row-major.  n < 2^31.  No synchronisation. */
TGB_API int32_t tgb_cell_directory_build(const void *positions, int64_t n,
                                         const tgb_cell_space *space,
                                         void *persistent, uint64_t persistent_bytes,
                                         void *temp, uint64_t temp_bytes,
                                         uint64_t stream);

/* row_ptr[0..n] (int64) of the radius relation and, in `candidate_pairs`
 * (one uint64 in device memory, may be null), the number of broad-phase
 * candidates (build_info["candidate_pairs"] of the reference).  An edge is a
 * pair with distance <= cutoff, minus i == j when exclude_self.
 * `temp` needs tgb_cell_directory_sizes' temp_bytes. */
TGB_API int32_t tgb_radius_row_ptr(const void *positions, int64_t n,
                                   const tgb_cell_space *space, const void *directory,
                                   float cutoff, int32_t exclude_self, void *row_ptr,
                                   void *candidate_pairs, void *temp, uint64_t temp_bytes,
                                   uint64_t stream);

/* col[E] (int64) in the reference's order and, when not null, distance[E] and
 * displacement[E, dims] (float32): the implicit edge fields. */
TGB_API int32_t tgb_radius_fill(const void *positions, int64_t n,
                                const tgb_cell_space *space, const void *directory,
                                float cutoff, int32_t exclude_self, const void *row_ptr,
                                void *col, void *distance, void *displacement,
                                uint64_t stream);

/* Weight of a pair in the fused consumer. */
enum { TGB_PAIR_WEIGHT_ONE = 0, TGB_PAIR_WEIGHT_DISTANCE = 1 };

/* out[i, :] = sum over the radius neighbours j of i, in the relation's edge
 * order, of weight(i, j) * x[j, :]; x, out float32 [n, F], F <= 128.  The sum
 * is the sequential float32 fold of the CSR kernels, so it equals
 * tgb_csr_reduce_fwd over the materialised relation bit for bit. */
TGB_API int32_t tgb_radius_wsum_fwd(const void *positions, int64_t n,
                                    const tgb_cell_space *space, const void *directory,
                                    float cutoff, int32_t exclude_self, int32_t weight,
                                    const void *x, int64_t F, void *out, uint64_t stream);

/* Position cotangent of the distance-weighted sum:
 * dpos[i, :] = - sum_j (dy[i,:].x[j,:] + dy[j,:].x[i,:]) * displacement(i, j) / distance(i, j),
 * pairs at distance zero contributing nothing (the subgradient Torch's
 * vector_norm uses).  Requires the symmetric relation of a scalar cutoff. */
TGB_API int32_t tgb_radius_wsum_bwd_pos(const void *positions, int64_t n,
                                        const tgb_cell_space *space, const void *directory,
                                        float cutoff, int32_t exclude_self, const void *x,
                                        const void *dy, int64_t F, void *dpos,
                                        uint64_t stream);

/* Exact k nearest candidates of every query, ascending by (squared distance,
 * candidate index): col[nq, k] int64 and, when not null, dist_sq[nq, k].
 * exclude_self drops candidate i of query i (self search).  dims <= 64,
 * 1 <= k <= 128, k <= nc - exclude_self. */
TGB_API int32_t tgb_knn(const void *queries, int64_t nq, const void *candidates,
                        int64_t nc, int32_t dims, int32_t k, int32_t exclude_self,
                        void *col, void *dist_sq, uint64_t stream);

/* The same selection as tgb_knn through a cell directory built over the
 * CANDIDATES (tgb_cell_directory_build, open boundary, dims <= 3): every query
 * walks the shells of cells around its own cell and stops once its k-th
 * distance is strictly below the distance to the boundary of the cells it has
 * covered, less `margin` (an absolute bound on the rounding of a coordinate:
 * a few ulps of the largest |coordinate|); queries not settled within six
 * shells are finished by a scan over all candidates, so the result is exact
 * and identical to tgb_knn for every input.  `unsettled`: int32[nq] scratch.
 * self_search != 0: the queries are the candidates themselves (nq == nc). */
TGB_API int32_t tgb_knn_grid(const void *queries, int64_t nq, const void *candidates,
                             int64_t nc, const tgb_cell_space *space,
                             const void *directory, int32_t k, int32_t exclude_self,
                             int32_t self_search, float margin, void *col,
                             void *dist_sq, void *unsettled, uint64_t stream);

/* Implicit edge fields of a stored relation: displacement[e, :] =
 * src_positions[col[e], :] - dst_positions[row of e, :] (minimum image when
 * `space` is periodic; only dims, periodic, lattice and inverse are read, dims
 * <= 8 for an open boundary) and distance[e]; either output may be null.
 * row_ptr, col int64. */
TGB_API int32_t tgb_edge_geometry(const void *dst_positions, const void *src_positions,
                                  const tgb_cell_space *space, const void *row_ptr,
                                  const void *col, int64_t num_dst, int64_t num_edges,
                                  void *displacement, void *distance, uint64_t stream);

/* ------------------------------------------------------------------------
 * Generic edge programs: an arbitrary element-wise edge expression folded over
 * CSR rows.  Replace the reference's generic CSR kernels gf_csr_additive_tile
 * (one row per program, lib/Target/Triton/Translate.cpp:2630-2783, expression
 * emitter :381-460) and gf_csr_scalar_reduce (:3452-3634) reached through
 * _execute_generic_csr (python/tiga/interop/torch/message_passing.py:2579-2815),
 * and the Torch autograd replay of the eager evaluator for their gradients.
 *
 * The expression is a register program: instruction i computes
 *   value[i] = op[i](value[a[i]], value[b[i]])
 * in float32, the last instruction is the message.  LOAD reads operand a[i]
 * (every operand is loaded by exactly one instruction), CONST reads
 * constants[a[i]].  An operand is a float32 array of per-entity rows: entity =
 * source of the edge (role 0), destination row (1), edge id (2) or none (3, a
 * tensor parameter); operand_modulus 0 = `width` elements per entity (element
 * f), 1 = one element per entity, m > 1 = m elements per entity (element f % m).
 * ------------------------------------------------------------------------ */
enum {
  TGB_EP_LOAD = 0, TGB_EP_CONST = 1, TGB_EP_ADD = 2, TGB_EP_SUB = 3, TGB_EP_MUL = 4,
  TGB_EP_DIV = 5, TGB_EP_MAX = 6, TGB_EP_EXP = 7, TGB_EP_NEG = 8
};
enum { TGB_EP_ROLE_SRC = 0, TGB_EP_ROLE_DST = 1, TGB_EP_ROLE_EDGE = 2, TGB_EP_ROLE_PARAM = 3 };
#define TGB_EP_MAX_INSTRUCTIONS 48
#define TGB_EP_MAX_OPERANDS 8
#define TGB_EP_MAX_CONSTANTS 16

typedef struct tgb_edge_program {
  int32_t num_instructions;
  int32_t num_operands;
  int32_t width; /* elements of one message */
  int32_t reserved;
  uint8_t op[TGB_EP_MAX_INSTRUCTIONS];
  uint8_t a[TGB_EP_MAX_INSTRUCTIONS];
  uint8_t b[TGB_EP_MAX_INSTRUCTIONS];
  float constants[TGB_EP_MAX_CONSTANTS];
  int32_t operand_role[TGB_EP_MAX_OPERANDS];
  int32_t operand_modulus[TGB_EP_MAX_OPERANDS];
} tgb_edge_program;

/* out[i, f] = reduce over the edges of row i, in edge order, of the message
 * element f.  reducer: TGB_REDUCER_SUM (rows without edges give `identity`),
 * _MEAN (NaN for rows without edges), _MAX (identity), _PROD (identity; the
 * reference's product monoid, python/tiga/reducer/core.py:146-158 of
 * walkerchi/TIGA-lang).  operands[k]: device pointer of operand k.
 * out: float32 [num_dst, width].
 * What the reverse mode of MAX and PROD needs is written when the pointers
 * are given (both may be null for a call without gradients):
 *   saved_index int32 [num_dst, width]  MAX: entry of the first message that
 *                                       reached the maximum (-1: none did);
 *                                       PROD: number of zero messages
 *   saved_value float32 [num_dst, width] PROD: the product with every zero
 *                                       message replaced by one */
TGB_API int32_t tgb_edge_program_fwd(const tgb_csr_plan *plan,
                                     const tgb_edge_program *program,
                                     const void *const *operands, int32_t reducer,
                                     float identity, void *out, void *saved_value,
                                     void *saved_index, uint64_t stream);

/* Reverse mode, destination-major pass: for every operand k with
 * grads[k] != null and role DST, EDGE or PARAM, writes its cotangent given
 * dy [num_dst, width]: DST -> [num_dst, elements], EDGE -> [E, elements],
 * PARAM -> one partial row per destination, [num_dst, elements], to be summed
 * with tgb_column_sum.  Cotangents are supported for modulus 0 and 1.
 * The cotangent of a message is dy (SUM), dy / degree (MEAN), dy for the
 * saved winner and 0 for the others (MAX), dy times the product of the row's
 * other messages (PROD: dy * saved_value / message in a row without zeros,
 * dy * saved_value for the only zero of a row, else 0 -- the zero-safe rule
 * of the reference's csr_segment_product_vjp, python/tiga/tensor/core.py:
 * 1586-1598).  saved_value / saved_index: as the forward wrote them. */
TGB_API int32_t tgb_edge_program_bwd_rows(const tgb_csr_plan *plan,
                                          const tgb_edge_program *program,
                                          const void *const *operands, int32_t reducer,
                                          const void *dy, void *const *grads,
                                          const void *saved_value,
                                          const void *saved_index, uint64_t stream);

/* Reverse mode, source-major pass over the plan's transposed relation (the
 * plan needs TGB_PLAN_TRANSPOSE): cotangents of the SRC operands with
 * grads[k] != null, [num_src, elements]; no atomics. */
TGB_API int32_t tgb_edge_program_bwd_sources(const tgb_csr_plan *plan,
                                             const tgb_edge_program *program,
                                             const void *const *operands, int32_t reducer,
                                             const void *dy, void *const *grads,
                                             const void *saved_value,
                                             const void *saved_index, uint64_t stream);

/* ---------------------------------------------------------------------------
 * Edge programs folded by a USER ALGEBRA: any associative reducer with a tuple
 * state (the reference's captured reducer regions,
 * python/tiga/compiler/reducer_capture.py:53-130 of walkerchi/TIGA-lang, run by
 * its generic tile gf_csr_algebra_tile, lib/Target/Triton/Translate.cpp:
 * 3065-3092).  Per (row, element):
 *     state = identity
 *     for the row's edges in order:  state = step(state, messages of the edge)
 *     out   = finalize(state)
 * with step(state, m) = combine(state, lift(m)).  A region is a register
 * program like tgb_edge_program whose TGB_EP_LOAD reads ARGUMENT a[i]:
 *     step      arguments: state[0..arity), then messages[0..num_messages)
 *     combine   arguments: left[0..arity), then right[0..arity)
 *     finalize  arguments: state[0..arity);  one output
 * out[k] names the instruction whose value is output k.  The messages of an
 * edge are the values of the instructions message_slot[j] of the edge program.
 * Rows above the plan's split threshold are folded in contiguous slices that
 * `combine` joins in order: the algebra must be associative with `identity`
 * neutral, as the reference requires of a parallel reducer; it need not be
 * commutative.
 * ------------------------------------------------------------------------ */
#define TGB_ALG_MAX_INSTRUCTIONS 40
#define TGB_ALG_MAX_STATE 4
#define TGB_ALG_MAX_MESSAGES 4
#define TGB_ALG_MAX_CONSTANTS 8

typedef struct tgb_region {
  int32_t num_instructions;
  uint8_t op[TGB_ALG_MAX_INSTRUCTIONS];
  uint8_t a[TGB_ALG_MAX_INSTRUCTIONS];
  uint8_t b[TGB_ALG_MAX_INSTRUCTIONS];
  uint8_t out[TGB_ALG_MAX_STATE];
  float constants[TGB_ALG_MAX_CONSTANTS];
} tgb_region;

typedef struct tgb_edge_algebra {
  int32_t arity;        /* state components, 1..TGB_ALG_MAX_STATE */
  int32_t num_messages; /* 1..TGB_ALG_MAX_MESSAGES */
  float identity[TGB_ALG_MAX_STATE];
  uint8_t message_slot[TGB_ALG_MAX_MESSAGES];
  tgb_region step;
  tgb_region combine;
  tgb_region finalize;
} tgb_edge_algebra;

/* out: float32 [num_dst, width]. */
TGB_API int32_t tgb_edge_algebra_fwd(const tgb_csr_plan *plan,
                                     const tgb_edge_program *program,
                                     const tgb_edge_algebra *algebra,
                                     const void *const *operands, void *out,
                                     uint64_t stream);

/* Reverse mode through the fold: the cotangent of every message of every
 * edge, message_grads float32 [num_messages, E, width], given
 * dy [num_dst, width].  prefix: scratch float32 [E, arity, width] (the state
 * before each edge, kept by the first sweep over a row for the backward sweep
 * over it). */
TGB_API int32_t tgb_edge_algebra_bwd_messages(const tgb_csr_plan *plan,
                                              const tgb_edge_program *program,
                                              const tgb_edge_algebra *algebra,
                                              const void *const *operands,
                                              const void *dy, void *prefix,
                                              void *message_grads, uint64_t stream);

/* From message cotangents to operand cotangents: the two passes of
 * tgb_edge_program_bwd_rows / _sources, seeded per edge and message slot from
 * message_grads [num_messages, E, width] instead of a reducer rule. */
TGB_API int32_t tgb_edge_algebra_bwd_rows(const tgb_csr_plan *plan,
                                          const tgb_edge_program *program,
                                          const tgb_edge_algebra *algebra,
                                          const void *const *operands,
                                          const void *message_grads,
                                          void *const *grads, uint64_t stream);
TGB_API int32_t tgb_edge_algebra_bwd_sources(const tgb_csr_plan *plan,
                                             const tgb_edge_program *program,
                                             const tgb_edge_algebra *algebra,
                                             const void *const *operands,
                                             const void *message_grads,
                                             void *const *grads, uint64_t stream);

/* ---------------------------------------------------------------------------
 * Runtime-compiled edge programs.  CUDA source generated for one staged edge
 * expression (straight-line code in place of the interpreter loop of the
 * tgb_edge_program kernels) is compiled for sm_100a by NVRTC and launched
 * through the driver's module interface: the role of the reference's provider
 * pipeline, which turns a captured UDF into generated kernel code compiled at
 * run time and cached per specialisation (python/tiga/codegen/ttir.py:103-121
 * of walkerchi/TIGA-lang; its compiler is Triton).
 *   tgb_jit_build    compiles `source`; needs NVRTC (opened with dlopen) but no
 *                    GPU.  The compiler's log is copied to `log` (may be null).
 *   tgb_jit_launch   loads the module on the current device on first use and
 *                    launches `kernel` (an extern "C" __global__ taking ONE
 *                    by-value argument block, pointed to by `arguments`) with
 *                    `grid` blocks of `block` threads on `stream`; block = 0:
 *                    the block size the kernel declares (__launch_bounds__).
 * ------------------------------------------------------------------------ */
typedef struct tgb_jit_module tgb_jit_module;
TGB_API int32_t tgb_jit_build(const char *source, tgb_jit_module **module,
                              char *log, int64_t log_capacity);
TGB_API int32_t tgb_jit_image_bytes(const tgb_jit_module *module, int64_t *bytes);
TGB_API int32_t tgb_jit_launch(tgb_jit_module *module, const char *kernel,
                               uint32_t grid, uint32_t block,
                               const void *arguments, uint64_t stream);
TGB_API void tgb_jit_destroy(tgb_jit_module *module);

/* The argument block of the generated edge-program kernels (`fwd`, `fwd_long`,
 * `bwd_rows`, `bwd_rows_long`, `bwd_sources`, `bwd_sources_long`); the
 * generated source declares the same structure.  The library fills it from the
 * plan and the call. */
typedef struct tgb_jit_edge_args {
  const float *in[TGB_EP_MAX_OPERANDS];
  float *sink[TGB_EP_MAX_OPERANDS];
  const void *ptr;          /* row pointers of the traversal */
  const void *idx;          /* neighbour per entry */
  const uint32_t *eid;      /* edge id per entry, or null: entry = edge */
  const int32_t *order;     /* plan row order: the long rows first */
  const void *degree_ptr;   /* forward row pointers (MEAN divides by the degree) */
  const float *dy;
  float *out;
  float *saved_value;
  int32_t *saved_index;
  int64_t n_rows;
  int64_t n_long;
  int64_t split_threshold;
  int32_t ptr_bits, idx_bits, degree_bits;
  float identity;
  float constants[TGB_EP_MAX_CONSTANTS];
  /* user algebras only */
  const float *seeds;       /* message cotangents [messages, E, width] (reverse passes) */
  float *prefix;            /* state before each edge [E, arity, width] */
  float *message_grads;     /* [messages, E, width] */
  int64_t num_edges;
} tgb_jit_edge_args;

/* tgb_edge_program_fwd / _bwd_rows / _bwd_sources with the kernels of a module
 * generated for this program (same reducer, width, operand roles and moduli;
 * the constants are read from `program` at every call).  source_major = 0:
 * the destination-major pass, 1: the source-major pass. */
TGB_API int32_t tgb_edge_program_jit_fwd(const tgb_csr_plan *plan, tgb_jit_module *module,
                                         const tgb_edge_program *program,
                                         const void *const *operands, int32_t reducer,
                                         float identity, void *out, void *saved_value,
                                         void *saved_index, uint64_t stream);
TGB_API int32_t tgb_edge_program_jit_bwd(const tgb_csr_plan *plan, tgb_jit_module *module,
                                         const tgb_edge_program *program,
                                         const void *const *operands, int32_t reducer,
                                         const void *dy, void *const *grads,
                                         const void *saved_value, const void *saved_index,
                                         int32_t source_major, uint64_t stream);

/* The user-algebra passes (tgb_edge_algebra_fwd / _bwd_messages / _bwd_rows /
 * _bwd_sources) through a module generated for the program AND the algebra:
 * kernels `alg_fwd`, `alg_fwd_long`, `alg_bwd_messages`,
 * `alg_bwd_messages_long`, and the four reverse passes seeded per edge from
 * message_grads.  The regions are part of the generated source, so only the
 * message count and state size are read from `algebra`. */
TGB_API int32_t tgb_edge_algebra_jit_fwd(const tgb_csr_plan *plan, tgb_jit_module *module,
                                         const tgb_edge_program *program,
                                         const void *const *operands, void *out,
                                         uint64_t stream);
TGB_API int32_t tgb_edge_algebra_jit_bwd_messages(const tgb_csr_plan *plan, tgb_jit_module *module,
                                                  const tgb_edge_program *program,
                                                  const void *const *operands, const void *dy,
                                                  void *prefix, void *message_grads,
                                                  uint64_t stream);
TGB_API int32_t tgb_edge_algebra_jit_bwd(const tgb_csr_plan *plan, tgb_jit_module *module,
                                         const tgb_edge_program *program,
                                         const void *const *operands,
                                         const void *message_grads, void *const *grads,
                                         int32_t source_major, uint64_t stream);

/* out[c] = sum over r of partial[r, c] (float32, rows added in a fixed order:
 * strips of rows by one thread each, then the strips in order). */
TGB_API int32_t tgb_column_sum(const void *partial, int64_t rows, int64_t cols,
                               void *out, uint64_t stream);

#ifdef __cplusplus
}
#endif
#endif /* TIGA_B200_H */
