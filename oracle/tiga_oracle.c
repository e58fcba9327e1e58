/*
 * tiga_oracle.c -- TEST INFRASTRUCTURE, not product code.
 *
 * A plain-C, CPU restatement of the reference algorithms that the CUDA path
 * of this repository replaces (walkerchi/TIGA-lang; every function cites the
 * reference file:line it follows, paths relative to the reference project).
 * It is compiled into oracle/libtiga_oracle.so and loaded by oracle/oracle.py.
 * Only the test-suite, the smoke check and the CPU-baseline legs of the
 * benchmark may load it; the product package never does.
 *
 * Parity of this restatement is pinned by tests/test_oracle_golden.py against
 * (a) literal known-answer vectors that the reference's README and tests hold
 * and (b) fixtures under tests/golden/ that were produced by running the
 * reference's own eager evaluator (kernel.reference() + torch.autograd) in the
 * build container.  The max reducer on vector features has no runnable
 * reference implementation (the reference raises NotImplementedError for it),
 * so for that one function parity is "unpinned": it follows the cited algebra.
 *
 * Conventions: int64 CSR indices, row-major contiguous float32 features.
 * Every loop over the edges of one destination row is sequential from the
 * first edge of the row, which is the reference's native CPU order
 * (lib/Transforms/LowerTensorToCPU.cpp:672-702, emitCSRSegmentSum) and the
 * order torch.index_add_ uses on CPU in the reference's eager evaluator
 * (python/tiga/interop/torch/reducer_oracle.py:44-57).  OpenMP only spreads
 * independent rows over threads, so results do not depend on the thread count.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define ORC_API __attribute__((visibility("default")))

ORC_API int orc_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

ORC_API void orc_set_num_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

/* ------------------------------------------------------------------------ */
/* CSR construction                                                          */
/* ------------------------------------------------------------------------ */

/* Graph.from_coo (python/tiga/interop/torch/graph.py:192-231): stable argsort
 * by destination, bincount, cumsum.  order[k] is the position in the COO
 * input of the k-th CSR edge. */
ORC_API int orc_coo_to_csr(const int64_t *src, const int64_t *dst, int64_t E,
                           int64_t num_dst, int64_t *row_ptr, int64_t *col_idx,
                           int64_t *order) {
  memset(row_ptr, 0, sizeof(int64_t) * (size_t)(num_dst + 1));
  for (int64_t e = 0; e < E; ++e) {
    if (dst[e] < 0 || dst[e] >= num_dst) return 1;
    row_ptr[dst[e] + 1]++;
  }
  for (int64_t r = 0; r < num_dst; ++r) row_ptr[r + 1] += row_ptr[r];
  int64_t *cursor = (int64_t *)malloc(sizeof(int64_t) * (size_t)(num_dst + 1));
  if (!cursor) return 3;
  memcpy(cursor, row_ptr, sizeof(int64_t) * (size_t)(num_dst + 1));
  for (int64_t e = 0; e < E; ++e) {
    int64_t slot = cursor[dst[e]]++;
    col_idx[slot] = src[e];
    if (order) order[slot] = e;
  }
  free(cursor);
  return 0;
}

/* Graph.destination_index (python/tiga/interop/torch/graph.py:1212-1222):
 * repeat_interleave(arange(N), degree). */
ORC_API void orc_destination_index(const int64_t *row_ptr, int64_t N,
                                   int64_t *dst_of_edge) {
  for (int64_t r = 0; r < N; ++r)
    for (int64_t e = row_ptr[r]; e < row_ptr[r + 1]; ++e) dst_of_edge[e] = r;
}

/* Transposed relation used by the generated source VJP
 * (python/tiga/interop/torch/relation_vjp.py:61-87) and Graph.transpose
 * (python/tiga/graph/core.py:1286-1299): order = argsort(col_idx, stable),
 * t_col = destination[order], t_ptr = cumsum(bincount(col_idx)). */
ORC_API int orc_csr_transpose(const int64_t *row_ptr, const int64_t *col_idx,
                              int64_t N, int64_t num_src, int64_t *t_ptr,
                              int64_t *t_col, int64_t *order) {
  int64_t E = row_ptr[N];
  memset(t_ptr, 0, sizeof(int64_t) * (size_t)(num_src + 1));
  for (int64_t e = 0; e < E; ++e) {
    if (col_idx[e] < 0 || col_idx[e] >= num_src) return 1;
    t_ptr[col_idx[e] + 1]++;
  }
  for (int64_t j = 0; j < num_src; ++j) t_ptr[j + 1] += t_ptr[j];
  int64_t *cursor = (int64_t *)malloc(sizeof(int64_t) * (size_t)(num_src + 1));
  if (!cursor) return 3;
  memcpy(cursor, t_ptr, sizeof(int64_t) * (size_t)(num_src + 1));
  for (int64_t r = 0; r < N; ++r)
    for (int64_t e = row_ptr[r]; e < row_ptr[r + 1]; ++e) {
      int64_t slot = cursor[col_idx[e]]++;
      t_col[slot] = r;
      order[slot] = e;
    }
  free(cursor);
  return 0;
}

/* Graph.degree_bounds / degree_statistics
 * (python/tiga/interop/torch/graph.py:1224-1245): min, max and sum of the
 * row lengths. stats = {min, max, sum}. */
ORC_API void orc_degree_stats(const int64_t *row_ptr, int64_t N,
                              int64_t *stats) {
  int64_t lo = N ? INT64_MAX : 0, hi = 0;
  for (int64_t r = 0; r < N; ++r) {
    int64_t d = row_ptr[r + 1] - row_ptr[r];
    if (d < lo) lo = d;
    if (d > hi) hi = d;
  }
  stats[0] = lo;
  stats[1] = hi;
  stats[2] = N ? row_ptr[N] - row_ptr[0] : 0;
}

/* ------------------------------------------------------------------------ */
/* Sum / mean reducers, weighted-sum edge function                           */
/* ------------------------------------------------------------------------ */

/* out[i,:] = identity + sum_{e in row i} w[e] * x[col[e],:]
 * (python/tiga/interop/torch/message_passing.py:2848-2894 with
 * reducer_oracle.py:44-57).  The product is rounded before it is added, as
 * torch evaluates `values * scales` and then index_add_.  w may be NULL
 * (unweighted `src.x` message).  mean != 0 divides the row sum by the float
 * row length, 0/0 = NaN for an empty row (reducer_oracle.py:140-158,
 * python/tiga/reducer/core.py:120-143). */
ORC_API void orc_csr_wsum_fwd_f32(const int64_t *row_ptr, const int64_t *col_idx,
                                  int64_t N, const float *x, int64_t F,
                                  const float *w, float identity, int mean,
                                  float *out) {
#pragma omp parallel for schedule(dynamic, 256)
  for (int64_t r = 0; r < N; ++r) {
    float *o = out + r * F;
    float init = mean ? 0.0f : identity;
    for (int64_t f = 0; f < F; ++f) o[f] = init;
    int64_t b = row_ptr[r], e_end = row_ptr[r + 1];
    for (int64_t e = b; e < e_end; ++e) {
      const float *xr = x + col_idx[e] * F;
      if (w) {
        float we = w[e];
        for (int64_t f = 0; f < F; ++f) {
          float m = we * xr[f]; /* built with -ffp-contract=off */
          o[f] = o[f] + m;
        }
      } else {
        for (int64_t f = 0; f < F; ++f) o[f] = o[f] + xr[f];
      }
    }
    if (mean) {
      float count = (float)(e_end - b);
      for (int64_t f = 0; f < F; ++f) o[f] = o[f] / count;
    }
  }
}

/* dx[j,:] = sum_{e: col[e]=j} w[e] * dy[dst(e),:] in ascending edge order,
 * which is the order of torch's CPU index_add_ in the autograd of the gather
 * `source[col_idx]` (python/tiga/interop/torch/message_passing.py:386-409) and
 * of the stable transposed relation (relation_vjp.py:61-87).  For the mean
 * reducer the cotangent of row i is first divided by the row length. */
ORC_API void orc_csr_wsum_bwd_dx_pre_f32(const int64_t *row_ptr,
                                         const int64_t *t_ptr,
                                         const int64_t *t_col,
                                         const int64_t *order, int64_t num_src,
                                         const float *dy, int64_t F,
                                         const float *w, int mean, float *dx) {
#pragma omp parallel for schedule(dynamic, 256)
  for (int64_t j = 0; j < num_src; ++j) {
    float *o = dx + j * F;
    for (int64_t f = 0; f < F; ++f) o[f] = 0.0f;
    for (int64_t t = t_ptr[j]; t < t_ptr[j + 1]; ++t) {
      int64_t r = t_col[t];
      const float *g = dy + r * F;
      float scale = w ? w[order[t]] : 1.0f;
      float count = (float)(row_ptr[r + 1] - row_ptr[r]);
      for (int64_t f = 0; f < F; ++f) {
        float gv = mean ? g[f] / count : g[f];
        float m = w ? scale * gv : gv;
        o[f] = o[f] + m;
      }
    }
  }
}

ORC_API int orc_csr_wsum_bwd_dx_f32(const int64_t *row_ptr,
                                    const int64_t *col_idx, int64_t N,
                                    int64_t num_src, const float *dy, int64_t F,
                                    const float *w, int mean, float *dx) {
  int64_t E = row_ptr[N];
  int64_t *t_ptr = (int64_t *)malloc(sizeof(int64_t) * (size_t)(num_src + 1));
  int64_t *t_col = (int64_t *)malloc(sizeof(int64_t) * (size_t)(E ? E : 1));
  int64_t *order = (int64_t *)malloc(sizeof(int64_t) * (size_t)(E ? E : 1));
  if (!t_ptr || !t_col || !order) return 3;
  int rc = orc_csr_transpose(row_ptr, col_idx, N, num_src, t_ptr, t_col, order);
  if (!rc)
    orc_csr_wsum_bwd_dx_pre_f32(row_ptr, t_ptr, t_col, order, num_src, dy, F, w,
                                mean, dx);
  free(t_ptr);
  free(t_col);
  free(order);
  return rc;
}

/* dw[e] = <dy[dst(e),:], x[col[e],:]>  (benchmark contract,
 * benchmarks/autograd/message_passing_backward.py:346-353; it is what
 * autograd of `values * scales` gives in message_passing.py:386-409). */
ORC_API void orc_csr_wsum_bwd_dw_f32(const int64_t *row_ptr,
                                     const int64_t *col_idx, int64_t N,
                                     const float *dy, const float *x, int64_t F,
                                     int mean, float *dw) {
#pragma omp parallel for schedule(dynamic, 256)
  for (int64_t r = 0; r < N; ++r) {
    const float *g = dy + r * F;
    float count = (float)(row_ptr[r + 1] - row_ptr[r]);
    for (int64_t e = row_ptr[r]; e < row_ptr[r + 1]; ++e) {
      const float *xr = x + col_idx[e] * F;
      float acc = 0.0f;
      for (int64_t f = 0; f < F; ++f) {
        float gv = mean ? g[f] / count : g[f];
        float m = gv * xr[f];
        acc = acc + m;
      }
      dw[e] = acc;
    }
  }
}

/* ------------------------------------------------------------------------ */
/* Product reducer (tg.prod)                                                  */
/* ------------------------------------------------------------------------ */

/* out[i,f] = product of the messages of row i, left to right from 1
 * (csr_segment_product, python/tiga/tensor/core.py:1575-1585; the Torch
 * interop folds the same way through index_reduce("prod") from
 * reducer.identity() = 1, python/tiga/interop/torch/reducer_oracle.py:160-178).
 * message: [E, F], one row per edge in CSR order. */
ORC_API void orc_csr_product_fwd_f32(const int64_t *row_ptr, int64_t N,
                                     const float *message, int64_t F, float *out) {
#pragma omp parallel for schedule(dynamic, 256)
  for (int64_t r = 0; r < N; ++r) {
    float *o = out + r * F;
    for (int64_t f = 0; f < F; ++f) o[f] = 1.0f;
    for (int64_t e = row_ptr[r]; e < row_ptr[r + 1]; ++e)
      for (int64_t f = 0; f < F; ++f) o[f] = o[f] * message[e * F + f];
  }
}

/* d message[e,f] = dy[row,f] times the product of the OTHER messages of the
 * row, taken in order (csr_segment_product_vjp, python/tiga/tensor/core.py:
 * 1586-1598): zero-safe by construction, O(degree^2) per row. */
ORC_API void orc_csr_product_vjp_f32(const int64_t *row_ptr, int64_t N,
                                     const float *message, int64_t F,
                                     const float *dy, float *d_message) {
#pragma omp parallel for schedule(dynamic, 64)
  for (int64_t r = 0; r < N; ++r)
    for (int64_t e = row_ptr[r]; e < row_ptr[r + 1]; ++e)
      for (int64_t f = 0; f < F; ++f) {
        float product = dy[r * F + f];
        for (int64_t other = row_ptr[r]; other < row_ptr[r + 1]; ++other)
          if (other != e) product = product * message[other * F + f];
        d_message[e * F + f] = product;
      }
}

/* ------------------------------------------------------------------------ */
/* Max reducer (user Reducer whose combine is tg.math.maximum)               */
/* ------------------------------------------------------------------------ */

/* NaN-propagating maximum = arith.maximumf, the op the reference emits for
 * tg.math.maximum (lib/Target/Triton/Translate.cpp:172-181). */
static inline float orc_maximumf(float a, float b) {
  if (isnan(a)) return a;
  if (isnan(b)) return b;
  return a > b ? a : b;
}

/* out[i,f] = fold(maximumf, identity, w[e]*x[col[e],f]) left to right, the
 * variadic-reduce algebra branch (lib/Target/Triton/Translate.cpp:3353-3402)
 * with Reducer.identity() as the start value
 * (python/tiga/reducer/core.py:24-58).  argmax[i,f] = the first edge (global
 * edge id) whose message equals the final value, -1 when the identity wins
 * (this routing rule is this repository's definition: the reference has no
 * differentiable maximum, docs/reducers.md:270-277).  PARITY UNPINNED. */
ORC_API void orc_csr_max_fwd_f32(const int64_t *row_ptr, const int64_t *col_idx,
                                 int64_t N, const float *x, int64_t F,
                                 const float *w, float identity, float *out,
                                 int64_t *argmax) {
#pragma omp parallel for schedule(dynamic, 256)
  for (int64_t r = 0; r < N; ++r) {
    float *o = out + r * F;
    int64_t *a = argmax + r * F;
    for (int64_t f = 0; f < F; ++f) {
      o[f] = identity;
      a[f] = -1;
    }
    for (int64_t e = row_ptr[r]; e < row_ptr[r + 1]; ++e) {
      const float *xr = x + col_idx[e] * F;
      for (int64_t f = 0; f < F; ++f) {
        float m = w ? w[e] * xr[f] : xr[f];
        float prev = o[f];
        float next = orc_maximumf(prev, m);
        /* the winner changes when the message is strictly larger, or when a
         * NaN message first poisons a non-NaN state */
        if ((m > prev) || (isnan(m) && !isnan(prev))) a[f] = e;
        o[f] = next;
      }
    }
  }
}

/* Subgradient routing: the cotangent of (row, f) goes to the winning edge
 * only.  dx[col[e],f] += w[e]*dy[row,f]; dw[e] += dy[row,f]*x[col[e],f]. */
ORC_API void orc_csr_max_bwd_f32(const int64_t *row_ptr, const int64_t *col_idx,
                                 int64_t N, int64_t num_src, const float *dy,
                                 const float *x, int64_t F, const float *w,
                                 const int64_t *argmax, float *dx, float *dw) {
  int64_t E = row_ptr[N];
  if (dx) memset(dx, 0, sizeof(float) * (size_t)(num_src * F));
  if (dw) memset(dw, 0, sizeof(float) * (size_t)E);
  for (int64_t r = 0; r < N; ++r)
    for (int64_t f = 0; f < F; ++f) {
      int64_t e = argmax[r * F + f];
      if (e < 0) continue;
      float g = dy[r * F + f];
      if (dx) dx[col_idx[e] * F + f] += w ? w[e] * g : g;
      if (dw) dw[e] += g * x[col_idx[e] * F + f];
    }
}

/* ------------------------------------------------------------------------ */
/* Online-softmax reducer                                                    */
/* ------------------------------------------------------------------------ */

/* Generic online softmax over materialised per-edge scores/values
 * (python/tiga/interop/torch/reducer_oracle.py:60-137):
 *   m = max_e s[e,h]; p = exp(s-m); out[i,h,:] = sum p*v / sum p;
 * empty row -> 0 (reducer_oracle.py:132-136).  score [E,H], value [E,H,D],
 * all float32 (the accumulation dtype for 16-bit inputs,
 * reducer_oracle.py:22-28).  m_out/l_out [N,H] receive the saved row maximum
 * and denominator (python/tiga/compiler/edge_nn_attention.py:330-334). */
ORC_API void orc_online_softmax_fwd_f32(const int64_t *row_ptr, int64_t N,
                                        const float *score, const float *value,
                                        int64_t H, int64_t D, float *out,
                                        float *m_out, float *l_out) {
#pragma omp parallel for schedule(dynamic, 64)
  for (int64_t r = 0; r < N; ++r) {
    int64_t b = row_ptr[r], e_end = row_ptr[r + 1];
    for (int64_t h = 0; h < H; ++h) {
      float *o = out + (r * H + h) * D;
      for (int64_t d = 0; d < D; ++d) o[d] = 0.0f;
      float m = -INFINITY;
      for (int64_t e = b; e < e_end; ++e) m = fmaxf(m, score[e * H + h]);
      float l = 0.0f;
      for (int64_t e = b; e < e_end; ++e) {
        float p = expf(score[e * H + h] - m);
        l += p;
        const float *v = value + (e * H + h) * D;
        for (int64_t d = 0; d < D; ++d) o[d] += p * v[d];
      }
      if (l > 0.0f)
        for (int64_t d = 0; d < D; ++d) o[d] = o[d] / l;
      else
        for (int64_t d = 0; d < D; ++d) o[d] = 0.0f;
      if (m_out) m_out[r * H + h] = m;
      if (l_out) l_out[r * H + h] = l;
    }
  }
}

/* Backward of the online softmax w.r.t. per-edge score and value
 * (python/tiga/compiler/edge_nn_attention.py:548-575):
 *   w_e = exp(s_e-m)/l;  dvalue[e] = w_e*dO[row];
 *   dscore[e] = w_e*(<dO,v_e> - <dO,O[row]>). */
ORC_API void orc_online_softmax_bwd_f32(const int64_t *row_ptr, int64_t N,
                                        const float *score, const float *value,
                                        const float *out, const float *dout,
                                        int64_t H, int64_t D, float *dscore,
                                        float *dvalue) {
#pragma omp parallel for schedule(dynamic, 64)
  for (int64_t r = 0; r < N; ++r) {
    int64_t b = row_ptr[r], e_end = row_ptr[r + 1];
    for (int64_t h = 0; h < H; ++h) {
      const float *o = out + (r * H + h) * D;
      const float *g = dout + (r * H + h) * D;
      float m = -INFINITY;
      for (int64_t e = b; e < e_end; ++e) m = fmaxf(m, score[e * H + h]);
      double l = 0.0;
      for (int64_t e = b; e < e_end; ++e) l += exp((double)score[e * H + h] - m);
      double go = 0.0;
      for (int64_t d = 0; d < D; ++d) go += (double)g[d] * o[d];
      for (int64_t e = b; e < e_end; ++e) {
        double we = exp((double)score[e * H + h] - m) / l;
        const float *v = value + (e * H + h) * D;
        double gv = 0.0;
        for (int64_t d = 0; d < D; ++d) {
          gv += (double)g[d] * v[d];
          if (dvalue) dvalue[(e * H + h) * D + d] = (float)(we * g[d]);
        }
        if (dscore) dscore[e * H + h] = (float)(we * (gv - go));
      }
    }
  }
}

/* bfloat16 helpers: round-to-nearest-even, the rounding torch uses. */
static inline float orc_bf16_to_f32(uint16_t v) {
  uint32_t u = (uint32_t)v << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}
static inline uint16_t orc_f32_to_bf16(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40u);
  uint32_t rounding = 0x7fffu + ((u >> 16) & 1u);
  return (uint16_t)((u + rounding) >> 16);
}
static inline float orc_round_bf16(float f) {
  return orc_bf16_to_f32(orc_f32_to_bf16(f));
}

ORC_API void orc_f32_to_bf16_array(const float *in, uint16_t *out, int64_t n) {
  for (int64_t i = 0; i < n; ++i) out[i] = orc_f32_to_bf16(in[i]);
}
ORC_API void orc_bf16_to_f32_array(const uint16_t *in, float *out, int64_t n) {
  for (int64_t i = 0; i < n; ++i) out[i] = orc_bf16_to_f32(in[i]);
}

/* GAT edge attention on bf16 fields, the program
 *   s = (src.x*a_src).sum(-1) + (dst.x*a_dst).sum(-1)
 *   return online_softmax(maximum(s, 0.2*s), src.x)
 * evaluated the way the reference's eager evaluator does
 * (python/tiga/interop/torch/message_passing.py:2848-2894): every elementwise
 * bf16 op rounds its result to bf16, `.sum(-1)` accumulates in float32 and
 * rounds once, and only then the score is widened to float32 for the softmax
 * (reducer_oracle.py:87-91).  x [N,H,D] bf16, a_src/a_dst [H,D] bf16,
 * out [N,H,D] bf16, m_out/l_out [N,H] float32, score_out [E,H] float32
 * (optional; the bf16-rounded logits, exposed for the backward checks). */
ORC_API void orc_gat_fwd_bf16(const int64_t *row_ptr, const int64_t *col_idx,
                              int64_t N, const uint16_t *x_src,
                              const uint16_t *x_dst, const uint16_t *a_src,
                              const uint16_t *a_dst, int64_t H, int64_t D,
                              float slope, uint16_t *out, float *m_out,
                              float *l_out, float *score_out) {
  float slope_bf = orc_round_bf16(slope);
#pragma omp parallel for schedule(dynamic, 64)
  for (int64_t r = 0; r < N; ++r) {
    int64_t b = row_ptr[r], e_end = row_ptr[r + 1];
    for (int64_t h = 0; h < H; ++h) {
      float sd = 0.0f;
      for (int64_t d = 0; d < D; ++d)
        sd += orc_round_bf16(orc_bf16_to_f32(x_dst[(r * H + h) * D + d]) *
                             orc_bf16_to_f32(a_dst[h * D + d]));
      sd = orc_round_bf16(sd);
      float m = -INFINITY;
      int64_t deg = e_end - b;
      float *sc = (float *)malloc(sizeof(float) * (size_t)(deg ? deg : 1));
      for (int64_t e = b; e < e_end; ++e) {
        const uint16_t *xs = x_src + (col_idx[e] * H + h) * D;
        float ss = 0.0f;
        for (int64_t d = 0; d < D; ++d)
          ss += orc_round_bf16(orc_bf16_to_f32(xs[d]) *
                               orc_bf16_to_f32(a_src[h * D + d]));
        ss = orc_round_bf16(ss);
        float s = orc_round_bf16(ss + sd);
        float scaled = orc_round_bf16(slope_bf * s);
        float logit = orc_maximumf(s, scaled);
        sc[e - b] = logit;
        if (score_out) score_out[e * H + h] = logit;
        m = fmaxf(m, logit);
      }
      float l = 0.0f;
      float acc[1024];
      for (int64_t d = 0; d < D; ++d) acc[d] = 0.0f;
      for (int64_t e = b; e < e_end; ++e) {
        float p = expf(sc[e - b] - m);
        l += p;
        const uint16_t *xs = x_src + (col_idx[e] * H + h) * D;
        for (int64_t d = 0; d < D; ++d) acc[d] += p * orc_bf16_to_f32(xs[d]);
      }
      for (int64_t d = 0; d < D; ++d)
        out[(r * H + h) * D + d] =
            orc_f32_to_bf16(l > 0.0f ? acc[d] / l : 0.0f);
      if (m_out) m_out[r * H + h] = m;
      if (l_out) l_out[r * H + h] = l;
      free(sc);
    }
  }
}

/* Analytic float32/float64 backward of the GAT program above; gradients for
 * x (as source and as destination, summed when x_src == x_dst is intended the
 * caller adds them), a_src and a_dst, all returned in float32.  The
 * leaky-relu derivative is taken at the bf16-rounded pre-activation, like
 * torch.maximum's subgradient (s >= 0.2*s picks s; ties split evenly in
 * torch, which only happens at s == 0). */
ORC_API void orc_gat_bwd_bf16(const int64_t *row_ptr, const int64_t *col_idx,
                              int64_t N, int64_t num_src, const uint16_t *x_src,
                              const uint16_t *x_dst, const uint16_t *a_src,
                              const uint16_t *a_dst, int64_t H, int64_t D,
                              float slope, const uint16_t *dout, float *dx_src,
                              float *dx_dst, float *da_src, float *da_dst) {
  float slope_bf = orc_round_bf16(slope);
  memset(dx_src, 0, sizeof(float) * (size_t)(num_src * H * D));
  memset(dx_dst, 0, sizeof(float) * (size_t)(N * H * D));
  double *das = (double *)calloc((size_t)(H * D), sizeof(double));
  double *dad = (double *)calloc((size_t)(H * D), sizeof(double));
  for (int64_t r = 0; r < N; ++r) {
    int64_t b = row_ptr[r], e_end = row_ptr[r + 1], deg = e_end - b;
    if (!deg) continue;
    for (int64_t h = 0; h < H; ++h) {
      float sd = 0.0f;
      for (int64_t d = 0; d < D; ++d)
        sd += orc_round_bf16(orc_bf16_to_f32(x_dst[(r * H + h) * D + d]) *
                             orc_bf16_to_f32(a_dst[h * D + d]));
      sd = orc_round_bf16(sd);
      double *logit = (double *)malloc(sizeof(double) * (size_t)deg);
      double *pre = (double *)malloc(sizeof(double) * (size_t)deg);
      double m = -INFINITY;
      for (int64_t e = b; e < e_end; ++e) {
        const uint16_t *xs = x_src + (col_idx[e] * H + h) * D;
        float ss = 0.0f;
        for (int64_t d = 0; d < D; ++d)
          ss += orc_round_bf16(orc_bf16_to_f32(xs[d]) *
                               orc_bf16_to_f32(a_src[h * D + d]));
        ss = orc_round_bf16(ss);
        float s = orc_round_bf16(ss + sd);
        float scaled = orc_round_bf16(slope_bf * s);
        pre[e - b] = s;
        logit[e - b] = orc_maximumf(s, scaled);
        if (logit[e - b] > m) m = logit[e - b];
      }
      double l = 0.0;
      for (int64_t k = 0; k < deg; ++k) l += exp(logit[k] - m);
      /* O[row] in float64 */
      double o[1024], g[1024];
      for (int64_t d = 0; d < D; ++d) {
        o[d] = 0.0;
        g[d] = orc_bf16_to_f32(dout[(r * H + h) * D + d]);
      }
      for (int64_t e = b; e < e_end; ++e) {
        double we = exp(logit[e - b] - m) / l;
        const uint16_t *xs = x_src + (col_idx[e] * H + h) * D;
        for (int64_t d = 0; d < D; ++d) o[d] += we * orc_bf16_to_f32(xs[d]);
      }
      double go = 0.0;
      for (int64_t d = 0; d < D; ++d) go += g[d] * o[d];
      for (int64_t e = b; e < e_end; ++e) {
        double we = exp(logit[e - b] - m) / l;
        const uint16_t *xs = x_src + (col_idx[e] * H + h) * D;
        double gv = 0.0;
        for (int64_t d = 0; d < D; ++d) gv += g[d] * orc_bf16_to_f32(xs[d]);
        double ds = we * (gv - go);
        double s = pre[e - b];
        double dpre = s > 0.0 ? ds : (s < 0.0 ? slope_bf * ds
                                              : 0.5 * (1.0 + slope_bf) * ds);
        for (int64_t d = 0; d < D; ++d) {
          double xv = orc_bf16_to_f32(xs[d]);
          double as = orc_bf16_to_f32(a_src[h * D + d]);
          double ad = orc_bf16_to_f32(a_dst[h * D + d]);
          double xd = orc_bf16_to_f32(x_dst[(r * H + h) * D + d]);
          dx_src[(col_idx[e] * H + h) * D + d] += (float)(we * g[d] + dpre * as);
          dx_dst[(r * H + h) * D + d] += (float)(dpre * ad);
          das[h * D + d] += dpre * xv;
          dad[h * D + d] += dpre * xd;
        }
      }
      free(logit);
      free(pre);
    }
  }
  for (int64_t k = 0; k < H * D; ++k) {
    da_src[k] = (float)das[k];
    da_dst[k] = (float)dad[k];
  }
  free(das);
  free(dad);
}

/* ------------------------------------------------------------------------ */
/* Dense (causal, variable-length) relation with the online-softmax reducer  */
/* ------------------------------------------------------------------------ */

/* softmax(q k^T * scale + causal) v inside each sequence of a packed batch:
 * position i of sequence k gathers from sources [start_k, i]
 * (Graph.cu_seqlens, python/tiga/interop/torch/graph.py:259-294; the streaming
 * kernel's mask `src <= row`, lib/Target/Triton/Translate.cpp:1774-1784).
 * q,k,v [T,H,D] float32 (bf16 values widened by the caller), out [T,H,D],
 * lse [T,H] = m + log(l).  Accumulation in float64. */
ORC_API void orc_varlen_attn_fwd(const int64_t *cu_seqlens, int64_t S,
                                 const float *q, const float *k, const float *v,
                                 int64_t H, int64_t D, float scale, int causal,
                                 float *out, float *lse) {
  for (int64_t s = 0; s < S; ++s) {
    int64_t b = cu_seqlens[s], e_end = cu_seqlens[s + 1];
#pragma omp parallel for schedule(dynamic, 8)
    for (int64_t i = b; i < e_end; ++i) {
      int64_t last = causal ? i + 1 : e_end;
      double *p = (double *)malloc(sizeof(double) * (size_t)(last - b));
      for (int64_t h = 0; h < H; ++h) {
        const float *qi = q + (i * H + h) * D;
        double m = -INFINITY;
        for (int64_t j = b; j < last; ++j) {
          const float *kj = k + (j * H + h) * D;
          double dot = 0.0;
          for (int64_t d = 0; d < D; ++d) dot += (double)qi[d] * kj[d];
          p[j - b] = dot * scale;
          if (p[j - b] > m) m = p[j - b];
        }
        double l = 0.0;
        for (int64_t j = b; j < last; ++j) {
          p[j - b] = exp(p[j - b] - m);
          l += p[j - b];
        }
        float *o = out + (i * H + h) * D;
        for (int64_t d = 0; d < D; ++d) {
          double acc = 0.0;
          for (int64_t j = b; j < last; ++j)
            acc += p[j - b] * v[(j * H + h) * D + d];
          o[d] = (float)(acc / l);
        }
        if (lse) lse[i * H + h] = (float)(m + log(l));
      }
      free(p);
    }
  }
}

/* Backward of the above (standard softmax-attention adjoint; the reference
 * has no dense backward, docs/roadmap.md "Backward unsupported"): with
 * P = softmax rows, dV = P^T dO, dP = dO V^T, dS = P*(dP - rowsum(dO*O)),
 * dQ = dS K * scale, dK = dS^T Q * scale.  Accumulation in float64. */
ORC_API void orc_varlen_attn_bwd(const int64_t *cu_seqlens, int64_t S,
                                 const float *q, const float *k, const float *v,
                                 const float *out, const float *dout, int64_t H,
                                 int64_t D, float scale, int causal, float *dq,
                                 float *dk, float *dv) {
  int64_t T = cu_seqlens[S];
  double *dk64 = (double *)calloc((size_t)(T * H * D), sizeof(double));
  double *dv64 = (double *)calloc((size_t)(T * H * D), sizeof(double));
  for (int64_t s = 0; s < S; ++s) {
    int64_t b = cu_seqlens[s], e_end = cu_seqlens[s + 1];
    for (int64_t i = b; i < e_end; ++i) {
      int64_t last = causal ? i + 1 : e_end;
      double *p = (double *)malloc(sizeof(double) * (size_t)(last - b));
      for (int64_t h = 0; h < H; ++h) {
        const float *qi = q + (i * H + h) * D;
        const float *gi = dout + (i * H + h) * D;
        const float *oi = out + (i * H + h) * D;
        double m = -INFINITY;
        for (int64_t j = b; j < last; ++j) {
          double dot = 0.0;
          for (int64_t d = 0; d < D; ++d)
            dot += (double)qi[d] * k[(j * H + h) * D + d];
          p[j - b] = dot * scale;
          if (p[j - b] > m) m = p[j - b];
        }
        double l = 0.0;
        for (int64_t j = b; j < last; ++j) {
          p[j - b] = exp(p[j - b] - m);
          l += p[j - b];
        }
        double delta = 0.0;
        for (int64_t d = 0; d < D; ++d) delta += (double)gi[d] * oi[d];
        double dqi[1024];
        for (int64_t d = 0; d < D; ++d) dqi[d] = 0.0;
        for (int64_t j = b; j < last; ++j) {
          double pj = p[j - b] / l;
          double dp = 0.0;
          for (int64_t d = 0; d < D; ++d)
            dp += (double)gi[d] * v[(j * H + h) * D + d];
          double ds = pj * (dp - delta) * scale;
          for (int64_t d = 0; d < D; ++d) {
            dqi[d] += ds * k[(j * H + h) * D + d];
            dk64[(j * H + h) * D + d] += ds * qi[d];
            dv64[(j * H + h) * D + d] += pj * gi[d];
          }
        }
        for (int64_t d = 0; d < D; ++d) dq[(i * H + h) * D + d] = (float)dqi[d];
      }
      free(p);
    }
  }
  for (int64_t t = 0; t < T * H * D; ++t) {
    dk[t] = (float)dk64[t];
    dv[t] = (float)dv64[t];
  }
  free(dk64);
  free(dv64);
}

/* ------------------------------------------------------------------------ */
/* Dense linear after the aggregation (user code `aggregate @ W`)             */
/* ------------------------------------------------------------------------ */

/* out[n,j] = sum_k a[n,k]*W[k,j], float32 data, float64 accumulation. */
ORC_API void orc_linear_f32(const float *a, const float *W, int64_t N,
                            int64_t K, int64_t J, float *out) {
#pragma omp parallel for schedule(static)
  for (int64_t n = 0; n < N; ++n)
    for (int64_t j = 0; j < J; ++j) {
      double acc = 0.0;
      for (int64_t kk = 0; kk < K; ++kk) acc += (double)a[n * K + kk] * W[kk * J + j];
      out[n * J + j] = (float)acc;
    }
}

/* ------------------------------------------------------------------------ */
/* Destination partitioning and halo maps                                    */
/* ------------------------------------------------------------------------ */

/* owned_range (python/tiga/distributed/model.py:124-130). */
ORC_API void orc_owned_range(int64_t entities, int64_t world, int64_t rank,
                             int64_t *begin, int64_t *end) {
  int64_t base = entities / world, rem = entities % world;
  *begin = rank * base + (rank < rem ? rank : rem);
  *end = *begin + base + (rank < rem ? 1 : 0);
}

/* destination_owner (python/tiga/distributed/model.py:113-121). */
ORC_API int64_t orc_destination_owner(int64_t entity, int64_t entities,
                                      int64_t world) {
  int64_t base = entities / world, rem = entities % world;
  int64_t wide = (base + 1) * rem;
  if (entity < wide) return entity / (base + 1);
  return base ? rem + (entity - wide) / base : rem;
}

static int orc_cmp_i64(const void *a, const void *b) {
  int64_t x = *(const int64_t *)a, y = *(const int64_t *)b;
  return (x > y) - (x < y);
}

/* derive_halo_map (python/tiga/distributed/model.py:133-194): ghosts = sorted
 * unique sources of the owned rows that lie outside the owned range.  Returns
 * the ghost count; ghost_ids must have room for every edge of the owned rows
 * (call with ghost_ids == NULL to get the count only). */
ORC_API int64_t orc_derive_ghosts(const int64_t *row_ptr, const int64_t *col_idx,
                                  int64_t num_entities, int64_t world,
                                  int64_t rank, int64_t *ghost_ids) {
  int64_t begin, end;
  orc_owned_range(num_entities, world, rank, &begin, &end);
  int64_t lo = row_ptr[begin], hi = row_ptr[end];
  int64_t *tmp = (int64_t *)malloc(sizeof(int64_t) * (size_t)(hi - lo + 1));
  int64_t n = 0;
  for (int64_t e = lo; e < hi; ++e)
    if (col_idx[e] < begin || col_idx[e] >= end) tmp[n++] = col_idx[e];
  qsort(tmp, (size_t)n, sizeof(int64_t), orc_cmp_i64);
  int64_t u = 0;
  for (int64_t k = 0; k < n; ++k)
    if (k == 0 || tmp[k] != tmp[k - 1]) {
      if (ghost_ids) ghost_ids[u] = tmp[k];
      ++u;
    }
  free(tmp);
  return u;
}

/* Local CSR of one rank: owned rows re-based to 0, owned sources renumbered
 * to [0, n_owned) and ghost sources to n_owned + position in the ascending
 * ghost list (python/tiga/distributed/transport.py:819-823).  local_ptr has
 * n_owned+1 entries, local_col as many as the owned rows hold edges. */
ORC_API void orc_local_csr(const int64_t *row_ptr, const int64_t *col_idx,
                           int64_t num_entities, int64_t world, int64_t rank,
                           const int64_t *ghost_ids, int64_t n_ghost,
                           int64_t *local_ptr, int64_t *local_col) {
  int64_t begin, end;
  orc_owned_range(num_entities, world, rank, &begin, &end);
  int64_t base = row_ptr[begin];
  for (int64_t r = begin; r <= end; ++r) local_ptr[r - begin] = row_ptr[r] - base;
  for (int64_t e = row_ptr[begin]; e < row_ptr[end]; ++e) {
    int64_t c = col_idx[e];
    if (c >= begin && c < end) {
      local_col[e - base] = c - begin;
    } else {
      int64_t lo = 0, hi = n_ghost;
      while (lo < hi) {
        int64_t mid = (lo + hi) / 2;
        if (ghost_ids[mid] < c) lo = mid + 1; else hi = mid;
      }
      local_col[e - base] = (end - begin) + lo;
    }
  }
}
