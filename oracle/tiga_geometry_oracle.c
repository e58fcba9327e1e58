/*
 * tiga_geometry_oracle.c -- CPU restatement of the reference's dynamic relation builders.
 * TEST INFRASTRUCTURE ONLY: linked into libtiga_oracle.so, called by tests, the smoke check and the
 * CPU-baseline leg of the benchmark; the product library never links or calls it.
 *
 * Restates, in plain C, what walkerchi/TIGA-lang does with Torch tensor operations:
 *   orc_radius_build    Graph.radius -> resolve_csr, uniform cell list broad phase and all-pairs path
 *                       (python/tiga/interop/torch/graph.py:947-1003 driver, :1023-1125 cell-list
 *                       candidates, :1127-1176 pair selection, :1203-1210 minimum image)
 *   orc_knn_build       Graph.knn -> resolve_csr (graph.py:854-895), ranked by (squared distance,
 *                       source index), the key tests/python/test_ranked_rebinding.py:88-104 pins
 *   orc_edge_geometry   Graph.implicit_edge_fields (graph.py:1403-1444)
 *
 * Arithmetic is float32 in the reference's operation order: the Euclidean norm is
 * sqrt(fma(z, z, fma(y, y, x * x))) and a [n, D] @ [D, D] product accumulates with fused
 * multiply-adds in increasing k, which is what the reference's Torch CPU build evaluates bit for bit
 * (pinned against tests/golden/geometry_cases.npz).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORC_API __attribute__((visibility("default")))
#define ORC_MAX_DIM 3

typedef struct {
  int64_t key;
  int64_t index;
} orc_keyed;

static int orc_cmp_keyed(const void *a, const void *b) {
  const orc_keyed *x = (const orc_keyed *)a, *y = (const orc_keyed *)b;
  if (x->key != y->key) return x->key < y->key ? -1 : 1;
  return x->index < y->index ? -1 : (x->index > y->index);
}

/* row [1, D] @ matrix [D, D], row-major, fused multiply-add chain in increasing k */
static void orc_row_times_matrix(const float *row, const float *m, int D, float *out) {
  for (int a = 0; a < D; ++a) {
    float acc = row[0] * m[a];
    for (int k = 1; k < D; ++k) acc = fmaf(row[k], m[k * D + a], acc);
    out[a] = acc;
  }
}

static float orc_norm(const float *v, int D) {
  float acc = v[0] * v[0];
  for (int k = 1; k < D; ++k) acc = fmaf(v[k], v[k], acc);
  return sqrtf(acc);
}

/* displacement = source - destination, mapped to the centred periodic cell when a lattice is given */
static void orc_displacement(const float *src, const float *dst, int D, const float *lattice,
                             const float *inverse, float *out) {
  float d[8];
  for (int a = 0; a < D; ++a) d[a] = src[a] - dst[a];
  if (lattice) {
    float f[8];
    orc_row_times_matrix(d, inverse, D, f);
    for (int a = 0; a < D; ++a) f[a] = f[a] - rintf(f[a]); /* torch.round: half to even */
    orc_row_times_matrix(f, lattice, D, d);
  }
  for (int a = 0; a < D; ++a) out[a] = d[a];
}

/*
 * Radius relation.  positions [n, D] float32; cutoff: one value (cutoff_count == 1) or one per
 * destination (cutoff_count == n); lattice / inverse [D, D] or NULL; extents [D] (periodic only: cells
 * per axis, computed by the caller exactly as graph.py:1051-1054).  use_cells = 0 runs the all-pairs
 * path (any D <= 8), 1 the cell list (D <= 3).  Two-call protocol: with col == NULL only row_ptr and
 * the counts are produced.  Returns the number of edges, or -1 on a bad argument.
 * Edge order: destination ascending; inside a row the cell list visits the 3^D neighbour cells in
 * meshgrid 'ij' order (first axis slowest) and the points of a cell in ascending index; the all-pairs
 * path visits sources in ascending index.
 */
ORC_API int64_t orc_radius_build(const float *positions, int64_t n, int32_t D, const float *cutoff,
                                 int64_t cutoff_count, int32_t exclude_self, const float *lattice,
                                 const float *inverse, const int64_t *extents_in, int32_t use_cells,
                                 int64_t *row_ptr, int64_t *col, float *distance, float *displacement,
                                 int64_t *candidate_pairs) {
  if (n < 0 || D < 1 || D > 8 || (use_cells && D > ORC_MAX_DIM)) return -1;
  if (cutoff_count != 1 && cutoff_count != n) return -1;
  int64_t edges = 0, candidates = 0;
  row_ptr[0] = 0;
  if (!use_cells) {
    for (int64_t i = 0; i < n; ++i) {
      for (int64_t j = 0; j < n; ++j) {
        float d[8];
        orc_displacement(positions + j * D, positions + i * D, D, lattice, inverse, d);
        const float dist = orc_norm(d, D);
        const float limit = cutoff[cutoff_count == 1 ? 0 : i];
        if (!(dist <= limit) || (exclude_self && i == j)) continue;
        if (col) {
          col[edges] = j;
          if (distance) distance[edges] = dist;
          if (displacement) memcpy(displacement + edges * D, d, sizeof(float) * D);
        }
        ++edges;
      }
      row_ptr[i + 1] = edges;
    }
    if (candidate_pairs) *candidate_pairs = n * n;
    return edges;
  }
  if (n == 0) {
    if (candidate_pairs) *candidate_pairs = 0;
    return 0;
  }
  const float cell_size = cutoff[0];
  int64_t *cells = (int64_t *)malloc(sizeof(int64_t) * n * D);
  orc_keyed *sorted = (orc_keyed *)malloc(sizeof(orc_keyed) * n);
  int64_t lower[ORC_MAX_DIM] = {0, 0, 0}, upper[ORC_MAX_DIM] = {0, 0, 0}, extents[ORC_MAX_DIM] = {1, 1, 1};
  if (lattice) {
    for (int a = 0; a < D; ++a) {
      extents[a] = extents_in[a];
      upper[a] = extents[a] - 1;
    }
    for (int64_t i = 0; i < n; ++i) {
      float f[ORC_MAX_DIM];
      orc_row_times_matrix(positions + i * D, inverse, D, f);
      for (int a = 0; a < D; ++a) {
        const float frac = f[a] - floorf(f[a]);
        int64_t c = (int64_t)floorf(frac * (float)extents[a]);
        cells[i * D + a] = c < extents[a] - 1 ? c : extents[a] - 1;
      }
    }
  } else {
    for (int64_t i = 0; i < n; ++i)
      for (int a = 0; a < D; ++a) {
        const int64_t c = (int64_t)floorf(positions[i * D + a] / cell_size);
        cells[i * D + a] = c;
        if (i == 0 || c < lower[a]) lower[a] = c;
        if (i == 0 || c > upper[a]) upper[a] = c;
      }
    for (int a = 0; a < D; ++a) extents[a] = upper[a] - lower[a] + 1;
  }
  int64_t strides[ORC_MAX_DIM] = {1, 1, 1};
  for (int a = 1; a < D; ++a) strides[a] = strides[a - 1] * extents[a - 1];
  for (int64_t i = 0; i < n; ++i) {
    int64_t key = 0;
    for (int a = 0; a < D; ++a) key += (cells[i * D + a] - lower[a]) * strides[a];
    sorted[i].key = key;
    sorted[i].index = i;
  }
  qsort(sorted, (size_t)n, sizeof(orc_keyed), orc_cmp_keyed);
  /* neighbour offsets per axis: periodic axes of extent 1 / 2 visit each image cell once */
  int axis_count[ORC_MAX_DIM] = {1, 1, 1};
  int64_t axis_value[ORC_MAX_DIM][3] = {{0, 0, 0}, {0, 0, 0}, {0, 0, 0}};
  for (int a = 0; a < D; ++a) {
    if (lattice && extents[a] == 1) {
      axis_count[a] = 1;
      axis_value[a][0] = 0;
    } else if (lattice && extents[a] == 2) {
      axis_count[a] = 2;
      axis_value[a][0] = 0;
      axis_value[a][1] = 1;
    } else {
      axis_count[a] = 3;
      axis_value[a][0] = -1;
      axis_value[a][1] = 0;
      axis_value[a][2] = 1;
    }
  }
  for (int64_t i = 0; i < n; ++i) {
    int o[ORC_MAX_DIM] = {0, 0, 0};
    for (;;) {
      int64_t key = 0;
      int valid = 1;
      for (int a = 0; a < D; ++a) {
        int64_t c = cells[i * D + a] + axis_value[a][o[a]];
        if (lattice) {
          c %= extents[a];
          if (c < 0) c += extents[a];
        } else if (c < lower[a] || c > upper[a]) {
          valid = 0;
        }
        key += (c - lower[a]) * strides[a];
      }
      if (valid) {
        int64_t lo = 0, hi = n; /* first entry of the cell in the sorted order */
        while (lo < hi) {
          const int64_t mid = (lo + hi) / 2;
          if (sorted[mid].key < key) lo = mid + 1; else hi = mid;
        }
        for (int64_t s = lo; s < n && sorted[s].key == key; ++s) {
          const int64_t j = sorted[s].index;
          ++candidates;
          float d[ORC_MAX_DIM];
          orc_displacement(positions + j * D, positions + i * D, D, lattice, inverse, d);
          const float dist = orc_norm(d, D);
          if (!(dist <= cell_size) || (exclude_self && i == j)) continue;
          if (col) {
            col[edges] = j;
            if (distance) distance[edges] = dist;
            if (displacement) memcpy(displacement + edges * D, d, sizeof(float) * D);
          }
          ++edges;
        }
      }
      int a = D - 1; /* meshgrid 'ij': last axis fastest */
      while (a >= 0 && ++o[a] == axis_count[a]) o[a--] = 0;
      if (a < 0) break;
    }
    row_ptr[i + 1] = edges;
  }
  free(cells);
  free(sorted);
  if (candidate_pairs) *candidate_pairs = candidates;
  return edges;
}

/*
 * Exact k nearest candidates of every query, ascending by (squared distance, candidate index).
 * col [nq, k] int64.  exclude_self drops candidate i of query i (self search only).
 */
ORC_API int32_t orc_knn_build(const float *queries, int64_t nq, const float *candidates, int64_t nc,
                              int32_t D, int32_t k, int32_t exclude_self, int64_t *col) {
  if (k < 1 || k > nc - (exclude_self ? 1 : 0) || D < 1) return -1;
  float *best = (float *)malloc(sizeof(float) * (size_t)k);
  for (int64_t i = 0; i < nq; ++i) {
    int filled = 0;
    int64_t *row = col + i * k;
    for (int64_t j = 0; j < nc; ++j) {
      if (exclude_self && i == j) continue;
      float acc = 0.0f;
      for (int a = 0; a < D; ++a) {
        const float d = candidates[j * D + a] - queries[i * D + a];
        acc = a == 0 ? d * d : fmaf(d, d, acc);
      }
      if (filled == k && !(acc < best[k - 1])) continue;
      int at = filled < k ? filled++ : k - 1;
      while (at > 0 && best[at - 1] > acc) {
        best[at] = best[at - 1];
        row[at] = row[at - 1];
        --at;
      }
      best[at] = acc;
      row[at] = j;
    }
  }
  free(best);
  return 0;
}

/* displacement [E, D] and distance [E] of stored edges (destination of edge e = dst[e]) */
ORC_API void orc_edge_geometry(const float *dst_positions, const float *src_positions, int32_t D,
                               const int64_t *dst, const int64_t *col, int64_t edges, const float *lattice,
                               const float *inverse, float *displacement, float *distance) {
  for (int64_t e = 0; e < edges; ++e) {
    float d[8];
    orc_displacement(src_positions + col[e] * D, dst_positions + dst[e] * D, D, lattice, inverse, d);
    if (displacement) memcpy(displacement + e * D, d, sizeof(float) * D);
    if (distance) distance[e] = orc_norm(d, D);
  }
}
