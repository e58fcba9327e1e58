// Dynamic relations on the device: radius (cell list) and exact k-nearest-neighbour builders, the
// implicit edge geometry, and a fused radius consumer that folds weight(i, j) * x[j] over the
// neighbours of i without ever writing the relation.
//
// Follows the behaviour of Graph.radius / Graph.knn of walkerchi/TIGA-lang
// (python/tiga/interop/torch/graph.py:851-1003 resolve_csr, :1023-1125 cell-list candidates,
// :1127-1176 pair selection, :1203-1210 minimum image, :1403-1444 implicit edge fields) with its own
// device data structure: points are sorted (stable radix sort) into modular hash buckets of their
// cells; a destination walks its 3^D neighbour cells in the reference's order, filters the bucket's
// points by exact cell coordinates (so hash collisions and wrapped duplicates cost time, never
// correctness) and applies the exact float32 distance test.  Count -> scan -> fill gives the CSR in
// the reference's edge order; the fused consumer runs the same walk and accumulates instead.
//
// Bound: latency / L2 (a few MB of points, gathered); algorithmic bytes per destination are
// 16 B (own point + cell) + 32 B per candidate + 4 B * F per accepted pair.
#include <cub/cub.cuh>

#include "tgb_common.cuh"

namespace tgb {
namespace {

constexpr int kThreads = 128;

inline unsigned grid_for(int64_t n, int per_block = kThreads) {
  return (unsigned)(n > 0 ? ceil_div(n, per_block) : 1);
}

// ---- the cell space as the kernels see it ------------------------------------------------------
struct Space {
  int dims;
  int periodic;
  float cell_size;
  float lattice[9];
  float inverse[9];
  int extents[3];
  int axis_count[3];     // neighbour offsets visited per axis
  int axis_first[3];     // first offset of the axis (-1 or 0)
  int bits;              // bucket bits per axis
};

// Directory arrays inside the caller's `persistent` block.
struct Directory {
  float4 *points;        // [n] x, y, z, index bits; sorted by bucket, ascending index inside
  int4 *cells;           // [n] cell coordinates of points[s]
  int4 *own_cell;        // [n] cell coordinates of point i (original order)
  int32_t *bucket_ptr;   // [buckets + 1]
  int64_t buckets;
};

int bucket_bits_per_axis(int64_t n, int dims) {
  int total = 1;
  while (((int64_t)1 << total) < 2 * (n > 1 ? n : 1)) ++total;   // about two buckets per point
  int bits = (total + dims - 1) / dims;
  const int cap = dims == 1 ? 26 : (dims == 2 ? 13 : 9);
  if (bits > cap) bits = cap;
  if (bits < 2) bits = 2;          // at least four residues per axis: the offsets -1, 0, 1 stay distinct
  return bits;
}

struct DirectoryLayout {
  uint64_t points, cells, own_cell, bucket_ptr, persistent_bytes;
  uint64_t k0, k1, v0, v1, counts, cub, cub_bytes, temp_bytes;
  int64_t buckets;
};

int32_t directory_layout(int64_t n, int dims, DirectoryLayout *L) {
  if (n < 0 || n >= ((int64_t)1 << 31)) TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "point count out of range");
  if (dims < 1 || dims > 3) TGB_FAIL(TGB_STATUS_UNSUPPORTED, "the cell list covers 1, 2 or 3 dimensions");
  const int64_t m = n > 0 ? n : 1;
  L->buckets = (int64_t)1 << (bucket_bits_per_axis(n, dims) * dims);
  uint64_t p = 0;
  auto take = [&](uint64_t bytes) {
    uint64_t at = p;
    p = align_up(p + bytes, 256);
    return at;
  };
  L->points = take((uint64_t)m * 16);
  L->cells = take((uint64_t)m * 16);
  L->own_cell = take((uint64_t)m * 16);
  L->bucket_ptr = take((uint64_t)(L->buckets + 1) * 4);
  L->persistent_bytes = p;
  size_t sort_bytes = 0, scan_bytes = 0;
  cub::DoubleBuffer<uint32_t> dk(nullptr, nullptr), dv(nullptr, nullptr);
  cudaError_t err = cub::DeviceRadixSort::SortPairs(nullptr, sort_bytes, dk, dv, (int64_t)m, 0, 32,
                                                    (cudaStream_t)0);
  if (err != cudaSuccess) TGB_FAIL(TGB_STATUS_INTERNAL, "cub sort size query failed: %s", cudaGetErrorString(err));
  err = cub::DeviceScan::ExclusiveSum(nullptr, scan_bytes, (int32_t *)nullptr, (int64_t *)nullptr,
                                      (int64_t)(m + 1), (cudaStream_t)0);
  if (err != cudaSuccess) TGB_FAIL(TGB_STATUS_INTERNAL, "cub scan size query failed: %s", cudaGetErrorString(err));
  p = 0;
  L->k0 = take((uint64_t)m * 4);
  L->k1 = take((uint64_t)m * 4);
  L->v0 = take((uint64_t)m * 4);
  L->v1 = take((uint64_t)m * 4);
  L->counts = take((uint64_t)(m + 1) * 4);
  L->cub_bytes = (sort_bytes > scan_bytes ? sort_bytes : scan_bytes) + 256;
  L->cub = take(L->cub_bytes);
  L->temp_bytes = p;
  return TGB_STATUS_OK;
}

int32_t make_space(const tgb_cell_space *in, int64_t n, Space *out) {
  if (!in) TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "null cell space");
  if (in->dims < 1 || in->dims > 3) TGB_FAIL(TGB_STATUS_UNSUPPORTED, "the cell list covers 1, 2 or 3 dimensions");
  if (!(in->cell_size > 0.0f)) TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "cell size must be positive");
  out->dims = in->dims;
  out->periodic = in->periodic ? 1 : 0;
  out->cell_size = in->cell_size;
  for (int i = 0; i < 9; ++i) {
    out->lattice[i] = in->lattice[i];
    out->inverse[i] = in->inverse[i];
  }
  for (int a = 0; a < 3; ++a) {
    out->extents[a] = a < in->dims ? in->extents[a] : 1;
    out->axis_count[a] = 1;
    out->axis_first[a] = 0;
    if (a >= in->dims) continue;
    if (out->periodic) {
      if (in->extents[a] < 1) TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "periodic extents must be at least 1");
      // axes of one or two cells visit every image cell once (graph.py:1075-1084)
      out->axis_count[a] = in->extents[a] == 1 ? 1 : (in->extents[a] == 2 ? 2 : 3);
      out->axis_first[a] = in->extents[a] <= 2 ? 0 : -1;
    } else {
      out->axis_count[a] = 3;
      out->axis_first[a] = -1;
    }
  }
  out->bits = bucket_bits_per_axis(n, in->dims);
  return TGB_STATUS_OK;
}

Directory directory_at(void *persistent, const DirectoryLayout &L) {
  char *base = static_cast<char *>(persistent);
  return Directory{reinterpret_cast<float4 *>(base + L.points), reinterpret_cast<int4 *>(base + L.cells),
                   reinterpret_cast<int4 *>(base + L.own_cell),
                   reinterpret_cast<int32_t *>(base + L.bucket_ptr), L.buckets};
}

// ---- float32 arithmetic in the reference's order ----------------------------------------------
// row [1, D] @ matrix [D, D]: fused multiply-add chain in increasing k
template <int D>
__device__ __forceinline__ void row_times_matrix(const float (&row)[3], const float *m, float (&out)[3]) {
#pragma unroll
  for (int a = 0; a < D; ++a) {
    float acc = __fmul_rn(row[0], m[a]);
#pragma unroll
    for (int k = 1; k < D; ++k) acc = __fmaf_rn(row[k], m[k * D + a], acc);
    out[a] = acc;
  }
}

template <int D>
__device__ __forceinline__ float norm_of(const float (&v)[3]) {
  float acc = __fmul_rn(v[0], v[0]);
#pragma unroll
  for (int k = 1; k < D; ++k) acc = __fmaf_rn(v[k], v[k], acc);
  return __fsqrt_rn(acc);
}

// displacement source - destination, mapped into the centred periodic cell
template <int D, bool PERIODIC>
__device__ __forceinline__ void displacement_of(const float (&src)[3], const float (&dst)[3], const Space &sp,
                                                float (&out)[3]) {
#pragma unroll
  for (int a = 0; a < D; ++a) out[a] = __fsub_rn(src[a], dst[a]);
  if (PERIODIC) {
    float f[3];
    row_times_matrix<D>(out, sp.inverse, f);
#pragma unroll
    for (int a = 0; a < D; ++a) f[a] = __fsub_rn(f[a], rintf(f[a]));
    row_times_matrix<D>(f, sp.lattice, out);
  }
}

template <int D>
__device__ __forceinline__ void cell_of(const float (&p)[3], const Space &sp, int (&cell)[3]) {
  if (sp.periodic) {
    float f[3];
    row_times_matrix<D>(p, sp.inverse, f);
#pragma unroll
    for (int a = 0; a < D; ++a) {
      const float frac = __fsub_rn(f[a], floorf(f[a]));
      const int c = (int)floorf(__fmul_rn(frac, (float)sp.extents[a]));
      cell[a] = c < sp.extents[a] - 1 ? c : sp.extents[a] - 1;
    }
  } else {
#pragma unroll
    for (int a = 0; a < D; ++a) cell[a] = (int)floorf(__fdiv_rn(p[a], sp.cell_size));
  }
#pragma unroll
  for (int a = D; a < 3; ++a) cell[a] = 0;
}

template <int D>
__device__ __forceinline__ uint32_t bucket_of(const int (&cell)[3], int bits) {
  const uint32_t mask = (1u << bits) - 1u;
  uint32_t b = (uint32_t)cell[0] & mask;
  if (D > 1) b |= ((uint32_t)cell[1] & mask) << bits;
  if (D > 2) b |= ((uint32_t)cell[2] & mask) << (2 * bits);
  return b;
}

template <int D>
__device__ __forceinline__ void load_point(const float *positions, int64_t i, float (&p)[3]) {
#pragma unroll
  for (int a = 0; a < D; ++a) p[a] = __ldg(positions + i * D + a);
#pragma unroll
  for (int a = D; a < 3; ++a) p[a] = 0.0f;
}

// ---- directory construction --------------------------------------------------------------------
template <int D>
__global__ void __launch_bounds__(kThreads)
k_cell_keys(const float *__restrict__ positions, int64_t n, Space sp, uint32_t *__restrict__ keys,
            uint32_t *__restrict__ values, int4 *__restrict__ own_cell) {
  const int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x;
  if (i >= n) return;
  float p[3];
  int cell[3];
  load_point<D>(positions, i, p);
  cell_of<D>(p, sp, cell);
  keys[i] = bucket_of<D>(cell, sp.bits);
  values[i] = (uint32_t)i;
  own_cell[i] = make_int4(cell[0], cell[1], cell[2], 0);
}

// sorted entry s: gathers its point and cell
template <int D>
__global__ void __launch_bounds__(kThreads)
k_directory_fill(const float *__restrict__ positions, int64_t n, const uint32_t *__restrict__ order,
                 const int4 *__restrict__ own_cell, Directory dir) {
  const int64_t s = (int64_t)blockIdx.x * kThreads + threadIdx.x;
  if (s >= n) return;
  const uint32_t i = order[s];
  float p[3];
  load_point<D>(positions, (int64_t)i, p);
  dir.points[s] = make_float4(p[0], p[1], p[2], __uint_as_float(i));
  dir.cells[s] = own_cell[i];
}

// bucket_ptr[b] = first sorted entry whose key is >= b (lower bound), b in [0, buckets]
__global__ void __launch_bounds__(kThreads)
k_bucket_ptr(const uint32_t *__restrict__ keys, int64_t n, Directory dir) {
  const int64_t b = (int64_t)blockIdx.x * kThreads + threadIdx.x;
  if (b > dir.buckets) return;
  int64_t lo = 0, hi = n;
  while (lo < hi) {
    const int64_t mid = (lo + hi) >> 1;
    if ((int64_t)__ldg(keys + mid) < b) lo = mid + 1; else hi = mid;
  }
  dir.bucket_ptr[b] = (int32_t)lo;
}

// ---- the neighbour walk ------------------------------------------------------------------------
// Calls visit(j, displacement, distance) for every radius neighbour j of destination i in the
// relation's edge order and returns the number of broad-phase candidates seen.
template <int D, bool PERIODIC, typename Visit>
__device__ __forceinline__ int64_t walk_neighbours(const Directory &dir, const Space &sp, int64_t i,
                                                   const float (&pi)[3], float cutoff, bool exclude_self,
                                                   Visit visit) {
  const int4 own = __ldg(dir.own_cell + i);
  int64_t candidates = 0;
  const int n0 = sp.axis_count[0], n1 = D > 1 ? sp.axis_count[1] : 1, n2 = D > 2 ? sp.axis_count[2] : 1;
  for (int o0 = 0; o0 < n0; ++o0)
    for (int o1 = 0; o1 < n1; ++o1)
      for (int o2 = 0; o2 < n2; ++o2) {        // meshgrid 'ij': the last axis runs fastest
        int target[3] = {own.x + sp.axis_first[0] + o0, own.y, own.z};
        if (D > 1) target[1] = own.y + sp.axis_first[1] + o1;
        if (D > 2) target[2] = own.z + sp.axis_first[2] + o2;
        if (PERIODIC) {
#pragma unroll
          for (int a = 0; a < D; ++a) {
            int c = target[a] % sp.extents[a];
            target[a] = c < 0 ? c + sp.extents[a] : c;
          }
        }
        const uint32_t bucket = bucket_of<D>(target, sp.bits);
        const int begin = __ldg(dir.bucket_ptr + bucket), end = __ldg(dir.bucket_ptr + bucket + 1);
        for (int s = begin; s < end; ++s) {
          const int4 cell = __ldg(dir.cells + s);
          if (cell.x != target[0] || (D > 1 && cell.y != target[1]) || (D > 2 && cell.z != target[2])) continue;
          ++candidates;
          const float4 q = __ldg(dir.points + s);
          const int64_t j = (int64_t)__float_as_uint(q.w);
          const float pj[3] = {q.x, q.y, q.z};
          float d[3];
          displacement_of<D, PERIODIC>(pj, pi, sp, d);
          const float distance = norm_of<D>(d);
          if (!(distance <= cutoff) || (exclude_self && j == i)) continue;
          visit(j, d, distance);
        }
      }
  return candidates;
}

// Destinations are processed in directory order (thread s owns the s-th sorted point), so that the
// threads of a warp walk the same few buckets.
__device__ __forceinline__ int64_t destination_of(const Directory &dir, int64_t s) {
  return (int64_t)__float_as_uint(__ldg(&dir.points[s].w));
}

template <int D, bool PERIODIC>
__global__ void __launch_bounds__(kThreads)
k_radius_count(const float *__restrict__ positions, int64_t n, Space sp, Directory dir, float cutoff,
               int exclude_self, int32_t *__restrict__ counts, unsigned long long *__restrict__ candidate_pairs) {
  const int64_t s = (int64_t)blockIdx.x * kThreads + threadIdx.x;
  unsigned long long candidates = 0;
  if (s < n) {
    const int64_t i = destination_of(dir, s);
    float pi[3];
    load_point<D>(positions, i, pi);
    int32_t count = 0;
    candidates = (unsigned long long)walk_neighbours<D, PERIODIC>(
        dir, sp, i, pi, cutoff, exclude_self != 0, [&](int64_t, const float (&)[3], float) { ++count; });
    counts[i] = count;
  }
  if (candidate_pairs) {
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) candidates += __shfl_xor_sync(0xffffffffu, candidates, offset);
    if ((threadIdx.x & 31) == 0 && candidates) atomicAdd(candidate_pairs, candidates);
  }
}

template <int D, bool PERIODIC>
__global__ void __launch_bounds__(kThreads)
k_radius_fill(const float *__restrict__ positions, int64_t n, Space sp, Directory dir, float cutoff,
              int exclude_self, const int64_t *__restrict__ row_ptr, int64_t *__restrict__ col,
              float *__restrict__ distance, float *__restrict__ displacement) {
  const int64_t s = (int64_t)blockIdx.x * kThreads + threadIdx.x;
  if (s >= n) return;
  const int64_t i = destination_of(dir, s);
  float pi[3];
  load_point<D>(positions, i, pi);
  int64_t e = row_ptr[i];
  walk_neighbours<D, PERIODIC>(dir, sp, i, pi, cutoff, exclude_self != 0,
                               [&](int64_t j, const float (&d)[3], float dist) {
                                 col[e] = j;
                                 if (distance) distance[e] = dist;
                                 if (displacement) {
#pragma unroll
                                   for (int a = 0; a < D; ++a) displacement[e * D + a] = d[a];
                                 }
                                 ++e;
                               });
}

// ---- fused consumer ----------------------------------------------------------------------------
// LANES lanes share one destination; lane l owns the features l, l + LANES, ... (at most kMaxPerLane).
constexpr int kMaxPerLane = 4;

template <int D, bool PERIODIC, int LANES, int WEIGHT>
__global__ void __launch_bounds__(kThreads)
k_radius_wsum(const float *__restrict__ positions, int64_t n, Space sp, Directory dir, float cutoff,
              int exclude_self, const float *__restrict__ x, int F, float *__restrict__ out) {
  const int64_t s = ((int64_t)blockIdx.x * kThreads + threadIdx.x) / LANES;
  const int lane = threadIdx.x % LANES;
  if (s >= n) return;
  const int64_t i = destination_of(dir, s);
  float pi[3];
  load_point<D>(positions, i, pi);
  float acc[kMaxPerLane];
#pragma unroll
  for (int q = 0; q < kMaxPerLane; ++q) acc[q] = 0.0f;
  walk_neighbours<D, PERIODIC>(dir, sp, i, pi, cutoff, exclude_self != 0,
                               [&](int64_t j, const float (&)[3], float dist) {
                                 const float *row = x + j * F;
#pragma unroll
                                 for (int q = 0; q < kMaxPerLane; ++q) {
                                   const int f = lane + q * LANES;
                                   if (f < F) {
                                     const float v = __ldg(row + f);
                                     acc[q] = WEIGHT == TGB_PAIR_WEIGHT_DISTANCE ? mul_add_rn(dist, v, acc[q])
                                                                                 : __fadd_rn(acc[q], v);
                                   }
                                 }
                               });
#pragma unroll
  for (int q = 0; q < kMaxPerLane; ++q) {
    const int f = lane + q * LANES;
    if (f < F) out[i * F + f] = acc[q];
  }
}

// dpos[i] = - sum_j (dy_i . x_j + dy_j . x_i) * displacement / distance; the LANES lanes of a
// destination split the feature dot products and combine them by shuffles.
template <int D, bool PERIODIC, int LANES>
__global__ void __launch_bounds__(kThreads)
k_radius_wsum_bwd_pos(const float *__restrict__ positions, int64_t n, Space sp, Directory dir, float cutoff,
                      int exclude_self, const float *__restrict__ x, const float *__restrict__ dy, int F,
                      float *__restrict__ dpos) {
  const int64_t s = ((int64_t)blockIdx.x * kThreads + threadIdx.x) / LANES;
  const int lane = threadIdx.x % LANES;
  if (s >= n) return;
  // the lanes of one destination run in lockstep; other groups of the warp walk other neighbourhoods,
  // so every shuffle names this group's lanes only
  const unsigned group_mask = LANES == 32 ? 0xffffffffu
                                          : ((1u << LANES) - 1u) << ((threadIdx.x & 31) / LANES * LANES);
  const int64_t i = destination_of(dir, s);
  float pi[3];
  load_point<D>(positions, i, pi);
  float xi[kMaxPerLane], dyi[kMaxPerLane];
#pragma unroll
  for (int q = 0; q < kMaxPerLane; ++q) {
    const int f = lane + q * LANES;
    xi[q] = f < F ? __ldg(x + i * F + f) : 0.0f;
    dyi[q] = f < F ? __ldg(dy + i * F + f) : 0.0f;
  }
  float g[3] = {0.0f, 0.0f, 0.0f};
  walk_neighbours<D, PERIODIC>(dir, sp, i, pi, cutoff, exclude_self != 0,
                               [&](int64_t j, const float (&d)[3], float dist) {
                                 float dot = 0.0f;
#pragma unroll
                                 for (int q = 0; q < kMaxPerLane; ++q) {
                                   const int f = lane + q * LANES;
                                   if (f < F) {
                                     dot = fmaf(dyi[q], __ldg(x + j * F + f), dot);
                                     dot = fmaf(__ldg(dy + j * F + f), xi[q], dot);
                                   }
                                 }
#pragma unroll
                                 for (int offset = LANES / 2; offset > 0; offset >>= 1)
                                   dot += __shfl_xor_sync(group_mask, dot, offset, LANES);
                                 if (dist > 0.0f) {
                                   const float scale = dot / dist;
#pragma unroll
                                   for (int a = 0; a < D; ++a) g[a] = fmaf(-scale, d[a], g[a]);
                                 }
                               });
  if (lane == 0) {
#pragma unroll
    for (int a = 0; a < D; ++a) dpos[i * D + a] = g[a];
  }
}

// ---- exact k nearest neighbours ----------------------------------------------------------------
// One thread per query.  The candidates stream through shared memory in tiles; the thread keeps its k
// best (squared distance, index) in shared memory, ascending, and the current k-th distance in a
// register: the inner loop is a distance and one compare, an insertion happens O(k log(nc / k)) times.
// Candidates arrive in ascending index, so "strictly closer than the k-th" plus insertion behind
// equal distances is exactly the (distance, index) order.
constexpr int kKnnThreads = 128;
constexpr int kKnnTile = 1024;       // candidates per tile, dims <= 3 (float4 each)
constexpr int kKnnWideTile = 64;     // candidates per tile, dims up to 64

__device__ __forceinline__ void knn_insert(float *best_d, int32_t *best_j, int k, float d, int32_t j) {
  // slot (r, thread) lives at [r * kKnnThreads + thread]: a warp's accesses hit 32 banks
  int at = k - 1;
  while (at > 0 && best_d[(at - 1) * kKnnThreads] > d) {
    best_d[at * kKnnThreads] = best_d[(at - 1) * kKnnThreads];
    best_j[at * kKnnThreads] = best_j[(at - 1) * kKnnThreads];
    --at;
  }
  best_d[at * kKnnThreads] = d;
  best_j[at * kKnnThreads] = j;
}

template <int D>
__global__ void __launch_bounds__(kKnnThreads)
k_knn_small(const float *__restrict__ queries, int64_t nq, const float *__restrict__ candidates, int64_t nc,
            int k, int exclude_self, int64_t *__restrict__ col, float *__restrict__ dist_sq) {
  extern __shared__ __align__(16) unsigned char knn_smem[];
  float4 *tile = reinterpret_cast<float4 *>(knn_smem);
  float *best_d = reinterpret_cast<float *>(knn_smem + sizeof(float4) * kKnnTile) + threadIdx.x;
  int32_t *best_j = reinterpret_cast<int32_t *>(best_d - threadIdx.x + (size_t)k * kKnnThreads) + threadIdx.x;
  const int64_t i = (int64_t)blockIdx.x * kKnnThreads + threadIdx.x;
  const bool live = i < nq;
  float q[3] = {0.0f, 0.0f, 0.0f};
  if (live) {
#pragma unroll
    for (int a = 0; a < D; ++a) q[a] = __ldg(queries + i * D + a);
  }
  for (int r = 0; r < k; ++r) {
    best_d[r * kKnnThreads] = __int_as_float(0x7f800000);
    best_j[r * kKnnThreads] = -1;
  }
  float worst = __int_as_float(0x7f800000);
  const int64_t self = exclude_self ? i : -1;
  for (int64_t base = 0; base < nc; base += kKnnTile) {
    const int count = (int)(nc - base < kKnnTile ? nc - base : kKnnTile);
    __syncthreads();
    for (int t = threadIdx.x; t < count; t += kKnnThreads) {
      const float *c = candidates + (base + t) * D;
      tile[t] = make_float4(__ldg(c), D > 1 ? __ldg(c + 1) : 0.0f, D > 2 ? __ldg(c + 2) : 0.0f, 0.0f);
    }
    __syncthreads();
    if (!live) continue;
#pragma unroll 4
    for (int t = 0; t < count; ++t) {
      const float4 c = tile[t];
      const float d0 = __fsub_rn(c.x, q[0]);
      float acc = __fmul_rn(d0, d0);
      if (D > 1) {
        const float d1 = __fsub_rn(c.y, q[1]);
        acc = __fmaf_rn(d1, d1, acc);
      }
      if (D > 2) {
        const float d2 = __fsub_rn(c.z, q[2]);
        acc = __fmaf_rn(d2, d2, acc);
      }
      if (acc < worst && base + t != self) {
        knn_insert(best_d, best_j, k, acc, (int32_t)(base + t));
        worst = best_d[(k - 1) * kKnnThreads];
      }
    }
  }
  if (!live) return;
  for (int r = 0; r < k; ++r) {
    col[i * k + r] = (int64_t)best_j[r * kKnnThreads];
    if (dist_sq) dist_sq[i * k + r] = best_d[r * kKnnThreads];
  }
}

// Any width up to 64: the query row and the candidate tile both sit in shared memory.
__global__ void __launch_bounds__(kKnnThreads)
k_knn_wide(const float *__restrict__ queries, int64_t nq, const float *__restrict__ candidates, int64_t nc,
           int D, int k, int exclude_self, int64_t *__restrict__ col, float *__restrict__ dist_sq) {
  extern __shared__ __align__(16) unsigned char knn_smem[];
  float *tile = reinterpret_cast<float *>(knn_smem);                      // [kKnnWideTile][D]
  float *query = tile + (size_t)kKnnWideTile * D + threadIdx.x;           // [D][threads]
  float *best_d = tile + (size_t)kKnnWideTile * D + (size_t)D * kKnnThreads + threadIdx.x;
  int32_t *best_j = reinterpret_cast<int32_t *>(best_d - threadIdx.x + (size_t)k * kKnnThreads) + threadIdx.x;
  const int64_t i = (int64_t)blockIdx.x * kKnnThreads + threadIdx.x;
  const bool live = i < nq;
  for (int a = 0; a < D; ++a) query[a * kKnnThreads] = live ? __ldg(queries + i * D + a) : 0.0f;
  for (int r = 0; r < k; ++r) {
    best_d[r * kKnnThreads] = __int_as_float(0x7f800000);
    best_j[r * kKnnThreads] = -1;
  }
  float worst = __int_as_float(0x7f800000);
  const int64_t self = exclude_self ? i : -1;
  for (int64_t base = 0; base < nc; base += kKnnWideTile) {
    const int count = (int)(nc - base < kKnnWideTile ? nc - base : kKnnWideTile);
    __syncthreads();
    for (int t = threadIdx.x; t < count * D; t += kKnnThreads) tile[t] = __ldg(candidates + base * D + t);
    __syncthreads();
    if (!live) continue;
    for (int t = 0; t < count; ++t) {
      const float *c = tile + t * D;
      const float d0 = __fsub_rn(c[0], query[0]);
      float acc = __fmul_rn(d0, d0);
      for (int a = 1; a < D; ++a) {
        const float d = __fsub_rn(c[a], query[a * kKnnThreads]);
        acc = __fmaf_rn(d, d, acc);
      }
      if (acc < worst && base + t != self) {
        knn_insert(best_d, best_j, k, acc, (int32_t)(base + t));
        worst = best_d[(k - 1) * kKnnThreads];
      }
    }
  }
  if (!live) return;
  for (int r = 0; r < k; ++r) {
    col[i * k + r] = (int64_t)best_j[r * kKnnThreads];
    if (dist_sq) dist_sq[i * k + r] = best_d[r * kKnnThreads];
  }
}

// ---- exact k nearest neighbours over the cell directory ---------------------------------------
// One thread per query walks the shells of cells around the query's cell (Chebyshev radius 0, 1,
// 2, ...), inserting candidates by the (squared distance, index) key, and stops as soon as its k-th
// best distance is strictly smaller than the distance to the boundary of the block of cells it has
// covered (minus a rounding margin): no closer candidate can lie outside.  With the cell edge chosen
// for about k points per ball of that radius, two shells (27 cells) settle almost every query, so the
// search costs O(k) distance evaluations per query instead of the number of candidates.  A query that
// is not settled within kKnnMaxShells shells is flagged and finished by the brute-force scan below
// (k_knn_flagged), so the result is exact for every input.
constexpr int kKnnMaxShells = 6;

__device__ __forceinline__ void knn_insert_keyed(float *best_d, int32_t *best_j, int k, float d, int32_t j) {
  // ascending by (d, j); candidates arrive in any order
  int at = k - 1;
  while (at > 0) {
    const float pd = best_d[(at - 1) * kKnnThreads];
    const int32_t pj = best_j[(at - 1) * kKnnThreads];
    if (pd < d || (pd == d && pj < j && pj >= 0)) break;
    best_d[at * kKnnThreads] = pd;
    best_j[at * kKnnThreads] = pj;
    --at;
  }
  best_d[at * kKnnThreads] = d;
  best_j[at * kKnnThreads] = j;
}

template <int D>
__global__ void __launch_bounds__(kKnnThreads)
k_knn_grid(const float *__restrict__ queries, int64_t nq, Space sp, Directory dir, int k, int exclude_self,
           int self_order, float margin, int64_t *__restrict__ col, float *__restrict__ dist_sq,
           int32_t *__restrict__ unsettled) {
  extern __shared__ __align__(16) unsigned char knn_smem[];
  float *best_d = reinterpret_cast<float *>(knn_smem) + threadIdx.x;
  int32_t *best_j = reinterpret_cast<int32_t *>(knn_smem + (size_t)k * kKnnThreads * 4) + threadIdx.x;
  const int64_t s = (int64_t)blockIdx.x * kKnnThreads + threadIdx.x;
  if (s >= nq) return;
  // a self search takes its queries in directory order: the threads of a warp share cells
  const int64_t i = self_order ? destination_of(dir, s) : s;
  float q[3];
  int cell[3];
  load_point<D>(queries, i, q);
  cell_of<D>(q, sp, cell);
  for (int r = 0; r < k; ++r) {
    best_d[r * kKnnThreads] = __int_as_float(0x7f800000);
    best_j[r * kKnnThreads] = -1;
  }
  float worst = __int_as_float(0x7f800000);
  int32_t worst_j = -1;
  const int64_t self = exclude_self ? i : -1;
  bool settled = false;
  for (int shell = 0; shell <= kKnnMaxShells && !settled; ++shell) {
    const int lo1 = D > 1 ? -shell : 0, hi1 = D > 1 ? shell : 0;
    const int lo2 = D > 2 ? -shell : 0, hi2 = D > 2 ? shell : 0;
    for (int o0 = -shell; o0 <= shell; ++o0)
      for (int o1 = lo1; o1 <= hi1; ++o1)
        for (int o2 = lo2; o2 <= hi2; ++o2) {
          const int reach = max(abs(o0), max(abs(o1), abs(o2)));
          if (reach != shell) continue;             // interior cells were covered by earlier shells
          const int target[3] = {cell[0] + o0, cell[1] + o1, cell[2] + o2};
          const uint32_t bucket = bucket_of<D>(target, sp.bits);
          const int begin = __ldg(dir.bucket_ptr + bucket), end = __ldg(dir.bucket_ptr + bucket + 1);
          for (int e = begin; e < end; ++e) {
            const int4 c = __ldg(dir.cells + e);
            if (c.x != target[0] || (D > 1 && c.y != target[1]) || (D > 2 && c.z != target[2])) continue;
            const float4 p = __ldg(dir.points + e);
            const int32_t j = (int32_t)__float_as_uint(p.w);
            const float d0 = __fsub_rn(p.x, q[0]);
            float acc = __fmul_rn(d0, d0);
            if (D > 1) {
              const float d1 = __fsub_rn(p.y, q[1]);
              acc = __fmaf_rn(d1, d1, acc);
            }
            if (D > 2) {
              const float d2 = __fsub_rn(p.z, q[2]);
              acc = __fmaf_rn(d2, d2, acc);
            }
            if ((acc < worst || (acc == worst && j < worst_j)) && (int64_t)j != self) {
              knn_insert_keyed(best_d, best_j, k, acc, j);
              worst = best_d[(k - 1) * kKnnThreads];
              worst_j = best_j[(k - 1) * kKnnThreads];
            }
          }
        }
    // everything outside the covered block [cell - shell, cell + shell + 1) * cell_size is at least
    // `cover` away from the query
    float cover = __int_as_float(0x7f800000);
#pragma unroll
    for (int a = 0; a < D; ++a) {
      const float low = q[a] - (float)(cell[a] - shell) * sp.cell_size;
      const float high = (float)(cell[a] + shell + 1) * sp.cell_size - q[a];
      cover = fminf(cover, fminf(low, high));
    }
    cover -= margin;
    settled = worst_j >= 0 && cover > 0.0f && worst < cover * cover * 0.99999f;
  }
  unsettled[i] = settled ? 0 : 1;
  if (!settled) return;
  for (int r = 0; r < k; ++r) {
    col[i * k + r] = (int64_t)best_j[r * kKnnThreads];
    if (dist_sq) dist_sq[i * k + r] = best_d[r * kKnnThreads];
  }
}

// Brute-force scan for the queries the shell search left unsettled (a handful in sparse regions,
// every query when the points sit in a few cells): same selection as k_knn_small, straight from
// global memory, candidates in ascending index.
template <int D>
__global__ void __launch_bounds__(kKnnThreads)
k_knn_flagged(const float *__restrict__ queries, int64_t nq, const float *__restrict__ candidates, int64_t nc,
              int k, int exclude_self, const int32_t *__restrict__ unsettled, int64_t *__restrict__ col,
              float *__restrict__ dist_sq) {
  extern __shared__ __align__(16) unsigned char knn_smem[];
  float *best_d = reinterpret_cast<float *>(knn_smem) + threadIdx.x;
  int32_t *best_j = reinterpret_cast<int32_t *>(knn_smem + (size_t)k * kKnnThreads * 4) + threadIdx.x;
  const int64_t i = (int64_t)blockIdx.x * kKnnThreads + threadIdx.x;
  if (i >= nq || !unsettled[i]) return;
  float q[3];
  load_point<D>(queries, i, q);
  for (int r = 0; r < k; ++r) {
    best_d[r * kKnnThreads] = __int_as_float(0x7f800000);
    best_j[r * kKnnThreads] = -1;
  }
  float worst = __int_as_float(0x7f800000);
  const int64_t self = exclude_self ? i : -1;
  for (int64_t j = 0; j < nc; ++j) {
    float p[3];
    load_point<D>(candidates, j, p);
    const float d0 = __fsub_rn(p[0], q[0]);
    float acc = __fmul_rn(d0, d0);
    if (D > 1) {
      const float d1 = __fsub_rn(p[1], q[1]);
      acc = __fmaf_rn(d1, d1, acc);
    }
    if (D > 2) {
      const float d2 = __fsub_rn(p[2], q[2]);
      acc = __fmaf_rn(d2, d2, acc);
    }
    if (acc < worst && j != self) {
      knn_insert(best_d, best_j, k, acc, (int32_t)j);
      worst = best_d[(k - 1) * kKnnThreads];
    }
  }
  for (int r = 0; r < k; ++r) {
    col[i * k + r] = (int64_t)best_j[r * kKnnThreads];
    if (dist_sq) dist_sq[i * k + r] = best_d[r * kKnnThreads];
  }
}

// ---- implicit edge fields of a stored relation ---------------------------------------------------
constexpr int kMaxGeometryDims = 8;

struct WideSpace {
  int dims;
  int periodic;
  float lattice[9];
  float inverse[9];
};

__global__ void __launch_bounds__(kThreads)
k_edge_geometry(const float *__restrict__ dst_positions, const float *__restrict__ src_positions, WideSpace sp,
                const int64_t *__restrict__ row_ptr, const int64_t *__restrict__ col, int64_t num_dst,
                int64_t edges, float *__restrict__ displacement, float *__restrict__ distance) {
  const int64_t e = (int64_t)blockIdx.x * kThreads + threadIdx.x;
  if (e >= edges) return;
  int64_t lo = 0, hi = num_dst;          // the row of edge e: last row whose first edge is <= e
  while (hi - lo > 1) {
    const int64_t mid = (lo + hi) >> 1;
    if (__ldg(row_ptr + mid) <= e) lo = mid; else hi = mid;
  }
  const int64_t i = lo, j = __ldg(col + e);
  const int D = sp.dims;
  float d[kMaxGeometryDims];
#pragma unroll
  for (int a = 0; a < kMaxGeometryDims; ++a)
    d[a] = a < D ? __fsub_rn(__ldg(src_positions + j * D + a), __ldg(dst_positions + i * D + a)) : 0.0f;
  if (sp.periodic) {                     // dims <= 3 here
    float f[3];
    for (int a = 0; a < D; ++a) {
      float acc = __fmul_rn(d[0], sp.inverse[a]);
      for (int k = 1; k < D; ++k) acc = __fmaf_rn(d[k], sp.inverse[k * D + a], acc);
      f[a] = __fsub_rn(acc, rintf(acc));
    }
    float w[3];
    for (int a = 0; a < D; ++a) {
      float acc = __fmul_rn(f[0], sp.lattice[a]);
      for (int k = 1; k < D; ++k) acc = __fmaf_rn(f[k], sp.lattice[k * D + a], acc);
      w[a] = acc;
    }
    for (int a = 0; a < D; ++a) d[a] = w[a];
  }
  float acc = __fmul_rn(d[0], d[0]);
#pragma unroll
  for (int a = 1; a < kMaxGeometryDims; ++a)
    if (a < D) acc = __fmaf_rn(d[a], d[a], acc);
  if (displacement) {
#pragma unroll
    for (int a = 0; a < kMaxGeometryDims; ++a)
      if (a < D) displacement[e * D + a] = d[a];
  }
  if (distance) distance[e] = __fsqrt_rn(acc);
}

// ---- host side -----------------------------------------------------------------------------------
#define TGB_DISPATCH_SPACE(sp, CALL)                                   \
  do {                                                                 \
    if ((sp).periodic) {                                               \
      if ((sp).dims == 1) { CALL(1, true); }                           \
      else if ((sp).dims == 2) { CALL(2, true); }                      \
      else { CALL(3, true); }                                          \
    } else {                                                           \
      if ((sp).dims == 1) { CALL(1, false); }                          \
      else if ((sp).dims == 2) { CALL(2, false); }                     \
      else { CALL(3, false); }                                         \
    }                                                                  \
  } while (0)

int lanes_for(int64_t F) {
  int lanes = 1;
  while (lanes < 32 && lanes * kMaxPerLane < F) lanes <<= 1;
  return lanes;
}

}  // namespace
}  // namespace tgb

using namespace tgb;

extern "C" int32_t tgb_cell_directory_sizes(int64_t n, int32_t dims, uint64_t *persistent_bytes,
                                            uint64_t *temp_bytes) {
  DirectoryLayout L;
  const int32_t status = directory_layout(n, dims, &L);
  if (status != TGB_STATUS_OK) return status;
  if (persistent_bytes) *persistent_bytes = L.persistent_bytes;
  if (temp_bytes) *temp_bytes = L.temp_bytes;
  return TGB_STATUS_OK;
}

extern "C" int32_t tgb_cell_directory_build(const void *positions, int64_t n, const tgb_cell_space *space,
                                            void *persistent, uint64_t persistent_bytes, void *temp,
                                            uint64_t temp_bytes, uint64_t stream) {
  Space sp;
  int32_t status = make_space(space, n, &sp);
  if (status != TGB_STATUS_OK) return status;
  DirectoryLayout L;
  status = directory_layout(n, sp.dims, &L);
  if (status != TGB_STATUS_OK) return status;
  if (!persistent || persistent_bytes < L.persistent_bytes || !temp || temp_bytes < L.temp_bytes)
    TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "directory buffers are missing or too small");
  if (n > 0 && !positions) TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "null positions");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  Directory dir = directory_at(persistent, L);
  char *t = static_cast<char *>(temp);
  uint32_t *k0 = reinterpret_cast<uint32_t *>(t + L.k0), *k1 = reinterpret_cast<uint32_t *>(t + L.k1);
  uint32_t *v0 = reinterpret_cast<uint32_t *>(t + L.v0), *v1 = reinterpret_cast<uint32_t *>(t + L.v1);
  const float *pos = static_cast<const float *>(positions);
  const uint32_t *sorted_keys = k0;
  if (n > 0) {
#define TGB_KEYS(DIMS, PER) k_cell_keys<DIMS><<<grid_for(n), kThreads, 0, st>>>(pos, n, sp, k0, v0, dir.own_cell)
    TGB_DISPATCH_SPACE(sp, TGB_KEYS);
#undef TGB_KEYS
    TGB_LAUNCHED();
    cub::DoubleBuffer<uint32_t> dk(k0, k1), dv(v0, v1);
    size_t cub_bytes = L.cub_bytes;
    TGB_CUDA(cub::DeviceRadixSort::SortPairs(t + L.cub, cub_bytes, dk, dv, n, 0, sp.bits * sp.dims, st));
    g_launches.fetch_add(3);
    sorted_keys = dk.Current();
#define TGB_FILL(DIMS, PER) \
  k_directory_fill<DIMS><<<grid_for(n), kThreads, 0, st>>>(pos, n, dv.Current(), dir.own_cell, dir)
    TGB_DISPATCH_SPACE(sp, TGB_FILL);
#undef TGB_FILL
    TGB_LAUNCHED();
  }
  k_bucket_ptr<<<grid_for(dir.buckets + 1), kThreads, 0, st>>>(sorted_keys, n, dir);
  TGB_LAUNCHED();
  return TGB_STATUS_OK;
}

namespace {

struct RadiusCall {
  Space sp;
  Directory dir;
  DirectoryLayout L;
};

int32_t radius_call(const tgb_cell_space *space, int64_t n, const void *directory, const void *positions,
                    RadiusCall *call) {
  int32_t status = make_space(space, n, &call->sp);
  if (status != TGB_STATUS_OK) return status;
  status = directory_layout(n, call->sp.dims, &call->L);
  if (status != TGB_STATUS_OK) return status;
  if (!directory) TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "null cell directory");
  if (n > 0 && !positions) TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "null positions");
  call->dir = directory_at(const_cast<void *>(directory), call->L);
  return TGB_STATUS_OK;
}

}  // namespace

extern "C" int32_t tgb_radius_row_ptr(const void *positions, int64_t n, const tgb_cell_space *space,
                                      const void *directory, float cutoff, int32_t exclude_self, void *row_ptr,
                                      void *candidate_pairs, void *temp, uint64_t temp_bytes, uint64_t stream) {
  RadiusCall c;
  const int32_t status = radius_call(space, n, directory, positions, &c);
  if (status != TGB_STATUS_OK) return status;
  if (!row_ptr || !temp || temp_bytes < c.L.temp_bytes)
    TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "row_ptr or scratch is missing or too small");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  char *t = static_cast<char *>(temp);
  int32_t *counts = reinterpret_cast<int32_t *>(t + c.L.counts);
  unsigned long long *pairs = static_cast<unsigned long long *>(candidate_pairs);
  if (pairs) TGB_CUDA(cudaMemsetAsync(pairs, 0, sizeof(unsigned long long), st));
  const float *pos = static_cast<const float *>(positions);
  // counts[n] = 0 closes the exclusive scan: row_ptr[n] = number of edges
  TGB_CUDA(cudaMemsetAsync(counts + n, 0, sizeof(int32_t), st));
  if (n > 0) {
#define TGB_COUNT(DIMS, PER)                                                                              \
  k_radius_count<DIMS, PER><<<grid_for(n), kThreads, 0, st>>>(pos, n, c.sp, c.dir, cutoff, exclude_self, \
                                                               counts, pairs)
    TGB_DISPATCH_SPACE(c.sp, TGB_COUNT);
#undef TGB_COUNT
    TGB_LAUNCHED();
  }
  size_t cub_bytes = c.L.cub_bytes;
  TGB_CUDA(cub::DeviceScan::ExclusiveSum(t + c.L.cub, cub_bytes, counts, static_cast<int64_t *>(row_ptr),
                                         (int64_t)(n + 1), st));
  g_launches.fetch_add(2);
  return TGB_STATUS_OK;
}

extern "C" int32_t tgb_radius_fill(const void *positions, int64_t n, const tgb_cell_space *space,
                                   const void *directory, float cutoff, int32_t exclude_self,
                                   const void *row_ptr, void *col, void *distance, void *displacement,
                                   uint64_t stream) {
  RadiusCall c;
  const int32_t status = radius_call(space, n, directory, positions, &c);
  if (status != TGB_STATUS_OK) return status;
  if (n == 0) return TGB_STATUS_OK;
  if (!row_ptr || !col) TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "null row_ptr or col");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const float *pos = static_cast<const float *>(positions);
#define TGB_FILL_EDGES(DIMS, PER)                                                                        \
  k_radius_fill<DIMS, PER><<<grid_for(n), kThreads, 0, st>>>(pos, n, c.sp, c.dir, cutoff, exclude_self, \
                                                              static_cast<const int64_t *>(row_ptr),     \
                                                              static_cast<int64_t *>(col),               \
                                                              static_cast<float *>(distance),            \
                                                              static_cast<float *>(displacement))
  TGB_DISPATCH_SPACE(c.sp, TGB_FILL_EDGES);
#undef TGB_FILL_EDGES
  TGB_LAUNCHED();
  return TGB_STATUS_OK;
}

namespace {

template <int D, bool PER, int WEIGHT>
void launch_wsum(int lanes, const float *pos, int64_t n, const RadiusCall &c, float cutoff, int exclude_self,
                 const float *x, int F, float *out, cudaStream_t st) {
  const unsigned blocks = grid_for(n * lanes);
  switch (lanes) {
#define TGB_CASE(L)                                                                                            \
  case L:                                                                                                      \
    k_radius_wsum<D, PER, L, WEIGHT><<<blocks, kThreads, 0, st>>>(pos, n, c.sp, c.dir, cutoff, exclude_self, x, \
                                                                   F, out);                                    \
    break;
    TGB_CASE(1) TGB_CASE(2) TGB_CASE(4) TGB_CASE(8) TGB_CASE(16) TGB_CASE(32)
#undef TGB_CASE
  }
}

template <int D, bool PER>
void launch_bwd_pos(int lanes, const float *pos, int64_t n, const RadiusCall &c, float cutoff, int exclude_self,
                    const float *x, const float *dy, int F, float *dpos, cudaStream_t st) {
  const unsigned blocks = grid_for(n * lanes);
  switch (lanes) {
#define TGB_CASE(L)                                                                                          \
  case L:                                                                                                    \
    k_radius_wsum_bwd_pos<D, PER, L><<<blocks, kThreads, 0, st>>>(pos, n, c.sp, c.dir, cutoff, exclude_self, \
                                                                   x, dy, F, dpos);                          \
    break;
    TGB_CASE(1) TGB_CASE(2) TGB_CASE(4) TGB_CASE(8) TGB_CASE(16) TGB_CASE(32)
#undef TGB_CASE
  }
}

}  // namespace

extern "C" int32_t tgb_radius_wsum_fwd(const void *positions, int64_t n, const tgb_cell_space *space,
                                       const void *directory, float cutoff, int32_t exclude_self, int32_t weight,
                                       const void *x, int64_t F, void *out, uint64_t stream) {
  RadiusCall c;
  const int32_t status = radius_call(space, n, directory, positions, &c);
  if (status != TGB_STATUS_OK) return status;
  if (F < 1 || F > 32 * kMaxPerLane) TGB_FAIL(TGB_STATUS_UNSUPPORTED, "feature width must be in [1, 128]");
  if (weight != TGB_PAIR_WEIGHT_ONE && weight != TGB_PAIR_WEIGHT_DISTANCE)
    TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "unknown pair weight");
  if (n == 0) return TGB_STATUS_OK;
  if (!x || !out) TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "null feature pointer");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int lanes = lanes_for(F);
  const float *pos = static_cast<const float *>(positions);
#define TGB_WSUM(DIMS, PER)                                                                                      \
  if (weight == TGB_PAIR_WEIGHT_DISTANCE)                                                                        \
    launch_wsum<DIMS, PER, TGB_PAIR_WEIGHT_DISTANCE>(lanes, pos, n, c, cutoff, exclude_self,                     \
                                                     static_cast<const float *>(x), (int)F,                      \
                                                     static_cast<float *>(out), st);                             \
  else                                                                                                           \
    launch_wsum<DIMS, PER, TGB_PAIR_WEIGHT_ONE>(lanes, pos, n, c, cutoff, exclude_self,                          \
                                                static_cast<const float *>(x), (int)F, static_cast<float *>(out), st)
  TGB_DISPATCH_SPACE(c.sp, TGB_WSUM);
#undef TGB_WSUM
  TGB_LAUNCHED();
  return TGB_STATUS_OK;
}

extern "C" int32_t tgb_radius_wsum_bwd_pos(const void *positions, int64_t n, const tgb_cell_space *space,
                                           const void *directory, float cutoff, int32_t exclude_self,
                                           const void *x, const void *dy, int64_t F, void *dpos,
                                           uint64_t stream) {
  RadiusCall c;
  const int32_t status = radius_call(space, n, directory, positions, &c);
  if (status != TGB_STATUS_OK) return status;
  if (F < 1 || F > 32 * kMaxPerLane) TGB_FAIL(TGB_STATUS_UNSUPPORTED, "feature width must be in [1, 128]");
  if (n == 0) return TGB_STATUS_OK;
  if (!x || !dy || !dpos) TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "null pointer");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int lanes = lanes_for(F);
  const float *pos = static_cast<const float *>(positions);
#define TGB_BWD(DIMS, PER)                                                                                   \
  launch_bwd_pos<DIMS, PER>(lanes, pos, n, c, cutoff, exclude_self, static_cast<const float *>(x),           \
                            static_cast<const float *>(dy), (int)F, static_cast<float *>(dpos), st)
  TGB_DISPATCH_SPACE(c.sp, TGB_BWD);
#undef TGB_BWD
  TGB_LAUNCHED();
  return TGB_STATUS_OK;
}

extern "C" int32_t tgb_knn(const void *queries, int64_t nq, const void *candidates, int64_t nc, int32_t dims,
                           int32_t k, int32_t exclude_self, void *col, void *dist_sq, uint64_t stream) {
  if (nq < 0 || nc < 0 || nc >= ((int64_t)1 << 31)) TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "point count out of range");
  if (dims < 1 || dims > 64) TGB_FAIL(TGB_STATUS_UNSUPPORTED, "positions must have 1 to 64 columns");
  if (k < 1 || k > 128) TGB_FAIL(TGB_STATUS_UNSUPPORTED, "k must be in [1, 128]");
  if ((int64_t)k > nc - (exclude_self ? 1 : 0))
    TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "k exceeds the number of admissible candidates");
  if (nq == 0) return TGB_STATUS_OK;
  if (!queries || !candidates || !col) TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "null pointer");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const float *q = static_cast<const float *>(queries), *c = static_cast<const float *>(candidates);
  int64_t *out = static_cast<int64_t *>(col);
  float *dist = static_cast<float *>(dist_sq);
  const unsigned blocks = grid_for(nq, kKnnThreads);
  const size_t list_bytes = (size_t)k * kKnnThreads * 8;
  if (dims <= 3) {
    const size_t smem = sizeof(float4) * kKnnTile + list_bytes;
#define TGB_KNN(DIMS)                                                                                       \
  do {                                                                                                      \
    TGB_CUDA(cudaFuncSetAttribute(k_knn_small<DIMS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
    k_knn_small<DIMS><<<blocks, kKnnThreads, smem, st>>>(q, nq, c, nc, k, exclude_self, out, dist);        \
  } while (0)
    if (dims == 1) TGB_KNN(1); else if (dims == 2) TGB_KNN(2); else TGB_KNN(3);
#undef TGB_KNN
  } else {
    const size_t smem = sizeof(float) * ((size_t)kKnnWideTile * dims + (size_t)dims * kKnnThreads) + list_bytes;
    TGB_CUDA(cudaFuncSetAttribute(k_knn_wide, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    k_knn_wide<<<blocks, kKnnThreads, smem, st>>>(q, nq, c, nc, dims, k, exclude_self, out, dist);
  }
  TGB_LAUNCHED();
  return TGB_STATUS_OK;
}

extern "C" int32_t tgb_knn_grid(const void *queries, int64_t nq, const void *candidates, int64_t nc,
                                const tgb_cell_space *space, const void *directory, int32_t k,
                                int32_t exclude_self, int32_t self_search, float margin, void *col,
                                void *dist_sq, void *unsettled, uint64_t stream) {
  RadiusCall c;
  const int32_t status = radius_call(space, nc, directory, candidates, &c);
  if (status != TGB_STATUS_OK) return status;
  if (c.sp.periodic) TGB_FAIL(TGB_STATUS_UNSUPPORTED, "the nearest-neighbour search has no periodic form");
  if (nq < 0 || (self_search && nq != nc)) TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "query count out of range");
  if (k < 1 || k > 128) TGB_FAIL(TGB_STATUS_UNSUPPORTED, "k must be in [1, 128]");
  if ((int64_t)k > nc - (exclude_self ? 1 : 0))
    TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "k exceeds the number of admissible candidates");
  if (!(margin >= 0.0f)) TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "margin must be non-negative");
  if (nq == 0) return TGB_STATUS_OK;
  if (!queries || !col || !unsettled) TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "null pointer");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const float *q = static_cast<const float *>(queries), *cand = static_cast<const float *>(candidates);
  const unsigned blocks = grid_for(nq, kKnnThreads);
  const size_t smem = (size_t)k * kKnnThreads * 8;
#define TGB_KNN_GRID(DIMS)                                                                                       \
  do {                                                                                                           \
    TGB_CUDA(cudaFuncSetAttribute(k_knn_grid<DIMS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));    \
    TGB_CUDA(cudaFuncSetAttribute(k_knn_flagged<DIMS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
    k_knn_grid<DIMS><<<blocks, kKnnThreads, smem, st>>>(q, nq, c.sp, c.dir, k, exclude_self, self_search, margin, \
                                                         static_cast<int64_t *>(col),                            \
                                                         static_cast<float *>(dist_sq),                          \
                                                         static_cast<int32_t *>(unsettled));                     \
    k_knn_flagged<DIMS><<<blocks, kKnnThreads, smem, st>>>(q, nq, cand, nc, k, exclude_self,                     \
                                                            static_cast<const int32_t *>(unsettled),             \
                                                            static_cast<int64_t *>(col),                         \
                                                            static_cast<float *>(dist_sq));                      \
  } while (0)
  if (c.sp.dims == 1) TGB_KNN_GRID(1); else if (c.sp.dims == 2) TGB_KNN_GRID(2); else TGB_KNN_GRID(3);
#undef TGB_KNN_GRID
  TGB_CUDA(cudaGetLastError());
  g_launches.fetch_add(2);
  return TGB_STATUS_OK;
}

extern "C" int32_t tgb_edge_geometry(const void *dst_positions, const void *src_positions,
                                     const tgb_cell_space *space, const void *row_ptr, const void *col,
                                     int64_t num_dst, int64_t num_edges, void *displacement, void *distance,
                                     uint64_t stream) {
  if (!space) TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "null cell space");
  if (space->dims < 1 || space->dims > kMaxGeometryDims || (space->periodic && space->dims > 3))
    TGB_FAIL(TGB_STATUS_UNSUPPORTED, "edge geometry covers up to 8 columns (3 with a periodic lattice)");
  if (num_edges < 0 || num_dst < 0) TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "negative count");
  if (num_edges == 0) return TGB_STATUS_OK;
  if (!dst_positions || !src_positions || !row_ptr || !col) TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "null pointer");
  WideSpace sp;
  sp.dims = space->dims;
  sp.periodic = space->periodic ? 1 : 0;
  for (int i = 0; i < 9; ++i) {
    sp.lattice[i] = space->lattice[i];
    sp.inverse[i] = space->inverse[i];
  }
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  k_edge_geometry<<<grid_for(num_edges), kThreads, 0, st>>>(
      static_cast<const float *>(dst_positions), static_cast<const float *>(src_positions), sp,
      static_cast<const int64_t *>(row_ptr), static_cast<const int64_t *>(col), num_dst, num_edges,
      static_cast<float *>(displacement), static_cast<float *>(distance));
  TGB_LAUNCHED();
  return TGB_STATUS_OK;
}
