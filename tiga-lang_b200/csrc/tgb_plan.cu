// Per-graph plan: degree-bucket row order, split-row segments and the stable
// transposed relation.  Built once per graph on the device; deterministic
// (stable radix sorts and scans, integer counters only).
//
// What it re-derives from the reference (as heuristics, not code): the degree
// bucket bounds 1,2,4,...,2^k of lib/Transforms/PlanDegreeBuckets.cpp:32-143,
// the fixed-size chunk split of long rows of lib/Transforms/PlanSplitRows.cpp:
// 34-117 and the histogram -> prefix -> scatter work list of
// include/tiga/Transforms/Passes.td:95-103; the transposed relation is
// argsort(col_idx, stable) of python/tiga/interop/torch/relation_vjp.py:61-87.
#include <cub/device/device_radix_sort.cuh>
#include <cub/device/device_scan.cuh>

#include <new>

#include "tgb_common.cuh"

namespace tgb {
namespace {

constexpr int kKeyBits = 4;        // bucket keys 0..11
constexpr int kThreads = 256;

struct Counters {  // device-side, read back once per side
  long long min_degree;
  long long max_degree;
  unsigned long long n_long;
  unsigned long long n_seg;
};

template <typename PtrT>
__device__ __forceinline__ long long row_degree(const PtrT *ptr, int64_t r) {
  return (long long)ptr[r + 1] - (long long)ptr[r];
}

// key 0: long row (split); 1..10: degree 257-512 ... 1; 11: empty row.
__device__ __forceinline__ uint32_t bucket_key(long long degree) {
  if (degree > kSplitThreshold) return 0u;
  if (degree <= 0) return 11u;
  int b = degree > 1 ? 32 - __clz((int)degree - 1) : 0;  // ceil(log2(degree))
  return (uint32_t)(10 - b);
}

template <typename PtrT>
__global__ void k_row_keys(const PtrT *ptr, int64_t n_rows, uint32_t *keys,
                           uint32_t *rows, Counters *counters) {
  int64_t r = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  long long lo = LLONG_MAX, hi = 0;
  unsigned is_long = 0;
  if (r < n_rows) {
    long long d = row_degree(ptr, r);
    uint32_t key = bucket_key(d);
    keys[r] = key;
    rows[r] = (uint32_t)r;
    lo = hi = d;
    is_long = key == 0u;
  }
  // block-level reduction of min / max / long count, then one atomic each
  __shared__ long long s_lo[kThreads / 32], s_hi[kThreads / 32];
  __shared__ unsigned s_long[kThreads / 32];
  for (int o = 16; o; o >>= 1) {
    lo = min(lo, __shfl_xor_sync(0xffffffffu, lo, o));
    hi = max(hi, __shfl_xor_sync(0xffffffffu, hi, o));
    is_long += __shfl_xor_sync(0xffffffffu, is_long, o);
  }
  int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) { s_lo[warp] = lo; s_hi[warp] = hi; s_long[warp] = is_long; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int i = 1; i < kThreads / 32; ++i) {
      lo = min(lo, s_lo[i]); hi = max(hi, s_hi[i]); is_long += s_long[i];
    }
    if (lo != LLONG_MAX) atomicMin(&counters->min_degree, lo);
    atomicMax(&counters->max_degree, hi);
    if (is_long) atomicAdd(&counters->n_long, (unsigned long long)is_long);
  }
}

__global__ void k_init_counters(Counters *c) {
  c->min_degree = LLONG_MAX;
  c->max_degree = 0;
  c->n_long = 0;
  c->n_seg = 0;
}

// The first n_long entries of the sorted order are the long rows.
template <typename PtrT>
__global__ void k_long_counts(const PtrT *ptr, const uint32_t *order,
                              const Counters *counters, int64_t bound,
                              int32_t *seg_count) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= bound) return;
  int32_t c = 0;
  if ((unsigned long long)i < counters->n_long) {
    long long d = row_degree(ptr, order[i]);
    c = (int32_t)((d + kSegmentEdges - 1) / kSegmentEdges);
  }
  seg_count[i] = c;
}

__global__ void k_fill_segments(const int32_t *seg_ptr, Counters *counters,
                                int64_t bound, int32_t *seg_row) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  unsigned long long n_long = counters->n_long;
  if (i == 0) counters->n_seg = (unsigned long long)seg_ptr[n_long];
  if (i >= bound || (unsigned long long)i >= n_long) return;
  for (int32_t s = seg_ptr[i]; s < seg_ptr[i + 1]; ++s) seg_row[s] = (int32_t)i;
}

template <typename IdxT>
__global__ void k_expand_edges(const IdxT *col, int64_t E, uint32_t *keys,
                               uint32_t *vals) {
  int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= E) return;
  keys[e] = (uint32_t)col[e];
  vals[e] = (uint32_t)e;
}

// t_ptr[j] = first position in the sorted keys whose key is >= j.
__global__ void k_transposed_ptr(const uint32_t *sorted_keys, int64_t E,
                                 int64_t num_src, int64_t *t_ptr) {
  int64_t j = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (j > num_src) return;
  int64_t lo = 0, hi = E;
  while (lo < hi) {
    int64_t mid = (lo + hi) >> 1;
    if ((int64_t)sorted_keys[mid] < j) lo = mid + 1; else hi = mid;
  }
  t_ptr[j] = lo;
}

// t_dst[k] = destination row of original edge eid[k] (last row whose start is
// <= the edge id, skipping empty rows).
template <typename PtrT>
__global__ void k_transposed_dst(const PtrT *row_ptr, int64_t num_dst,
                                 const uint32_t *sorted_eid, int64_t E,
                                 uint32_t *eid_out, int32_t *t_dst) {
  int64_t k = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (k >= E) return;
  uint32_t e = sorted_eid[k];
  int64_t lo = 0, hi = num_dst;  // find the largest r with row_ptr[r] <= e
  while (hi - lo > 1) {
    int64_t mid = (lo + hi) >> 1;
    if ((int64_t)row_ptr[mid] <= (int64_t)e) lo = mid; else hi = mid;
  }
  eid_out[k] = e;
  t_dst[k] = (int32_t)lo;
}

// Work item of group g: segments of split rows first (g < n_seg), then whole
// rows in bucket order.
template <typename PtrT>
__global__ void k_fill_items(const PtrT *ptr, const int32_t *order, const int32_t *seg_row,
                             const int32_t *seg_ptr, int64_t n_rows, int64_t n_long,
                             int64_t n_seg, WorkItem *items) {
  const int64_t g = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (g >= n_seg + (n_rows - n_long)) return;
  WorkItem it;
  if (g < n_seg) {
    const int32_t lr = seg_row[g];
    const int32_t row = order[lr];
    const long long rb = (long long)ptr[row], re = (long long)ptr[row + 1];
    const long long beg = rb + (long long)(g - seg_ptr[lr]) * kSegmentEdges;
    it.beg = beg;
    it.row = row;
    it.count = (int32_t)((beg + kSegmentEdges < re ? beg + kSegmentEdges : re) - beg);
  } else {
    const int32_t row = order[n_long + (g - n_seg)];
    it.beg = (long long)ptr[row];
    it.row = row;
    it.count = (int32_t)((long long)ptr[row + 1] - it.beg);
  }
  items[g] = it;
}

__global__ void k_copy_u32(const uint32_t *src, int64_t n, int32_t *dst) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) dst[i] = (int32_t)src[i];
}

inline unsigned grid_for(int64_t n) {
  return (unsigned)(n > 0 ? ceil_div(n, kThreads) : 1);
}

int64_t long_row_bound(int64_t E, int64_t n_rows) {
  int64_t b = E / (kSplitThreshold + 1) + 1;
  return b < n_rows ? b : (n_rows > 0 ? n_rows : 1);
}
int64_t segment_bound(int64_t E, int64_t n_rows) {
  return E / kSegmentEdges + long_row_bound(E, n_rows) + 1;
}

int bits_for(int64_t n) {
  int b = 1;
  while (b < 32 && ((int64_t)1 << b) < n) ++b;
  return b;
}

struct Layout {
  // persistent
  uint64_t order_f, seg_ptr_f, seg_row_f, items_f;
  uint64_t t_ptr, t_dst, eid, order_b, seg_ptr_b, seg_row_b, items_b;
  uint64_t persistent_bytes;
  // temp
  uint64_t counters, k0, k1, v0, v1, seg_count, cub, cub_bytes;
  uint64_t temp_bytes;
};

int32_t compute_layout(int64_t num_dst, int64_t num_src, int64_t E, int flags,
                       Layout *L) {
  uint64_t p = 0;
  auto take = [&](uint64_t bytes) {
    uint64_t at = p;
    p = align_up(p + bytes, 256);
    return at;
  };
  L->order_f = take((uint64_t)(num_dst > 0 ? num_dst : 1) * 4);
  L->seg_ptr_f = take((uint64_t)(long_row_bound(E, num_dst) + 1) * 4);
  L->seg_row_f = take((uint64_t)segment_bound(E, num_dst) * 4);
  L->items_f = take((uint64_t)(segment_bound(E, num_dst) + num_dst) * sizeof(WorkItem));
  if (flags & TGB_PLAN_TRANSPOSE) {
    L->t_ptr = take((uint64_t)(num_src + 1) * 8);
    L->t_dst = take((uint64_t)(E > 0 ? E : 1) * 4);
    L->eid = take((uint64_t)(E > 0 ? E : 1) * 4);
    L->order_b = take((uint64_t)(num_src > 0 ? num_src : 1) * 4);
    L->seg_ptr_b = take((uint64_t)(long_row_bound(E, num_src) + 1) * 4);
    L->seg_row_b = take((uint64_t)segment_bound(E, num_src) * 4);
    L->items_b = take((uint64_t)(segment_bound(E, num_src) + num_src) * sizeof(WorkItem));
  }
  L->persistent_bytes = p;

  int64_t n_sort = num_dst;
  if (flags & TGB_PLAN_TRANSPOSE) {
    if (num_src > n_sort) n_sort = num_src;
    if (E > n_sort) n_sort = E;
  }
  if (n_sort < 1) n_sort = 1;
  // CUB temp: the larger of the sort and the scan requirements
  size_t sort_bytes = 0, scan_bytes = 0;
  cub::DoubleBuffer<uint32_t> dk(nullptr, nullptr), dv(nullptr, nullptr);
  cudaError_t err = cub::DeviceRadixSort::SortPairs(
      nullptr, sort_bytes, dk, dv, (int64_t)n_sort, 0, 32, (cudaStream_t)0);
  if (err != cudaSuccess)
    TGB_FAIL(TGB_STATUS_INTERNAL, "cub sort size query failed: %s",
             cudaGetErrorString(err));
  int64_t lb = long_row_bound(E, num_dst > num_src ? num_dst : num_src) + 1;
  err = cub::DeviceScan::ExclusiveSum(nullptr, scan_bytes, (int32_t *)nullptr,
                                      (int32_t *)nullptr, (int64_t)lb,
                                      (cudaStream_t)0);
  if (err != cudaSuccess)
    TGB_FAIL(TGB_STATUS_INTERNAL, "cub scan size query failed: %s",
             cudaGetErrorString(err));
  p = 0;
  L->counters = take(sizeof(Counters));
  L->k0 = take((uint64_t)n_sort * 4);
  L->k1 = take((uint64_t)n_sort * 4);
  L->v0 = take((uint64_t)n_sort * 4);
  L->v1 = take((uint64_t)n_sort * 4);
  L->seg_count = take((uint64_t)lb * 4);
  L->cub_bytes = (sort_bytes > scan_bytes ? sort_bytes : scan_bytes) + 256;
  L->cub = take(L->cub_bytes);
  L->temp_bytes = p;
  return TGB_STATUS_OK;
}

// Builds order / segments for one side.  `ptr` is the side's row pointer
// array; results go to order_out, seg_ptr_out, seg_row_out.
template <typename PtrT>
int32_t build_side(const PtrT *ptr, int64_t n_rows, int64_t E, char *temp,
                   const Layout &L, int32_t *order_out, int32_t *seg_ptr_out,
                   int32_t *seg_row_out, WorkItem *items_out, cudaStream_t stream, Side *side) {
  Counters *counters = reinterpret_cast<Counters *>(temp + L.counters);
  uint32_t *k0 = reinterpret_cast<uint32_t *>(temp + L.k0);
  uint32_t *k1 = reinterpret_cast<uint32_t *>(temp + L.k1);
  uint32_t *v0 = reinterpret_cast<uint32_t *>(temp + L.v0);
  uint32_t *v1 = reinterpret_cast<uint32_t *>(temp + L.v1);
  int32_t *seg_count = reinterpret_cast<int32_t *>(temp + L.seg_count);
  void *cub_temp = temp + L.cub;
  size_t cub_bytes = L.cub_bytes;

  k_init_counters<<<1, 1, 0, stream>>>(counters);
  TGB_LAUNCHED();
  if (n_rows > 0) {
    k_row_keys<PtrT><<<grid_for(n_rows), kThreads, 0, stream>>>(
        ptr, n_rows, k0, v0, counters);
    TGB_LAUNCHED();
    cub::DoubleBuffer<uint32_t> dk(k0, k1), dv(v0, v1);
    TGB_CUDA(cub::DeviceRadixSort::SortPairs(cub_temp, cub_bytes, dk, dv,
                                             (int64_t)n_rows, 0, kKeyBits,
                                             stream));
    g_launches.fetch_add(3);
    const uint32_t *sorted_rows = dv.Current();
    k_copy_u32<<<grid_for(n_rows), kThreads, 0, stream>>>(sorted_rows, n_rows,
                                                         order_out);
    TGB_LAUNCHED();
    int64_t bound = long_row_bound(E, n_rows);
    k_long_counts<PtrT><<<grid_for(bound + 1), kThreads, 0, stream>>>(
        ptr, sorted_rows, counters, bound + 1, seg_count);
    TGB_LAUNCHED();
    TGB_CUDA(cub::DeviceScan::ExclusiveSum(cub_temp, cub_bytes, seg_count,
                                           seg_ptr_out, (int64_t)(bound + 1),
                                           stream));
    g_launches.fetch_add(2);
    k_fill_segments<<<grid_for(bound), kThreads, 0, stream>>>(
        seg_ptr_out, counters, bound, seg_row_out);
    TGB_LAUNCHED();
  }
  Counters host;
  TGB_CUDA(cudaMemcpyAsync(&host, counters, sizeof(Counters),
                           cudaMemcpyDeviceToHost, stream));
  TGB_CUDA(cudaStreamSynchronize(stream));
  side->order = order_out;
  side->seg_ptr = seg_ptr_out;
  side->seg_row = seg_row_out;
  side->n_rows = n_rows;
  side->n_long = (int64_t)host.n_long;
  side->n_seg = (int64_t)host.n_seg;
  side->min_degree = n_rows > 0 && host.min_degree != LLONG_MAX ? host.min_degree : 0;
  side->max_degree = host.max_degree;
  side->items = items_out;
  const int64_t groups = side->n_seg + (n_rows - side->n_long);
  if (groups > 0) {
    k_fill_items<PtrT><<<grid_for(groups), kThreads, 0, stream>>>(
        ptr, order_out, seg_row_out, seg_ptr_out, n_rows, side->n_long, side->n_seg, items_out);
    TGB_LAUNCHED();
  }
  return TGB_STATUS_OK;
}

template <typename IdxT>
int32_t create_typed(const IdxT *row_ptr, const IdxT *col_idx, int64_t num_dst,
                     int64_t num_src, int64_t E, int flags, char *persistent,
                     char *temp, const Layout &L, cudaStream_t stream,
                     tgb_csr_plan *plan) {
  plan->fwd.ptr = row_ptr;
  plan->fwd.idx = col_idx;
  plan->fwd.ptr_bits = plan->fwd.idx_bits = (int)sizeof(IdxT) * 8;
  int32_t rc = build_side<IdxT>(
      row_ptr, num_dst, E, temp, L,
      reinterpret_cast<int32_t *>(persistent + L.order_f),
      reinterpret_cast<int32_t *>(persistent + L.seg_ptr_f),
      reinterpret_cast<int32_t *>(persistent + L.seg_row_f),
      reinterpret_cast<WorkItem *>(persistent + L.items_f), stream, &plan->fwd);
  if (rc) return rc;
  if (!(flags & TGB_PLAN_TRANSPOSE)) return TGB_STATUS_OK;

  int64_t *t_ptr = reinterpret_cast<int64_t *>(persistent + L.t_ptr);
  int32_t *t_dst = reinterpret_cast<int32_t *>(persistent + L.t_dst);
  uint32_t *eid = reinterpret_cast<uint32_t *>(persistent + L.eid);
  uint32_t *k0 = reinterpret_cast<uint32_t *>(temp + L.k0);
  uint32_t *k1 = reinterpret_cast<uint32_t *>(temp + L.k1);
  uint32_t *v0 = reinterpret_cast<uint32_t *>(temp + L.v0);
  uint32_t *v1 = reinterpret_cast<uint32_t *>(temp + L.v1);
  const uint32_t *sorted_keys = k0;
  if (E > 0) {
    k_expand_edges<IdxT><<<grid_for(E), kThreads, 0, stream>>>(col_idx, E, k0, v0);
    TGB_LAUNCHED();
    cub::DoubleBuffer<uint32_t> dk(k0, k1), dv(v0, v1);
    size_t cub_bytes = L.cub_bytes;
    TGB_CUDA(cub::DeviceRadixSort::SortPairs(temp + L.cub, cub_bytes, dk, dv,
                                             (int64_t)E, 0, bits_for(num_src),
                                             stream));
    g_launches.fetch_add(2 * ((bits_for(num_src) + 7) / 8) + 1);
    sorted_keys = dk.Current();
    k_transposed_dst<IdxT><<<grid_for(E), kThreads, 0, stream>>>(
        row_ptr, num_dst, dv.Current(), E, eid, t_dst);
    TGB_LAUNCHED();
  }
  k_transposed_ptr<<<grid_for(num_src + 1), kThreads, 0, stream>>>(
      sorted_keys, E, num_src, t_ptr);
  TGB_LAUNCHED();
  // the sort buffers are reused by build_side: wait until t_ptr is complete
  TGB_CUDA(cudaStreamSynchronize(stream));
  plan->t_ptr = t_ptr;
  plan->t_dst = t_dst;
  plan->bwd.ptr = t_ptr;
  plan->bwd.idx = t_dst;
  plan->bwd.eid = eid;
  plan->bwd.ptr_bits = 64;
  plan->bwd.idx_bits = 32;
  return build_side<int64_t>(
      t_ptr, num_src, E, temp, L,
      reinterpret_cast<int32_t *>(persistent + L.order_b),
      reinterpret_cast<int32_t *>(persistent + L.seg_ptr_b),
      reinterpret_cast<int32_t *>(persistent + L.seg_row_b),
      reinterpret_cast<WorkItem *>(persistent + L.items_b), stream, &plan->bwd);
}

int32_t check_sizes(int64_t num_dst, int64_t num_src, int64_t E, int32_t bits) {
  if (bits != 32 && bits != 64)
    TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "index_bits must be 32 or 64, got %d", bits);
  if (num_dst < 0 || num_src < 0 || E < 0)
    TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "negative graph dimension");
  if (num_dst >= ((int64_t)1 << 31) || num_src >= ((int64_t)1 << 31))
    TGB_FAIL(TGB_STATUS_UNSUPPORTED, "more than 2^31-1 rows are not supported");
  if (E >= ((int64_t)1 << 32))
    TGB_FAIL(TGB_STATUS_UNSUPPORTED, "more than 2^32-1 edges are not supported");
  return TGB_STATUS_OK;
}

}  // namespace
}  // namespace tgb

extern "C" {

int32_t tgb_csr_plan_sizes(int64_t num_dst, int64_t num_src, int64_t num_edges,
                           int32_t index_bits, int32_t flags,
                           uint64_t *persistent_bytes, uint64_t *temp_bytes) {
  if (!persistent_bytes || !temp_bytes)
    TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "null size output");
  int32_t rc = tgb::check_sizes(num_dst, num_src, num_edges, index_bits);
  if (rc) return rc;
  tgb::Layout L{};
  rc = tgb::compute_layout(num_dst, num_src, num_edges, flags, &L);
  if (rc) return rc;
  *persistent_bytes = L.persistent_bytes;
  *temp_bytes = L.temp_bytes;
  return TGB_STATUS_OK;
}

int32_t tgb_csr_plan_create(const void *row_ptr, const void *col_idx,
                            int64_t num_dst, int64_t num_src, int64_t num_edges,
                            int32_t index_bits, int32_t flags, void *persistent,
                            uint64_t persistent_bytes, void *temp,
                            uint64_t temp_bytes, uint64_t stream,
                            tgb_csr_plan **out_plan) {
  if (!out_plan) TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "null plan output");
  *out_plan = nullptr;
  int32_t rc = tgb::check_sizes(num_dst, num_src, num_edges, index_bits);
  if (rc) return rc;
  if (!row_ptr || (num_edges > 0 && !col_idx))
    TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "null CSR pointer");
  tgb::Layout L{};
  rc = tgb::compute_layout(num_dst, num_src, num_edges, flags, &L);
  if (rc) return rc;
  if (!persistent || persistent_bytes < L.persistent_bytes)
    TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT,
             "persistent buffer too small: %llu < %llu bytes",
             (unsigned long long)persistent_bytes,
             (unsigned long long)L.persistent_bytes);
  if (!temp || temp_bytes < L.temp_bytes)
    TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "temp buffer too small: %llu < %llu bytes",
             (unsigned long long)temp_bytes, (unsigned long long)L.temp_bytes);
  if (((uintptr_t)persistent & 255u) || ((uintptr_t)temp & 255u))
    TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "plan buffers must be 256-byte aligned");
  tgb_csr_plan *plan = new (std::nothrow) tgb_csr_plan();
  if (!plan) TGB_FAIL(TGB_STATUS_OUT_OF_MEMORY, "host allocation failed");
  plan->num_dst = num_dst;
  plan->num_src = num_src;
  plan->num_edges = num_edges;
  plan->index_bits = index_bits;
  plan->flags = flags;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (index_bits == 32)
    rc = tgb::create_typed<int32_t>((const int32_t *)row_ptr, (const int32_t *)col_idx,
                                    num_dst, num_src, num_edges, flags,
                                    (char *)persistent, (char *)temp, L, s, plan);
  else
    rc = tgb::create_typed<int64_t>((const int64_t *)row_ptr, (const int64_t *)col_idx,
                                    num_dst, num_src, num_edges, flags,
                                    (char *)persistent, (char *)temp, L, s, plan);
  if (rc) {
    delete plan;
    return rc;
  }
  *out_plan = plan;
  return TGB_STATUS_OK;
}

int32_t tgb_csr_plan_destroy(tgb_csr_plan *plan) {
  delete plan;
  return TGB_STATUS_OK;
}

namespace tgb {
namespace {
// eid_t[k] <- map[eid_t[k]]: the transposed side then addresses weights directly
__global__ void k_compose_edge_map(uint32_t *eid_t, const uint32_t *map, int64_t E) {
  int64_t k = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (k < E) eid_t[k] = map[eid_t[k]];
}
}  // namespace
}  // namespace tgb

int32_t tgb_csr_plan_set_edge_map(tgb_csr_plan *plan, const void *edge_map, uint64_t stream) {
  if (!plan || !edge_map) TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "null plan or edge map");
  if (plan->fwd.eid) TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "the plan already has an edge map");
  plan->fwd.eid = static_cast<const uint32_t *>(edge_map);
  if ((plan->flags & TGB_PLAN_TRANSPOSE) && plan->num_edges > 0) {
    tgb::k_compose_edge_map<<<tgb::grid_for(plan->num_edges), tgb::kThreads, 0,
                              reinterpret_cast<cudaStream_t>(stream)>>>(
        const_cast<uint32_t *>(plan->bwd.eid), plan->fwd.eid, plan->num_edges);
    TGB_LAUNCHED();
  }
  return TGB_STATUS_OK;
}

int32_t tgb_csr_plan_info(const tgb_csr_plan *plan, int64_t *info) {
  if (!plan || !info) TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "null plan or output");
  for (int i = 0; i < 16; ++i) info[i] = 0;
  info[0] = plan->num_dst;
  info[1] = plan->num_src;
  info[2] = plan->num_edges;
  info[3] = plan->fwd.min_degree;
  info[4] = plan->fwd.max_degree;
  info[5] = plan->fwd.n_long;
  info[6] = plan->fwd.n_seg;
  info[7] = plan->bwd.n_long;
  info[8] = plan->bwd.n_seg;
  info[9] = tgb::kSplitThreshold;
  info[10] = tgb::kSegmentEdges;
  info[11] = plan->bwd.min_degree;
  info[12] = plan->bwd.max_degree;
  return TGB_STATUS_OK;
}

int32_t tgb_csr_plan_array(const tgb_csr_plan *plan, int32_t which,
                           uint64_t *device_ptr, int64_t *count) {
  if (!plan || !device_ptr || !count)
    TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "null plan or output");
  bool t = plan->flags & TGB_PLAN_TRANSPOSE;
  switch (which) {
    case 0: *device_ptr = (uint64_t)plan->fwd.order; *count = plan->num_dst; break;
    case 1: *device_ptr = (uint64_t)plan->t_ptr; *count = t ? plan->num_src + 1 : 0; break;
    case 2: *device_ptr = (uint64_t)plan->t_dst; *count = t ? plan->num_edges : 0; break;
    case 3: *device_ptr = (uint64_t)plan->bwd.eid; *count = t ? plan->num_edges : 0; break;
    case 4: *device_ptr = (uint64_t)plan->bwd.order; *count = t ? plan->num_src : 0; break;
    default: TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "unknown plan array %d", which);
  }
  return TGB_STATUS_OK;
}

}  // extern "C"
