// Shared host/device helpers of libtiga_b200: status handling, the plan
// structure, and small load/store wrappers.  sm_100a only.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>
#include <cstdarg>
#include <cstdio>

#include "tiga_b200.h"

namespace tgb {

// ---- status + thread-local error text -------------------------------------
void set_error(const char *format, ...);
extern std::atomic<int64_t> g_launches;

#define TGB_FAIL(status, ...)   \
  do {                          \
    ::tgb::set_error(__VA_ARGS__); \
    return (status);            \
  } while (0)

#define TGB_CUDA(expr)                                                        \
  do {                                                                        \
    cudaError_t tgb_err_ = (expr);                                            \
    if (tgb_err_ != cudaSuccess) {                                            \
      ::tgb::set_error("%s failed: %s", #expr, cudaGetErrorString(tgb_err_)); \
      return tgb_err_ == cudaErrorMemoryAllocation ? TGB_STATUS_OUT_OF_MEMORY \
                                                   : TGB_STATUS_INTERNAL;     \
    }                                                                         \
  } while (0)

// Checks the launch that has just been enqueued and counts it.
#define TGB_LAUNCHED()                         \
  do {                                         \
    TGB_CUDA(cudaGetLastError());              \
    ::tgb::g_launches.fetch_add(1);            \
  } while (0)

// ---- plan -------------------------------------------------------------------
// Rows whose degree exceeds kSplitThreshold are cut into segments of
// kSegmentEdges edges; each segment is reduced by its own thread group into a
// partial row and a finalize kernel adds the partial rows in segment order.
constexpr int kSplitThreshold = 512;
constexpr int kSegmentEdges = 256;

// One unit of work of the CSR kernels: a whole row, or one segment of a split
// row.  16 bytes, so a thread group fetches its assignment with one 128-bit
// load instead of chasing order[] -> row_ptr[row], row_ptr[row + 1].
struct WorkItem {
  long long beg;   // first edge
  int32_t row;     // row the edges belong to
  int32_t count;   // number of edges
};

// One traversal direction: rows are destinations (forward, dw) or sources
// (dx over the transposed relation).
struct Side {
  const void *ptr = nullptr;     // row pointers: user's (32/64 bit) or int64
  const void *idx = nullptr;     // neighbour ids: user's col_idx or int32
  const uint32_t *eid = nullptr; // transposed only: original edge id per entry
  const int32_t *order = nullptr;     // [n_rows] long rows first, then buckets
  const int32_t *seg_row = nullptr;   // [n_seg] ordinal of the long row
  const int32_t *seg_ptr = nullptr;   // [n_long+1] first segment of long row
  const WorkItem *items = nullptr;    // [n_seg + n_rows - n_long] segments first, then rows in bucket order
  int64_t n_rows = 0;
  int64_t n_long = 0;
  int64_t n_seg = 0;
  int ptr_bits = 64;
  int idx_bits = 32;
  int64_t min_degree = 0;
  int64_t max_degree = 0;
};

}  // namespace tgb

struct tgb_csr_plan {
  int64_t num_dst = 0, num_src = 0, num_edges = 0;
  int index_bits = 64;
  int flags = 0;
  tgb::Side fwd;   // over CSR rows
  tgb::Side bwd;   // over transposed rows (flags & TGB_PLAN_TRANSPOSE)
  const int64_t *t_ptr = nullptr;  // == bwd.ptr
  const int32_t *t_dst = nullptr;  // == bwd.idx
};

namespace tgb {

// ---- device helpers ---------------------------------------------------------
__device__ __forceinline__ float4 ldg_f4(const float *p) {
  return __ldg(reinterpret_cast<const float4 *>(p));
}

template <typename T>
__device__ __forceinline__ T ld_stream(const T *p) {
  return __ldcs(p);
}

__device__ __forceinline__ void st_stream_f4(float *p, float4 v) {
  __stcs(reinterpret_cast<float4 *>(p), v);
}

// acc + a*b with the product rounded first (no fused multiply-add): keeps the
// bits of the sequential CPU definition of the row sum.
__device__ __forceinline__ float mul_add_rn(float a, float b, float acc) {
  return __fadd_rn(acc, __fmul_rn(a, b));
}

// Work list of one traversal side as the kernels see it.  Thread groups
// [0, n_seg) own segments of split rows, the rest own whole rows in bucket order.
struct WorkList {
  const void *ptr;
  const void *idx;
  const uint32_t *eid;
  const int32_t *order;
  const int32_t *seg_row;
  const int32_t *seg_ptr;
  const WorkItem *items;
  int64_t n_rows, n_long, n_seg;
};

inline WorkList work_list(const Side &side) {
  return WorkList{side.ptr, side.idx, side.eid, side.order, side.seg_row, side.seg_ptr, side.items,
                  side.n_rows, side.n_long, side.n_seg};
}

// The (row, edge range) of group `gid`: one 128-bit load of its work item.
__device__ __forceinline__ void load_work_item(const WorkItem *items, int64_t n_seg, int64_t gid,
                                               int64_t &row, int64_t &beg, int64_t &end, int64_t &seg) {
  const int4 raw = __ldg(reinterpret_cast<const int4 *>(items) + gid);
  beg = (int64_t)(((unsigned long long)(unsigned)raw.y << 32) | (unsigned long long)(unsigned)raw.x);
  row = raw.z;
  end = beg + raw.w;
  seg = gid < n_seg ? gid : -1;
}

template <typename PtrT>
__device__ __forceinline__ void decode_group(const WorkList &w, int64_t gid, int64_t &row,
                                             int64_t &beg, int64_t &end, int64_t &seg) {
  load_work_item(w.items, w.n_seg, gid, row, beg, end, seg);
}

inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }
inline uint64_t align_up(uint64_t v, uint64_t a) { return (v + a - 1) / a * a; }

}  // namespace tgb
