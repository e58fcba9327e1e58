// Online-softmax reducer with the score stored per edge and the value per source:
//
//   edge():  return self.reducer(edge.score, src.value)
//   out[i, h, :] = sum_{e in row i} p[e, h] * value[col[e], h, :],
//   p[e, h] = exp(score[e, h] - m[i, h]) / l[i, h],  m = row maximum, l = sum of exp(score - m)
//
// (the reference's stable-weighted reduction tile, lib/Target/Triton/Translate.cpp:3296-3352, and
// its eager definition, python/tiga/interop/torch/reducer_oracle.py:60-137: float32 state, an
// empty row yields exactly 0, (m, l) are kept for the backward).
//
// HBM bound: one gathered value row (H*D elements) per edge.  One warp owns a destination row; lane
// h < H keeps the head's running (m, l), every lane keeps up to kMaxPerLane output elements and
// fetches its head's weight by shuffle, so exp is evaluated once per (edge, head).  Rows wider
// than 32 * kMaxPerLane elements are processed in column passes.
//
// Backward, no atomics:
//   k_fs_bwd_dst  destination-major: delta[i,h] = <dout[i,h,:], out[i,h,:]>,
//                 d_score[e,h] = p (<dout[i,h,:], value[col[e],h,:]> - delta), and p is stored
//   k_fs_bwd_src  source-major over the plan's transposed relation:
//                 d_value[j,h,:] = sum_k p[eid[k],h] * dout[t_dst[k],h,:]
#include <cuda_bf16.h>

#include "tgb_common.cuh"

namespace tgb {
namespace {

constexpr int kWarpsPerBlock = 4;
constexpr int kMaxPerLane = 8;          // output elements a lane keeps per column pass

template <typename T>
__device__ __forceinline__ float load_value(const T *p);
template <>
__device__ __forceinline__ float load_value<float>(const float *p) { return __ldg(p); }
template <>
__device__ __forceinline__ float load_value<__nv_bfloat16>(const __nv_bfloat16 *p) {
  return __bfloat162float(*p);
}

struct FieldArgs {
  const void *ptr;          // row pointers of the traversed side
  const void *idx;          // neighbour ids of the traversed side
  const uint32_t *eid;      // transposed side: position of the entry in the edge arrays
  int64_t n_rows;
  const float *score;       // [E, H]
  const void *value;        // [num_src, H*D], float32 or bf16
  float *out;               // [N, H*D]
  float *m, *l;             // [N, H]
  const float *dout;        // [N, H*D]
  float *p;                 // [E, H] softmax weights, written by the destination-major pass
  float *d_score;           // [E, H]
  float *d_value;           // [num_src, H*D]
  int H, D;
};

// ------------------------------------------------------------------------------------------ forward
template <typename PtrT, typename IdxT, typename ValueT>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
k_fs_fwd(const FieldArgs a) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  if (row >= a.n_rows) return;
  const PtrT *ptr = static_cast<const PtrT *>(a.ptr);
  const IdxT *idx = static_cast<const IdxT *>(a.idx);
  const ValueT *value = static_cast<const ValueT *>(a.value);
  const int64_t beg = (int64_t)ptr[row], end = (int64_t)ptr[row + 1];
  const int H = a.H, D = a.D, HD = H * D;
  for (int f0 = 0; f0 < HD; f0 += 32 * kMaxPerLane) {
    // heads of this column pass are re-scanned per pass; lane h serves head h0 + h
    const int h0 = f0 / D;
    float m = -INFINITY, l = 0.0f;
    float acc[kMaxPerLane];
#pragma unroll
    for (int v = 0; v < kMaxPerLane; ++v) acc[v] = 0.0f;
    for (int64_t e = beg; e < end; ++e) {
      const int64_t c = (int64_t)idx[e];
      // lanes 0..31 cover heads h0 .. h0+31 (a pass spans at most 32 * kMaxPerLane / D + 1 heads)
      const int my_head = h0 + lane;
      float scale = 1.0f, weight = 0.0f;
      if (my_head < H) {
        const float s = __ldg(a.score + e * H + my_head);
        const float m_new = fmaxf(m, s);
        // m_new == -inf only while every score so far is -inf: keep the state at zero
        scale = m_new == -INFINITY ? 1.0f : expf(m - m_new);
        weight = m_new == -INFINITY ? 0.0f : expf(s - m_new);
        l = l * scale + weight;
        m = m_new;
      }
#pragma unroll
      for (int v = 0; v < kMaxPerLane; ++v) {
        const int f = f0 + lane + 32 * v;
        const int src_lane = f < HD ? f / D - h0 : 0;
        const float sc = __shfl_sync(0xffffffffu, scale, src_lane);
        const float wt = __shfl_sync(0xffffffffu, weight, src_lane);
        if (f < HD) acc[v] = acc[v] * sc + wt * load_value(value + c * HD + f);
      }
    }
#pragma unroll
    for (int v = 0; v < kMaxPerLane; ++v) {
      const int f = f0 + lane + 32 * v;
      const int src_lane = f < HD ? f / D - h0 : 0;
      const float denom = __shfl_sync(0xffffffffu, l, src_lane);
      if (f < HD) a.out[row * HD + f] = denom > 0.0f ? acc[v] / denom : 0.0f;
    }
    // a head may be visited by two consecutive passes; both compute the same (m, l)
    const int my_head = h0 + lane;
    const int last_head = (min(f0 + 32 * kMaxPerLane, HD) - 1) / D;
    if (my_head <= last_head && my_head < H) {
      a.m[row * H + my_head] = m;
      a.l[row * H + my_head] = l;
    }
  }
}

// ---------------------------------------------------------------------- backward, destination-major
template <typename PtrT, typename IdxT, typename ValueT>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
k_fs_bwd_dst(const FieldArgs a) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  if (row >= a.n_rows) return;
  const PtrT *ptr = static_cast<const PtrT *>(a.ptr);
  const IdxT *idx = static_cast<const IdxT *>(a.idx);
  const ValueT *value = static_cast<const ValueT *>(a.value);
  const int64_t beg = (int64_t)ptr[row], end = (int64_t)ptr[row + 1];
  const int H = a.H, D = a.D, HD = H * D;
  // one head at a time: the warp's lanes stride over the head's D elements
  for (int h = 0; h < H; ++h) {
    const float m = a.m[row * H + h], l = a.l[row * H + h];
    const float *g = a.dout + row * HD + h * D;
    const float *o = a.out + row * HD + h * D;
    float delta = 0.0f;
    for (int d = lane; d < D; d += 32) delta += g[d] * o[d];
#pragma unroll
    for (int s = 16; s; s >>= 1) delta += __shfl_xor_sync(0xffffffffu, delta, s);
    for (int64_t e = beg; e < end; ++e) {
      const int64_t c = (int64_t)idx[e];
      float dot = 0.0f;
      for (int d = lane; d < D; d += 32) dot += g[d] * load_value(value + c * HD + h * D + d);
#pragma unroll
      for (int s = 16; s; s >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, s);
      if (lane == 0) {
        const float score = a.score[e * H + h];
        const float p = l > 0.0f && m != -INFINITY ? expf(score - m) / l : 0.0f;
        a.p[e * H + h] = p;
        a.d_score[e * H + h] = p * (dot - delta);
      }
    }
  }
}

// --------------------------------------------------------------------------- backward, source-major
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
k_fs_bwd_src(const FieldArgs a) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);   // a source
  if (row >= a.n_rows) return;
  const int64_t *ptr = static_cast<const int64_t *>(a.ptr);
  const int32_t *dst = static_cast<const int32_t *>(a.idx);
  const int64_t beg = ptr[row], end = ptr[row + 1];
  const int H = a.H, D = a.D, HD = H * D;
  for (int f0 = 0; f0 < HD; f0 += 32 * kMaxPerLane) {
    float acc[kMaxPerLane];
#pragma unroll
    for (int v = 0; v < kMaxPerLane; ++v) acc[v] = 0.0f;
    for (int64_t k = beg; k < end; ++k) {
      const int64_t i = dst[k];
      const int64_t e = a.eid[k];
#pragma unroll
      for (int v = 0; v < kMaxPerLane; ++v) {
        const int f = f0 + lane + 32 * v;
        if (f < HD) acc[v] += __ldg(a.p + e * H + f / D) * __ldg(a.dout + i * HD + f);
      }
    }
#pragma unroll
    for (int v = 0; v < kMaxPerLane; ++v) {
      const int f = f0 + lane + 32 * v;
      if (f < HD) a.d_value[row * HD + f] = acc[v];
    }
  }
}

inline unsigned blocks_for_rows(int64_t rows) { return (unsigned)ceil_div(rows > 0 ? rows : 1, kWarpsPerBlock); }

int32_t check_shapes(const tgb_csr_plan *plan, int32_t H, int32_t D, int32_t value_dtype) {
  if (!plan) TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "null plan");
  if (H <= 0 || D <= 0) TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "heads and payload width must be positive");
  if (H > 32 * kMaxPerLane) TGB_FAIL(TGB_STATUS_UNSUPPORTED, "more than %d softmax lanes per row", 32 * kMaxPerLane);
  if (value_dtype != TGB_DTYPE_F32 && value_dtype != TGB_DTYPE_BF16)
    TGB_FAIL(TGB_STATUS_UNSUPPORTED, "values must be float32 or bfloat16");
  // a column pass of 32 * kMaxPerLane elements must not span more than 32 heads (one lane per head)
  if (D <= kMaxPerLane && H > 32)
    TGB_FAIL(TGB_STATUS_UNSUPPORTED, "payload of at most %d elements with more than 32 heads", kMaxPerLane);
  return TGB_STATUS_OK;
}

}  // namespace
}  // namespace tgb

using namespace tgb;

extern "C" int32_t tgb_softmax_field_fwd(const tgb_csr_plan *plan, const void *score, const void *value,
                                         int32_t value_dtype, void *out, void *m, void *l, int32_t H, int32_t D,
                                         uint64_t stream) {
  int32_t rc = check_shapes(plan, H, D, value_dtype);
  if (rc) return rc;
  if (plan->num_dst == 0) return TGB_STATUS_OK;
  if (!out || !m || !l || (plan->num_edges > 0 && (!score || !value)))
    TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "null pointer");
  FieldArgs a{};
  a.ptr = plan->fwd.ptr;
  a.idx = plan->fwd.idx;
  a.n_rows = plan->num_dst;
  a.score = (const float *)score;
  a.value = value;
  a.out = (float *)out;
  a.m = (float *)m;
  a.l = (float *)l;
  a.H = H;
  a.D = D;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const unsigned blocks = blocks_for_rows(plan->num_dst);
  const bool bf = value_dtype == TGB_DTYPE_BF16;
  if (plan->index_bits == 32) {
    if (bf) k_fs_fwd<int32_t, int32_t, __nv_bfloat16><<<blocks, kWarpsPerBlock * 32, 0, st>>>(a);
    else k_fs_fwd<int32_t, int32_t, float><<<blocks, kWarpsPerBlock * 32, 0, st>>>(a);
  } else {
    if (bf) k_fs_fwd<int64_t, int64_t, __nv_bfloat16><<<blocks, kWarpsPerBlock * 32, 0, st>>>(a);
    else k_fs_fwd<int64_t, int64_t, float><<<blocks, kWarpsPerBlock * 32, 0, st>>>(a);
  }
  TGB_LAUNCHED();
  return TGB_STATUS_OK;
}

extern "C" int32_t tgb_softmax_field_bwd(const tgb_csr_plan *plan, const void *score, const void *value,
                                         int32_t value_dtype, const void *out, const void *dout, const void *m,
                                         const void *l, int32_t H, int32_t D, void *d_score, void *d_value,
                                         void *p_scratch, uint64_t stream) {
  int32_t rc = check_shapes(plan, H, D, value_dtype);
  if (rc) return rc;
  if (!(plan->flags & TGB_PLAN_TRANSPOSE))
    TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "plan was created without TGB_PLAN_TRANSPOSE");
  if (plan->fwd.eid) TGB_FAIL(TGB_STATUS_UNSUPPORTED, "the softmax reducer does not take a plan with an edge map");
  if ((plan->num_src > 0 && !d_value) || (plan->num_edges > 0 && (!d_score || !p_scratch || !score || !value)) ||
      (plan->num_dst > 0 && (!out || !dout || !m || !l)))
    TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "null pointer");
  FieldArgs a{};
  a.score = (const float *)score;
  a.value = value;
  a.out = (float *)const_cast<void *>(out);
  a.m = (float *)const_cast<void *>(m);
  a.l = (float *)const_cast<void *>(l);
  a.dout = (const float *)dout;
  a.p = (float *)p_scratch;
  a.d_score = (float *)d_score;
  a.d_value = (float *)d_value;
  a.H = H;
  a.D = D;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const bool bf = value_dtype == TGB_DTYPE_BF16;
  if (plan->num_dst > 0 && plan->num_edges > 0) {
    a.ptr = plan->fwd.ptr;
    a.idx = plan->fwd.idx;
    a.n_rows = plan->num_dst;
    const unsigned blocks = blocks_for_rows(plan->num_dst);
    if (plan->index_bits == 32) {
      if (bf) k_fs_bwd_dst<int32_t, int32_t, __nv_bfloat16><<<blocks, kWarpsPerBlock * 32, 0, st>>>(a);
      else k_fs_bwd_dst<int32_t, int32_t, float><<<blocks, kWarpsPerBlock * 32, 0, st>>>(a);
    } else {
      if (bf) k_fs_bwd_dst<int64_t, int64_t, __nv_bfloat16><<<blocks, kWarpsPerBlock * 32, 0, st>>>(a);
      else k_fs_bwd_dst<int64_t, int64_t, float><<<blocks, kWarpsPerBlock * 32, 0, st>>>(a);
    }
    TGB_LAUNCHED();
  }
  if (plan->num_src > 0) {
    a.ptr = plan->bwd.ptr;
    a.idx = plan->bwd.idx;
    a.eid = plan->bwd.eid;
    a.n_rows = plan->num_src;
    k_fs_bwd_src<<<blocks_for_rows(plan->num_src), kWarpsPerBlock * 32, 0, st>>>(a);
    TGB_LAUNCHED();
  }
  return TGB_STATUS_OK;
}
