// Fused gather + reduce over CSR rows: forward (sum / mean / max), dx over the
// stable transposed relation, and dw as a per-edge dot product.
//
// Mapping.  A row is owned by a group of G lanes (G = 16-byte vectors per
// feature row, capped at a warp); a lane keeps VPL float4 accumulators.  Groups
// take rows from the plan's degree-bucket order, so the groups of one CTA hold
// rows of similar length.  Rows above the split threshold are cut into
// fixed-size segments reduced by separate groups into partial rows; a finalize
// kernel adds the partial rows in segment order (the cross-CTA reduction).
// Per step a group loads G neighbour ids (and weights) with one coalesced
// load, broadcasts them by shuffle and gathers whole feature rows with 128-bit
// loads, several in flight per lane.
//
// HBM roofline bound.  Algorithmic bytes per edge are index + weight + one
// feature row (F*4 bytes); per row the pointer and one written row.
//
// Summation order inside a row is the edge order and the product is rounded
// before the add, i.e. the sequential CPU definition of the reference
// (lib/Transforms/LowerTensorToCPU.cpp:672-702) for every unsplit row.
#include "tgb_common.cuh"

namespace tgb {
namespace {

// Tunables (overridable at build time for sweeps).  Measured on B200 with the
// GCN-layer workload: 128-thread CTAs and 4 rows in flight per lane were the
// fastest of {128, 256} x {2, 4, 6, 8}; forcing fewer registers or a rolling
// software pipeline was slower.
#ifndef TGB_BLOCK
#define TGB_BLOCK 128
#endif
#ifndef TGB_MIN_BLOCKS
#define TGB_MIN_BLOCKS 1
#endif
#ifndef TGB_U32
#define TGB_U32 4
#endif
// Index pipeline of the gather kernel (ids of batch b+2 load while batch b is gathered): measured
// on B200 at 128 / 64 floats per row, forward 2.36 -> 2.31 / 1.35 -> 1.27 ms and the transposed pass
// 2.93 -> 2.70 / 1.93 -> 1.70 ms on the 60 M-edge R-MAT; the per-edge dot kernel measured 2 % slower
// with the same pipeline (2.42 -> 2.47 ms), so it keeps the plain loop.
#ifndef TGB_PREFETCH
#define TGB_PREFETCH 1
#endif
#ifndef TGB_PREFETCH_DOT
#define TGB_PREFETCH_DOT 0
#endif

constexpr int kBlock = TGB_BLOCK;

enum Mode { kSum = 0, kMax = 2 };

struct GatherArgs {
  const void *ptr;        // row pointers of this side
  const void *idx;        // neighbour ids of this side
  const uint32_t *eid;    // transposed side: original edge id (weights, argmax)
  const int32_t *order;   // plan row order
  const int32_t *seg_row; // segment -> long-row ordinal
  const int32_t *seg_ptr; // long-row ordinal -> first segment
  const WorkItem *items;  // one per thread group: (first edge, row, edge count)
  int64_t n_rows, n_long, n_seg;
  const float *x;         // gathered rows [*, F]
  const float *w;         // per-edge weight or null
  float *out;             // [n_rows, F]
  float *partial;         // [n_seg, F] partial rows of split rows
  int32_t *arg_out;       // max forward: winning edge per element
  int32_t *arg_partial;   // max forward: per-segment winners
  const int32_t *arg_in;  // max dx: winners [num_dst, F] (gathered with x)
  const void *deg_ptr;    // mean: row pointers used for the final divide
  int64_t F;
  float identity;
  int mean;               // divide finished rows by their length
  int accumulate;         // add to the rows already in `out`; rows without edges stay untouched
};

template <typename T>
__device__ __forceinline__ T shfl_group(unsigned mask, T v, int src, int width) {
  return __shfl_sync(mask, v, src, width);
}

// Which (row, edge range) group `gid` owns: groups [0, n_seg) own segments of
// long rows, the rest whole rows in bucket order.  The plan stores the answer
// as one 16-byte work item per group.
template <typename PtrT>
__device__ __forceinline__ void decode_work(const GatherArgs &a, int64_t gid,
                                            int64_t &row, int64_t &beg,
                                            int64_t &end, int64_t &seg) {
  load_work_item(a.items, a.n_seg, gid, row, beg, end, seg);
}

__device__ __forceinline__ void max_update(float m, int32_t e, float &acc,
                                           int32_t &arg) {
  // arith.maximumf: NaN poisons the state; the first winner is kept
  if (m > acc || (m != m && acc == acc)) {
    acc = m;
    arg = e;
  }
}

// ---------------------------------------------------------------------------
// Vector path: F % 4 == 0, 16-byte aligned rows.
//   G    lanes per row (power of two <= 32)
//   VPL  float4 per lane: 4 when F = 16 * G (the usual widths), else 1 and the
//        row may use fewer than G lanes
//   U    gathered rows in flight per lane
// ---------------------------------------------------------------------------
template <typename PtrT, typename IdxT, int G, int VPL, int U, int MODE,
          bool HAS_W, bool W_BY_EID, bool ARG_FILTER>
__global__ void __launch_bounds__(kBlock, TGB_MIN_BLOCKS)
k_gather_vec(const GatherArgs a) {
  const int lane = threadIdx.x & (G - 1);
  const int64_t gid = ((int64_t)blockIdx.x * kBlock + threadIdx.x) / G;
  if (gid >= a.n_seg + (a.n_rows - a.n_long)) return;
  // lanes of this group inside the warp
  const unsigned gmask = G == 32 ? 0xffffffffu
                                 : (((1u << G) - 1u) << ((threadIdx.x & 31) & ~(G - 1)));
  int64_t row, beg, end, seg;
  decode_work<PtrT>(a, gid, row, beg, end, seg);
  const IdxT *idx = static_cast<const IdxT *>(a.idx);
  const int64_t F = a.F;
  const int vecs = (int)(F >> 2);            // float4 per row
  const bool active = lane < vecs;           // G may exceed the row's vectors
  const float start = (seg >= 0 || a.mean) ? (MODE == kMax ? a.identity : 0.0f)
                                           : a.identity;
  if (a.accumulate && beg == end) return;

  float4 acc[VPL];
  int4 arg[MODE == kMax ? VPL : 1];
#pragma unroll
  for (int v = 0; v < VPL; ++v) {
    acc[v] = make_float4(start, start, start, start);
    if (a.accumulate && seg < 0 && active) acc[v] = *reinterpret_cast<const float4 *>(a.out + row * F + 4 * (lane + v * G));
    if constexpr (MODE == kMax) arg[v] = make_int4(-1, -1, -1, -1);
  }

  // Index pipeline: while the rows of batch b are gathered, the neighbour ids (and edge ids /
  // direct weights) of batch b+2 are already loading and the edge-mapped weights of batch b+1,
  // whose edge ids arrived one batch ago, are issued; no gather waits on an index load after the
  // first batch of a row.
  auto load_ids = [&](int64_t at, int32_t &c_, uint32_t &eid_, float &w_) {
    c_ = 0; eid_ = 0; w_ = 1.0f;
    const int64_t e_ = at + lane;
    if (e_ < end) {
      c_ = (int32_t)ld_stream(idx + e_);
      if (W_BY_EID || ARG_FILTER) eid_ = ld_stream(a.eid + e_);
      if (HAS_W && !W_BY_EID) w_ = ld_stream(a.w + e_);
    }
  };
  int32_t c, c1, c2;
  uint32_t my_eid, eid1, eid2;
  float wv, w1, w2;
  load_ids(beg, c, my_eid, wv);
#if TGB_PREFETCH
  load_ids(beg + G, c1, eid1, w1);
#endif
  if (HAS_W && W_BY_EID && beg + lane < end) wv = __ldg(a.w + my_eid);
  for (int64_t base = beg; base < end; base += G) {
#if TGB_PREFETCH
    load_ids(base + 2 * G, c2, eid2, w2);
    if (HAS_W && W_BY_EID && base + G + lane < end) w1 = __ldg(a.w + eid1);
#endif
    const int n = (int)(end - base < G ? end - base : G);
    for (int k0 = 0; k0 < n; k0 += U) {
      float4 val[U][VPL];
      int4 win[ARG_FILTER ? U : 1][ARG_FILTER ? VPL : 1];
      float ww[U];
      int32_t ee[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int k = k0 + u;
        const int src = k < n ? k : n - 1;
        const int32_t cc = shfl_group(gmask, c, src, G);
        ww[u] = HAS_W ? shfl_group(gmask, wv, src, G) : 1.0f;
        if constexpr (ARG_FILTER) ee[u] = (int32_t)shfl_group(gmask, my_eid, src, G);
        else ee[u] = (int32_t)(base + k);
        if (k < n && active) {
          const float *xr = a.x + (int64_t)cc * F;
#pragma unroll
          for (int v = 0; v < VPL; ++v) {
            val[u][v] = ldg_f4(xr + 4 * (lane + v * G));
            if constexpr (ARG_FILTER)
              win[u][v] = __ldg(reinterpret_cast<const int4 *>(
                  a.arg_in + (int64_t)cc * F + 4 * (lane + v * G)));
          }
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (k0 + u < n && active) {
#pragma unroll
          for (int v = 0; v < VPL; ++v) {
            float4 m = val[u][v];
            if (HAS_W) {
              m.x = __fmul_rn(ww[u], m.x); m.y = __fmul_rn(ww[u], m.y);
              m.z = __fmul_rn(ww[u], m.z); m.w = __fmul_rn(ww[u], m.w);
            }
            if constexpr (MODE == kMax) {
              max_update(m.x, ee[u], acc[v].x, arg[v].x);
              max_update(m.y, ee[u], acc[v].y, arg[v].y);
              max_update(m.z, ee[u], acc[v].z, arg[v].z);
              max_update(m.w, ee[u], acc[v].w, arg[v].w);
            } else if constexpr (ARG_FILTER) {
              // only the winning edge of (row, element) passes its cotangent
              if (win[u][v].x == ee[u]) acc[v].x = __fadd_rn(acc[v].x, m.x);
              if (win[u][v].y == ee[u]) acc[v].y = __fadd_rn(acc[v].y, m.y);
              if (win[u][v].z == ee[u]) acc[v].z = __fadd_rn(acc[v].z, m.z);
              if (win[u][v].w == ee[u]) acc[v].w = __fadd_rn(acc[v].w, m.w);
            } else {
              acc[v].x = __fadd_rn(acc[v].x, m.x); acc[v].y = __fadd_rn(acc[v].y, m.y);
              acc[v].z = __fadd_rn(acc[v].z, m.z); acc[v].w = __fadd_rn(acc[v].w, m.w);
            }
          }
        }
      }
    }
#if TGB_PREFETCH
    c = c1; my_eid = eid1; wv = w1;
    c1 = c2; eid1 = eid2; w1 = w2;
#else
    load_ids(base + G, c, my_eid, wv);
    if (HAS_W && W_BY_EID && base + G + lane < end) wv = __ldg(a.w + my_eid);
#endif
  }
  if (!active) return;
  if (seg < 0 && a.mean) {
    const float count = (float)(end - beg);
#pragma unroll
    for (int v = 0; v < VPL; ++v) {
      acc[v].x = __fdiv_rn(acc[v].x, count); acc[v].y = __fdiv_rn(acc[v].y, count);
      acc[v].z = __fdiv_rn(acc[v].z, count); acc[v].w = __fdiv_rn(acc[v].w, count);
    }
  }
  float *dst = seg >= 0 ? a.partial + seg * F : a.out + row * F;
#pragma unroll
  for (int v = 0; v < VPL; ++v) st_stream_f4(dst + 4 * (lane + v * G), acc[v]);
  if constexpr (MODE == kMax) {
    int32_t *adst = seg >= 0 ? a.arg_partial + seg * F : a.arg_out + row * F;
#pragma unroll
    for (int v = 0; v < VPL; ++v)
      *reinterpret_cast<int4 *>(adst + 4 * (lane + v * G)) = arg[v];
  }
}

// Scalar path: any F, no alignment requirement.  A group of G lanes strides
// over the F elements of the row.
template <typename PtrT, typename IdxT, int G, int MODE, bool HAS_W,
          bool W_BY_EID, bool ARG_FILTER>
__global__ void __launch_bounds__(kBlock)
k_gather_scalar(const GatherArgs a) {
  const int lane = threadIdx.x & (G - 1);
  const int64_t gid = ((int64_t)blockIdx.x * kBlock + threadIdx.x) / G;
  if (gid >= a.n_seg + (a.n_rows - a.n_long)) return;
  int64_t row, beg, end, seg;
  decode_work<PtrT>(a, gid, row, beg, end, seg);
  const IdxT *idx = static_cast<const IdxT *>(a.idx);
  const int64_t F = a.F;
  const float start = (seg >= 0 || a.mean) ? (MODE == kMax ? a.identity : 0.0f)
                                           : a.identity;
  if (a.accumulate && beg == end) return;
  for (int64_t f = lane; f < F; f += G) {
    float acc = (a.accumulate && seg < 0) ? a.out[row * F + f] : start;
    int32_t arg = -1;
    for (int64_t e = beg; e < end; ++e) {
      const int64_t c = (int64_t)idx[e];
      const uint32_t oe = (W_BY_EID || ARG_FILTER) ? a.eid[e] : (uint32_t)e;
      float m = __ldg(a.x + c * F + f);
      if (HAS_W) m = __fmul_rn(W_BY_EID ? a.w[oe] : a.w[e], m);
      if (MODE == kMax) {
        max_update(m, (int32_t)e, acc, arg);
      } else if (ARG_FILTER) {
        if (a.arg_in[c * F + f] == (int32_t)oe) acc = __fadd_rn(acc, m);
      } else {
        acc = __fadd_rn(acc, m);
      }
    }
    if (seg < 0 && a.mean) acc = __fdiv_rn(acc, (float)(end - beg));
    if (seg >= 0) {
      a.partial[seg * F + f] = acc;
      if (MODE == kMax) a.arg_partial[seg * F + f] = arg;
    } else {
      a.out[row * F + f] = acc;
      if (MODE == kMax) a.arg_out[row * F + f] = arg;
    }
  }
}

// Adds (or max-combines) the partial rows of every split row in segment order.
template <typename PtrT, int MODE>
__global__ void __launch_bounds__(kBlock)
k_finalize_split(const GatherArgs a) {
  const int64_t lr = blockIdx.x;  // one CTA per long row
  if (lr >= a.n_long) return;
  const int64_t row = a.order[lr];
  const int32_t s0 = a.seg_ptr[lr], s1 = a.seg_ptr[lr + 1];
  const PtrT *ptr = static_cast<const PtrT *>(a.ptr);
  const float count = (float)((int64_t)ptr[row + 1] - (int64_t)ptr[row]);
  for (int64_t f = threadIdx.x; f < a.F; f += kBlock) {
    float acc = a.accumulate ? a.out[row * a.F + f] : (a.mean ? 0.0f : a.identity);
    int32_t arg = -1;
    // 16 partial rows are fetched at once (the longest row of a power-law graph
    // has hundreds of segments and one CTA walks them), then folded in order
    for (int32_t s = s0; s < s1; s += 16) {
      float p[16];
      int32_t q[MODE == kMax ? 16 : 1];
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const bool in = s + j < s1;
        p[j] = in ? __ldcs(a.partial + (int64_t)(s + j) * a.F + f) : 0.0f;
        if constexpr (MODE == kMax) q[j] = in ? __ldcs(a.arg_partial + (int64_t)(s + j) * a.F + f) : -1;
      }
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        if (s + j < s1) {
          if constexpr (MODE == kMax) max_update(p[j], q[j], acc, arg);
          else acc = __fadd_rn(acc, p[j]);
        }
      }
    }
    if (a.mean) acc = __fdiv_rn(acc, count);
    a.out[row * a.F + f] = acc;
    if (MODE == kMax) a.arg_out[row * a.F + f] = arg;
  }
}

// dy / row length, the mean reducer's cotangent (row-wise, vectorised by 1).
template <typename PtrT>
__global__ void k_scale_by_degree(const PtrT *ptr, const float *dy, int64_t N,
                                  int64_t F, float *out) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= N * F) return;
  const int64_t r = i / F;
  out[i] = __fdiv_rn(dy[i], (float)((int64_t)ptr[r + 1] - (int64_t)ptr[r]));
}

// ---------------------------------------------------------------------------
// dw[e] = <dy[row,:], x[col[e],:]>: the row's cotangent stays in registers, one
// gathered row per edge, group-wide shuffle reduction, coalesced store of up
// to G results per step.  MAX keeps only elements whose winner is the edge.
// ---------------------------------------------------------------------------
template <typename PtrT, typename IdxT, int G, int VPL, int U, bool ARG_FILTER>
__global__ void __launch_bounds__(kBlock, TGB_MIN_BLOCKS)
k_edge_dot_vec(const GatherArgs a, const float *dy, float *dw) {
  const int lane = threadIdx.x & (G - 1);
  const int64_t gid = ((int64_t)blockIdx.x * kBlock + threadIdx.x) / G;
  if (gid >= a.n_seg + (a.n_rows - a.n_long)) return;
  const unsigned gmask = G == 32 ? 0xffffffffu
                                 : (((1u << G) - 1u) << ((threadIdx.x & 31) & ~(G - 1)));
  int64_t row, beg, end, seg;
  decode_work<PtrT>(a, gid, row, beg, end, seg);
  const IdxT *idx = static_cast<const IdxT *>(a.idx);
  const int64_t F = a.F;
  const int vecs = (int)(F >> 2);
  const bool active = lane < vecs;
  float4 g[VPL];
  int4 win[ARG_FILTER ? VPL : 1];
#pragma unroll
  for (int v = 0; v < VPL; ++v) {
    g[v] = active ? ldg_f4(dy + row * F + 4 * (lane + v * G)) : make_float4(0, 0, 0, 0);
    if constexpr (ARG_FILTER)
      win[v] = active ? __ldg(reinterpret_cast<const int4 *>(a.arg_in + row * F + 4 * (lane + v * G)))
                      : make_int4(-1, -1, -1, -1);
  }
  // the neighbour ids (and mapped edge ids) of the next batch load while this batch is gathered
  auto load_ids = [&](int64_t at, int32_t &c_, int64_t &slot_) {
    const int64_t e_ = at + lane;
    c_ = 0;
    slot_ = e_;
    if (e_ < end) {
      c_ = (int32_t)ld_stream(idx + e_);
      if (a.eid) slot_ = (int64_t)ld_stream(a.eid + e_);
    }
  };
  int32_t c, c_next = 0;
  int64_t slot, slot_next = 0;
  load_ids(beg, c, slot);
  for (int64_t base = beg; base < end; base += G) {
    const int64_t e = base + lane;
#if TGB_PREFETCH_DOT
    load_ids(base + G, c_next, slot_next);
#endif
    const int n = (int)(end - base < G ? end - base : G);
    float mine = 0.0f;
    for (int k0 = 0; k0 < n; k0 += U) {
      float4 val[U][VPL];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int k = k0 + u;
        const int32_t cc = shfl_group(gmask, c, k < n ? k : n - 1, G);
#pragma unroll
        for (int v = 0; v < VPL; ++v)
          val[u][v] = (k < n && active) ? ldg_f4(a.x + (int64_t)cc * F + 4 * (lane + v * G))
                                        : make_float4(0, 0, 0, 0);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int32_t ee = (int32_t)(base + k0 + u);
        float p = 0.0f;
#pragma unroll
        for (int v = 0; v < VPL; ++v) {
          if constexpr (ARG_FILTER) {
            if (win[v].x == ee) p = fmaf(g[v].x, val[u][v].x, p);
            if (win[v].y == ee) p = fmaf(g[v].y, val[u][v].y, p);
            if (win[v].z == ee) p = fmaf(g[v].z, val[u][v].z, p);
            if (win[v].w == ee) p = fmaf(g[v].w, val[u][v].w, p);
          } else {
            p = fmaf(g[v].x, val[u][v].x, p); p = fmaf(g[v].y, val[u][v].y, p);
            p = fmaf(g[v].z, val[u][v].z, p); p = fmaf(g[v].w, val[u][v].w, p);
          }
        }
#pragma unroll
        for (int o = G >> 1; o; o >>= 1) p += __shfl_xor_sync(gmask, p, o, G);
        if (lane == k0 + u) mine = p;
      }
    }
    if (e < end) dw[slot] = mine;
#if TGB_PREFETCH_DOT
    c = c_next; slot = slot_next;
#else
    load_ids(base + G, c, slot);
#endif
  }
}

template <typename PtrT, typename IdxT, bool ARG_FILTER>
__global__ void __launch_bounds__(kBlock)
k_edge_dot_scalar(const GatherArgs a, const float *dy, float *dw) {
  // one thread per (row or segment); any F
  const int64_t gid = (int64_t)blockIdx.x * kBlock + threadIdx.x;
  if (gid >= a.n_seg + (a.n_rows - a.n_long)) return;
  int64_t row, beg, end, seg;
  decode_work<PtrT>(a, gid, row, beg, end, seg);
  const IdxT *idx = static_cast<const IdxT *>(a.idx);
  const int64_t F = a.F;
  for (int64_t e = beg; e < end; ++e) {
    const int64_t c = (int64_t)idx[e];
    float p = 0.0f;
    for (int64_t f = 0; f < F; ++f) {
      if (ARG_FILTER && a.arg_in[row * F + f] != (int32_t)e) continue;
      p = __fadd_rn(p, __fmul_rn(dy[row * F + f], a.x[c * F + f]));
    }
    dw[a.eid ? (int64_t)a.eid[e] : e] = p;
  }
}

// ---------------------------------------------------------------------------
// Host dispatch
// ---------------------------------------------------------------------------
inline unsigned blocks_for_groups(int64_t groups, int G) {
  int64_t threads = groups * G;
  return (unsigned)(threads > 0 ? ceil_div(threads, kBlock) : 0);
}

struct Shape {
  bool vec;   // vector path usable
  int G;      // lanes per row
  int VPL;    // float4 per lane
  int U;      // gathered rows in flight per lane
};

Shape scalar_shape(int64_t F) {
  Shape s{false, 1, 1, 1};
  int g = 1;
  while (g < F && g < 32) g <<= 1;
  s.G = g;
  return s;
}

// Lanes per row, float4 per lane and gathered rows in flight for a feature
// width.  The usual widths give a row only 4-16 lanes with several float4 per
// lane, so that a warp keeps 2-8 destination rows in flight: measured on
// fixed-degree and R-MAT graphs this is 1.3-2.7x faster than one full warp per
// 512-byte row at every degree (fewer index broadcasts per byte, more
// independent rows per warp).  The per-edge dot product prefers 8 lanes where
// the width allows and more gathered rows in flight (at 256 floats a full warp
// with two float4 per lane measured faster).  Other widths use one float4 per
// lane.
Shape pick_shape(int64_t F, const void *x, const void *out, bool dot = false) {
  Shape s{false, 1, 1, 1};
  bool aligned = (((uintptr_t)x | (uintptr_t)out) & 15u) == 0;
  if (F % 4 == 0 && aligned && F <= 4 * 32 * 4) {
    const int64_t vecs = F / 4;
    s.vec = true;
    switch (vecs) {
      case 8: s = dot ? Shape{true, 4, 2, 4} : Shape{true, 4, 2, 1}; break;
      case 16: s = dot ? Shape{true, 8, 2, 4} : Shape{true, 4, 4, 1}; break;
      case 32: s = dot ? Shape{true, 8, 4, 2} : Shape{true, 8, 4, 1}; break;
      case 64: s = dot ? Shape{true, 32, 2, 2} : Shape{true, 16, 4, 1}; break;
      case 128: s = Shape{true, 32, 4, 1}; break;
      default:
        if (vecs <= 32) {
          int g = 1;
          while (g < vecs) g <<= 1;
          s.G = g;
          s.VPL = 1;
          s.U = g < 4 ? g : 4;
        } else {
          s.vec = false;
        }
    }
  }
  if (!s.vec) s = scalar_shape(F);
  return s;
}

template <typename PtrT, typename IdxT, int MODE, bool HAS_W, bool W_BY_EID,
          bool ARG_FILTER>
int32_t launch_gather(const GatherArgs &a, const Shape &s, cudaStream_t stream) {
  const int64_t groups = a.n_seg + (a.n_rows - a.n_long);
  if (groups <= 0) return TGB_STATUS_OK;
  const unsigned blocks = blocks_for_groups(groups, s.G);
#define TGB_VEC(GG, VV, UU)                                                    \
  k_gather_vec<PtrT, IdxT, GG, VV, UU, MODE, HAS_W, W_BY_EID, ARG_FILTER>     \
      <<<blocks, kBlock, 0, stream>>>(a)
#define TGB_SCL(GG)                                                            \
  k_gather_scalar<PtrT, IdxT, GG, MODE, HAS_W, W_BY_EID, ARG_FILTER>          \
      <<<blocks, kBlock, 0, stream>>>(a)
  if (s.vec) {
    switch (s.G * 100 + s.VPL * 10 + s.U) {
      case 111: TGB_VEC(1, 1, 1); break;
      case 212: TGB_VEC(2, 1, 2); break;
      case 414: TGB_VEC(4, 1, 4); break;
      case 814: TGB_VEC(8, 1, 4); break;
      case 1614: TGB_VEC(16, 1, 4); break;
      case 3214: TGB_VEC(32, 1, TGB_U32); break;
      case 421: TGB_VEC(4, 2, 1); break;
      case 441: TGB_VEC(4, 4, 1); break;
      case 841: TGB_VEC(8, 4, 1); break;
      case 1641: TGB_VEC(16, 4, 1); break;
      case 3222: TGB_VEC(32, 2, 2); break;
      case 3241: TGB_VEC(32, 4, 1); break;
      default: TGB_FAIL(TGB_STATUS_INTERNAL, "no gather kernel for shape %d/%d/%d", s.G, s.VPL, s.U);
    }
  } else {
    switch (s.G) {
      case 1: TGB_SCL(1); break;
      case 2: TGB_SCL(2); break;
      case 4: TGB_SCL(4); break;
      case 8: TGB_SCL(8); break;
      case 16: TGB_SCL(16); break;
      default: TGB_SCL(32); break;
    }
  }
#undef TGB_VEC
#undef TGB_SCL
  TGB_LAUNCHED();
  if (a.n_long > 0) {
    k_finalize_split<PtrT, MODE><<<(unsigned)a.n_long, kBlock, 0, stream>>>(a);
    TGB_LAUNCHED();
  }
  return TGB_STATUS_OK;
}

template <typename PtrT, typename IdxT, bool ARG_FILTER>
int32_t launch_edge_dot(const GatherArgs &a, const Shape &s, const float *dy,
                        float *dw, cudaStream_t stream) {
  const int64_t groups = a.n_seg + (a.n_rows - a.n_long);
  if (groups <= 0) return TGB_STATUS_OK;
#define TGB_DOT(GG, VV, UU)                                                    \
  k_edge_dot_vec<PtrT, IdxT, GG, VV, UU, ARG_FILTER>                          \
      <<<blocks_for_groups(groups, GG), kBlock, 0, stream>>>(a, dy, dw)
  if (s.vec) {
    switch (s.G * 100 + s.VPL * 10 + s.U) {
      case 111: TGB_DOT(1, 1, 1); break;
      case 212: TGB_DOT(2, 1, 2); break;
      case 414: TGB_DOT(4, 1, 4); break;
      case 814: TGB_DOT(8, 1, 4); break;
      case 1614: TGB_DOT(16, 1, 4); break;
      case 3214: TGB_DOT(32, 1, TGB_U32); break;
      case 424: TGB_DOT(4, 2, 4); break;
      case 824: TGB_DOT(8, 2, 4); break;
      case 842: TGB_DOT(8, 4, 2); break;
      case 1641: TGB_DOT(16, 4, 1); break;
      case 3222: TGB_DOT(32, 2, 2); break;
      case 3241: TGB_DOT(32, 4, 1); break;
      default: TGB_FAIL(TGB_STATUS_INTERNAL, "no edge-dot kernel for shape %d/%d/%d", s.G, s.VPL, s.U);
    }
  } else {
    k_edge_dot_scalar<PtrT, IdxT, ARG_FILTER>
        <<<blocks_for_groups(groups, 1), kBlock, 0, stream>>>(a, dy, dw);
  }
#undef TGB_DOT
  TGB_LAUNCHED();
  return TGB_STATUS_OK;
}

void fill_side(GatherArgs &a, const Side &side) {
  a.ptr = side.ptr;
  a.idx = side.idx;
  a.eid = side.eid;
  a.order = side.order;
  a.seg_row = side.seg_row;
  a.seg_ptr = side.seg_ptr;
  a.items = side.items;
  a.n_rows = side.n_rows;
  a.n_long = side.n_long;
  a.n_seg = side.n_seg;
}

uint64_t partial_bytes(const Side &side, int32_t reducer, int64_t F) {
  uint64_t b = align_up((uint64_t)side.n_seg * (uint64_t)F * 4, 256);
  return reducer == TGB_REDUCER_MAX ? 2 * b : b;
}

// dx over the transposed relation needs w[eid[k]] for entry k.  Reading it inside the gather
// kernel puts a dependent random 4-byte load in front of every row gather; a streaming pass that
// writes the weights in transposed order first (what the reference's generated VJP keeps as its
// `jacobian = w[order]`, python/tiga/interop/torch/relation_vjp.py:61-87) lets the gather kernel
// read them in order.  Measured on the 2^24-node R-MAT with 64 floats per row: 33.0 -> 23.7 ms per
// transposed pass including the permutation.  The max reducer filters by edge id and keeps the
// in-kernel lookup.
bool permute_weights_first(int32_t reducer) { return reducer != TGB_REDUCER_MAX; }

__global__ void k_permute_weights(const float *__restrict__ w, const uint32_t *__restrict__ eid, int64_t E,
                                  float *__restrict__ out) {
  const int64_t k = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (k < E) out[k] = __ldg(w + ld_stream(eid + k));
}

int32_t check_common(const tgb_csr_plan *plan, int32_t reducer, int64_t F,
                     int32_t dtype) {
  if (!plan) TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "null plan");
  if (reducer != TGB_REDUCER_SUM && reducer != TGB_REDUCER_MEAN &&
      reducer != TGB_REDUCER_MAX)
    TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "unknown reducer %d", reducer);
  if (F <= 0) TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "feature width must be positive");
  if (dtype != TGB_DTYPE_F32)
    TGB_FAIL(TGB_STATUS_UNSUPPORTED, "csr reduce kernels take float32 features");
  if (reducer == TGB_REDUCER_MAX && plan->num_edges >= ((int64_t)1 << 31))
    TGB_FAIL(TGB_STATUS_UNSUPPORTED, "max reducer needs fewer than 2^31 edges");
  // winners are stored as CSR positions; an edge map renames the transposed side's edge ids, so the
  // winner comparison of the backward would never match
  if (reducer == TGB_REDUCER_MAX && plan->fwd.eid)
    TGB_FAIL(TGB_STATUS_UNSUPPORTED, "the max reducer does not take a plan with an edge map");
  return TGB_STATUS_OK;
}

}  // namespace
}  // namespace tgb

using namespace tgb;

extern "C" {

int32_t tgb_csr_plan_scratch_bytes(const tgb_csr_plan *plan, int32_t direction,
                                   int32_t reducer, int64_t feature_elems,
                                   int32_t dtype, uint64_t *bytes) {
  if (!bytes) TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "null output");
  int32_t rc = check_common(plan, reducer, feature_elems, dtype);
  if (rc) return rc;
  if (direction < 0 || direction > 2) TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "direction must be 0, 1 or 2");
  if (direction >= 1 && !(plan->flags & TGB_PLAN_TRANSPOSE))
    TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "plan has no transposed relation");
  const Side &side = direction >= 1 ? plan->bwd : plan->fwd;
  uint64_t b = partial_bytes(side, reducer, feature_elems);
  if (direction == 1 && permute_weights_first(reducer))
    b += align_up((uint64_t)plan->num_edges * 4, 256);   // weights in transposed order
  // the mean reducer's backward also stores dy / degree
  if (reducer == TGB_REDUCER_MEAN)
    b += align_up((uint64_t)plan->num_dst * (uint64_t)feature_elems * 4, 256);
  *bytes = b;
  return TGB_STATUS_OK;
}

int32_t tgb_csr_reduce_fwd(const tgb_csr_plan *plan, int32_t reducer,
                           const void *x, const void *w, void *out, void *aux,
                           int64_t F, int32_t dtype, float identity,
                           int32_t flags, void *scratch, uint64_t scratch_bytes,
                           uint64_t stream) {
  int32_t rc = check_common(plan, reducer, F, dtype);
  if (rc) return rc;
  if ((flags & TGB_REDUCE_ACCUMULATE) && reducer != TGB_REDUCER_SUM)
    TGB_FAIL(TGB_STATUS_UNSUPPORTED, "accumulation into existing rows is defined for the sum reducer only");
  if ((!x && plan->num_src > 0 && plan->num_edges > 0) || (!out && plan->num_dst > 0))
    TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "null feature pointer");
  if (reducer == TGB_REDUCER_MAX && !aux && plan->num_dst > 0)
    TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "max reducer needs the aux (argmax) buffer");
  const Side &side = plan->fwd;
  uint64_t need = partial_bytes(side, reducer, F);
  if (side.n_seg > 0 && (!scratch || scratch_bytes < need))
    TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "scratch too small: %llu < %llu bytes",
             (unsigned long long)scratch_bytes, (unsigned long long)need);
  GatherArgs a{};
  fill_side(a, side);
  a.x = (const float *)x;
  a.w = (const float *)w;
  a.out = (float *)out;
  a.partial = (float *)scratch;
  a.arg_out = (int32_t *)aux;
  a.arg_partial = reducer == TGB_REDUCER_MAX
                      ? (int32_t *)((char *)scratch + need / 2) : nullptr;
  a.F = F;
  a.identity = identity;
  a.mean = reducer == TGB_REDUCER_MEAN;
  a.accumulate = (flags & TGB_REDUCE_ACCUMULATE) != 0;
  Shape s = pick_shape(F, x, out);
  if (reducer == TGB_REDUCER_MAX && s.vec && (((uintptr_t)aux | (uintptr_t)a.arg_partial) & 15u))
    s = scalar_shape(F);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (side.eid && w) {   // weights are addressed through the plan's edge map
    return plan->index_bits == 32 ? launch_gather<int32_t, int32_t, kSum, true, true, false>(a, s, st)
                                  : launch_gather<int64_t, int64_t, kSum, true, true, false>(a, s, st);
  }
#define TGB_FWD(PT, MODE, HW) launch_gather<PT, PT, MODE, HW, false, false>(a, s, st)
  if (plan->index_bits == 32) {
    if (reducer == TGB_REDUCER_MAX) return w ? TGB_FWD(int32_t, kMax, true) : TGB_FWD(int32_t, kMax, false);
    return w ? TGB_FWD(int32_t, kSum, true) : TGB_FWD(int32_t, kSum, false);
  }
  if (reducer == TGB_REDUCER_MAX) return w ? TGB_FWD(int64_t, kMax, true) : TGB_FWD(int64_t, kMax, false);
  return w ? TGB_FWD(int64_t, kSum, true) : TGB_FWD(int64_t, kSum, false);
#undef TGB_FWD
}

int32_t tgb_csr_reduce_bwd_dx(const tgb_csr_plan *plan, int32_t reducer,
                              const void *dy, const void *w, const void *aux,
                              void *dx, int64_t F, int32_t dtype, void *scratch,
                              uint64_t scratch_bytes, uint64_t stream) {
  int32_t rc = check_common(plan, reducer, F, dtype);
  if (rc) return rc;
  if (!(plan->flags & TGB_PLAN_TRANSPOSE))
    TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "plan was created without TGB_PLAN_TRANSPOSE");
  if ((!dy && plan->num_dst > 0 && plan->num_edges > 0) || (!dx && plan->num_src > 0))
    TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "null gradient pointer");
  if (reducer == TGB_REDUCER_MAX && !aux && plan->num_edges > 0)
    TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "max reducer needs the aux (argmax) buffer");
  const Side &side = plan->bwd;
  uint64_t part = partial_bytes(side, TGB_REDUCER_SUM, F);
  uint64_t need = part;
  if (reducer == TGB_REDUCER_MEAN)
    need += align_up((uint64_t)plan->num_dst * (uint64_t)F * 4, 256);
  // SUM / MEAN: `aux`, when given, holds the weights already in transposed order
  const float *ready = reducer != TGB_REDUCER_MAX ? (const float *)aux : nullptr;
  const bool permute = w && !ready && permute_weights_first(reducer) && plan->num_edges > 0;
  const uint64_t permuted_at = need;
  if (permute) need += align_up((uint64_t)plan->num_edges * 4, 256);
  if (need > 0 && (side.n_seg > 0 || reducer == TGB_REDUCER_MEAN || permute) &&
      (!scratch || scratch_bytes < need))
    TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "scratch too small: %llu < %llu bytes",
             (unsigned long long)scratch_bytes, (unsigned long long)need);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const float *grad = (const float *)dy;
  if (reducer == TGB_REDUCER_MEAN && plan->num_dst > 0) {
    float *scaled = (float *)((char *)scratch + part);
    int64_t total = plan->num_dst * F;
    unsigned blocks = (unsigned)ceil_div(total, 256);
    if (plan->index_bits == 32)
      k_scale_by_degree<int32_t><<<blocks, 256, 0, st>>>((const int32_t *)plan->fwd.ptr, grad, plan->num_dst, F, scaled);
    else
      k_scale_by_degree<int64_t><<<blocks, 256, 0, st>>>((const int64_t *)plan->fwd.ptr, grad, plan->num_dst, F, scaled);
    TGB_LAUNCHED();
    grad = scaled;
  }
  GatherArgs a{};
  fill_side(a, side);
  a.x = grad;
  a.w = (const float *)w;
  a.out = (float *)dx;
  a.partial = (float *)scratch;
  a.arg_in = (const int32_t *)aux;
  a.F = F;
  a.identity = 0.0f;
  a.mean = 0;
  Shape s = pick_shape(F, grad, dx);
  if (reducer == TGB_REDUCER_MAX && s.vec && ((uintptr_t)aux & 15u))
    s = scalar_shape(F);
  if (reducer == TGB_REDUCER_MAX)
    return w ? launch_gather<int64_t, int32_t, kSum, true, true, true>(a, s, st)
             : launch_gather<int64_t, int32_t, kSum, false, false, true>(a, s, st);
  if (ready) {
    a.w = ready;
    return launch_gather<int64_t, int32_t, kSum, true, false, false>(a, s, st);
  }
  if (permute) {
    float *w_t = (float *)((char *)scratch + permuted_at);
    k_permute_weights<<<(unsigned)ceil_div(plan->num_edges, 256), 256, 0, st>>>(
        (const float *)w, side.eid, plan->num_edges, w_t);
    TGB_LAUNCHED();
    a.w = w_t;
    return launch_gather<int64_t, int32_t, kSum, true, false, false>(a, s, st);
  }
  return w ? launch_gather<int64_t, int32_t, kSum, true, true, false>(a, s, st)
           : launch_gather<int64_t, int32_t, kSum, false, false, false>(a, s, st);
}

int32_t tgb_csr_transposed_weights(const tgb_csr_plan *plan, const void *w, void *w_t, uint64_t stream) {
  if (!plan) TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "null plan");
  if (!(plan->flags & TGB_PLAN_TRANSPOSE))
    TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "plan was created without TGB_PLAN_TRANSPOSE");
  if (plan->num_edges == 0) return TGB_STATUS_OK;
  if (!w || !w_t) TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "null pointer");
  k_permute_weights<<<(unsigned)ceil_div(plan->num_edges, 256), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      (const float *)w, plan->bwd.eid, plan->num_edges, (float *)w_t);
  TGB_LAUNCHED();
  return TGB_STATUS_OK;
}

int32_t tgb_csr_reduce_bwd_dw(const tgb_csr_plan *plan, int32_t reducer,
                              const void *dy, const void *x, const void *aux,
                              void *dw, int64_t F, int32_t dtype, void *scratch,
                              uint64_t scratch_bytes, uint64_t stream) {
  int32_t rc = check_common(plan, reducer, F, dtype);
  if (rc) return rc;
  if (plan->num_edges == 0) return TGB_STATUS_OK;
  if (!dy || !x || !dw) TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "null pointer");
  if (reducer == TGB_REDUCER_MAX && !aux)
    TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "max reducer needs the aux (argmax) buffer");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const float *grad = (const float *)dy;
  if (reducer == TGB_REDUCER_MEAN) {
    uint64_t need = align_up((uint64_t)plan->num_dst * (uint64_t)F * 4, 256);
    if (!scratch || scratch_bytes < need)
      TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "scratch too small: %llu < %llu bytes",
               (unsigned long long)scratch_bytes, (unsigned long long)need);
    float *scaled = (float *)scratch;
    int64_t total = plan->num_dst * F;
    unsigned blocks = (unsigned)ceil_div(total, 256);
    if (plan->index_bits == 32)
      k_scale_by_degree<int32_t><<<blocks, 256, 0, st>>>((const int32_t *)plan->fwd.ptr, grad, plan->num_dst, F, scaled);
    else
      k_scale_by_degree<int64_t><<<blocks, 256, 0, st>>>((const int64_t *)plan->fwd.ptr, grad, plan->num_dst, F, scaled);
    TGB_LAUNCHED();
    grad = scaled;
  }
  GatherArgs a{};
  fill_side(a, plan->fwd);
  a.x = (const float *)x;
  a.arg_in = (const int32_t *)aux;
  a.F = F;
  Shape s = pick_shape(F, x, grad, true);
  if (reducer == TGB_REDUCER_MAX && s.vec && ((uintptr_t)aux & 15u))
    s = scalar_shape(F);
  float *out = (float *)dw;
  if (plan->index_bits == 32)
    return reducer == TGB_REDUCER_MAX
               ? launch_edge_dot<int32_t, int32_t, true>(a, s, grad, out, st)
               : launch_edge_dot<int32_t, int32_t, false>(a, s, grad, out, st);
  return reducer == TGB_REDUCER_MAX
             ? launch_edge_dot<int64_t, int64_t, true>(a, s, grad, out, st)
             : launch_edge_dot<int64_t, int64_t, false>(a, s, grad, out, st);
}

}  // extern "C"

// ---------------------------------------------------------------------------
// Allocation-free forward sum.
//
// Some callers may not allocate device memory at the point where they need the
// aggregation: code running inside a region where cudaMalloc is forbidden or
// would synchronise the device (a real-time control loop, a section that holds
// a driver-level lock, a plug-in host that hands out no allocator).  The
// regular entry point needs a scratch buffer for the partial rows of split
// (long) rows; this variant keeps that scratch in a fixed array that is part
// of the library image, so the call needs nothing but its inputs and outputs.
// ---------------------------------------------------------------------------
#include <mutex>

namespace {
// 2 Mi floats = 8 MiB, resident on every GPU that loads the library until the
// process exits.  Bounds (split-row segments) x (feature width).
constexpr size_t kNoAllocScratchFloats = size_t(2) << 20;
constexpr int kNoAllocMaxDevices = 64;
}  // namespace

static __device__ __align__(256) float g_noalloc_partials[kNoAllocScratchFloats];

namespace {
std::mutex g_noalloc_mutex;
float *g_noalloc_address[kNoAllocMaxDevices] = {};

// The array's name is only a host-side handle; the device address has to be
// asked for, once per device, with that device current.
int32_t noalloc_scratch_address(float **address) {
  int device = -1;
  TGB_CUDA(cudaGetDevice(&device));
  if (device < 0 || device >= kNoAllocMaxDevices)
    TGB_FAIL(TGB_STATUS_UNSUPPORTED, "device ordinal %d is outside the supported range", device);
  std::lock_guard<std::mutex> lock(g_noalloc_mutex);
  if (!g_noalloc_address[device]) {
    void *pointer = nullptr;
    cudaError_t err = cudaGetSymbolAddress(&pointer, g_noalloc_partials);
    if (err != cudaSuccess || !pointer)
      TGB_FAIL(TGB_STATUS_INTERNAL, "cudaGetSymbolAddress(scratch) failed: %s", cudaGetErrorString(err));
    g_noalloc_address[device] = static_cast<float *>(pointer);
  }
  *address = g_noalloc_address[device];
  return TGB_STATUS_OK;
}
}  // namespace

extern "C" int32_t tgb_csr_wsum_fwd_noalloc(const tgb_csr_plan *plan, const void *x, const void *w,
                                            void *out, int64_t F, float identity, uint64_t stream) {
  int32_t rc = check_common(plan, TGB_REDUCER_SUM, F, TGB_DTYPE_F32);
  if (rc) return rc;
  if ((!x && plan->num_src > 0 && plan->num_edges > 0) || (!out && plan->num_dst > 0))
    TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "null feature pointer");
  const Side &side = plan->fwd;
  const uint64_t need = (uint64_t)side.n_seg * (uint64_t)F;
  if (need > kNoAllocScratchFloats)
    TGB_FAIL(TGB_STATUS_UNSUPPORTED,
             "graph too large for the built-in scratch: %lld split-row segments x %lld features = %llu floats, "
             "the limit is %llu (use tgb_csr_reduce_fwd with a caller-provided scratch buffer)",
             (long long)side.n_seg, (long long)F, (unsigned long long)need,
             (unsigned long long)kNoAllocScratchFloats);
  float *scratch = nullptr;
  rc = noalloc_scratch_address(&scratch);
  if (rc) return rc;
  GatherArgs a{};
  fill_side(a, side);
  a.x = (const float *)x;
  a.w = (const float *)w;
  a.out = (float *)out;
  a.partial = scratch;   // every segment overwrites its whole partial row before the finalize kernel reads it
  a.F = F;
  a.identity = identity;
  Shape s = pick_shape(F, x, out);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (side.eid && w)   // the plan carries an edge map: weights are read as w[map[e]], as the regular entry does
    return plan->index_bits == 32 ? launch_gather<int32_t, int32_t, kSum, true, true, false>(a, s, st)
                                  : launch_gather<int64_t, int64_t, kSum, true, true, false>(a, s, st);
  if (plan->index_bits == 32)
    return w ? launch_gather<int32_t, int32_t, kSum, true, false, false>(a, s, st)
             : launch_gather<int32_t, int32_t, kSum, false, false, false>(a, s, st);
  return w ? launch_gather<int64_t, int64_t, kSum, true, false, false>(a, s, st)
           : launch_gather<int64_t, int64_t, kSum, false, false, false>(a, s, st);
}
