// GAT-style edge attention over CSR rows with the online-softmax reducer,
// bf16 features, float32 state, and its backward without atomics.
//
// Program (reference spelling):
//   s     = (src.x * a_src).sum(-1) + (dst.x * a_dst).sum(-1)        per head
//   score = maximum(s, slope * s)                                     leaky-relu
//   out   = online_softmax(score, src.x)                              per head
//
// Algorithm: the row-centric online softmax of the reference's
// gf_edge_nn_attention kernels (python/tiga/compiler/edge_nn_attention.py:
// 127-338 forward, 344-611 backward): running (m, l, acc) per destination row
// and head, epilogue acc/l (0 for an empty row), (m, l) saved; backward
// w_e = exp(s_e-m)/l, d_value = w_e*dO, d_s = w_e*(<dO,v_e> - <dO,O>).
// Semantics of the scores follow the reference's eager evaluator for bf16
// inputs (python/tiga/interop/torch/message_passing.py:2848-2894 with
// reducer_oracle.py:87-91): every bf16 elementwise op rounds to bf16, the
// sum over the head dimension accumulates in float32 and rounds once.
//
// Layout: a feature row is H*D bf16 = G lanes x 16 bytes; a head spans
// D/8 adjacent lanes.  Per-node score halves s_src[n,h], s_dst[n,h] are
// computed once per call by k_node_scores (a streaming pass), so the edge loop
// gathers one 16-byte vector per lane plus one float per lane.
//
// Backward, atomics-free:
//   pass 1 (destination-major): per edge w_e and d_pre -> P[e,h], Q[e,h];
//          per row d_sdst[r,h] = sum_e d_pre
//   pass 2 (source-major over the transposed relation):
//          dx_src[j] = sum_e P*dO[dst] + (sum_e Q) * a_src;  d_ssrc[j,h] = sum_e Q
//   pass 3 (streaming): dx_dst = d_sdst*a_dst,  da_src = sum_j d_ssrc*x_src,
//          da_dst = sum_r d_sdst*x_dst  (two-stage deterministic reduction)
// HBM roofline bound; algorithmic bytes per edge: forward 8 + 512 (+32 score),
// backward 8 + 512 + 32 + 64 written, then 8 + 512 + 64 gathered.
#include <cuda_bf16.h>

#include "tgb_common.cuh"

namespace tgb {
namespace {

constexpr int kBlock = 128;
constexpr int kU = 4;           // gathered rows in flight per lane
#ifndef TGB_GAT_HEAD_LANES
#define TGB_GAT_HEAD_LANES 1
#endif
#ifndef TGB_GAT_BWD_U
#define TGB_GAT_BWD_U 1
#endif
constexpr int kReduceBlocks = 592;  // 4 CTAs per SM for the parameter-gradient reduction

__device__ __forceinline__ float bf16_round(float v) {
  return __bfloat162float(__float2bfloat16_rn(v));
}

__device__ __forceinline__ void unpack8(const uint4 &q, float (&f)[8]) {
  f[0] = __uint_as_float(q.x << 16); f[1] = __uint_as_float(q.x & 0xffff0000u);
  f[2] = __uint_as_float(q.y << 16); f[3] = __uint_as_float(q.y & 0xffff0000u);
  f[4] = __uint_as_float(q.z << 16); f[5] = __uint_as_float(q.z & 0xffff0000u);
  f[6] = __uint_as_float(q.w << 16); f[7] = __uint_as_float(q.w & 0xffff0000u);
}

__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t *>(&v);
}

__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  return make_uint4(pack2(f[0], f[1]), pack2(f[2], f[3]), pack2(f[4], f[5]), pack2(f[6], f[7]));
}

__device__ __forceinline__ uint4 ldg_u4(const void *p) {
  return __ldg(reinterpret_cast<const uint4 *>(p));
}

// leaky-relu logit from the two bf16-rounded halves, in bf16 arithmetic
__device__ __forceinline__ float logit_of(float s_src, float s_dst, float slope_bf, float &pre) {
  pre = bf16_round(s_src + s_dst);
  const float scaled = bf16_round(slope_bf * pre);
  return fmaxf(pre, scaled);
}

// d(maximum(s, slope*s))/ds as torch's maximum backward gives it (ties split)
__device__ __forceinline__ float leaky_grad(float pre, float slope_bf) {
  return pre > 0.0f ? 1.0f : (pre < 0.0f ? slope_bf : 0.5f * (1.0f + slope_bf));
}

struct GatArgs {
  WorkList work;
  const __nv_bfloat16 *x_src;   // [num_src, H*D]
  const __nv_bfloat16 *x_dst;   // [N, H*D]
  const float *s_src;           // [num_src, H]
  const float *s_dst;           // [N, H]
  __nv_bfloat16 *out;           // [N, H*D]
  float *m;                     // [N, H]
  float *l;                     // [N, H]
  float *part_acc;              // [n_seg, H*D]
  float *part_ml;               // [n_seg, 2*H]
  int H, D, lph;                // lph = lanes per head = D/8
  float slope_bf;
  // backward
  const __nv_bfloat16 *o;       // forward output
  const __nv_bfloat16 *dout;
  float *P;                     // [E, H] softmax weight of the edge
  float *Q;                     // [E, H] cotangent of the pre-activation
  float *d_sdst;                // [N, H]
  float *d_ssrc;                // [num_src, H]
  const __nv_bfloat16 *a_src;   // [H*D]
  const __nv_bfloat16 *a_dst;
  __nv_bfloat16 *dx_src;        // [num_src, H*D]
  __nv_bfloat16 *dx_dst;        // [N, H*D]
  float *part_h;                // [n_seg, H] partial sums of Q per segment
};

// s[n,h] = bf16( sum_d bf16(x[n,h,d] * a[h,d]) ), one thread group of G lanes per node
template <int G>
__global__ void __launch_bounds__(kBlock)
k_node_scores(const __nv_bfloat16 *x, const __nv_bfloat16 *a, int64_t n, int H, int lph, float *s) {
  const int lane = threadIdx.x & (G - 1);
  const int64_t node = ((int64_t)blockIdx.x * kBlock + threadIdx.x) / G;
  if (node >= n) return;
  const unsigned gmask = G == 32 ? 0xffffffffu : (((1u << G) - 1u) << ((threadIdx.x & 31) & ~(G - 1)));
  float xv[8], av[8];
  unpack8(ldg_u4(x + (node * G + lane) * 8), xv);
  unpack8(ldg_u4(a + lane * 8), av);
  float p = 0.0f;
#pragma unroll
  for (int i = 0; i < 8; ++i) p += bf16_round(xv[i] * av[i]);
  for (int o = lph >> 1; o; o >>= 1) p += __shfl_xor_sync(gmask, p, o, G);
  if ((lane & (lph - 1)) == 0) s[node * H + lane / lph] = bf16_round(p);
}

// ---------------------------------------------------------------------------
// forward
// ---------------------------------------------------------------------------
template <typename PtrT, typename IdxT, int G>
__global__ void __launch_bounds__(kBlock)
k_gat_fwd(const GatArgs a) {
  const int lane = threadIdx.x & (G - 1);
  const int64_t gid = ((int64_t)blockIdx.x * kBlock + threadIdx.x) / G;
  if (gid >= a.work.n_seg + (a.work.n_rows - a.work.n_long)) return;
  const unsigned gmask = G == 32 ? 0xffffffffu : (((1u << G) - 1u) << ((threadIdx.x & 31) & ~(G - 1)));
  int64_t row, beg, end, seg;
  decode_group<PtrT>(a.work, gid, row, beg, end, seg);
  const IdxT *idx = static_cast<const IdxT *>(a.work.idx);
  const int H = a.H, head = lane / a.lph;
  const float sd = __ldg(a.s_dst + row * H + head);
  float m = -INFINITY, l = 0.0f;
  float acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.0f;

  for (int64_t base = beg; base < end; base += G) {
    const int64_t e = base + lane;
    const int32_t c = e < end ? (int32_t)ld_stream(idx + e) : 0;
    const int n = (int)(end - base < G ? end - base : G);
    for (int k0 = 0; k0 < n; k0 += kU) {
      uint4 raw[kU];
      float logit[kU];
      float mc = m;
#pragma unroll
      for (int u = 0; u < kU; ++u) {
        const int k = k0 + u;
        const int32_t cc = __shfl_sync(gmask, c, k < n ? k : n - 1, G);
        logit[u] = -INFINITY;
        if (k < n) {
          raw[u] = ldg_u4(a.x_src + ((int64_t)cc * G + lane) * 8);
          float pre;
          logit[u] = logit_of(__ldg(a.s_src + (int64_t)cc * H + head), sd, a.slope_bf, pre);
          mc = fmaxf(mc, logit[u]);
        }
      }
      // one rescale per chunk of kU edges
      const float scale = m == -INFINITY ? 0.0f : __expf(m - mc);
      l *= scale;
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] *= scale;
      m = mc;
#pragma unroll
      for (int u = 0; u < kU; ++u) {
        if (k0 + u < n) {
          const float p = __expf(logit[u] - m);
          float v[8];
          unpack8(raw[u], v);
          l += p;
#pragma unroll
          for (int i = 0; i < 8; ++i) acc[i] = fmaf(p, v[i], acc[i]);
        }
      }
    }
  }
  if (seg >= 0) {
    float *pa = a.part_acc + (seg * G + lane) * 8;
    *reinterpret_cast<float4 *>(pa) = make_float4(acc[0], acc[1], acc[2], acc[3]);
    *reinterpret_cast<float4 *>(pa + 4) = make_float4(acc[4], acc[5], acc[6], acc[7]);
    if ((lane & (a.lph - 1)) == 0) {
      a.part_ml[seg * 2 * H + head] = m;
      a.part_ml[seg * 2 * H + H + head] = l;
    }
    return;
  }
  float o[8];
  const float inv = l > 0.0f ? 1.0f / l : 0.0f;   // empty row -> exact zeros
#pragma unroll
  for (int i = 0; i < 8; ++i) o[i] = acc[i] * inv;
  *reinterpret_cast<uint4 *>(a.out + (row * G + lane) * 8) = pack8(o);
  if ((lane & (a.lph - 1)) == 0) {
    a.m[row * H + head] = m;
    a.l[row * H + head] = l;
  }
}

// combines the (m, l, acc) partial states of a split row in segment order
template <int G>
__global__ void __launch_bounds__(32)
k_gat_fwd_finalize(const GatArgs a) {
  const int lane = threadIdx.x;
  const int64_t lr = blockIdx.x;
  if (lane >= G) return;
  const int64_t row = a.work.order[lr];
  const int32_t s0 = a.work.seg_ptr[lr], s1 = a.work.seg_ptr[lr + 1];
  const int H = a.H, head = lane / a.lph;
  float m = -INFINITY;
  for (int32_t s = s0; s < s1; ++s) m = fmaxf(m, a.part_ml[(int64_t)s * 2 * H + head]);
  float l = 0.0f, acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.0f;
  for (int32_t s = s0; s < s1; ++s) {
    const float ms = a.part_ml[(int64_t)s * 2 * H + head];
    const float f = ms == -INFINITY ? 0.0f : __expf(ms - m);
    l += f * a.part_ml[(int64_t)s * 2 * H + H + head];
    const float *pa = a.part_acc + ((int64_t)s * G + lane) * 8;
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = fmaf(f, pa[i], acc[i]);
  }
  const float inv = l > 0.0f ? 1.0f / l : 0.0f;
  float o[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) o[i] = acc[i] * inv;
  *reinterpret_cast<uint4 *>(a.out + (row * G + lane) * 8) = pack8(o);
  if ((lane & (a.lph - 1)) == 0) {
    a.m[row * H + head] = m;
    a.l[row * H + head] = l;
  }
}

// ---------------------------------------------------------------------------
// backward pass 1: destination-major, writes P, Q per edge and d_sdst per row
// ---------------------------------------------------------------------------
template <typename PtrT, typename IdxT, int G>
__global__ void __launch_bounds__(kBlock)
k_gat_bwd_dst(const GatArgs a) {
  const int lane = threadIdx.x & (G - 1);
  const int64_t gid = ((int64_t)blockIdx.x * kBlock + threadIdx.x) / G;
  if (gid >= a.work.n_seg + (a.work.n_rows - a.work.n_long)) return;
  const unsigned gmask = G == 32 ? 0xffffffffu : (((1u << G) - 1u) << ((threadIdx.x & 31) & ~(G - 1)));
  int64_t row, beg, end, seg;
  decode_group<PtrT>(a.work, gid, row, beg, end, seg);
  const IdxT *idx = static_cast<const IdxT *>(a.work.idx);
  const int H = a.H, lph = a.lph, head = lane / lph;
  const bool writer = (lane & (lph - 1)) == 0;
  const float sd = __ldg(a.s_dst + row * H + head);
  const float m = __ldg(a.m + row * H + head);
  const float l = __ldg(a.l + row * H + head);
  const float inv_l = l > 0.0f ? 1.0f / l : 0.0f;
  float g[8], ov[8];
  unpack8(ldg_u4(a.dout + (row * G + lane) * 8), g);
  unpack8(ldg_u4(a.o + (row * G + lane) * 8), ov);
  float delta = 0.0f;
#pragma unroll
  for (int i = 0; i < 8; ++i) delta = fmaf(g[i], ov[i], delta);
  for (int o = lph >> 1; o; o >>= 1) delta += __shfl_xor_sync(gmask, delta, o, G);
  float dsd = 0.0f;

  for (int64_t base = beg; base < end; base += G) {
    const int64_t e = base + lane;
    const int32_t c = e < end ? (int32_t)ld_stream(idx + e) : 0;
    const int n = (int)(end - base < G ? end - base : G);
    for (int k0 = 0; k0 < n; k0 += kU) {
      uint4 raw[kU];
      float ss[kU];
#pragma unroll
      for (int u = 0; u < kU; ++u) {
        const int k = k0 + u;
        const int32_t cc = __shfl_sync(gmask, c, k < n ? k : n - 1, G);
        if (k < n) {
          raw[u] = ldg_u4(a.x_src + ((int64_t)cc * G + lane) * 8);
          ss[u] = __ldg(a.s_src + (int64_t)cc * H + head);
        }
      }
#pragma unroll
      for (int u = 0; u < kU; ++u) {
        if (k0 + u < n) {   // uniform across the group
          float v[8], pre;
          unpack8(raw[u], v);
          const float logit = logit_of(ss[u], sd, a.slope_bf, pre);
          const float w = __expf(logit - m) * inv_l;
          float gv = 0.0f;
#pragma unroll
          for (int i = 0; i < 8; ++i) gv = fmaf(g[i], v[i], gv);
          for (int o = lph >> 1; o; o >>= 1) gv += __shfl_xor_sync(gmask, gv, o, G);
          const float dpre = w * (gv - delta) * leaky_grad(pre, a.slope_bf);
          dsd += dpre;
          if (writer) {
            const int64_t at = (base + k0 + u) * H + head;
            __stcs(a.P + at, w);
            __stcs(a.Q + at, dpre);
          }
        }
      }
    }
  }
  if (writer) {
    if (seg >= 0) a.part_h[seg * H + head] = dsd;
    else a.d_sdst[row * H + head] = dsd;
  }
}

// sums per-segment partial head sums of split rows (one thread per head)
__global__ void k_sum_head_partials(const WorkList work, const float *part_h, int H, float *out) {
  const int64_t lr = blockIdx.x;
  const int head = threadIdx.x;
  if (head >= H) return;
  const int64_t row = work.order[lr];
  float acc = 0.0f;
  for (int32_t s = work.seg_ptr[lr]; s < work.seg_ptr[lr + 1]; ++s) acc += part_h[(int64_t)s * H + head];
  out[row * H + head] = acc;
}

// ---------------------------------------------------------------------------
// backward pass 2: source-major over the transposed relation
// ---------------------------------------------------------------------------
template <int G>
__global__ void __launch_bounds__(kBlock)
k_gat_bwd_src(const GatArgs a) {
  const int lane = threadIdx.x & (G - 1);
  const int64_t gid = ((int64_t)blockIdx.x * kBlock + threadIdx.x) / G;
  if (gid >= a.work.n_seg + (a.work.n_rows - a.work.n_long)) return;
  const unsigned gmask = G == 32 ? 0xffffffffu : (((1u << G) - 1u) << ((threadIdx.x & 31) & ~(G - 1)));
  int64_t row, beg, end, seg;
  decode_group<int64_t>(a.work, gid, row, beg, end, seg);
  const int32_t *idx = static_cast<const int32_t *>(a.work.idx);
  const int H = a.H, lph = a.lph, head = lane / lph;
  float acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.0f;
  float dss = 0.0f;
  for (int64_t base = beg; base < end; base += G) {
    const int64_t e = base + lane;
    int32_t c = 0;
    uint32_t my_eid = 0;
    if (e < end) {
      c = ld_stream(idx + e);
      my_eid = ld_stream(a.work.eid + e);
    }
    const int n = (int)(end - base < G ? end - base : G);
    for (int k0 = 0; k0 < n; k0 += kU) {
      uint4 raw[kU];
      float p[kU], q[kU];
#pragma unroll
      for (int u = 0; u < kU; ++u) {
        const int k = k0 + u;
        const int src = k < n ? k : n - 1;
        const int32_t cc = __shfl_sync(gmask, c, src, G);
        const uint32_t ee = __shfl_sync(gmask, my_eid, src, G);
        if (k < n) {
          raw[u] = ldg_u4(a.dout + ((int64_t)cc * G + lane) * 8);
          p[u] = __ldg(a.P + (int64_t)ee * H + head);
          q[u] = __ldg(a.Q + (int64_t)ee * H + head);
        }
      }
#pragma unroll
      for (int u = 0; u < kU; ++u) {
        if (k0 + u < n) {
          float gv[8];
          unpack8(raw[u], gv);
#pragma unroll
          for (int i = 0; i < 8; ++i) acc[i] = fmaf(p[u], gv[i], acc[i]);
          dss += q[u];
        }
      }
    }
  }
  if (seg >= 0) {
    float *pa = a.part_acc + (seg * G + lane) * 8;
    *reinterpret_cast<float4 *>(pa) = make_float4(acc[0], acc[1], acc[2], acc[3]);
    *reinterpret_cast<float4 *>(pa + 4) = make_float4(acc[4], acc[5], acc[6], acc[7]);
    if ((lane & (lph - 1)) == 0) a.part_h[seg * H + head] = dss;
    return;
  }
  float av[8], o[8];
  unpack8(ldg_u4(a.a_src + lane * 8), av);
#pragma unroll
  for (int i = 0; i < 8; ++i) o[i] = fmaf(dss, av[i], acc[i]);
  *reinterpret_cast<uint4 *>(a.dx_src + (row * G + lane) * 8) = pack8(o);
  if ((lane & (lph - 1)) == 0) a.d_ssrc[row * H + head] = dss;
}

template <int G>
__global__ void __launch_bounds__(32)
k_gat_bwd_src_finalize(const GatArgs a) {
  const int lane = threadIdx.x;
  const int64_t lr = blockIdx.x;
  if (lane >= G) return;
  const int64_t row = a.work.order[lr];
  const int H = a.H, head = lane / a.lph;
  float acc[8], dss = 0.0f;
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.0f;
  for (int32_t s = a.work.seg_ptr[lr]; s < a.work.seg_ptr[lr + 1]; ++s) {
    const float *pa = a.part_acc + ((int64_t)s * G + lane) * 8;
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] += pa[i];
    dss += a.part_h[(int64_t)s * H + head];
  }
  float av[8], o[8];
  unpack8(ldg_u4(a.a_src + lane * 8), av);
#pragma unroll
  for (int i = 0; i < 8; ++i) o[i] = fmaf(dss, av[i], acc[i]);
  *reinterpret_cast<uint4 *>(a.dx_src + (row * G + lane) * 8) = pack8(o);
  if ((lane & (a.lph - 1)) == 0) a.d_ssrc[row * H + head] = dss;
}

// ---------------------------------------------------------------------------
// Rows of 32 vectors (H*D = 256 bf16) with heads of at most 8 vectors: the
// forward pass with 8 lanes per row and 4 vectors per lane (lane l holds
// vectors l, l+8, l+16, l+24, each of a different head), so a warp keeps four
// rows in flight and broadcasts an edge's source id once per 512 bytes
// gathered.  The running maximum moves only when an edge exceeds it.  Partial
// rows of split rows keep the layout of the one-vector-per-lane kernel, so the
// finalize kernel is shared.  Measured on the 2^21-node R-MAT case: forward
// 7.23 -> 6.54 ms.  The same shape for the two backward passes was slower
// (step 23.8 -> 31.9 ms: four per-head scalars per lane and edge instead of
// one) and is not used.
// ---------------------------------------------------------------------------
constexpr int kQG = 8, kQV = 4, kQVecs = kQG * kQV;

template <typename PtrT, typename IdxT, int U>
__global__ void __launch_bounds__(kBlock)
k_gat_fwd_q(const GatArgs a) {
  const int lane = threadIdx.x & (kQG - 1);
  const int64_t gid = ((int64_t)blockIdx.x * kBlock + threadIdx.x) / kQG;
  if (gid >= a.work.n_seg + (a.work.n_rows - a.work.n_long)) return;
  const unsigned gmask = 0xffu << ((threadIdx.x & 31) & ~(kQG - 1));
  int64_t row, beg, end, seg;
  decode_group<PtrT>(a.work, gid, row, beg, end, seg);
  const IdxT *idx = static_cast<const IdxT *>(a.work.idx);
  const int H = a.H, sh = __ffs(a.lph) - 1;
  const uint4 *xs = reinterpret_cast<const uint4 *>(a.x_src);
  int hv[kQV];
  float sd[kQV], m[kQV], l[kQV], acc[kQV][8];
#pragma unroll
  for (int v = 0; v < kQV; ++v) {
    hv[v] = (lane + v * kQG) >> sh;
    sd[v] = __ldg(a.s_dst + row * H + hv[v]);
    m[v] = -INFINITY;
    l[v] = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[v][i] = 0.0f;
  }
  for (int64_t base = beg; base < end; base += kQG) {
    const int64_t e = base + lane;
    const int32_t c = e < end ? (int32_t)ld_stream(idx + e) : 0;
    const int n = (int)(end - base < kQG ? end - base : kQG);
    for (int k0 = 0; k0 < n; k0 += U) {
      uint4 raw[U][kQV];
      float ss[U][kQV];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int k = k0 + u;
        const int32_t cc = __shfl_sync(gmask, c, k < n ? k : n - 1, kQG);
        if (k < n) {
#pragma unroll
          for (int v = 0; v < kQV; ++v) {
            raw[u][v] = __ldg(xs + (int64_t)cc * kQVecs + lane + v * kQG);
            ss[u][v] = __ldg(a.s_src + (int64_t)cc * H + hv[v]);
          }
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (k0 + u < n) {
#pragma unroll
          for (int v = 0; v < kQV; ++v) {
            float pre;
            const float logit = logit_of(ss[u][v], sd[v], a.slope_bf, pre);
            if (logit > m[v]) {                       // rare after the first edges of a row
              const float scale = m[v] == -INFINITY ? 0.0f : __expf(m[v] - logit);
              l[v] *= scale;
#pragma unroll
              for (int i = 0; i < 8; ++i) acc[v][i] *= scale;
              m[v] = logit;
            }
            const float p = __expf(logit - m[v]);
            float val[8];
            unpack8(raw[u][v], val);
            l[v] += p;
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[v][i] = fmaf(p, val[i], acc[v][i]);
          }
        }
      }
    }
  }
  const bool writer = (lane & (a.lph - 1)) == 0;
#pragma unroll
  for (int v = 0; v < kQV; ++v) {
    const int j = lane + v * kQG;
    if (seg >= 0) {
      float *pa = a.part_acc + (seg * kQVecs + j) * 8;
      *reinterpret_cast<float4 *>(pa) = make_float4(acc[v][0], acc[v][1], acc[v][2], acc[v][3]);
      *reinterpret_cast<float4 *>(pa + 4) = make_float4(acc[v][4], acc[v][5], acc[v][6], acc[v][7]);
      if (writer) {
        a.part_ml[seg * 2 * H + hv[v]] = m[v];
        a.part_ml[seg * 2 * H + H + hv[v]] = l[v];
      }
    } else {
      float o[8];
      const float inv = l[v] > 0.0f ? 1.0f / l[v] : 0.0f;   // empty row -> exact zeros
#pragma unroll
      for (int i = 0; i < 8; ++i) o[i] = acc[v][i] * inv;
      *reinterpret_cast<uint4 *>(a.out + (row * kQVecs + j) * 8) = pack8(o);
      if (writer) {
        a.m[row * H + hv[v]] = m[v];
        a.l[row * H + hv[v]] = l[v];
      }
    }
  }
}

// ---------------------------------------------------------------------------
// Backward passes for rows of 8 heads x 32 elements with one lane per HEAD: a row is owned by
// 8 lanes, lane h keeps the 4 vectors (64 contiguous bytes) of head h.  Everything a head needs
// then lives in one lane: its logit, softmax weight and exp are evaluated once per (edge, head)
// instead of once per lane of the head, the dot products <dO, x> and <dO, O> need no shuffles, the
// per-edge (P, Q) pair is written and read by one lane, and a warp keeps four rows (and four
// gathered rows per step) in flight.  Partial rows of split rows keep the vector-major layout of
// the one-vector-per-lane kernels, so the finalize kernels are shared.
// ---------------------------------------------------------------------------
constexpr int kHL = 8, kHV = 4;     // lanes per row, vectors per lane

template <typename PtrT, typename IdxT, int U>
__global__ void __launch_bounds__(kBlock)
k_gat_bwd_dst_h(const GatArgs a) {
  const int lane = threadIdx.x & (kHL - 1);          // = head
  const int64_t gid = ((int64_t)blockIdx.x * kBlock + threadIdx.x) / kHL;
  if (gid >= a.work.n_seg + (a.work.n_rows - a.work.n_long)) return;
  const unsigned gmask = 0xffu << ((threadIdx.x & 31) & ~(kHL - 1));
  int64_t row, beg, end, seg;
  decode_group<PtrT>(a.work, gid, row, beg, end, seg);
  const IdxT *idx = static_cast<const IdxT *>(a.work.idx);
  const uint4 *xs = reinterpret_cast<const uint4 *>(a.x_src);
  constexpr int H = kHL;
  const float sd = __ldg(a.s_dst + row * H + lane);
  const float m = __ldg(a.m + row * H + lane);
  const float l = __ldg(a.l + row * H + lane);
  const float inv_l = l > 0.0f ? 1.0f / l : 0.0f;
  uint4 graw[kHV];
  float delta = 0.0f;
#pragma unroll
  for (int v = 0; v < kHV; ++v) {
    graw[v] = ldg_u4(a.dout + ((row * kHL + lane) * kHV + v) * 8);
    float g[8], ov[8];
    unpack8(graw[v], g);
    unpack8(ldg_u4(a.o + ((row * kHL + lane) * kHV + v) * 8), ov);
#pragma unroll
    for (int i = 0; i < 8; ++i) delta = fmaf(g[i], ov[i], delta);
  }
  float dsd = 0.0f;
  for (int64_t base = beg; base < end; base += kHL) {
    const int64_t e = base + lane;
    const int32_t c = e < end ? (int32_t)ld_stream(idx + e) : 0;
    const int n = (int)(end - base < kHL ? end - base : kHL);
    for (int k0 = 0; k0 < n; k0 += U) {
      uint4 raw[U][kHV];
      float ss[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int k = k0 + u;
        const int32_t cc = __shfl_sync(gmask, c, k < n ? k : n - 1, kHL);
        if (k < n) {
#pragma unroll
          for (int v = 0; v < kHV; ++v) raw[u][v] = __ldg(xs + ((int64_t)cc * kHL + lane) * kHV + v);
          ss[u] = __ldg(a.s_src + (int64_t)cc * H + lane);
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (k0 + u < n) {
          float pre;
          const float logit = logit_of(ss[u], sd, a.slope_bf, pre);
          const float w = __expf(logit - m) * inv_l;
          float gv = 0.0f;
#pragma unroll
          for (int v = 0; v < kHV; ++v) {
            float g[8], x[8];
            unpack8(graw[v], g);
            unpack8(raw[u][v], x);
#pragma unroll
            for (int i = 0; i < 8; ++i) gv = fmaf(g[i], x[i], gv);
          }
          const float dpre = w * (gv - delta) * leaky_grad(pre, a.slope_bf);
          dsd += dpre;
          const int64_t at = (base + k0 + u) * H + lane;      // 8 lanes: one 32-byte line per edge
          __stcs(a.P + at, w);
          __stcs(a.Q + at, dpre);
        }
      }
    }
  }
  if (seg >= 0) a.part_h[seg * H + lane] = dsd;
  else a.d_sdst[row * H + lane] = dsd;
}

template <int U>
__global__ void __launch_bounds__(kBlock)
k_gat_bwd_src_h(const GatArgs a) {
  const int lane = threadIdx.x & (kHL - 1);          // = head
  const int64_t gid = ((int64_t)blockIdx.x * kBlock + threadIdx.x) / kHL;
  if (gid >= a.work.n_seg + (a.work.n_rows - a.work.n_long)) return;
  const unsigned gmask = 0xffu << ((threadIdx.x & 31) & ~(kHL - 1));
  int64_t row, beg, end, seg;
  decode_group<int64_t>(a.work, gid, row, beg, end, seg);
  const int32_t *idx = static_cast<const int32_t *>(a.work.idx);
  const uint4 *go = reinterpret_cast<const uint4 *>(a.dout);
  constexpr int H = kHL;
  float acc[kHV][8];
#pragma unroll
  for (int v = 0; v < kHV; ++v)
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[v][i] = 0.0f;
  float dss = 0.0f;
  for (int64_t base = beg; base < end; base += kHL) {
    const int64_t e = base + lane;
    int32_t c = 0;
    uint32_t my_eid = 0;
    if (e < end) {
      c = ld_stream(idx + e);
      my_eid = ld_stream(a.work.eid + e);
    }
    const int n = (int)(end - base < kHL ? end - base : kHL);
    for (int k0 = 0; k0 < n; k0 += U) {
      uint4 raw[U][kHV];
      float p[U], q[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int k = k0 + u;
        const int src = k < n ? k : n - 1;
        const int32_t cc = __shfl_sync(gmask, c, src, kHL);
        const uint32_t ee = __shfl_sync(gmask, my_eid, src, kHL);
        if (k < n) {
#pragma unroll
          for (int v = 0; v < kHV; ++v) raw[u][v] = __ldg(go + ((int64_t)cc * kHL + lane) * kHV + v);
          p[u] = __ldg(a.P + (int64_t)ee * H + lane);
          q[u] = __ldg(a.Q + (int64_t)ee * H + lane);
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (k0 + u < n) {
#pragma unroll
          for (int v = 0; v < kHV; ++v) {
            float gv[8];
            unpack8(raw[u][v], gv);
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[v][i] = fmaf(p[u], gv[i], acc[v][i]);
          }
          dss += q[u];
        }
      }
    }
  }
  if (seg >= 0) {
#pragma unroll
    for (int v = 0; v < kHV; ++v) {
      float *pa = a.part_acc + ((seg * kHL + lane) * kHV + v) * 8;
      *reinterpret_cast<float4 *>(pa) = make_float4(acc[v][0], acc[v][1], acc[v][2], acc[v][3]);
      *reinterpret_cast<float4 *>(pa + 4) = make_float4(acc[v][4], acc[v][5], acc[v][6], acc[v][7]);
    }
    a.part_h[seg * H + lane] = dss;
    return;
  }
#pragma unroll
  for (int v = 0; v < kHV; ++v) {
    float av[8], o[8];
    unpack8(ldg_u4(a.a_src + (lane * kHV + v) * 8), av);
#pragma unroll
    for (int i = 0; i < 8; ++i) o[i] = fmaf(dss, av[i], acc[v][i]);
    *reinterpret_cast<uint4 *>(a.dx_src + ((row * kHL + lane) * kHV + v) * 8) = pack8(o);
  }
  a.d_ssrc[row * H + lane] = dss;
}

// ---------------------------------------------------------------------------
// backward pass 3: dx_dst rows and the two parameter gradients
//   dx_dst[r] = d_sdst[r,h] * a_dst ;  partial[b] = sum_{rows of CTA b} d_s[r,h] * x[r]
// One thread per 8-element vector of the row; CTAs stride over rows.
// ---------------------------------------------------------------------------
template <int G>
__global__ void __launch_bounds__(256)
k_param_grad(const __nv_bfloat16 *x, const float *d_s, const __nv_bfloat16 *a_vec, int64_t n, int H, int lph,
             __nv_bfloat16 *dx_out, float *partial) {
  constexpr int kRowsPerCta = 256 / G;
  const int lane = threadIdx.x % G, sub = threadIdx.x / G;
  const int head = lane / lph;
  float acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.0f;
  float av[8];
  unpack8(ldg_u4(a_vec + lane * 8), av);
  for (int64_t r = (int64_t)blockIdx.x * kRowsPerCta + sub; r < n; r += (int64_t)gridDim.x * kRowsPerCta) {
    const float d = __ldg(d_s + r * H + head);
    float xv[8];
    unpack8(ldg_u4(x + (r * G + lane) * 8), xv);
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = fmaf(d, xv[i], acc[i]);
    if (dx_out) {
      float o[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) o[i] = d * av[i];
      *reinterpret_cast<uint4 *>(dx_out + (r * G + lane) * 8) = pack8(o);
    }
  }
  __shared__ float tile[256 * 8];
#pragma unroll
  for (int i = 0; i < 8; ++i) tile[(sub * G + lane) * 8 + i] = acc[i];
  __syncthreads();
  if (sub == 0) {
    for (int s = 1; s < kRowsPerCta; ++s)
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] += tile[(s * G + lane) * 8 + i];
    float *dst = partial + ((int64_t)blockIdx.x * G + lane) * 8;
#pragma unroll
    for (int i = 0; i < 8; ++i) dst[i] = acc[i];
  }
}

__global__ void k_sum_partials(const float *partial, int blocks, int width, float *out) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= width) return;
  float acc = 0.0f;
  for (int b = 0; b < blocks; ++b) acc += partial[(int64_t)b * width + i];
  out[i] = acc;
}

struct GatShape {
  int G;     // 16-byte vectors per row
  int lph;   // lanes per head
};

int32_t gat_shape(int32_t H, int32_t D, GatShape *s) {
  if (H <= 0 || D <= 0) TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "heads and head width must be positive");
  if (D % 8 != 0) TGB_FAIL(TGB_STATUS_UNSUPPORTED, "edge attention needs a head width that is a multiple of 8");
  const int lph = D / 8, vecs = H * lph;
  if ((lph & (lph - 1)) != 0 || (vecs & (vecs - 1)) != 0 || vecs > 32)
    TGB_FAIL(TGB_STATUS_UNSUPPORTED,
             "edge attention supports heads*width/8 in {1,2,4,8,16,32} with a power-of-two head width "
             "(got H=%d, D=%d)", H, D);
  s->G = vecs;
  s->lph = lph;
  return TGB_STATUS_OK;
}

constexpr int kQU = 1;   // gathered rows in flight per lane of the 8-lane forward kernel

// rows of 32 vectors whose heads span at most 8 of them take the 8-lane forward kernel
inline bool quarter_shape(const GatShape &s) { return s.G == kQVecs && s.lph <= kQG; }

struct GatScratch {
  uint64_t part_acc, part_ml, part_h, P, Q, d_sdst, d_ssrc, red, total;
};

GatScratch gat_scratch(const tgb_csr_plan *plan, int H, int D, bool backward) {
  GatScratch s{};
  uint64_t p = 0;
  auto take = [&](uint64_t bytes) { uint64_t at = p; p = align_up(p + bytes, 256); return at; };
  const uint64_t F = (uint64_t)H * D;
  const uint64_t seg = (uint64_t)(plan->fwd.n_seg > plan->bwd.n_seg ? plan->fwd.n_seg : plan->bwd.n_seg);
  s.part_acc = take(seg * F * 4);
  s.part_ml = take(seg * 2 * H * 4);
  s.part_h = take(seg * H * 4);
  if (backward) {
    s.P = take((uint64_t)plan->num_edges * H * 4);
    s.Q = take((uint64_t)plan->num_edges * H * 4);
    s.d_sdst = take((uint64_t)plan->num_dst * H * 4);
    s.d_ssrc = take((uint64_t)plan->num_src * H * 4);
    s.red = take((uint64_t)kReduceBlocks * F * 4);
  }
  s.total = p;
  return s;
}

#define TGB_DISPATCH_G(G_, ...)                             \
  switch (G_) {                                             \
    case 1: { constexpr int GG = 1; __VA_ARGS__; } break;   \
    case 2: { constexpr int GG = 2; __VA_ARGS__; } break;   \
    case 4: { constexpr int GG = 4; __VA_ARGS__; } break;   \
    case 8: { constexpr int GG = 8; __VA_ARGS__; } break;   \
    case 16: { constexpr int GG = 16; __VA_ARGS__; } break; \
    default: { constexpr int GG = 32; __VA_ARGS__; } break; \
  }

inline unsigned blocks_for(int64_t groups, int G) {
  return (unsigned)ceil_div(groups * G, kBlock);
}

}  // namespace
}  // namespace tgb

using namespace tgb;

extern "C" {

int32_t tgb_gat_scratch_bytes(const tgb_csr_plan *plan, int32_t H, int32_t D, int32_t backward,
                              uint64_t *bytes) {
  if (!plan || !bytes) TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "null plan or output");
  GatShape shape;
  int32_t rc = gat_shape(H, D, &shape);
  if (rc) return rc;
  *bytes = gat_scratch(plan, H, D, backward != 0).total;
  return TGB_STATUS_OK;
}

int32_t tgb_gat_node_scores(const void *x, const void *a, int64_t n, int32_t H, int32_t D, void *scores,
                            uint64_t stream) {
  GatShape shape;
  int32_t rc = gat_shape(H, D, &shape);
  if (rc) return rc;
  if (n == 0) return TGB_STATUS_OK;
  if (!x || !a || !scores) TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "null pointer");
  if (((uintptr_t)x | (uintptr_t)a) & 15u) TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "features must be 16-byte aligned");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  TGB_DISPATCH_G(shape.G, k_node_scores<GG><<<blocks_for(n, GG), kBlock, 0, st>>>(
      (const __nv_bfloat16 *)x, (const __nv_bfloat16 *)a, n, H, shape.lph, (float *)scores));
  TGB_LAUNCHED();
  return TGB_STATUS_OK;
}

int32_t tgb_gat_fwd(const tgb_csr_plan *plan, const void *x_src, const void *s_src, const void *s_dst,
                    void *out, void *m, void *l, int32_t H, int32_t D, float slope, void *scratch,
                    uint64_t scratch_bytes, uint64_t stream) {
  if (!plan) TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "null plan");
  GatShape shape;
  int32_t rc = gat_shape(H, D, &shape);
  if (rc) return rc;
  if (plan->num_dst == 0) return TGB_STATUS_OK;
  if (!s_dst || !out || !m || !l || (plan->num_edges > 0 && (!x_src || !s_src)))
    TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "null pointer");
  if (((uintptr_t)x_src | (uintptr_t)out) & 15u)
    TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "features must be 16-byte aligned");
  GatScratch sc = gat_scratch(plan, H, D, false);
  if (plan->fwd.n_seg > 0 && (!scratch || scratch_bytes < sc.total))
    TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "scratch too small: %llu < %llu bytes",
             (unsigned long long)scratch_bytes, (unsigned long long)sc.total);
  GatArgs a{};
  a.work = work_list(plan->fwd);
  a.x_src = (const __nv_bfloat16 *)x_src;
  a.s_src = (const float *)s_src;
  a.s_dst = (const float *)s_dst;
  a.out = (__nv_bfloat16 *)out;
  a.m = (float *)m;
  a.l = (float *)l;
  a.part_acc = (float *)((char *)scratch + sc.part_acc);
  a.part_ml = (float *)((char *)scratch + sc.part_ml);
  a.H = H;
  a.D = D;
  a.lph = shape.lph;
  a.slope_bf = __bfloat162float(__float2bfloat16_rn(slope));
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int64_t groups = a.work.n_seg + (a.work.n_rows - a.work.n_long);
  if (quarter_shape(shape)) {
    if (plan->index_bits == 32) k_gat_fwd_q<int32_t, int32_t, kQU><<<blocks_for(groups, kQG), kBlock, 0, st>>>(a);
    else k_gat_fwd_q<int64_t, int64_t, kQU><<<blocks_for(groups, kQG), kBlock, 0, st>>>(a);
  } else if (plan->index_bits == 32) {
    TGB_DISPATCH_G(shape.G, k_gat_fwd<int32_t, int32_t, GG><<<blocks_for(groups, GG), kBlock, 0, st>>>(a));
  } else {
    TGB_DISPATCH_G(shape.G, k_gat_fwd<int64_t, int64_t, GG><<<blocks_for(groups, GG), kBlock, 0, st>>>(a));
  }
  TGB_LAUNCHED();
  if (a.work.n_long > 0) {
    TGB_DISPATCH_G(shape.G, k_gat_fwd_finalize<GG><<<(unsigned)a.work.n_long, 32, 0, st>>>(a));
    TGB_LAUNCHED();
  }
  return TGB_STATUS_OK;
}

int32_t tgb_gat_bwd(const tgb_csr_plan *plan, const void *x_src, const void *x_dst, const void *a_src,
                    const void *a_dst, const void *s_src, const void *s_dst, const void *out,
                    const void *dout, const void *m, const void *l, int32_t H, int32_t D, float slope,
                    void *dx_src, void *dx_dst, void *da_src, void *da_dst, void *scratch,
                    uint64_t scratch_bytes, uint64_t stream) {
  if (!plan) TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "null plan");
  if (!(plan->flags & TGB_PLAN_TRANSPOSE))
    TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "plan was created without TGB_PLAN_TRANSPOSE");
  GatShape shape;
  int32_t rc = gat_shape(H, D, &shape);
  if (rc) return rc;
  if (!x_src || !x_dst || !a_src || !a_dst || !s_src || !s_dst || !out || !dout || !m || !l || !dx_src ||
      !dx_dst || !da_src || !da_dst)
    TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "null pointer");
  GatScratch sc = gat_scratch(plan, H, D, true);
  if (!scratch || scratch_bytes < sc.total)
    TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "scratch too small: %llu < %llu bytes",
             (unsigned long long)scratch_bytes, (unsigned long long)sc.total);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int F = H * D;
  GatArgs a{};
  a.x_src = (const __nv_bfloat16 *)x_src;
  a.x_dst = (const __nv_bfloat16 *)x_dst;
  a.s_src = (const float *)s_src;
  a.s_dst = (const float *)s_dst;
  a.m = (float *)m;
  a.l = (float *)l;
  a.o = (const __nv_bfloat16 *)out;
  a.dout = (const __nv_bfloat16 *)dout;
  a.a_src = (const __nv_bfloat16 *)a_src;
  a.a_dst = (const __nv_bfloat16 *)a_dst;
  a.dx_src = (__nv_bfloat16 *)dx_src;
  a.dx_dst = (__nv_bfloat16 *)dx_dst;
  a.part_acc = (float *)((char *)scratch + sc.part_acc);
  a.part_h = (float *)((char *)scratch + sc.part_h);
  a.P = (float *)((char *)scratch + sc.P);
  a.Q = (float *)((char *)scratch + sc.Q);
  a.d_sdst = (float *)((char *)scratch + sc.d_sdst);
  a.d_ssrc = (float *)((char *)scratch + sc.d_ssrc);
  float *red = (float *)((char *)scratch + sc.red);
  a.H = H;
  a.D = D;
  a.lph = shape.lph;
  a.slope_bf = __bfloat162float(__float2bfloat16_rn(slope));

  // pass 1: destination-major
  a.work = work_list(plan->fwd);
  int64_t groups = a.work.n_seg + (a.work.n_rows - a.work.n_long);
  const bool head_lanes = H == kHL && D == 8 * kHV && TGB_GAT_HEAD_LANES;   // one lane per head (8 x 32 rows)
  if (groups > 0) {
    if (head_lanes) {
      if (plan->index_bits == 32)
        k_gat_bwd_dst_h<int32_t, int32_t, TGB_GAT_BWD_U><<<blocks_for(groups, kHL), kBlock, 0, st>>>(a);
      else
        k_gat_bwd_dst_h<int64_t, int64_t, TGB_GAT_BWD_U><<<blocks_for(groups, kHL), kBlock, 0, st>>>(a);
    } else if (plan->index_bits == 32) {
      TGB_DISPATCH_G(shape.G, k_gat_bwd_dst<int32_t, int32_t, GG><<<blocks_for(groups, GG), kBlock, 0, st>>>(a));
    } else {
      TGB_DISPATCH_G(shape.G, k_gat_bwd_dst<int64_t, int64_t, GG><<<blocks_for(groups, GG), kBlock, 0, st>>>(a));
    }
    TGB_LAUNCHED();
    if (a.work.n_long > 0) {
      k_sum_head_partials<<<(unsigned)a.work.n_long, 32, 0, st>>>(a.work, a.part_h, H, a.d_sdst);
      TGB_LAUNCHED();
    }
  }
  // pass 2: source-major over the transposed relation
  a.work = work_list(plan->bwd);
  groups = a.work.n_seg + (a.work.n_rows - a.work.n_long);
  if (groups > 0) {
    if (head_lanes) {
      k_gat_bwd_src_h<TGB_GAT_BWD_U><<<blocks_for(groups, kHL), kBlock, 0, st>>>(a);
    } else {
      TGB_DISPATCH_G(shape.G, k_gat_bwd_src<GG><<<blocks_for(groups, GG), kBlock, 0, st>>>(a));
    }
    TGB_LAUNCHED();
    if (a.work.n_long > 0) {
      TGB_DISPATCH_G(shape.G, k_gat_bwd_src_finalize<GG><<<(unsigned)a.work.n_long, 32, 0, st>>>(a));
      TGB_LAUNCHED();
    }
  }
  // pass 3: dx_dst and the parameter gradients
  TGB_DISPATCH_G(shape.G, k_param_grad<GG><<<kReduceBlocks, 256, 0, st>>>(
      a.x_dst, a.d_sdst, a.a_dst, plan->num_dst, H, shape.lph, a.dx_dst, red));
  TGB_LAUNCHED();
  k_sum_partials<<<(unsigned)ceil_div(F, 128), 128, 0, st>>>(red, kReduceBlocks, F, (float *)da_dst);
  TGB_LAUNCHED();
  TGB_DISPATCH_G(shape.G, k_param_grad<GG><<<kReduceBlocks, 256, 0, st>>>(
      a.x_src, a.d_ssrc, a.a_src, plan->num_src, H, shape.lph, (__nv_bfloat16 *)nullptr, red));
  TGB_LAUNCHED();
  k_sum_partials<<<(unsigned)ceil_div(F, 128), 128, 0, st>>>(red, kReduceBlocks, F, (float *)da_src);
  TGB_LAUNCHED();
  return TGB_STATUS_OK;
}

}  // extern "C"
