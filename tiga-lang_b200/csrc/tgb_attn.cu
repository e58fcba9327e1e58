// Dense-relation attention with the online-softmax reducer over packed
// variable-length sequences (causal or full inside each sequence), bf16 inputs,
// float32 softmax state, on the 5th-generation tensor cores.
//
// It is the reference's streaming kernel gf_dense_streaming_reduce
// (lib/Target/Triton/Translate.cpp:1603-1912: S = Q K^T * scale * log2e, causal
// mask src <= row, online softmax with exp2, O += P V, O / l) rebuilt for
// sm_100a, extended to bf16, to a block-diagonal (cu_seqlens) relation that is
// never materialised (Graph.cu_seqlens / Graph.cat of triangular blocks,
// python/tiga/graph/core.py:314-351,650-709), and to a backward pass, which the
// reference does not have.
//
// Forward, one CTA (four softmax warps + one issue warp) per (128-query tile, head):
//   TMA loads Q once and K/V blocks of 64 keys into two-stage rings
//   (128-byte rows, 128-byte swizzle; a 128-wide head is two 64-column boxes);
//   one thread of the issue warp issues tcgen05.mma: S = Q K^T into one of two
//   buffers in tensor memory, one block ahead of the softmax; the four warps
//   read their 32 rows of S, keep the running max / denominator in registers,
//   write P as bf16 into a swizzled shared-memory tile; a second MMA group
//   accumulates P V in tensor memory over all key blocks (V is consumed
//   MN-major as loaded).  The accumulator is rescaled in place only when a
//   row's maximum has grown by more than 2^8 since its reference was set.
// Tensor-core bound: 4*D flops per (query, key) pair forward.
#include <cuda_bf16.h>

#include "tgb_common.cuh"
#include "tgb_tcgen05.cuh"

namespace tgb {
namespace {

using namespace sm100;

constexpr int kTile = 128;                 // queries per CTA and keys per block
constexpr int kBoxBytes = kTile * 128;     // one TMA box: 128 rows x 128 bytes (64 bf16)
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t *>(&v);
}

// Writes 8 consecutive bf16 of row `r`, 16-byte chunk `chunk` (0..7) of a
// K-major tile of 128-byte rows with the 128-byte swizzle.
__device__ __forceinline__ void store_swizzled_chunk(uint8_t *tile, int r, int chunk, uint4 value) {
  *reinterpret_cast<uint4 *>(tile + r * 128 + ((chunk ^ (r & 7)) << 4)) = value;
}

struct Tile {           // one 128-token tile of one sequence, for one head
  int32_t q_begin;      // first query (or key) of the tile (token index)
  int32_t seq_begin;    // first token of the sequence
  int32_t seq_end;      // one past the last token of the sequence
  int32_t head;
};

// Keys per block of the forward and dQ kernels.  64 keeps a CTA at 112 KB of
// shared memory, 256 registers x 128 threads and 256 tensor-memory columns, so
// two CTAs share an SM and one CTA's softmax overlaps the other's MMAs.
constexpr int kKeyBlock = 64;
constexpr int kKeyBoxBytes = kKeyBlock * 128;

template <int HALVES>   // head width = 64 * HALVES
struct FwdSmem {
  alignas(1024) uint8_t q[HALVES][kBoxBytes];
  alignas(1024) uint8_t k[2][HALVES][kKeyBoxBytes];
  alignas(1024) uint8_t v[2][HALVES][kKeyBoxBytes];
  alignas(1024) uint8_t p[kBoxBytes];              // [128 queries x 64 keys] bf16
  uint64_t q_full, k_full[2], v_full[2], s_done[2], s_free[2], p_ready, o_done;
  uint32_t tmem_base;
  int abort_flag;
};

// The output accumulates in tensor memory against a reference maximum that is
// only moved (and the accumulator rescaled) when the running maximum has grown
// by more than this many powers of two; p = 2^(s - reference) then stays below
// 2^8 and the final O / l is the same quotient as with the exact maximum.
constexpr float kRescaleGap = 8.0f;

constexpr int kFwdThreads = 160;   // warps 0-3: softmax (one query row per thread); warp 4: TMA + MMA issue

template <int HALVES>
__global__ void __launch_bounds__(kFwdThreads, 2)
k_attn_fwd(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
           const __grid_constant__ CUtensorMap map_v, const Tile *__restrict__ tiles, int H, int group,
           float scale_log2, int causal, __nv_bfloat16 *__restrict__ out, float *__restrict__ lse, int *error) {
  constexpr int D = 64 * HALVES;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  FwdSmem<HALVES> &sm = *reinterpret_cast<FwdSmem<HALVES> *>(smem_raw);
  if (smem_u32(smem_raw) & 1023u) {                  // swizzled tiles need a 1024-byte aligned base
    if (threadIdx.x == 0) atomicCAS(error, 0, 19);
    return;
  }
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const Tile tile = tiles[blockIdx.x];
  const int head = tile.head;
  const int kv_head = head / group;                  // grouped queries: `group` query heads read one K/V head
  const int key_limit = causal ? min(tile.q_begin + kTile, tile.seq_end) : tile.seq_end;
  const int n_blocks = (key_limit - tile.seq_begin + kKeyBlock - 1) / kKeyBlock;

  if (tid == 0) {
    sm.abort_flag = 0;
    mbar_init(&sm.q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&sm.k_full[i], 1);
      mbar_init(&sm.v_full[i], 1);
      mbar_init(&sm.s_done[i], 1);
      mbar_init(&sm.s_free[i], 4);        // one arrival per softmax warp
    }
    mbar_init(&sm.p_ready, 4);
    mbar_init(&sm.o_done, 1);
    mbar_fence_init();
    tma_prefetch_descriptor(&map_q);
    tma_prefetch_descriptor(&map_k);
    tma_prefetch_descriptor(&map_v);
  }
  __syncthreads();
  if (warp == 0) tmem_alloc(&sm.tmem_base, 256);    // S: two buffers at columns 0-63 and 64-127, O: columns 128-255
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_s = sm.tmem_base, tmem_o = sm.tmem_base + 128;
  volatile int *abort_flag = &sm.abort_flag;

  if (warp == 4) {
    // ---- issue warp: one thread loads Q, K, V and issues the MMAs.  S of block kb+1 is issued before
    // the softmax of block kb has run (two S buffers), P V of block kb while the softmax warps are
    // already on block kb+1; issuing can stall on the tensor pipe, so this thread does nothing else.
    if (lane == 0 && n_blocks > 0) {
      auto load_k = [&](int block) {
        const int stage = block & 1, y = tile.seq_begin + block * kKeyBlock;
        mbar_arrive_expect_tx(&sm.k_full[stage], HALVES * kKeyBoxBytes);
#pragma unroll
        for (int j = 0; j < HALVES; ++j) tma_load_2d(sm.k[stage][j], &map_k, kv_head * D + 64 * j, y, &sm.k_full[stage]);
      };
      auto load_v = [&](int block) {
        const int stage = block & 1, y = tile.seq_begin + block * kKeyBlock;
        mbar_arrive_expect_tx(&sm.v_full[stage], HALVES * kKeyBoxBytes);
#pragma unroll
        for (int j = 0; j < HALVES; ++j) tma_load_2d(sm.v[stage][j], &map_v, kv_head * D + 64 * j, y, &sm.v_full[stage]);
      };
      constexpr uint32_t idesc_s = instr_desc(kFmtBF16, kFmtBF16, kTile, kKeyBlock, 0, 0);
      constexpr uint32_t idesc_o = instr_desc(kFmtBF16, kFmtBF16, kTile, D, 0, 1);   // V is MN-major
      auto issue_s = [&](int block) {
        const int st = block & 1;
        mbar_wait(&sm.k_full[st], (uint32_t)((block >> 1) & 1), abort_flag, error, 12);
        if (block >= 2)       // the softmax of block-2 has read this S buffer
          mbar_wait(&sm.s_free[st], (uint32_t)(((block >> 1) - 1) & 1), abort_flag, error, 17);
        tc_fence_after_sync();
#pragma unroll
        for (int k16 = 0; k16 < D / 16; ++k16) {       // 16 bf16 = 32 bytes of the 128-byte row per MMA
          const int j = k16 >> 2;
          const uint32_t off = (k16 & 3) * 32;
          mma_f16(tmem_s + (uint32_t)st * kKeyBlock, smem_desc_k_major_sw128(smem_u32(sm.q[j]) + off),
                  smem_desc_k_major_sw128(smem_u32(sm.k[st][j]) + off), idesc_s, k16 != 0);
        }
        mma_commit(&sm.s_done[st]);
      };
      mbar_arrive_expect_tx(&sm.q_full, HALVES * kBoxBytes);
#pragma unroll
      for (int j = 0; j < HALVES; ++j) tma_load_2d(sm.q[j], &map_q, head * D + 64 * j, tile.q_begin, &sm.q_full);
      load_k(0);
      load_v(0);
      if (n_blocks > 1) {
        load_k(1);
        load_v(1);
      }
      mbar_wait(&sm.q_full, 0, abort_flag, error, 11);
      issue_s(0);
      for (int kb = 0; kb < n_blocks; ++kb) {
        const int st = kb & 1;
        if (kb + 1 < n_blocks) issue_s(kb + 1);
        if (kb + 2 < n_blocks) {                        // K stage of block kb is free once S(kb) is complete
          mbar_wait(&sm.s_done[st], (uint32_t)((kb >> 1) & 1), abort_flag, error, 13);
          load_k(kb + 2);
        }
        mbar_wait(&sm.p_ready, (uint32_t)(kb & 1), abort_flag, error, 18);
        // the softmax threads waited for P V of block kb-1 before they wrote P: its V stage is free
        if (kb >= 1 && kb + 1 < n_blocks) load_v(kb + 1);
        mbar_wait(&sm.v_full[st], (uint32_t)((kb >> 1) & 1), abort_flag, error, 15);
        tc_fence_after_sync();
#pragma unroll
        for (int k16 = 0; k16 < kKeyBlock / 16; ++k16) {   // 16 keys per MMA, accumulated over all blocks
          const uint64_t a_desc = smem_desc_k_major_sw128(smem_u32(sm.p) + k16 * 32);
          const uint64_t b_desc = smem_desc_mn_major_sw128(smem_u32(sm.v[st][0]) + k16 * 16 * 128, kKeyBoxBytes);
          mma_f16(tmem_o, a_desc, b_desc, idesc_o, (kb | k16) != 0);
        }
        mma_commit(&sm.o_done);
      }
    }
  } else {
    // ---- softmax warps -----------------------------------------------------------------------------
    const int row = warp * 32 + lane;                 // query row of this thread inside the tile
    const int q_index = tile.q_begin + row;
    const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
    float m = -INFINITY, l = 0.0f;                    // reference maximum (log2 domain) and denominator
    for (int kb = 0; kb < n_blocks; ++kb) {
      const int st = kb & 1;
      const int key0 = tile.seq_begin + kb * kKeyBlock;
      const uint32_t s_addr = tmem_s + (uint32_t)st * kKeyBlock + lane_base;
      mbar_wait(&sm.s_done[st], (uint32_t)((kb >> 1) & 1), abort_flag, error, 13);
      tc_fence_after_sync();
      const bool masked = (key0 + kKeyBlock > tile.seq_end) || (causal && key0 + kKeyBlock - 1 > tile.q_begin);
      // The 64 scores of the row stay in registers for both passes; the S buffer is released at once.
      // Maximum and sum run as four independent chains: with two warps per scheduler every dependent
      // instruction would otherwise wait out its full latency.
      uint32_t r0[32], r1[32];
      tmem_ld_32x32(s_addr, r0);
      tmem_ld_32x32(s_addr + 32, r1);
      tmem_ld_wait();
      tc_fence_before_sync();
      mbar_arrive_warp(&sm.s_free[st]);                // this S buffer may be overwritten
      float sc[kKeyBlock];
#pragma unroll
      for (int c = 0; c < 32; ++c) {
        sc[c] = __uint_as_float(r0[c]);
        sc[32 + c] = __uint_as_float(r1[c]);
      }
      if (masked) {
#pragma unroll
        for (int c = 0; c < kKeyBlock; ++c) {
          const int key = key0 + c;
          if (!(key < tile.seq_end && (!causal || key <= q_index))) sc[c] = -INFINITY;
        }
      }
      float bm[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int c = 0; c < kKeyBlock; ++c) bm[c & 3] = fmaxf(bm[c & 3], sc[c]);
      const float block_max = fmaxf(fmaxf(bm[0], bm[1]), fmaxf(bm[2], bm[3]));
      const float m_blk = fmaxf(m, block_max * scale_log2);
      float alpha = 1.0f;
      if (m == -INFINITY) {
        m = m_blk;                                     // nothing accumulated for this row yet
      } else if (m_blk - m > kRescaleGap) {
        alpha = fast_exp2(m - m_blk);
        m = m_blk;
      }
      const float m_use = m == -INFINITY ? 0.0f : m;   // a fully masked row keeps p = 0
      // p = 2^(s - m); masked scores are -inf and give exactly 0
      float bs[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
      for (int c = 0; c < kKeyBlock; ++c) {
        sc[c] = fast_exp2(fmaf(sc[c], scale_log2, -m_use));
        bs[c & 3] += sc[c];
      }
      l = l * alpha + ((bs[0] + bs[1]) + (bs[2] + bs[3]));
      if (kb > 0) {
        // P V of the previous block read the P tile and the accumulator
        mbar_wait(&sm.o_done, (uint32_t)((kb - 1) & 1), abort_flag, error, 14);
        tc_fence_after_sync();
      }
      if (__any_sync(0xffffffffu, alpha != 1.0f)) {    // rare: move the reference maximum of these 32 rows
#pragma unroll 1
        for (int c0 = 0; c0 < D; c0 += 32) {
          uint32_t r[32];
          tmem_ld_32x32(tmem_o + lane_base + c0, r);
          tmem_ld_wait();
#pragma unroll
          for (int c = 0; c < 32; ++c) r[c] = __float_as_uint(__uint_as_float(r[c]) * alpha);
          tmem_st_32x32(tmem_o + lane_base + c0, r);
        }
        tmem_st_wait();
      }
#pragma unroll
      for (int g = 0; g < kKeyBlock / 8; ++g)
        store_swizzled_chunk(sm.p, row, g,
                             make_uint4(pack_bf16(sc[8 * g], sc[8 * g + 1]), pack_bf16(sc[8 * g + 2], sc[8 * g + 3]),
                                        pack_bf16(sc[8 * g + 4], sc[8 * g + 5]), pack_bf16(sc[8 * g + 6], sc[8 * g + 7])));
      tc_fence_before_sync();
      fence_proxy_async_smem();
      mbar_arrive_warp(&sm.p_ready);                   // P written, accumulator rescaled
    }
    if (n_blocks > 0) {
      mbar_wait(&sm.o_done, (uint32_t)((n_blocks - 1) & 1), abort_flag, error, 16);
      tc_fence_after_sync();
    }
    const bool writes = q_index < tile.seq_end && !*abort_flag;
    const float inv = l > 0.0f ? 1.0f / l : 0.0f;
    __nv_bfloat16 *dst = out + ((int64_t)q_index * H + head) * D;
#pragma unroll 1
    for (int c0 = 0; c0 < D; c0 += 32) {
      uint32_t r[32];
      if (n_blocks > 0) {
        tmem_ld_32x32(tmem_o + lane_base + c0, r);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int c = 0; c < 32; ++c) r[c] = 0u;
      }
      if (writes) {
#pragma unroll
        for (int d = 0; d < 32; d += 8)
          *reinterpret_cast<uint4 *>(dst + c0 + d) = make_uint4(
              pack_bf16(__uint_as_float(r[d]) * inv, __uint_as_float(r[d + 1]) * inv),
              pack_bf16(__uint_as_float(r[d + 2]) * inv, __uint_as_float(r[d + 3]) * inv),
              pack_bf16(__uint_as_float(r[d + 4]) * inv, __uint_as_float(r[d + 5]) * inv),
              pack_bf16(__uint_as_float(r[d + 6]) * inv, __uint_as_float(r[d + 7]) * inv));
      }
    }
    if (writes) lse[(int64_t)q_index * H + head] = l > 0.0f ? (m + log2f(l)) * kLn2 : -INFINITY;
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(sm.tmem_base, 256);
}

// ---------------------------------------------------------------------------
// Backward.  delta[i,h] = <dO[i,h,:], O[i,h,:]>; with P = exp(S*scale - lse):
//   dV = P^T dO,  dP = dO V^T,  dS = P o (dP - delta),  dQ = scale dS K,  dK = scale dS^T Q.
// Two kernels, both without atomics:
//   k_attn_bwd_dkv  one CTA per (128-key tile, head), loops over the query
//                   blocks that see those keys; works on the TRANSPOSED score
//                   tile (rows = keys), so every thread owns one key row of the
//                   dV / dK accumulators in tensor memory (S^T, dP^T, dV, dK:
//                   512 columns);
//   k_attn_bwd_dq   one CTA per (128-query tile, head), loops over key blocks
//                   (S, dP, dQ in tensor memory).
// Every operand is used in the orientation TMA delivers it: [rows, D] tiles are
// K-major for the score products and MN-major for the gradient products.
// ---------------------------------------------------------------------------
__global__ void k_attn_delta(const __nv_bfloat16 *__restrict__ o, const __nv_bfloat16 *__restrict__ d_o,
                             int64_t rows, int D, float *__restrict__ delta) {
  const int lane = threadIdx.x & 31;
  const int64_t r = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  if (r >= rows) return;
  float acc = 0.0f;
  for (int d = lane * 2; d < D; d += 64) {
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(o + r * D + d));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(d_o + r * D + d));
    acc = fmaf(a.x, b.x, fmaf(a.y, b.y, acc));
  }
  for (int s = 16; s; s >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, s);
  if (lane == 0) delta[r] = acc;
}


// [128 x 128] score-like product of two K-major tiles of width D into `tmem`
template <int HALVES, int BOX_A, int BOX_B>
__device__ __forceinline__ void issue_scores(uint32_t tmem, uint8_t (*a)[BOX_A], uint8_t (*b)[BOX_B],
                                             uint32_t idesc) {
#pragma unroll
  for (int k16 = 0; k16 < HALVES * 4; ++k16) {
    const uint32_t off = (k16 & 3) * 32;
    mma_f16(tmem, smem_desc_k_major_sw128(smem_u32(a[k16 >> 2]) + off),
            smem_desc_k_major_sw128(smem_u32(b[k16 >> 2]) + off), idesc, k16 != 0);
  }
}

// dK/dV kernel: CTA = (128-key tile, head), eight compute warps (a thread owns a key row of the
// transposed score tile and half of the block's queries) + one issue warp.  Queries stream in blocks of 64 through two stages; S^T and
// dP^T have two buffers each in tensor memory (queries stream through three shared-memory stages), so the issue thread puts the score MMAs of block qb+1 in
// flight while the compute warps turn block qb into P^T and dS^T, and issues the gradient MMAs of block
// qb as soon as those tiles are written.  Tensor memory: S^T 0/64, dP^T 128/192, dV 256, dK 384.
constexpr int kQBlock = 64;
constexpr int kQBoxBytes = kQBlock * 128;
constexpr int kDkvStages = 3;              // query-block stages: the TMA of block qb+2 starts when block qb-1 is done
constexpr int kDkvComputeThreads = 256;   // eight compute warps: two per 32-lane quadrant, 32 queries of the block each
constexpr int kDkvThreads = kDkvComputeThreads + 32;

template <int HALVES>
struct DkvSmem {
  alignas(1024) uint8_t k[HALVES][kBoxBytes];
  alignas(1024) uint8_t v[HALVES][kBoxBytes];
  alignas(1024) uint8_t q[kDkvStages][HALVES][kQBoxBytes];
  alignas(1024) uint8_t d_o[kDkvStages][HALVES][kQBoxBytes];
  alignas(1024) uint8_t p[2][kBoxBytes];     // P^T  [128 keys x 64 queries] bf16
  alignas(1024) uint8_t ds[2][kBoxBytes];    // dS^T
  float lse2[2][kQBlock];
  float delta[2][kQBlock];
  uint64_t fixed_full, stream_full[kDkvStages], s_done[2], s_free[2], pd_ready[2], g_done[2];
  uint32_t tmem_base;
  int abort_flag;
};

template <int HALVES>
__global__ void __launch_bounds__(kDkvThreads, 1)
k_attn_bwd_dkv(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
               const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_do,
               const Tile *__restrict__ tiles, int H, int H_kv, float scale, int causal,
               const float *__restrict__ lse, const float *__restrict__ delta, __nv_bfloat16 *__restrict__ dk,
               __nv_bfloat16 *__restrict__ dv, int *error) {
  constexpr int D = 64 * HALVES;
  extern __shared__ uint8_t smem_raw[];
  DkvSmem<HALVES> &sm =
      *reinterpret_cast<DkvSmem<HALVES> *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const Tile tile = tiles[blockIdx.x];               // q_begin holds the first key of this tile
  const int head = tile.head;                        // a K/V head
  const int group = H / H_kv;                        // query heads that read this K/V head
  const int q_first = causal ? tile.q_begin : tile.seq_begin;
  const int blocks_per_head = (tile.seq_end - q_first + kQBlock - 1) / kQBlock;
  // The streamed blocks run over every query head of the group in turn: block b is query block
  // b % blocks_per_head of query head head * group + b / blocks_per_head.  dK and dV accumulate in
  // tensor memory over all of them.
  const int n_blocks = blocks_per_head * group;
  const float scale_log2 = scale * kLog2e;
  auto q_head_of = [&](int block) { return head * group + block / blocks_per_head; };
  auto q_begin_of = [&](int block) { return q_first + (block % blocks_per_head) * kQBlock; };

  if (tid == 0) {
    sm.abort_flag = 0;
    mbar_init(&sm.fixed_full, 1);
    for (int i = 0; i < kDkvStages; ++i) mbar_init(&sm.stream_full[i], 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&sm.s_done[i], 1);
      mbar_init(&sm.s_free[i], kDkvComputeThreads / 32);   // one arrival per compute warp
      mbar_init(&sm.pd_ready[i], kDkvComputeThreads / 32);
      mbar_init(&sm.g_done[i], 1);
    }
    mbar_fence_init();
  }
  __syncthreads();
  if (warp == 0) tmem_alloc(&sm.tmem_base, 512);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_st = sm.tmem_base, tmem_dpt = sm.tmem_base + 128, tmem_dv = sm.tmem_base + 256,
                 tmem_dk = sm.tmem_base + 384;
  volatile int *abort_flag = &sm.abort_flag;

  if (warp == kDkvComputeThreads / 32) {
    if (lane == 0 && n_blocks > 0) {
      constexpr uint32_t idesc_s = instr_desc(kFmtBF16, kFmtBF16, kTile, kQBlock, 0, 0);
      constexpr uint32_t idesc_g = instr_desc(kFmtBF16, kFmtBF16, kTile, D, 0, 1);
      auto load_stream = [&](int block) {
        const int st = block % kDkvStages, q0 = q_begin_of(block), qh = q_head_of(block);
        mbar_arrive_expect_tx(&sm.stream_full[st], 2 * HALVES * kQBoxBytes);
#pragma unroll
        for (int j = 0; j < HALVES; ++j) {
          tma_load_2d(sm.q[st][j], &map_q, qh * D + 64 * j, q0, &sm.stream_full[st]);
          tma_load_2d(sm.d_o[st][j], &map_do, qh * D + 64 * j, q0, &sm.stream_full[st]);
        }
      };
      auto issue_scores_of = [&](int block) {
        const int st = block & 1, stage = block % kDkvStages;
        mbar_wait(&sm.stream_full[stage], (uint32_t)((block / kDkvStages) & 1), abort_flag, error, 22);
        if (block >= 2)       // the compute warps have read this pair of score buffers
          mbar_wait(&sm.s_free[st], (uint32_t)(((block >> 1) - 1) & 1), abort_flag, error, 25);
        tc_fence_after_sync();
        issue_scores<HALVES, kBoxBytes, kQBoxBytes>(tmem_st + st * kQBlock, sm.k, sm.q[stage], idesc_s);     // S^T  = K Q^T
        issue_scores<HALVES, kBoxBytes, kQBoxBytes>(tmem_dpt + st * kQBlock, sm.v, sm.d_o[stage], idesc_s);  // dP^T = V dO^T
        mma_commit(&sm.s_done[st]);
      };
      mbar_arrive_expect_tx(&sm.fixed_full, 2 * HALVES * kBoxBytes);
#pragma unroll
      for (int j = 0; j < HALVES; ++j) {
        tma_load_2d(sm.k[j], &map_k, head * D + 64 * j, tile.q_begin, &sm.fixed_full);
        tma_load_2d(sm.v[j], &map_v, head * D + 64 * j, tile.q_begin, &sm.fixed_full);
      }
      for (int blk = 0; blk < kDkvStages && blk < n_blocks; ++blk) load_stream(blk);
      mbar_wait(&sm.fixed_full, 0, abort_flag, error, 21);
      issue_scores_of(0);
      for (int qb = 0; qb < n_blocks; ++qb) {
        const int st = qb & 1, stage = qb % kDkvStages;
        if (qb + 1 < n_blocks) issue_scores_of(qb + 1);
        if (qb >= 1 && qb + 2 < n_blocks) {             // the stage of block qb-1 is free once its gradient MMAs are complete
          mbar_wait(&sm.g_done[(qb - 1) & 1], (uint32_t)(((qb - 1) >> 1) & 1), abort_flag, error, 24);
          load_stream(qb + 2);
        }
        mbar_wait(&sm.pd_ready[st], (uint32_t)((qb >> 1) & 1), abort_flag, error, 26);
        tc_fence_after_sync();
#pragma unroll
        for (int k16 = 0; k16 < kQBlock / 16; ++k16) {   // 16 queries per MMA; dO and Q consumed MN-major as loaded
          const uint32_t boff = k16 * 16 * 128;
          mma_f16(tmem_dv, smem_desc_k_major_sw128(smem_u32(sm.p[st]) + k16 * 32),                       // dV += P^T dO
                  smem_desc_mn_major_sw128(smem_u32(sm.d_o[stage][0]) + boff, kQBoxBytes), idesc_g, (qb | k16) != 0);
          mma_f16(tmem_dk, smem_desc_k_major_sw128(smem_u32(sm.ds[st]) + k16 * 32),                      // dK += dS^T Q
                  smem_desc_mn_major_sw128(smem_u32(sm.q[stage][0]) + boff, kQBoxBytes), idesc_g, (qb | k16) != 0);
        }
        mma_commit(&sm.g_done[st]);
      }
    }
  } else {
    const int quad = warp & 3, h = warp >> 2;          // tensor-memory lane quadrant, half of the block's queries
    const int row = quad * 32 + lane;
    const int key_index = tile.q_begin + row;
    const bool key_ok = key_index < tile.seq_end;
    const uint32_t lane_base = (uint32_t)(quad * 32) << 16;
    // per-query softmax statistics: threads 0-63 fetch those of block qb+1 while block qb is computed
    auto fetch_stats = [&](int block, float &l2, float &dl) {
      const int qi = q_begin_of(block) + tid;
      const bool ok = qi < tile.seq_end;
      const int qh = q_head_of(block);
      l2 = ok ? lse[(int64_t)qi * H + qh] * kLog2e : INFINITY;
      dl = ok ? delta[(int64_t)qi * H + qh] : 0.0f;
    };
    if (tid < kQBlock && n_blocks > 0) fetch_stats(0, sm.lse2[0][tid], sm.delta[0][tid]);
    for (int qb = 0; qb < n_blocks; ++qb) {
      const int st = qb & 1;
      const int q0 = q_begin_of(qb);
      float next_lse2 = INFINITY, next_delta = 0.0f;
      const bool prefetch = tid < kQBlock && qb + 1 < n_blocks;
      if (prefetch) fetch_stats(qb + 1, next_lse2, next_delta);
      asm volatile("bar.sync 1, 256;" ::: "memory");   // the eight compute warps only; their control flow never diverges
      mbar_wait(&sm.s_done[st], (uint32_t)((qb >> 1) & 1), abort_flag, error, 23);
      tc_fence_after_sync();
      uint32_t rs[32], rp[32];
      tmem_ld_32x32(tmem_st + st * kQBlock + lane_base + 32 * h, rs);
      tmem_ld_32x32(tmem_dpt + st * kQBlock + lane_base + 32 * h, rp);
      tmem_ld_wait();
      tc_fence_before_sync();
      mbar_arrive_warp(&sm.s_free[st]);                 // the score buffers may be overwritten
      if (qb >= 2)                                      // the gradient MMAs of block qb-2 have read these P^T / dS^T tiles
        mbar_wait(&sm.g_done[st], (uint32_t)(((qb >> 1) - 1) & 1), abort_flag, error, 27);
      float p[32], ds[32];
#pragma unroll
      for (int c = 0; c < 32; ++c) {
        const int qi = q0 + 32 * h + c;
        const bool valid = key_ok && (!causal || key_index <= qi);
        p[c] = valid ? fast_exp2(fmaf(__uint_as_float(rs[c]), scale_log2, -sm.lse2[st][32 * h + c])) : 0.0f;
        ds[c] = p[c] * (__uint_as_float(rp[c]) - sm.delta[st][32 * h + c]);
      }
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        store_swizzled_chunk(sm.p[st], row, 4 * h + g,
                             make_uint4(pack_bf16(p[8 * g], p[8 * g + 1]), pack_bf16(p[8 * g + 2], p[8 * g + 3]),
                                        pack_bf16(p[8 * g + 4], p[8 * g + 5]), pack_bf16(p[8 * g + 6], p[8 * g + 7])));
        store_swizzled_chunk(sm.ds[st], row, 4 * h + g,
                             make_uint4(pack_bf16(ds[8 * g], ds[8 * g + 1]), pack_bf16(ds[8 * g + 2], ds[8 * g + 3]),
                                        pack_bf16(ds[8 * g + 4], ds[8 * g + 5]), pack_bf16(ds[8 * g + 6], ds[8 * g + 7])));
      }
      fence_proxy_async_smem();
      mbar_arrive_warp(&sm.pd_ready[st]);
      if (prefetch) {       // every compute warp is past this iteration's barrier, so block qb-1's statistics are dead
        sm.lse2[st ^ 1][tid] = next_lse2;
        sm.delta[st ^ 1][tid] = next_delta;
      }
    }
    if (n_blocks > 0) {                                 // the last commit covers every MMA issued before it
      mbar_wait(&sm.g_done[(n_blocks - 1) & 1], (uint32_t)(((n_blocks - 1) >> 1) & 1), abort_flag, error, 28);
      tc_fence_after_sync();
    }
    // warps 0-3 write dV, warps 4-7 write dK (scaled)
    const bool store = key_ok && !*abort_flag && n_blocks > 0;
    __nv_bfloat16 *dst = (h == 0 ? dv : dk) + ((int64_t)key_index * H_kv + head) * D;
    const float factor = h == 0 ? 1.0f : scale;
    const uint32_t src = (h == 0 ? tmem_dv : tmem_dk) + lane_base;
#pragma unroll 1
    for (int c0 = 0; c0 < D; c0 += 32) {
      uint32_t r[32];
      tmem_ld_32x32(src + c0, r);
      tmem_ld_wait();
      if (store) {
#pragma unroll
        for (int g = 0; g < 4; ++g)
          *reinterpret_cast<uint4 *>(dst + c0 + 8 * g) = make_uint4(
              pack_bf16(__uint_as_float(r[8 * g]) * factor, __uint_as_float(r[8 * g + 1]) * factor),
              pack_bf16(__uint_as_float(r[8 * g + 2]) * factor, __uint_as_float(r[8 * g + 3]) * factor),
              pack_bf16(__uint_as_float(r[8 * g + 4]) * factor, __uint_as_float(r[8 * g + 5]) * factor),
              pack_bf16(__uint_as_float(r[8 * g + 6]) * factor, __uint_as_float(r[8 * g + 7]) * factor));
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(sm.tmem_base, 512);
}

template <int HALVES>
struct DqSmem {
  alignas(1024) uint8_t q[HALVES][kBoxBytes];
  alignas(1024) uint8_t d_o[HALVES][kBoxBytes];
  alignas(1024) uint8_t k[HALVES][kKeyBoxBytes];
  alignas(1024) uint8_t v[HALVES][kKeyBoxBytes];
  alignas(1024) uint8_t ds[kBoxBytes];              // [128 queries x 64 keys] bf16
  uint64_t fixed_full, stream_full, s_done, acc_done;
  uint32_t tmem_base;
  int abort_flag;
};

// 64-key blocks: 112 KB of shared memory and 256 tensor-memory columns per CTA,
// two CTAs per SM.
template <int HALVES>
__global__ void __launch_bounds__(128, 2)
k_attn_bwd_dq(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
              const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_do,
              const Tile *__restrict__ tiles, int H, int group, float scale, int causal,
              const float *__restrict__ lse, const float *__restrict__ delta, __nv_bfloat16 *__restrict__ dq,
              int *error) {
  constexpr int D = 64 * HALVES;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  DqSmem<HALVES> &sm = *reinterpret_cast<DqSmem<HALVES> *>(smem_raw);
  if (smem_u32(smem_raw) & 1023u) {
    if (threadIdx.x == 0) atomicCAS(error, 0, 39);
    return;
  }
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const Tile tile = tiles[blockIdx.x];
  const int head = tile.head;
  const int kv_head = head / group;
  const int row = warp * 32 + lane;
  const int q_index = tile.q_begin + row;
  const int key_limit = causal ? min(tile.q_begin + kTile, tile.seq_end) : tile.seq_end;
  const int n_blocks = (key_limit - tile.seq_begin + kKeyBlock - 1) / kKeyBlock;
  const float scale_log2 = scale * kLog2e;

  if (tid == 0) {
    sm.abort_flag = 0;
    mbar_init(&sm.fixed_full, 1);
    mbar_init(&sm.stream_full, 1);
    mbar_init(&sm.s_done, 1);
    mbar_init(&sm.acc_done, 1);
    mbar_fence_init();
  }
  __syncthreads();
  if (warp == 0) tmem_alloc(&sm.tmem_base, 256);     // S: 0-63, dP: 64-127, dQ: 128-255
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_s = sm.tmem_base, tmem_dp = sm.tmem_base + 64, tmem_dq = sm.tmem_base + 128;
  const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
  volatile int *abort_flag = &sm.abort_flag;

  if (tid == 0) {
    mbar_arrive_expect_tx(&sm.fixed_full, 2 * HALVES * kBoxBytes);
#pragma unroll
    for (int j = 0; j < HALVES; ++j) {
      tma_load_2d(sm.q[j], &map_q, head * D + 64 * j, tile.q_begin, &sm.fixed_full);
      tma_load_2d(sm.d_o[j], &map_do, head * D + 64 * j, tile.q_begin, &sm.fixed_full);
    }
  }
  const bool q_ok = q_index < tile.seq_end;
  const float lse2 = q_ok ? lse[(int64_t)q_index * H + head] * kLog2e : INFINITY;
  const float my_delta = q_ok ? delta[(int64_t)q_index * H + head] : 0.0f;
  constexpr uint32_t idesc_s = instr_desc(kFmtBF16, kFmtBF16, kTile, kKeyBlock, 0, 0);
  constexpr uint32_t idesc_g = instr_desc(kFmtBF16, kFmtBF16, kTile, D, 0, 1);
  mbar_wait(&sm.fixed_full, 0, abort_flag, error, 31);

  for (int kb = 0; kb < n_blocks; ++kb) {
    const int key0 = tile.seq_begin + kb * kKeyBlock;
    if (tid == 0) {                                   // the previous block's readers finished (acc_done)
      mbar_arrive_expect_tx(&sm.stream_full, 2 * HALVES * kKeyBoxBytes);
#pragma unroll
      for (int j = 0; j < HALVES; ++j) {
        tma_load_2d(sm.k[j], &map_k, kv_head * D + 64 * j, key0, &sm.stream_full);
        tma_load_2d(sm.v[j], &map_v, kv_head * D + 64 * j, key0, &sm.stream_full);
      }
    }
    mbar_wait(&sm.stream_full, (uint32_t)(kb & 1), abort_flag, error, 32);
    if (tid == 0) {
      tc_fence_after_sync();
      issue_scores<HALVES, kBoxBytes, kKeyBoxBytes>(tmem_s, sm.q, sm.k, idesc_s);      // S  = Q K^T
      issue_scores<HALVES, kBoxBytes, kKeyBoxBytes>(tmem_dp, sm.d_o, sm.v, idesc_s);   // dP = dO V^T
      mma_commit(&sm.s_done);
    }
    mbar_wait(&sm.s_done, (uint32_t)(kb & 1), abort_flag, error, 33);
    tc_fence_after_sync();
#pragma unroll 1
    for (int c0 = 0; c0 < kKeyBlock; c0 += 32) {
      uint32_t rs[32], rp[32];
      tmem_ld_32x32(tmem_s + lane_base + c0, rs);
      tmem_ld_32x32(tmem_dp + lane_base + c0, rp);
      tmem_ld_wait();
      float ds[32];
#pragma unroll
      for (int c = 0; c < 32; ++c) {
        const int key = key0 + c0 + c;
        const bool valid = key < tile.seq_end && (!causal || key <= q_index);
        const float p = valid ? fast_exp2(__uint_as_float(rs[c]) * scale_log2 - lse2) : 0.0f;
        ds[c] = p * (__uint_as_float(rp[c]) - my_delta);
      }
#pragma unroll
      for (int g = 0; g < 4; ++g)
        store_swizzled_chunk(sm.ds, row, (c0 >> 3) + g,
                             make_uint4(pack_bf16(ds[8 * g], ds[8 * g + 1]), pack_bf16(ds[8 * g + 2], ds[8 * g + 3]),
                                        pack_bf16(ds[8 * g + 4], ds[8 * g + 5]), pack_bf16(ds[8 * g + 6], ds[8 * g + 7])));
    }
    fence_proxy_async_smem();
    tc_fence_before_sync();
    __syncthreads();
    if (tid == 0) {
      tc_fence_after_sync();
#pragma unroll
      for (int k16 = 0; k16 < kKeyBlock / 16; ++k16)   // dQ += dS K, 16 keys per MMA, K consumed MN-major
        mma_f16(tmem_dq, smem_desc_k_major_sw128(smem_u32(sm.ds) + k16 * 32),
                smem_desc_mn_major_sw128(smem_u32(sm.k[0]) + k16 * 16 * 128, kKeyBoxBytes), idesc_g,
                kb != 0 || k16 != 0);
      mma_commit(&sm.acc_done);
    }
    mbar_wait(&sm.acc_done, (uint32_t)(kb & 1), abort_flag, error, 34);
    tc_fence_after_sync();
  }

  const bool store = q_ok && !*abort_flag;
  __nv_bfloat16 *dst = dq + ((int64_t)q_index * H + head) * D;
#pragma unroll 1
  for (int c0 = 0; c0 < D; c0 += 32) {
    uint32_t r[32];
    tmem_ld_32x32(tmem_dq + lane_base + c0, r);
    tmem_ld_wait();
    if (store) {
#pragma unroll
      for (int g = 0; g < 4; ++g)
        *reinterpret_cast<uint4 *>(dst + c0 + 8 * g) = make_uint4(
            pack_bf16(__uint_as_float(r[8 * g]) * scale, __uint_as_float(r[8 * g + 1]) * scale),
            pack_bf16(__uint_as_float(r[8 * g + 2]) * scale, __uint_as_float(r[8 * g + 3]) * scale),
            pack_bf16(__uint_as_float(r[8 * g + 4]) * scale, __uint_as_float(r[8 * g + 5]) * scale),
            pack_bf16(__uint_as_float(r[8 * g + 6]) * scale, __uint_as_float(r[8 * g + 7]) * scale));
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(sm.tmem_base, 256);
}

int32_t check_attn(const void *q, const void *k, const void *v, int64_t tokens, int32_t H, int32_t H_kv, int32_t D) {
  if (!q || !k || !v) TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "null pointer");
  if (H <= 0 || tokens < 0) TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "invalid shape");
  if (H_kv <= 0 || H % H_kv != 0)
    TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "the %d query heads must be a multiple of the %d key/value heads", H, H_kv);
  if (D != 64 && D != 128) TGB_FAIL(TGB_STATUS_UNSUPPORTED, "dense attention supports head widths 64 and 128 (got %d)", D);
  if (tokens > (int64_t)INT32_MAX - 256) TGB_FAIL(TGB_STATUS_UNSUPPORTED, "too many tokens");
  return TGB_STATUS_OK;
}

int32_t head_map(CUtensorMap *map, const void *base, int64_t tokens, int32_t H, int32_t D, int box_rows = kTile) {
  return make_tensor_map_2d(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, base, (uint64_t)tokens, (uint64_t)H * D,
                            (uint64_t)H * D * 2, 64, (uint32_t)box_rows);
}

}  // namespace
}  // namespace tgb

using namespace tgb;

extern "C" int32_t tgb_varlen_attn_fwd(const void *q, const void *k, const void *v, void *out, void *lse,
                                       const void *tiles, int64_t n_tiles, int64_t tokens, int32_t H, int32_t H_kv,
                                       int32_t D, float scale, int32_t causal, void *error_flag, uint64_t stream) {
  int32_t rc = check_attn(q, k, v, tokens, H, H_kv, D);
  if (rc) return rc;
  if (n_tiles == 0) return TGB_STATUS_OK;
  if (!out || !lse || !tiles || !error_flag) TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "null pointer");
  CUtensorMap map_q, map_k, map_v;
  if ((rc = head_map(&map_q, q, tokens, H, D))) return rc;
  if ((rc = head_map(&map_k, k, tokens, H_kv, D, kKeyBlock))) return rc;
  if ((rc = head_map(&map_v, v, tokens, H_kv, D, kKeyBlock))) return rc;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const unsigned grid = (unsigned)n_tiles;
  const float scale_log2 = scale * kLog2e;
  const int group = H / H_kv;
  if (D == 128) {
    const size_t smem = sizeof(FwdSmem<2>);
    // the attribute belongs to the current device's context, so it is set on every call (cheap)
    TGB_CUDA(cudaFuncSetAttribute(k_attn_fwd<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    k_attn_fwd<2><<<grid, kFwdThreads, smem, st>>>(map_q, map_k, map_v, (const Tile *)tiles, H, group, scale_log2, causal,
                                           (__nv_bfloat16 *)out, (float *)lse, (int *)error_flag);
  } else {
    const size_t smem = sizeof(FwdSmem<1>);
    // the attribute belongs to the current device's context, so it is set on every call (cheap)
    TGB_CUDA(cudaFuncSetAttribute(k_attn_fwd<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    k_attn_fwd<1><<<grid, kFwdThreads, smem, st>>>(map_q, map_k, map_v, (const Tile *)tiles, H, group, scale_log2, causal,
                                           (__nv_bfloat16 *)out, (float *)lse, (int *)error_flag);
  }
  TGB_LAUNCHED();
  return TGB_STATUS_OK;
}

extern "C" int32_t tgb_varlen_attn_bwd(const void *q, const void *k, const void *v, const void *out,
                                       const void *dout, const void *lse, void *dq, void *dk, void *dv,
                                       void *delta, const void *query_tiles, const void *key_tiles,
                                       int64_t n_tiles, int64_t n_key_tiles, int64_t tokens, int32_t H,
                                       int32_t H_kv, int32_t D, float scale, int32_t causal, void *error_flag,
                                       uint64_t stream) {
  int32_t rc = check_attn(q, k, v, tokens, H, H_kv, D);
  if (rc) return rc;
  if (n_tiles == 0) return TGB_STATUS_OK;
  if (!out || !dout || !lse || !dq || !dk || !dv || !delta || !query_tiles || !key_tiles || !error_flag)
    TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "null pointer");
  CUtensorMap map_q, map_k, map_v, map_do;
  if ((rc = head_map(&map_q, q, tokens, H, D))) return rc;
  if ((rc = head_map(&map_k, k, tokens, H_kv, D))) return rc;
  if ((rc = head_map(&map_v, v, tokens, H_kv, D))) return rc;
  if ((rc = head_map(&map_do, dout, tokens, H, D))) return rc;
  CUtensorMap map_k64, map_v64, map_q64, map_do64;
  if ((rc = head_map(&map_k64, k, tokens, H_kv, D, kKeyBlock))) return rc;
  if ((rc = head_map(&map_v64, v, tokens, H_kv, D, kKeyBlock))) return rc;
  if ((rc = head_map(&map_q64, q, tokens, H, D, kQBlock))) return rc;
  if ((rc = head_map(&map_do64, dout, tokens, H, D, kQBlock))) return rc;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int64_t rows = tokens * H;
  k_attn_delta<<<(unsigned)ceil_div(rows * 32, 256), 256, 0, st>>>((const __nv_bfloat16 *)out,
                                                                  (const __nv_bfloat16 *)dout, rows, D,
                                                                  (float *)delta);
  TGB_LAUNCHED();
  const unsigned grid = (unsigned)n_tiles, key_grid = (unsigned)n_key_tiles;
  const int group = H / H_kv;
#define TGB_BWD(HV)                                                                                         \
  {                                                                                                         \
    const size_t smem = sizeof(DkvSmem<HV>) + 1024;                                                         \
    const size_t smem_dq = sizeof(DqSmem<HV>);                                                              \
    /* per-device attribute: set on every call */                                                          \
    TGB_CUDA(cudaFuncSetAttribute(k_attn_bwd_dkv<HV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
    TGB_CUDA(cudaFuncSetAttribute(k_attn_bwd_dq<HV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_dq)); \
    k_attn_bwd_dkv<HV><<<key_grid, kDkvThreads, smem, st>>>(map_q64, map_k, map_v, map_do64, (const Tile *)key_tiles, H, H_kv, scale, \
                                                causal, (const float *)lse, (const float *)delta,           \
                                                (__nv_bfloat16 *)dk, (__nv_bfloat16 *)dv, (int *)error_flag); \
    TGB_LAUNCHED();                                                                                         \
    k_attn_bwd_dq<HV><<<grid, 128, smem_dq, st>>>(map_q, map_k64, map_v64, map_do, (const Tile *)query_tiles, H, group, scale, \
                                               causal, (const float *)lse, (const float *)delta,            \
                                               (__nv_bfloat16 *)dq, (int *)error_flag);                     \
    TGB_LAUNCHED();                                                                                         \
  }
  if (D == 128) TGB_BWD(2) else TGB_BWD(1)
#undef TGB_BWD
  return TGB_STATUS_OK;
}
