// Dense float32 linear  out[M, N] = a[M, K] @ b_t[N, K]^T  on the 5th-generation
// tensor cores (tcgen05.mma kind::tf32, accumulators in tensor memory) with an
// error-compensated 3xTF32 split, so results stay within float32 tolerance:
//   a = a_hi + a_lo (a_hi = a rounded to tf32), same for b,
//   a*b ~= a_hi*b_hi + a_lo*b_hi + a_hi*b_lo      (dropped term <= 2^-22 |a||b|).
// This is the GCN layer's dense linear (the reference leaves it to user Torch
// code after the kernel; its own f16-only tt.dot GEMM is
// lib/Target/Triton/Translate.cpp:6306-6322).
//
// One persistent CTA per SM.  b_t (N x K, at most 128 x 128) is loaded once,
// split into hi/lo and kept in shared memory.  Tiles of 128 rows of `a` stream
// through a two-stage ring: TMA loads a [128 x 32] float chunk (128-byte rows,
// 128-byte swizzle), the CTA splits it into hi/lo in shared memory, one thread
// issues 12 MMAs (M=128, N, K=8) per chunk, and after the last chunk the four
// warps read the accumulator from tensor memory and store their rows.
// Tensor-core bound in flops but HBM bound in practice: 2*M*K*4 bytes per call.
#include <cstdlib>

#include "tgb_common.cuh"
#include "tgb_tcgen05.cuh"

namespace tgb {

int32_t make_tensor_map_2d(CUtensorMap *map, CUtensorMapDataType dtype, uint32_t elem_bytes, const void *base,
                           uint64_t rows, uint64_t cols, uint64_t pitch_bytes, uint32_t box_cols,
                           uint32_t box_rows, bool swizzle_base32) {
  static EncodeTiledFn encode = nullptr;
  if (!encode) {
    void *fn = nullptr;
    cudaDriverEntryPointQueryResult query;
    cudaError_t err = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &query);
    if (err != cudaSuccess || query != cudaDriverEntryPointSuccess || !fn)
      TGB_FAIL(TGB_STATUS_INTERNAL, "cuTensorMapEncodeTiled is not available from the driver");
    encode = reinterpret_cast<EncodeTiledFn>(fn);
  }
  // The encoder is a driver call and needs the primary context bound to this
  // thread; a thread that has made no runtime call yet (an autograd worker) has none.
  TGB_CUDA(cudaFree(nullptr));
  if (((uintptr_t)base & 15u) || (pitch_bytes & 15u) || box_cols * elem_bytes != 128)
    TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "tensor map needs a 16-byte aligned base and pitch and a 128-byte box row");
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {pitch_bytes};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t elem_strides[2] = {1, 1};
  CUresult rc = encode(map, dtype, 2, const_cast<void *>(base), dims, strides, box, elem_strides,
                       CU_TENSOR_MAP_INTERLEAVE_NONE,
                       swizzle_base32 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
                       CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                       CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (rc != CUDA_SUCCESS) TGB_FAIL(TGB_STATUS_INTERNAL, "cuTensorMapEncodeTiled failed with code %d", (int)rc);
  return TGB_STATUS_OK;
}

namespace {

using namespace sm100;

constexpr int kTileM = 128;
constexpr int kChunkK = 32;                       // floats per 128-byte row
constexpr int kChunkBytes = kTileM * 128;         // [128 rows x 128 bytes]
constexpr int kMaxChunks = 4;                     // K <= 128

struct LinearSmem {
  alignas(1024) uint8_t b_hi[kMaxChunks][kChunkBytes];
  alignas(1024) uint8_t b_lo[kMaxChunks][kChunkBytes];
  alignas(1024) uint8_t a_hi[2][kChunkBytes];
  alignas(1024) uint8_t a_lo[2][kChunkBytes];
  uint64_t full[2];       // TMA chunk landed
  uint64_t mma_done[2];   // MMAs that read ring slot s have finished
  uint64_t acc_done;      // accumulator of the current tile is complete
  uint64_t b_full;
  uint32_t tmem_base;
  int abort_flag;
};

// hi = x rounded to tf32 (low 13 mantissa bits zero), lo = x - hi (exact)
__device__ __forceinline__ void split_tf32(float x, float &hi, float &lo) {
  uint32_t h;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(h) : "f"(x));
  hi = __uint_as_float(h);
  lo = x - hi;
}

// Element-wise split of one [rows x 128 B] chunk; the swizzle only permutes
// 16-byte units, so the same unit index is used for the hi and the lo copy.
__device__ __forceinline__ void split_chunk(uint8_t *hi_inplace, uint8_t *lo_out, int bytes, int tid, int threads) {
  float4 *hi = reinterpret_cast<float4 *>(hi_inplace);
  float4 *lo = reinterpret_cast<float4 *>(lo_out);
  for (int i = tid; i < bytes / 16; i += threads) {
    float4 v = hi[i], h, l;
    split_tf32(v.x, h.x, l.x);
    split_tf32(v.y, h.y, l.y);
    split_tf32(v.z, h.z, l.z);
    split_tf32(v.w, h.w, l.w);
    hi[i] = h;
    lo[i] = l;
  }
}

template <int N>
__global__ void __launch_bounds__(128, 1)
k_linear_3xtf32(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                float *__restrict__ out, int64_t M, int k_chunks, int *error) {
  extern __shared__ uint8_t smem_raw[];
  LinearSmem &sm = *reinterpret_cast<LinearSmem *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int b_bytes = N * 128;                       // one chunk of b_t: [N rows x 128 B]
  if (tid == 0) {
    sm.abort_flag = 0;
    mbar_init(&sm.full[0], 1);
    mbar_init(&sm.full[1], 1);
    mbar_init(&sm.mma_done[0], 1);
    mbar_init(&sm.mma_done[1], 1);
    mbar_init(&sm.acc_done, 1);
    mbar_init(&sm.b_full, 1);
    mbar_fence_init();
    tma_prefetch_descriptor(&map_a);
    tma_prefetch_descriptor(&map_b);
  }
  __syncthreads();
  if (warp == 0) tmem_alloc(&sm.tmem_base, N);       // N float32 columns x 128 lanes
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = sm.tmem_base;
  volatile int *abort_flag = &sm.abort_flag;

  const int64_t n_tiles = (M + kTileM - 1) / kTileM;
  const int64_t my_tiles = blockIdx.x < n_tiles ? (n_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
  const int64_t total_chunks = my_tiles * k_chunks;

  // b_t: load every chunk, split once
  if (tid == 0) {
    mbar_arrive_expect_tx(&sm.b_full, (uint32_t)(b_bytes * k_chunks));
    for (int kc = 0; kc < k_chunks; ++kc) tma_load_2d(sm.b_hi[kc], &map_b, kc * kChunkK, 0, &sm.b_full);
    if (total_chunks > 0) {   // first chunk of the first tile
      mbar_arrive_expect_tx(&sm.full[0], kChunkBytes);
      tma_load_2d(sm.a_hi[0], &map_a, 0, (int32_t)(blockIdx.x * kTileM), &sm.full[0]);
    }
  }
  mbar_wait(&sm.b_full, 0, abort_flag, error, 1);
  for (int kc = 0; kc < k_chunks; ++kc) split_chunk(sm.b_hi[kc], sm.b_lo[kc], b_bytes, tid, 128);
  fence_proxy_async_smem();
  __syncthreads();

  constexpr uint32_t idesc = instr_desc(kFmtTF32, kFmtTF32, kTileM, N, 0, 0);
  int64_t it = 0;
  for (int64_t t = 0; t < my_tiles; ++t) {
    const int64_t row0 = (blockIdx.x + t * gridDim.x) * kTileM;
    for (int kc = 0; kc < k_chunks; ++kc, ++it) {
      const int s = (int)(it & 1);
      const uint32_t use = (uint32_t)(it >> 1);
      if (tid == 0 && it + 1 < total_chunks) {        // prefetch the next chunk into the other slot
        const int64_t nx = it + 1;
        const int s1 = (int)(nx & 1);
        const uint32_t use1 = (uint32_t)(nx >> 1);
        if (use1 >= 1) mbar_wait(&sm.mma_done[s1], (use1 - 1) & 1, abort_flag, error, 2);
        const int kc1 = (int)(nx % k_chunks);
        const int64_t row1 = (blockIdx.x + (nx / k_chunks) * gridDim.x) * kTileM;
        mbar_arrive_expect_tx(&sm.full[s1], kChunkBytes);
        tma_load_2d(sm.a_hi[s1], &map_a, kc1 * kChunkK, (int32_t)row1, &sm.full[s1]);
      }
      mbar_wait(&sm.full[s], use & 1, abort_flag, error, 3);
      split_chunk(sm.a_hi[s], sm.a_lo[s], kChunkBytes, tid, 128);
      fence_proxy_async_smem();
      __syncthreads();
      if (tid == 0) {
        tc_fence_after_sync();
        const uint32_t a_hi = smem_u32(sm.a_hi[s]), a_lo = smem_u32(sm.a_lo[s]);
        const uint32_t b_hi = smem_u32(sm.b_hi[kc]), b_lo = smem_u32(sm.b_lo[kc]);
#pragma unroll
        for (int k = 0; k < kChunkK / 8; ++k) {       // K = 8 per MMA: 32 bytes along the row
          const uint32_t off = k * 32;
          const uint64_t ah = smem_desc_k_major_sw128(a_hi + off), al = smem_desc_k_major_sw128(a_lo + off);
          const uint64_t bh = smem_desc_k_major_sw128(b_hi + off), bl = smem_desc_k_major_sw128(b_lo + off);
          mma_tf32(tmem, al, bh, idesc, (kc | k) != 0);   // small terms first
          mma_tf32(tmem, ah, bl, idesc, 1);
          mma_tf32(tmem, ah, bh, idesc, 1);
        }
        mma_commit(&sm.mma_done[s]);
        if (kc == k_chunks - 1) mma_commit(&sm.acc_done);
      }
    }
    // epilogue: every warp reads its 32 lanes (rows) of the accumulator
    mbar_wait(&sm.acc_done, (uint32_t)(t & 1), abort_flag, error, 4);
    tc_fence_after_sync();
    const int64_t row = row0 + warp * 32 + lane;
#pragma unroll 1
    for (int c0 = 0; c0 < N; c0 += 32) {
      uint32_t r[32];
      tmem_ld_32x32(tmem + ((uint32_t)(warp * 32) << 16) + c0, r);
      tmem_ld_wait();
      if (row < M && !*abort_flag) {
        float4 *dst = reinterpret_cast<float4 *>(out + row * N + c0);
#pragma unroll
        for (int q = 0; q < 8; ++q)
          dst[q] = make_float4(__uint_as_float(r[4 * q]), __uint_as_float(r[4 * q + 1]),
                               __uint_as_float(r[4 * q + 2]), __uint_as_float(r[4 * q + 3]));
      }
    }
    tc_fence_before_sync();
    __syncthreads();     // the next tile's first MMA overwrites the accumulator
  }
  // teardown: drain the ring so no TMA or MMA is in flight, then free tensor memory
  if (tid == 0 && total_chunks > 0) {
    const int64_t last = total_chunks - 1;
    mbar_wait(&sm.mma_done[last & 1], (uint32_t)((last >> 1) & 1), abort_flag, error, 5);
    if (total_chunks > 1) mbar_wait(&sm.mma_done[(last - 1) & 1], (uint32_t)(((last - 1) >> 1) & 1), abort_flag, error, 6);
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, N);
}


// ---------------------------------------------------------------------------
// N = 128: the same product with the operand roles swapped, out^T = b_t a^T.
// The resident matrix b_t (hi and lo parts, 2 x 128 columns) lives in tensor
// memory as the A operand of the MMA, so shared memory holds nothing but the
// streamed rows of `a`: a ring of six TMA slots (96 KB in flight per SM) and
// three hi/lo operand slots.  One thread of a warp of its own refills the ring
// and issues the MMAs: issuing stalls while the tensor pipe is busy, and a
// thread that also splits would hold the other split threads at their barrier
// (measured: 365 us with a shared thread, 253 us with the dedicated one).  The accumulator is the transposed tile (lane =
// output feature, column = row of the tile), which makes the epilogue's
// stores full 128-byte lines: 32 lanes write 32 consecutive features of a row.
// Tensor memory: b_t hi [0,128), lo [128,256), two accumulators [256,512).
// ---------------------------------------------------------------------------
constexpr int kWtRing = 6;
constexpr int kWtOps = 3;         // hi/lo operand slots
constexpr int kWtThreads = 288;   // warps 0-3: split; warps 4-7: epilogue; warp 8: TMA + MMA issue

struct LinearWtSmem {
  alignas(1024) uint8_t raw[kWtRing][kChunkBytes];   // TMA destination ring
  alignas(1024) uint8_t a_hi[kWtOps][kChunkBytes];
  alignas(1024) uint8_t a_lo[kWtOps][kChunkBytes];
  uint64_t raw_full[kWtRing];   // TMA chunk landed in raw[r]
  uint64_t op_full[kWtOps];     // operand slot s holds the split chunk (and its TMA slot has been read)
  uint64_t mma_done[kWtOps];    // MMAs that read operand slot s have finished
  uint64_t acc_full[2];         // accumulator b of a tile is complete
  uint64_t acc_empty[2];        // the epilogue warps have read accumulator b
  uint32_t tmem_base;
  int abort_flag;
};

// Same split from a separate source buffer (the TMA ring) into an operand slot.
__device__ __forceinline__ void split_chunk_from(const uint8_t *raw, uint8_t *hi_out, uint8_t *lo_out, int bytes,
                                                 int tid, int threads) {
  const float4 *src = reinterpret_cast<const float4 *>(raw);
  float4 *hi = reinterpret_cast<float4 *>(hi_out);
  float4 *lo = reinterpret_cast<float4 *>(lo_out);
#pragma unroll 4
  for (int i = tid; i < bytes / 16; i += threads) {
    float4 v = src[i], h, l;
    split_tf32(v.x, h.x, l.x);
    split_tf32(v.y, h.y, l.y);
    split_tf32(v.z, h.z, l.z);
    split_tf32(v.w, h.w, l.w);
    hi[i] = h;
    lo[i] = l;
  }
}

// Bounded wait used only while tearing down: it ignores the abort flag (copies
// or MMAs still in flight must land before shared and tensor memory go away)
// and records nothing.
__device__ __forceinline__ void mbar_wait_teardown(uint64_t *bar, uint32_t parity) {
  for (uint32_t spin = 0; spin < kSpinLimit; ++spin)
    if (mbar_try_wait(bar, parity)) return;
}

__global__ void __launch_bounds__(kWtThreads, 1)
k_linear_wt_3xtf32(const __grid_constant__ CUtensorMap map_a, const float *__restrict__ b_t,
                   float *__restrict__ out, int64_t M, int k_chunks, int n_out, int pair, int *error) {
  // The accumulator always has 128 feature rows (the M of the MMA).  With n_out = 64 output
  // features the upper 64 rows of the resident matrix are zero and are never stored: the kernel is
  // bound by the rows of `a` it streams, not by MMA work.
  // pair (n_out = 64, K = 64): one accumulator serves TWO row tiles.  The resident matrix is the
  // block-diagonal [b_t 0; 0 b_t] (128 x 2K) and the streamed operand stacks the chunks of rows
  // [r, r + 128) on those of rows [r + 128, r + 256) along K, so accumulator rows 0..63 hold the
  // features of the first tile and rows 64..127 those of the second: 256 rows per accumulator at the
  // chunk and MMA count of a 128 x 128 tile, all epilogue lanes storing.
  constexpr int N = 128;
  const int tile_chunks = pair ? 2 * k_chunks : k_chunks;      // chunks feeding one accumulator
  const int tile_rows = pair ? 2 * kTileM : kTileM;            // rows of `a` behind one accumulator
  extern __shared__ uint8_t smem_raw[];
  LinearWtSmem &sm =
      *reinterpret_cast<LinearWtSmem *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    sm.abort_flag = 0;
    for (int i = 0; i < kWtRing; ++i) mbar_init(&sm.raw_full[i], 1);
    for (int i = 0; i < kWtOps; ++i) {
      mbar_init(&sm.op_full[i], 4);      // one arrival per split warp
      mbar_init(&sm.mma_done[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&sm.acc_full[i], 1);
      mbar_init(&sm.acc_empty[i], 4);    // one arrival per epilogue warp
    }
    mbar_fence_init();
    tma_prefetch_descriptor(&map_a);
  }
  __syncthreads();
  if (warp == 0) tmem_alloc(&sm.tmem_base, 512);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = sm.tmem_base;
  const uint32_t w_hi = tmem, w_lo = tmem + 128, acc0 = tmem + 256;
  volatile int *abort_flag = &sm.abort_flag;

  const int64_t n_tiles = (M + tile_rows - 1) / tile_rows;
  const int64_t my_tiles = blockIdx.x < n_tiles ? (n_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
  const int64_t total_chunks = my_tiles * tile_chunks;
  auto load_chunk = [&](int64_t chunk) {             // thread 0 only
    const int r = (int)(chunk % kWtRing);
    const int kc = (int)(chunk % tile_chunks);
    // second half of a pair: the same columns, 128 rows further down (rows past M read as zero)
    const int64_t row = (blockIdx.x + (chunk / tile_chunks) * gridDim.x) * tile_rows + (kc / k_chunks) * kTileM;
    mbar_arrive_expect_tx(&sm.raw_full[r], kChunkBytes);
    tma_load_2d(sm.raw[r], &map_a, (kc % k_chunks) * kChunkK, (int32_t)row, &sm.raw_full[r]);
  };
  if (tid == 0)
    for (int64_t c = 0; c < kWtRing && c < total_chunks; ++c) load_chunk(c);

  if (warp < 4) {
    // b_t row `tid` (an output feature) -> hi/lo -> this thread's lane of tensor memory
    const int K = k_chunks * kChunkK;
    const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
    // pair: accumulator row `tid` is feature tid % 64 of tile half tid / 64, fed by that half's chunks only
    const int feature = pair ? (tid & 63) : tid;
#pragma unroll 1
    for (int kc = 0; kc < tile_chunks; ++kc) {
      uint32_t hi[32], lo[32];
      const bool fed = feature < n_out && (!pair || kc / k_chunks == tid / 64);
      const float4 *src = reinterpret_cast<const float4 *>(b_t + (int64_t)(fed ? feature : 0) * K +
                                                           (kc % k_chunks) * kChunkK);
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        const float4 v = fed ? __ldg(src + q) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        float h, l;
        split_tf32(v.x, h, l); hi[4 * q] = __float_as_uint(h); lo[4 * q] = __float_as_uint(l);
        split_tf32(v.y, h, l); hi[4 * q + 1] = __float_as_uint(h); lo[4 * q + 1] = __float_as_uint(l);
        split_tf32(v.z, h, l); hi[4 * q + 2] = __float_as_uint(h); lo[4 * q + 2] = __float_as_uint(l);
        split_tf32(v.w, h, l); hi[4 * q + 3] = __float_as_uint(h); lo[4 * q + 3] = __float_as_uint(l);
      }
      tmem_st_32x32(w_hi + lane_base + kc * kChunkK, hi);
      tmem_st_32x32(w_lo + lane_base + kc * kChunkK, lo);
    }
    tmem_st_wait();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();

  if (warp < 4) {
    // ---- split warps: raw chunk -> hi/lo operand slot --------------------------------------------
    for (int64_t it = 0; it < total_chunks; ++it) {
      const int r = (int)(it % kWtRing);
      const uint32_t use_r = (uint32_t)(it / kWtRing);
      const int s = (int)(it % kWtOps);
      const uint32_t use_s = (uint32_t)(it / kWtOps);
      mbar_wait(&sm.raw_full[r], use_r & 1, abort_flag, error, 3);
      if (use_s >= 1) mbar_wait(&sm.mma_done[s], (use_s - 1) & 1, abort_flag, error, 2);   // operand slot free
      split_chunk_from(sm.raw[r], sm.a_hi[s], sm.a_lo[s], kChunkBytes, tid, 128);
      fence_proxy_async_smem();
      mbar_arrive_warp(&sm.op_full[s]);               // operands written, raw[r] read
    }
  } else if (warp == 8) {
    // ---- issue warp: one thread refills the TMA ring and issues the MMAs; issuing can stall on the
    // tensor pipe, so this thread does nothing else -------------------------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc = instr_desc(kFmtTF32, kFmtTF32, N, kTileM, 0, 0);   // M = features, N = rows of the tile
      int64_t it = 0;
      for (int64_t t = 0; t < my_tiles; ++t) {
        const uint32_t acc = acc0 + (uint32_t)(t & 1) * kTileM;
        for (int kc = 0; kc < tile_chunks; ++kc, ++it) {
          const int s = (int)(it % kWtOps);
          mbar_wait(&sm.op_full[s], (uint32_t)((it / kWtOps) & 1), abort_flag, error, 8);
          if (it + kWtRing < total_chunks) load_chunk(it + kWtRing);   // its slot raw[it % ring] has been read
          if (kc == 0 && t >= 2)                              // the epilogue of tile t-2 has drained this accumulator
            mbar_wait(&sm.acc_empty[t & 1], (uint32_t)(((t >> 1) - 1) & 1), abort_flag, error, 7);
          tc_fence_after_sync();
          const uint32_t a_hi = smem_u32(sm.a_hi[s]), a_lo = smem_u32(sm.a_lo[s]);
#pragma unroll
          for (int k = 0; k < kChunkK / 8; ++k) {       // K = 8 per MMA: 8 columns of b_t, 32 bytes of the row of a
            const uint32_t col = (uint32_t)(kc * kChunkK + k * 8);
            const uint64_t ah = smem_desc_k_major_sw128(a_hi + k * 32), al = smem_desc_k_major_sw128(a_lo + k * 32);
            mma_tf32_a_tmem(acc, w_lo + col, ah, idesc, (kc | k) != 0);   // small terms first
            mma_tf32_a_tmem(acc, w_hi + col, al, idesc, 1);
            mma_tf32_a_tmem(acc, w_hi + col, ah, idesc, 1);
          }
          mma_commit(&sm.mma_done[s]);
          if (kc == tile_chunks - 1) mma_commit(&sm.acc_full[t & 1]);
        }
      }
      // no TMA or MMA may be in flight when shared and tensor memory go away
      if (total_chunks > 0) {
        for (int64_t c = total_chunks - 1; c >= 0 && c > total_chunks - 1 - kWtOps; --c)
          mbar_wait_teardown(&sm.mma_done[c % kWtOps], (uint32_t)((c / kWtOps) & 1));
        // after an abort some chunk may still be on its way into the ring: give it a bounded 2 ms to land
        if (*abort_flag)
          for (int i = 0; i < 2000; ++i) __nanosleep(1000);
      }
    }
  } else {
    // ---- epilogue warps (4-7): lane = output feature, column = row of the tile ------------------------
    const int ew = warp - 4;
    const int n = ew * 32 + lane;
    const uint32_t lane_base = (uint32_t)(ew * 32) << 16;
    for (int64_t t = 0; t < my_tiles; ++t) {
      const int b = (int)(t & 1);
      mbar_wait(&sm.acc_full[b], (uint32_t)((t >> 1) & 1), abort_flag, error, 4);
      tc_fence_after_sync();
      // pair: lanes 64..127 hold the second row tile of the pair
      const int feature = pair ? (n & 63) : n;
      const int64_t row0 = (blockIdx.x + t * gridDim.x) * tile_rows + (pair ? (n >> 6) * kTileM : 0);
      const bool live = !*abort_flag;
#pragma unroll 1
      for (int c0 = 0; c0 < kTileM; c0 += 32) {
        uint32_t r[32];
        tmem_ld_32x32(acc0 + (uint32_t)(b * kTileM) + lane_base + c0, r);
        tmem_ld_wait();
        float *dst = out + (row0 + c0) * n_out + feature;
#pragma unroll
        for (int c = 0; c < 32; ++c)
          if (live && feature < n_out && row0 + c0 + c < M) __stcs(dst + (int64_t)c * n_out, __uint_as_float(r[c]));
      }
      tc_fence_before_sync();
      mbar_arrive_warp(&sm.acc_empty[b]);
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 512);
}

// ---------------------------------------------------------------------------
// Weight gradient  dw[K, N] = a[M, K]^T @ dout[M, N]  (a reduction over the M rows).
// Both operands are used MN-major exactly as TMA delivers them: a tile of 32
// rows is, per block of 32 columns, a [32 rows x 128 bytes] box whose rows are
// the reduction index (32-byte-base swizzle, the layout tf32 needs MN-major).
// Two TMA slots stay in flight while the tile before them is split into one of
// two hi/lo operand slots.  Persistent CTAs stride over the row tiles and keep one
// [K x N] accumulator in tensor memory for all of them (3xTF32 split as above);
// each CTA then writes its partial matrix and a second kernel adds the partials
// in CTA order (deterministic split-K, no atomics).
// ---------------------------------------------------------------------------
constexpr int kDwRows = 32;                        // rows (reduction) per tile
constexpr int kDwBoxBytes = kDwRows * 128;         // one [32 rows x 32 floats] box
constexpr int kDwChunkRowsPerCta = 8192;           // rows one accumulator sees before it is written out

constexpr int kDwSplitWarps = 8;
constexpr int kDwThreads = (kDwSplitWarps + 1) * 32;   // warps 0-7 split, warp 8 issues TMA and MMAs
constexpr int kDwMaxOpSlots = 3;                       // hi/lo operand slots at most
constexpr int kDwMaxRing = 6;                          // TMA slots in flight at most

// Shared-memory plan of the kernel for KR real columns of `a` (64 or 128) and N columns of dout.
// The TMA ring holds only boxes that exist in memory; an operand slot always has four `a` positions
// (the MMA's M is 128), of which the ones beyond KR stay zero for the whole kernel.
template <int KR, int N>
struct DwPlan {
  static constexpr int kARealBoxes = KR / 32, kDBoxes = N / 32;
  static constexpr int kRawBoxes = kARealBoxes + kDBoxes;          // boxes one tile brings in
  static constexpr int kOpBoxes = 4 + kDBoxes;                     // boxes of one hi (or lo) operand slot
  // two operand slots: a third one (the split warps two tiles ahead of the MMAs) measured no faster
  static constexpr int kOpSlots = 2;
  static constexpr int kOperandBytes = 2 * kOpSlots * kOpBoxes * kDwBoxBytes;
  static constexpr int kBudget = 216 * 1024 - kOperandBytes;
  static constexpr int kRingFit = kBudget / (kRawBoxes * kDwBoxBytes);
  static constexpr int kRing = kRingFit > kDwMaxRing ? kDwMaxRing : (kRingFit < 2 ? 2 : kRingFit);
  static constexpr int kRawOffset = 0;
  static constexpr int kHiOffset = kRing * kRawBoxes * kDwBoxBytes;
  static constexpr int kLoOffset = kHiOffset + kOpSlots * kOpBoxes * kDwBoxBytes;
  static constexpr int kBarOffset = kLoOffset + kOpSlots * kOpBoxes * kDwBoxBytes;
  static constexpr int kBytes = kBarOffset + 256;
};

struct DwBarriers {
  uint64_t raw_full[kDwMaxRing];    // tile landed in TMA slot r
  uint64_t op_full[kDwMaxOpSlots];  // operand slot s holds the split tile (and its TMA slot has been read)
  uint64_t mma_done[kDwMaxOpSlots]; // the MMAs that read operand slot s have finished
  uint64_t acc_done;
  uint32_t tmem_base;
  int abort_flag;
};

template <int KR, int N>
__global__ void __launch_bounds__(kDwThreads, 1)
k_linear_dw_3xtf32(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_d,
                   float *__restrict__ partial, int64_t M, int *error) {
  using P = DwPlan<KR, N>;
  constexpr int K = 128;                             // rows of the accumulator = M dimension of the MMA
  constexpr int kRing = P::kRing;
  constexpr int kDwOpSlots = P::kOpSlots;
  extern __shared__ uint8_t smem_raw[];
  uint8_t *base = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t *raw = base + P::kRawOffset;               // [kRing][kRawBoxes][box]
  uint8_t *hi = base + P::kHiOffset;                 // [slots][kOpBoxes][box]: four `a` positions, then dout
  uint8_t *lo = base + P::kLoOffset;
  DwBarriers &sm = *reinterpret_cast<DwBarriers *>(base + P::kBarOffset);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    sm.abort_flag = 0;
    for (int i = 0; i < kRing; ++i) mbar_init(&sm.raw_full[i], 1);
    for (int i = 0; i < kDwOpSlots; ++i) {
      mbar_init(&sm.op_full[i], kDwSplitWarps);   // one arrival per split warp
      mbar_init(&sm.mma_done[i], 1);
    }
    mbar_init(&sm.acc_done, 1);
    mbar_fence_init();
    tma_prefetch_descriptor(&map_a);
    tma_prefetch_descriptor(&map_d);
  }
  if (P::kARealBoxes < 4) {
    // the `a` positions no tile ever fills: zero once, in both parts of both operand slots
    constexpr int kZeroBytes = (4 - P::kARealBoxes) * kDwBoxBytes;
    for (int slot = 0; slot < kDwOpSlots; ++slot) {
      float4 *zh = reinterpret_cast<float4 *>(hi + (slot * P::kOpBoxes + P::kARealBoxes) * kDwBoxBytes);
      float4 *zl = reinterpret_cast<float4 *>(lo + (slot * P::kOpBoxes + P::kARealBoxes) * kDwBoxBytes);
      for (int i = tid; i < kZeroBytes / 16; i += kDwThreads) {
        zh[i] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        zl[i] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
      }
    }
    fence_proxy_async_smem();
  }
  __syncthreads();
  if (warp == 0) tmem_alloc(&sm.tmem_base, N);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = sm.tmem_base;
  volatile int *abort_flag = &sm.abort_flag;

  const int64_t n_tiles = (M + kDwRows - 1) / kDwRows;
  const int64_t my_tiles = blockIdx.x < n_tiles ? (n_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
  auto load_tile = [&](int64_t t) {                   // issue thread only; tile t goes to TMA slot t % kRing
    const int r = (int)(t % kRing);
    const int32_t row0 = (int32_t)((blockIdx.x + t * gridDim.x) * kDwRows);
    uint8_t *slot = raw + (size_t)r * P::kRawBoxes * kDwBoxBytes;
    mbar_arrive_expect_tx(&sm.raw_full[r], P::kRawBoxes * kDwBoxBytes);
#pragma unroll
    for (int j = 0; j < P::kARealBoxes; ++j) tma_load_2d(slot + j * kDwBoxBytes, &map_a, 32 * j, row0, &sm.raw_full[r]);
#pragma unroll
    for (int j = 0; j < P::kDBoxes; ++j)
      tma_load_2d(slot + (P::kARealBoxes + j) * kDwBoxBytes, &map_d, 32 * j, row0, &sm.raw_full[r]);
  };

  if (warp < kDwSplitWarps) {
    // ---- split warps: raw tile -> hi/lo operand slot ------------------------------------------
    for (int64_t t = 0; t < my_tiles; ++t) {
      const int r = (int)(t % kRing);
      const int s = (int)(t % kDwOpSlots);
      const uint32_t use_s = (uint32_t)(t / kDwOpSlots);
      mbar_wait(&sm.raw_full[r], (uint32_t)((t / kRing) & 1), abort_flag, error, 52);
      if (use_s >= 1) mbar_wait(&sm.mma_done[s], (use_s - 1) & 1, abort_flag, error, 51);   // operand slot free
      const uint8_t *src = raw + (size_t)r * P::kRawBoxes * kDwBoxBytes;
      uint8_t *h = hi + (size_t)s * P::kOpBoxes * kDwBoxBytes, *l = lo + (size_t)s * P::kOpBoxes * kDwBoxBytes;
      split_chunk_from(src, h, l, P::kARealBoxes * kDwBoxBytes, tid, kDwSplitWarps * 32);
      split_chunk_from(src + P::kARealBoxes * kDwBoxBytes, h + 4 * kDwBoxBytes, l + 4 * kDwBoxBytes,
                       P::kDBoxes * kDwBoxBytes, tid, kDwSplitWarps * 32);
      fence_proxy_async_smem();
      mbar_arrive_warp(&sm.op_full[s]);               // operands written, the TMA slot read
    }
  } else if (lane == 0) {
    // ---- issue thread: refills the TMA ring and issues the MMAs, nothing else ------------------
    constexpr uint32_t idesc = instr_desc(kFmtTF32, kFmtTF32, K, N, 1, 1);    // both operands MN-major
    for (int64_t t = 0; t < kRing && t < my_tiles; ++t) load_tile(t);
    for (int64_t t = 0; t < my_tiles; ++t) {
      const int s = (int)(t % kDwOpSlots);
      mbar_wait(&sm.op_full[s], (uint32_t)((t / kDwOpSlots) & 1), abort_flag, error, 55);
      if (t + kRing < my_tiles) load_tile(t + kRing);  // every split thread has read TMA slot t % kRing
      tc_fence_after_sync();
      const uint32_t a_hi = smem_u32(hi + (size_t)s * P::kOpBoxes * kDwBoxBytes);
      const uint32_t a_lo = smem_u32(lo + (size_t)s * P::kOpBoxes * kDwBoxBytes);
      const uint32_t d_hi = a_hi + 4 * kDwBoxBytes, d_lo = a_lo + 4 * kDwBoxBytes;
#pragma unroll
      for (int k = 0; k < kDwRows / 8; ++k) {          // 8 reduction rows = one 1024-byte swizzle atom per MMA
        const uint32_t off = k * 1024;
        const uint64_t ah = smem_desc_mn_major_sw128_base32(a_hi + off, kDwBoxBytes);
        const uint64_t al = smem_desc_mn_major_sw128_base32(a_lo + off, kDwBoxBytes);
        const uint64_t dh = smem_desc_mn_major_sw128_base32(d_hi + off, kDwBoxBytes);
        const uint64_t dl = smem_desc_mn_major_sw128_base32(d_lo + off, kDwBoxBytes);
        mma_tf32(tmem, al, dh, idesc, (t | k) != 0);
        mma_tf32(tmem, ah, dl, idesc, 1);
        mma_tf32(tmem, ah, dh, idesc, 1);
      }
      mma_commit(&sm.mma_done[s]);
      if (t == my_tiles - 1) mma_commit(&sm.acc_done);
    }
    if (my_tiles > 1) {                                // the tile before the last: its MMAs must be complete too
      const int64_t prev = my_tiles - 2;
      mbar_wait_teardown(&sm.mma_done[prev % kDwOpSlots], (uint32_t)((prev / kDwOpSlots) & 1));
    }
  }
  // epilogue: warps 0-3 write this CTA's partial matrix (row of dw = column of a = tensor-memory lane)
  float *mine = partial + (int64_t)blockIdx.x * K * N;
  if (warp < 4) {
    if (my_tiles > 0) {
      mbar_wait(&sm.acc_done, 0, abort_flag, error, 53);
      tc_fence_after_sync();
    }
    const int row = warp * 32 + lane;
#pragma unroll 1
    for (int c0 = 0; c0 < N; c0 += 32) {
      uint32_t r[32];
      if (my_tiles > 0) {
        tmem_ld_32x32(tmem + ((uint32_t)(warp * 32) << 16) + c0, r);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int q = 0; q < 32; ++q) r[q] = 0u;
      }
      float4 *dst = reinterpret_cast<float4 *>(mine + (int64_t)row * N + c0);
#pragma unroll
      for (int q = 0; q < 8; ++q)
        dst[q] = make_float4(__uint_as_float(r[4 * q]), __uint_as_float(r[4 * q + 1]), __uint_as_float(r[4 * q + 2]),
                             __uint_as_float(r[4 * q + 3]));
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, N);
}

// Adds the CTAs' partial matrices in CTA order (deterministic).  A partial matrix always has 128
// rows; only the first `elems / N` of them belong to the result.
__global__ void k_sum_dw_partials(const float *__restrict__ partial, int blocks, int elems, int64_t stride,
                                  float *__restrict__ out) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= elems) return;
  float acc = 0.0f;
  for (int b = 0; b < blocks; ++b) acc += partial[(int64_t)b * stride + i];
  out[i] = acc;
}

}  // namespace
}  // namespace tgb

using namespace tgb;

// Self-test of the bounded-wait path every tensor-core kernel relies on: one warp waits, with a
// caller-chosen poll limit, on an mbarrier that nothing ever arrives on.  The wait must give up,
// raise the CTA's abort flag, store its code in the error word, let the following wait fall
// through, and the kernel must return.  Nothing faults and nothing spins without a bound.
namespace tgb {
namespace {
__global__ void k_selftest_bounded_wait(int *error, uint32_t polls, int *fell_through) {
  __shared__ uint64_t never_signalled;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(&never_signalled, 1);
    mbar_fence_init();
  }
  __syncthreads();
  volatile int *flag = &abort_flag;
  if (threadIdx.x == 0) {
    mbar_wait_limited(&never_signalled, 0, flag, error, 99, polls);      // runs out of polls
    mbar_wait_limited(&never_signalled, 0, flag, error, 98, polls);      // must return at once
    *fell_through = *flag;
  }
}
}  // namespace
}  // namespace tgb

extern "C" int32_t tgb_selftest_bounded_wait(void *error_flag, uint32_t polls, void *fell_through,
                                             uint64_t stream) {
  if (!error_flag || !fell_through) TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "null pointer");
  if (polls == 0 || polls > (1u << 20))
    TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "poll limit must be in [1, 2^20]");
  k_selftest_bounded_wait<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>((int *)error_flag, polls,
                                                                               (int *)fell_through);
  TGB_LAUNCHED();
  return TGB_STATUS_OK;
}

// K = N = 64 runs two row tiles per accumulator; TGB_LINEAR_PAIR=0 in the environment selects the
// older kernel (both operands in shared memory), for comparisons.
static bool linear_pair_enabled() {
  static const bool enabled = [] {
    const char *text = getenv("TGB_LINEAR_PAIR");
    return text ? atoi(text) != 0 : true;
  }();
  return enabled;
}

extern "C" int32_t tgb_linear_f32(const void *a, const void *b_t, void *out, int64_t M, int32_t K, int32_t N,
                                  void *error_flag, uint64_t stream) {
  if (M < 0) TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "negative row count");
  if (M == 0) return TGB_STATUS_OK;
  if (!a || !b_t || !out || !error_flag) TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "null pointer");
  if ((N != 64 && N != 128) || K % 32 != 0 || K <= 0 || K > 128)
    TGB_FAIL(TGB_STATUS_UNSUPPORTED, "tensor-core linear supports N in {64, 128} and K in {32, 64, 96, 128} (got K=%d, N=%d)", K, N);
  if (M > (int64_t)INT32_MAX - 256) TGB_FAIL(TGB_STATUS_UNSUPPORTED, "more than 2^31 rows");
  if ((uintptr_t)out & 15u) TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "output must be 16-byte aligned");
  CUtensorMap map_a, map_b;
  int32_t rc = make_tensor_map_2d(&map_a, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, a, (uint64_t)M, (uint64_t)K,
                                  (uint64_t)K * 4, 32, 128);
  if (rc) return rc;
  rc = make_tensor_map_2d(&map_b, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, b_t, (uint64_t)N, (uint64_t)K, (uint64_t)K * 4,
                          32, (uint32_t)N);
  if (rc) return rc;
  int device = 0, sms = 0;
  TGB_CUDA(cudaGetDevice(&device));
  TGB_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
  const int64_t tiles = ceil_div(M, kTileM);
  const unsigned grid = (unsigned)(tiles < sms ? tiles : sms);
  const size_t smem = sizeof(LinearSmem) + 1024;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const bool pair = N == 64 && K == 64 && linear_pair_enabled();
  if ((N == 128 || pair) && ((uintptr_t)b_t & 15u) == 0) {
    // resident matrix in tensor memory, rows of `a` through a six-slot TMA ring.  A tile costs about
    // 5 us whatever its MMA count, so 64 output features with the upper half of the resident matrix
    // zero measured slower than the kernel with both operands in shared memory (4.43 vs 3.65 ms for
    // 2^24 rows, K = 64); K = N = 64 therefore runs PAIRED: two row tiles per accumulator behind a
    // block-diagonal resident matrix, 256 rows at the cost of one tile.
    const size_t smem_wt = sizeof(LinearWtSmem) + 1024;
    const int64_t wt_tiles = ceil_div(M, pair ? 2 * kTileM : kTileM);
    const unsigned wt_grid = (unsigned)(wt_tiles < sms ? wt_tiles : sms);
    // the attribute belongs to the current device's context, so it is set on every call (cheap)
    TGB_CUDA(cudaFuncSetAttribute(k_linear_wt_3xtf32, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_wt));
    k_linear_wt_3xtf32<<<wt_grid, kWtThreads, smem_wt, st>>>(map_a, (const float *)b_t, (float *)out, M, K / 32, N,
                                                            pair ? 1 : 0, (int *)error_flag);
  } else if (N == 128) {
    // the attribute belongs to the current device's context, so it is set on every call (cheap)
    TGB_CUDA(cudaFuncSetAttribute(k_linear_3xtf32<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    k_linear_3xtf32<128><<<grid, 128, smem, st>>>(map_a, map_b, (float *)out, M, K / 32, (int *)error_flag);
  } else {
    // the attribute belongs to the current device's context, so it is set on every call (cheap)
    TGB_CUDA(cudaFuncSetAttribute(k_linear_3xtf32<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    k_linear_3xtf32<64><<<grid, 128, smem, st>>>(map_a, map_b, (float *)out, M, K / 32, (int *)error_flag);
  }
  TGB_LAUNCHED();
  return TGB_STATUS_OK;
}

extern "C" int32_t tgb_linear_dw_f32(const void *a, const void *dout, void *dw, void *partial,
                                     uint64_t partial_bytes, int64_t M, int32_t K, int32_t N, void *error_flag,
                                     uint64_t stream) {
  if (M < 0) TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "negative row count");
  // The MMA always produces a 128-row accumulator.  A narrower `a` (K = 32, 64, 96) is read through a
  // tensor map of its true width: the boxes beyond column K come back zero-filled by the TMA unit
  // (no memory traffic), and only the first K rows of the accumulator are summed into dw.
  if (K <= 0 || K > 128 || K % 32 != 0 || (N != 64 && N != 128))
    TGB_FAIL(TGB_STATUS_UNSUPPORTED, "tensor-core weight gradient supports K in {32, 64, 96, 128} and N in {64, 128} (got K=%d, N=%d)", K, N);
  if (!a || !dout || !dw || !partial || !error_flag) TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "null pointer");
  if (M > (int64_t)INT32_MAX - 256) TGB_FAIL(TGB_STATUS_UNSUPPORTED, "more than 2^31 rows");
  if (M == 0) {
    TGB_CUDA(cudaMemsetAsync(dw, 0, (size_t)K * N * 4, reinterpret_cast<cudaStream_t>(stream)));
    return TGB_STATUS_OK;
  }
  int device = 0, sms = 0;
  TGB_CUDA(cudaGetDevice(&device));
  TGB_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
  // The rows are processed in chunks of at most kDwChunkRowsPerCta rows per CTA, one launch per chunk.
  // A tensor-memory accumulator adds with round-toward-zero, so its error grows with the number of
  // additions times the size of the running sum; bounding the rows one accumulator sees keeps the
  // result within a few tens of float32 ulps of sum |a * dout| however large M is.  Chunk results are
  // added in chunk order (deterministic).
  const int64_t chunk_rows = (int64_t)sms * kDwChunkRowsPerCta;
  const int64_t chunks = ceil_div(M, chunk_rows);
  const int64_t first_tiles = ceil_div(M < chunk_rows ? M : chunk_rows, kDwRows);
  const unsigned max_grid = (unsigned)(first_tiles < sms ? first_tiles : sms);
  const uint64_t need = ((uint64_t)max_grid + (chunks > 1 ? (uint64_t)chunks : 0)) * 128 * N * 4;
  if (partial_bytes < need)
    TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "partial buffer too small: %llu < %llu bytes",
             (unsigned long long)partial_bytes, (unsigned long long)need);
  float *cta_partials = (float *)partial;
  float *chunk_sums = cta_partials + (size_t)max_grid * 128 * N;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  // columns of `a` that exist in memory, in whole 64-column halves of the accumulator's 128 rows
  const int kr = K <= 64 ? 64 : 128;
  // the attribute belongs to the current device's context, so it is set on every call (cheap)
#define TGB_DW_CASE(KR_, N_)                                                                                   \
  if (kr == KR_ && N == N_)                                                                                    \
    TGB_CUDA(cudaFuncSetAttribute(k_linear_dw_3xtf32<KR_, N_>, cudaFuncAttributeMaxDynamicSharedMemorySize,    \
                                  DwPlan<KR_, N_>::kBytes + 1024));
  TGB_DW_CASE(64, 64) TGB_DW_CASE(64, 128) TGB_DW_CASE(128, 64) TGB_DW_CASE(128, 128)
#undef TGB_DW_CASE
  for (int64_t c = 0; c < chunks; ++c) {
    const int64_t row0 = c * chunk_rows;
    const int64_t rows = M - row0 < chunk_rows ? M - row0 : chunk_rows;
    const int64_t tiles = ceil_div(rows, kDwRows);
    const unsigned grid = (unsigned)(tiles < sms ? tiles : sms);
    CUtensorMap map_a, map_d;
    int32_t rc = make_tensor_map_2d(&map_a, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, (const float *)a + row0 * K,
                                    (uint64_t)rows, (uint64_t)K, (uint64_t)K * 4, 32, kDwRows, true);
    if (rc) return rc;
    rc = make_tensor_map_2d(&map_d, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, (const float *)dout + row0 * N,
                            (uint64_t)rows, (uint64_t)N, (uint64_t)N * 4, 32, kDwRows, true);
    if (rc) return rc;
#define TGB_DW_CASE(KR_, N_)                                                                       \
  if (kr == KR_ && N == N_)                                                                        \
    k_linear_dw_3xtf32<KR_, N_><<<grid, kDwThreads, DwPlan<KR_, N_>::kBytes + 1024, st>>>(         \
        map_a, map_d, cta_partials, rows, (int *)error_flag);
    TGB_DW_CASE(64, 64) TGB_DW_CASE(64, 128) TGB_DW_CASE(128, 64) TGB_DW_CASE(128, 128)
#undef TGB_DW_CASE
    TGB_LAUNCHED();
    float *target = chunks > 1 ? chunk_sums + (size_t)c * K * N : (float *)dw;
    k_sum_dw_partials<<<(unsigned)ceil_div((int64_t)K * N, 256), 256, 0, st>>>(cta_partials, (int)grid, K * N,
                                                                              (int64_t)128 * N, target);
    TGB_LAUNCHED();
  }
  if (chunks > 1) {
    k_sum_dw_partials<<<(unsigned)ceil_div((int64_t)K * N, 256), 256, 0, st>>>(chunk_sums, (int)chunks, K * N,
                                                                              (int64_t)K * N, (float *)dw);
    TGB_LAUNCHED();
  }
  return TGB_STATUS_OK;
}

/* number of [128, N] float matrices the `partial` scratch of tgb_linear_dw_f32 must hold for M rows */
extern "C" int32_t tgb_linear_dw_partials(int64_t M, int32_t *count) {
  if (!count) TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "null output");
  int device = 0, sms = 0;
  TGB_CUDA(cudaGetDevice(&device));
  TGB_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
  if (M < 1) M = 1;
  const int64_t chunk_rows = (int64_t)sms * kDwChunkRowsPerCta;
  const int64_t chunks = ceil_div(M, chunk_rows);
  const int64_t tiles = ceil_div(M < chunk_rows ? M : chunk_rows, kDwRows);
  *count = (int32_t)((tiles < sms ? tiles : sms) + (chunks > 1 ? chunks : 0));
  return TGB_STATUS_OK;
}
