// Blackwell (sm_100a) building blocks in inline PTX: mbarrier with bounded
// waits, TMA tiled loads (no multicast anywhere), tensor-memory allocation,
// tcgen05.mma issue / commit / load, and the shared-memory and instruction
// descriptors of the 5th-generation tensor cores.
//
// Every wait is bounded: after kSpinLimit polls the waiter raises the CTA's
// abort flag and records an error code for the host; all later waits return
// at once, control flow stays convergent, tensor memory is released at the
// end of the kernel and the context stays usable.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace tgb {
namespace sm100 {

constexpr uint32_t kSpinLimit = 1u << 24;   // polls of mbarrier.try_wait before giving up

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ---- mbarrier ---------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t *bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// One arrival per warp: every lane has finished its part (and issued whatever
// proxy / tensor-memory fence its writes need) before the warp synchronises,
// then lane 0 arrives for all of them.  A barrier that 128 or 256 threads
// arrive on one by one serialises that many shared-memory atomics per phase.
__device__ __forceinline__ void mbar_arrive_warp(uint64_t *bar) {
  __syncwarp();
  if ((threadIdx.x & 31) == 0) mbar_arrive(bar);
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return done != 0;
}

// Bounded wait.  `abort_flag` lives in shared memory (one per CTA), `error`
// in global memory (one per launch); `code` says which wait gave up.
__device__ __forceinline__ void mbar_wait_limited(uint64_t *bar, uint32_t parity, volatile int *abort_flag,
                                                  int *error, int code, uint32_t limit) {
  if (*abort_flag) return;
  for (uint32_t spin = 0; spin < limit; ++spin) {
    if (mbar_try_wait(bar, parity)) return;
    if ((spin & 1023u) == 1023u && *abort_flag) return;
  }
  *abort_flag = 1;
  atomicCAS(error, 0, code);
}

__device__ __forceinline__ void mbar_wait(uint64_t *bar, uint32_t parity, volatile int *abort_flag,
                                          int *error, int code) {
  mbar_wait_limited(bar, parity, abort_flag, error, code, kSpinLimit);
}

// ---- proxies / fences ---------------------------------------------------------
// generic-proxy writes to shared memory -> visible to the async proxy (TMA, tcgen05.mma)
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// ---- TMA (tiled, 2-D, no multicast) -------------------------------------------
// x is the innermost coordinate in elements; x * element size must be a
// multiple of 16 bytes.
__device__ __forceinline__ void tma_load_2d(void *smem_dst, const CUtensorMap *map, int32_t x, int32_t y,
                                            uint64_t *bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(smem_u32(bar))
      : "memory");
}

__device__ __forceinline__ void tma_prefetch_descriptor(const CUtensorMap *map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

// ---- tensor memory ------------------------------------------------------------
// Executed by one full warp; columns is a power of two in [32, 512].
__device__ __forceinline__ void tmem_alloc(uint32_t *smem_result, uint32_t columns) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
               "r"(columns)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t columns) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(columns) : "memory");
}

// ---- descriptors ----------------------------------------------------------------
// Shared-memory matrix descriptor of a K-major operand tile stored as rows of
// 128 bytes with the 128-byte swizzle (what a TMA box of 128 bytes x rows with
// CU_TENSOR_MAP_SWIZZLE_128B writes): 8-row groups are 1024 bytes apart.
// The tile base must be 1024-byte aligned; advancing along K inside the
// 128-byte row adds the byte offset to the start address.
__device__ __forceinline__ uint64_t smem_desc_k_major_sw128(uint32_t smem_addr) {
  uint64_t desc = 0;
  desc |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);   // start address, 16-byte units
  desc |= (uint64_t)1 << 16;                         // leading byte offset (unused with swizzle)
  desc |= (uint64_t)(1024 >> 4) << 32;               // stride byte offset: next 8-row group
  desc |= (uint64_t)1 << 46;                         // descriptor version of sm_100
  desc |= (uint64_t)2 << 61;                         // SWIZZLE_128B
  return desc;
}

// MN-major operand tile made of 128-byte rows (64 16-bit elements along MN per
// row, consecutive rows = consecutive K), 128-byte swizzle.  `mn_atom_stride`
// is the distance in bytes between two 64-element column blocks.
__device__ __forceinline__ uint64_t smem_desc_mn_major_sw128(uint32_t smem_addr, uint32_t mn_atom_stride) {
  uint64_t desc = 0;
  desc |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
  desc |= (uint64_t)((mn_atom_stride >> 4) & 0x3FFFu) << 16;   // leading byte offset: next MN block
  desc |= (uint64_t)(1024 >> 4) << 32;                         // stride byte offset: next 8 rows of K
  desc |= (uint64_t)1 << 46;
  desc |= (uint64_t)2 << 61;
  return desc;
}

// MN-major operand of 32-bit elements (tf32): the only layout the tensor core
// accepts is the 128-byte swizzle with a 32-byte base -- 128-byte rows (32
// floats along MN, consecutive rows = consecutive K), 32-byte chunks permuted
// inside groups of 4 rows (512 bytes).  It is what TMA writes with
// CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B.
__device__ __forceinline__ uint64_t smem_desc_mn_major_sw128_base32(uint32_t smem_addr, uint32_t mn_atom_stride) {
  uint64_t desc = 0;
  desc |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
  desc |= (uint64_t)((mn_atom_stride >> 4) & 0x3FFFu) << 16;   // leading byte offset: next block of 32 floats
  desc |= (uint64_t)(512 >> 4) << 32;                          // stride byte offset: next 4 rows of K
  desc |= (uint64_t)1 << 46;
  desc |= (uint64_t)1 << 61;                                   // SWIZZLE_128B_BASE32B
  return desc;
}

enum : uint32_t { kFmtF16 = 0, kFmtBF16 = 1, kFmtTF32 = 2 };

// Instruction descriptor of tcgen05.mma kind::f16 / kind::tf32 with float32
// accumulation: D format bits [4,6), A format [7,10), B format [10,13),
// A/B major bits 15/16 (0 = K-major), N>>3 at [17,23), M>>4 at [24,29).
__host__ __device__ constexpr uint32_t instr_desc(uint32_t a_fmt, uint32_t b_fmt, uint32_t m, uint32_t n,
                                                  uint32_t a_mn_major, uint32_t b_mn_major) {
  return (1u << 4) | (a_fmt << 7) | (b_fmt << 10) | (a_mn_major << 15) | (b_mn_major << 16) | ((n >> 3) << 17) |
         ((m >> 4) << 24);
}

// ---- MMA issue (one thread) -------------------------------------------------------
__device__ __forceinline__ void mma_tf32(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                         uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Same with the A operand in tensor memory (row i of A in lane i, one 32-bit
// column per tf32 element along K).
__device__ __forceinline__ void mma_tf32_a_tmem(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                                uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

__device__ __forceinline__ void mma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// The mbarrier gets one arrival when every tcgen05 operation issued so far by
// this thread has completed.
__device__ __forceinline__ void mma_commit(uint64_t *bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}

// ---- TMEM -> registers: warp w of a warpgroup reads lanes 32*(w%4)..+31, one
// lane per thread, 32 consecutive 32-bit columns starting at `taddr`.
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}

__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// registers -> TMEM, same shape as tmem_ld_32x32
__device__ __forceinline__ void tmem_st_32x32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
        "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
        "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}

__device__ __forceinline__ void tmem_st_wait() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

}  // namespace sm100

// ---- host: tensor maps through the driver entry point (no link against libcuda)
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

// 2-D row-major tensor [rows, cols] of `elem_bytes` elements with row pitch
// `pitch_bytes`; box = box_cols x box_rows, 128-byte swizzle (box_cols *
// elem_bytes must be 128).  Returns a TGB status.
int32_t make_tensor_map_2d(CUtensorMap *map, CUtensorMapDataType dtype, uint32_t elem_bytes, const void *base,
                           uint64_t rows, uint64_t cols, uint64_t pitch_bytes, uint32_t box_cols,
                           uint32_t box_rows, bool swizzle_base32 = false);

}  // namespace tgb
