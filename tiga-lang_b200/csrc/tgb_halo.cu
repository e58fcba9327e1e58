// Row movers of the halo exchange.
//   tgb_rows_gather       packed[i, :]  = rows[ids[i], :]     (pack the rows a peer asked for)
//   tgb_rows_scatter_add  rows[ids[i], :] += packed[i, :]     (add the cotangents a peer sent back)
// They replace the reference's pack / unpack / segment-sum steps of the device halo path
// (python/tiga/distributed/transport.py:1060-1133 pack and per-run copies, :446-574
// reverse_halo_device).  The ids of one call are unique (a peer asks for / returns each row
// once), so the add is a plain read-modify-write: no atomics, deterministic.
// HBM bound: F*4 bytes read + written (gather), read + read + written (scatter-add) per row.
#include <cstring>

#include "tgb_common.cuh"

namespace tgb {
namespace {

constexpr int kBlock = 256;

constexpr int kLanes = 8;    // lanes per row on the vector path: four rows per warp
constexpr int kInFlight = 4; // float4 per lane and pass: 8 x 4 x 16 = 512 bytes of a row per pass

template <bool ADD>
__global__ void __launch_bounds__(kBlock)
k_move_rows(float *__restrict__ rows, const int64_t *__restrict__ ids, float *__restrict__ packed, int64_t n,
            int64_t F) {
  const bool vec = (F & 3) == 0 && ((((uintptr_t)rows | (uintptr_t)packed) & 15u) == 0);
  if (vec) {
    // eight lanes per row, every lane keeps four 128-bit accesses in flight
    const int lane = threadIdx.x & (kLanes - 1);
    const int64_t i = ((int64_t)blockIdx.x * kBlock + threadIdx.x) / kLanes;
    if (i >= n) return;
    float *row = rows + ids[i] * F;
    float *pack = packed + i * F;
    for (int64_t f0 = 0; f0 < F; f0 += 4 * kLanes * kInFlight) {
      float4 a[kInFlight], b[kInFlight];
#pragma unroll
      for (int q = 0; q < kInFlight; ++q) {
        const int64_t f = f0 + 4 * (lane + kLanes * q);
        if (f < F) {
          a[q] = *reinterpret_cast<const float4 *>(row + f);
          if (ADD) b[q] = __ldcs(reinterpret_cast<const float4 *>(pack + f));
        }
      }
#pragma unroll
      for (int q = 0; q < kInFlight; ++q) {
        const int64_t f = f0 + 4 * (lane + kLanes * q);
        if (f < F) {
          if (ADD) {
            a[q].x += b[q].x; a[q].y += b[q].y; a[q].z += b[q].z; a[q].w += b[q].w;
            *reinterpret_cast<float4 *>(row + f) = a[q];
          } else {
            __stcs(reinterpret_cast<float4 *>(pack + f), a[q]);
          }
        }
      }
    }
  } else {
    // any width or alignment: the same eight lanes stride over the row's elements
    const int lane = threadIdx.x & (kLanes - 1);
    const int64_t i = ((int64_t)blockIdx.x * kBlock + threadIdx.x) / kLanes;
    if (i >= n) return;
    float *row = rows + ids[i] * F;
    float *pack = packed + i * F;
    for (int64_t f = lane; f < F; f += kLanes) {
      if (ADD) row[f] += pack[f];
      else pack[f] = row[f];
    }
  }
}

int32_t move_rows(bool add, void *rows, const void *ids, void *packed, int64_t n, int64_t F, uint64_t stream) {
  if (n < 0 || F <= 0) TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "invalid row count or width");
  if (n == 0) return TGB_STATUS_OK;
  if (!rows || !ids || !packed) TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "null pointer");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const unsigned blocks = (unsigned)ceil_div(n * kLanes, kBlock);
  if (add)
    k_move_rows<true><<<blocks, kBlock, 0, st>>>((float *)rows, (const int64_t *)ids, (float *)packed, n, F);
  else
    k_move_rows<false><<<blocks, kBlock, 0, st>>>((float *)rows, (const int64_t *)ids, (float *)packed, n, F);
  TGB_LAUNCHED();
  return TGB_STATUS_OK;
}

}  // namespace
}  // namespace tgb

extern "C" int32_t tgb_rows_gather(const void *rows, const void *ids, void *packed, int64_t n, int64_t F,
                                   uint64_t stream) {
  return tgb::move_rows(false, const_cast<void *>(rows), ids, packed, n, F, stream);
}

extern "C" int32_t tgb_rows_scatter_add(void *rows, const void *ids, const void *packed, int64_t n, int64_t F,
                                        uint64_t stream) {
  return tgb::move_rows(true, rows, ids, const_cast<void *>(packed), n, F, stream);
}

// ---------------------------------------------------------------------------
// Peer windows: device memory of another process on the same node, mapped into this process so that
// the row movers above (and plain copies) can store straight into a peer's halo buffer over NVLink.
// Legacy CUDA IPC only (no multicast object is ever created).  The reference moves halo rows through
// its transport's send / recv (python/tiga/distributed/nccl.py:256-284); a window replaces the pack
// buffer + send + receive of one direction by stores into the receiver's own buffer.
// ---------------------------------------------------------------------------
#include <cuda.h>

namespace {

typedef CUresult (*AddressRangeFn)(CUdeviceptr *, size_t *, CUdeviceptr);

int32_t allocation_base(const void *ptr, uint64_t *base) {
  static AddressRangeFn fn = nullptr;
  if (!fn) {
    void *entry = nullptr;
    cudaDriverEntryPointQueryResult query;
    cudaError_t err = cudaGetDriverEntryPoint("cuMemGetAddressRange", &entry, cudaEnableDefault, &query);
    if (err != cudaSuccess || query != cudaDriverEntryPointSuccess || !entry)
      TGB_FAIL(TGB_STATUS_INTERNAL, "cuMemGetAddressRange is not available from the driver");
    fn = reinterpret_cast<AddressRangeFn>(entry);
  }
  CUdeviceptr start = 0;
  size_t size = 0;
  const CUresult rc = fn(&start, &size, reinterpret_cast<CUdeviceptr>(ptr));
  if (rc != CUDA_SUCCESS) TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "not a device allocation (driver code %d)", (int)rc);
  *base = static_cast<uint64_t>(start);
  return TGB_STATUS_OK;
}

}  // namespace

extern "C" int32_t tgb_peer_export(const void *ptr, void *handle64, uint64_t *offset) {
  if (!ptr || !handle64 || !offset) TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "null pointer");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handles are 64 bytes");
  uint64_t base = 0;
  const int32_t rc = allocation_base(ptr, &base);
  if (rc) return rc;
  cudaIpcMemHandle_t handle;
  TGB_CUDA(cudaIpcGetMemHandle(&handle, reinterpret_cast<void *>(base)));
  memcpy(handle64, &handle, 64);
  *offset = reinterpret_cast<uint64_t>(ptr) - base;
  return TGB_STATUS_OK;
}

extern "C" int32_t tgb_peer_open(const void *handle64, uint64_t *mapped_base) {
  if (!handle64 || !mapped_base) TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "null pointer");
  cudaIpcMemHandle_t handle;
  memcpy(&handle, handle64, 64);
  void *mapped = nullptr;
  TGB_CUDA(cudaIpcOpenMemHandle(&mapped, handle, cudaIpcMemLazyEnablePeerAccess));
  *mapped_base = reinterpret_cast<uint64_t>(mapped);
  return TGB_STATUS_OK;
}

extern "C" int32_t tgb_peer_close(uint64_t mapped_base) {
  if (!mapped_base) return TGB_STATUS_OK;
  TGB_CUDA(cudaIpcCloseMemHandle(reinterpret_cast<void *>(mapped_base)));
  return TGB_STATUS_OK;
}

extern "C" int32_t tgb_peer_copy(uint64_t dst, const void *src, uint64_t bytes, uint64_t stream) {
  if (bytes == 0) return TGB_STATUS_OK;
  if (!dst || !src) TGB_FAIL(TGB_STATUS_INVALID_ARGUMENT, "null pointer");
  TGB_CUDA(cudaMemcpyAsync(reinterpret_cast<void *>(dst), src, bytes, cudaMemcpyDeviceToDevice,
                           reinterpret_cast<cudaStream_t>(stream)));
  return TGB_STATUS_OK;
}
