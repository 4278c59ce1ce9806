// Tiled TMA (cp.async.bulk.tensor) support for the tile kernels: encoding a 2-D tensor map on the
// host and the device-side load / store wrappers.
//
// The kernels move [rows x 16 or 32 floats] boxes of row-major fp32 matrices (the forward's output,
// the backward's upstream gradient) between global and shared memory with the TMA engine, so the
// transfer costs no load/store-unit wavefronts and arrives in the 64- or 128-byte swizzled layout
// that lets a lane read or write the 16 bytes of its own row without bank conflicts:
//   box row r (64 or 128 bytes), 16-byte chunk q of that row  ->  byte offset
//     64-byte rows :  64 r + 16 (q ^ ((r >> 1) & 3))      (CU_TENSOR_MAP_SWIZZLE_64B)
//     128-byte rows: 128 r + 16 (q ^ (r & 7))             (CU_TENSOR_MAP_SWIZZLE_128B)
// The shared-memory box has to start on a 1024-byte boundary for these formulas to hold.
// No multicast anywhere: every copy is between this GPU's memory and this CTA's shared memory.
#pragma once

#include <cuda.h>

#include "ht_common.cuh"

namespace ht {
namespace tma {

// cuTensorMapEncodeTiled, looked up through the runtime so that the library has no link-time
// dependency on the driver library.  Returns nullptr when the driver does not offer it.
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = []() -> EncodeTiledFn {
    void *p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      return nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

// Tensor map of a row-major fp32 matrix [rows, cols] (row pitch = cols floats) moved in boxes of
// box_rows x box_cols, box_cols = 16 (64-byte swizzle) or 32 (128-byte swizzle).  The base must be
// 16-byte aligned and cols a multiple of 4; rows and cols below 2^31.  Boxes that reach past the
// matrix are clipped by the hardware (stores) or filled with zeros (loads).
inline bool encode_matrix_f32(CUtensorMap *map, const void *base, int64_t rows, int64_t cols, int box_rows, int box_cols) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (fn == nullptr) return false;
  if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0 || (cols & 3) != 0 || rows < 1 || cols < 1) return false;
  if (rows > 0x7fffffff || cols > 0x7fffffff || box_rows < 1 || box_rows > 256) return false;
  if (box_cols != 16 && box_cols != 32) return false;
  const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)cols * 4u};
  const cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
  const cuuint32_t elem[2] = {1u, 1u};
  const CUresult rc = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void *>(base), dims, strides, box, elem,
                         CU_TENSOR_MAP_INTERLEAVE_NONE,
                         box_cols == 16 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B,
                         CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return rc == CUDA_SUCCESS;
}

// Byte offset of 16-byte chunk q of box row r in the swizzled shared-memory box.
template <int BOX_COLS>
__device__ __forceinline__ uint32_t swizzled_offset(uint32_t r, uint32_t q) {
  if (BOX_COLS == 16) return 64u * r + 16u * (q ^ ((r >> 1) & 3u));
  return 128u * r + 16u * (q ^ (r & 7u));
}

#ifdef __CUDACC__
__device__ __forceinline__ uint32_t shared_addr(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

// Makes this thread's earlier shared-memory writes visible to the TMA engine (the async proxy).
__device__ __forceinline__ void fence_async_shared() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// shared -> global, box at (col, row); completion is tracked by the issuing thread's bulk groups.
__device__ __forceinline__ void store_2d(const CUtensorMap *map, uint32_t src, int col, int row) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];" ::"l"(map), "r"(col), "r"(row),
               "r"(src)
               : "memory");
}
__device__ __forceinline__ void commit_group() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Until the issuing thread's earlier stores have finished READING shared memory (the source may be reused).
__device__ __forceinline__ void wait_stores_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }

// global -> shared, box at (col, row); completes on the mbarrier with the box's byte count.
__device__ __forceinline__ void load_2d(uint32_t dst, const CUtensorMap *map, int col, int row, uint64_t *bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cta.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
      "l"(map), "r"(col), "r"(row), "r"(shared_addr(bar))
      : "memory");
}

__device__ __forceinline__ void prefetch_map(const CUtensorMap *map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}
#endif

}  // namespace tma
}  // namespace ht
