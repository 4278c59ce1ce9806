// Per-evaluation records: the arrays through which the tile kernels of the forest backward hand their
// results to the reductions, and through which a forward that saves its traversal hands it to the backward.
#pragma once

#include <type_traits>

#include "ht_common.cuh"

namespace ht {

// Three arrays, each laid out [sample block of 256][tree][256] so that a sample-stationary kernel streams
// each sample block's records sequentially and a tree-stationary one reads contiguous runs.  `where` packs the
// deciding vertex (1-based) and the reference leaf key — 8 + 8 bits for depths up to 8, 16 + 16 bits beyond.
// The two float arrays hold
//   * after the backward's traversal kernel: `dx` = sign * w * g (the x-gradient term; the threshold term is
//     -dx) and `dw` = |margin| * g (the leaf-weight term);
//   * after a forward that saves its traversal: `dx` = threshold - feature at the deciding vertex (the negated
//     signed margin); the backward then fills `dw` with the upstream gradient in this layout.
// The reductions move 10 or 12 bytes per evaluation through HBM and are bound by it, so every byte saved here
// is time saved there.
struct EvalRecords {
  float *dx;
  float *dw;
  void *where;
};

constexpr int kRecordBlock = 256;

__host__ __device__ inline int64_t record_index(int64_t sample, int64_t tree, int64_t trees) {
  return ((sample / kRecordBlock) * trees + tree) * kRecordBlock + (sample % kRecordBlock);
}

inline size_t record_array_bytes(const ht_forest_problem *p, size_t element) {
  const int64_t blocks = (p->B * p->K + kRecordBlock - 1) / kRecordBlock;
  return align_up((size_t)(blocks * kRecordBlock * p->T) * element, 256);
}
inline size_t where_bytes(int depth) { return depth <= 8 ? 2 : 4; }

// The three arrays inside one scratch area of backward_records_bytes() bytes.
inline EvalRecords eval_record_arrays(const ht_forest_problem *p, void *area) {
  const size_t floats = record_array_bytes(p, 4);
  unsigned char *base = static_cast<unsigned char *>(area);
  return EvalRecords{reinterpret_cast<float *>(base), reinterpret_cast<float *>(base + floats), base + 2 * floats};
}

// `where` as the kernels use it: vertex in the low 16 bits, leaf key in the high 16.
template <typename WT>
__device__ __forceinline__ void store_where(void *base, int64_t at, uint32_t vertex, uint32_t key) {
  if (sizeof(WT) == 2)
    __stcs(static_cast<unsigned short *>(base) + at, (unsigned short)(vertex | (key << 8)));
  else
    __stcs(static_cast<uint32_t *>(base) + at, vertex | (key << 16));
}
// Streaming loads as volatile statements: the compiler keeps a batch of them together at the point
// where the prefetch was written instead of sinking each load to its first use.
__device__ __forceinline__ float stream_f32(const float *p) {
  float v;
  asm volatile("ld.global.cs.f32 %0, [%1];" : "=f"(v) : "l"(p));
  return v;
}
template <typename WT>
__device__ __forceinline__ uint32_t stream_raw_where(const void *base, int64_t at) {
  uint32_t v;
  if (sizeof(WT) == 2)
    asm volatile("ld.global.cs.u16 %0, [%1];" : "=r"(v) : "l"(static_cast<const unsigned short *>(base) + at));
  else
    asm volatile("ld.global.cs.u32 %0, [%1];" : "=r"(v) : "l"(static_cast<const uint32_t *>(base) + at));
  return v;
}
// The same with a compile-time byte offset from a base pointer, which ends up in the instruction's immediate field
// (a volatile statement that is handed a computed address costs two integer instructions per load to form it).
template <int BYTES>
__device__ __forceinline__ float stream_f32_at(const float *base) {
  float v;
  asm volatile("ld.global.cs.f32 %0, [%1+%2];" : "=f"(v) : "l"(base), "n"(BYTES));
  return v;
}
template <typename WT, int ELEMENTS>
__device__ __forceinline__ uint32_t stream_raw_where_at(const WT *base) {
  uint32_t v;
  if (sizeof(WT) == 2)
    asm volatile("ld.global.cs.u16 %0, [%1+%2];" : "=r"(v) : "l"(base), "n"(ELEMENTS * 2));
  else
    asm volatile("ld.global.cs.u32 %0, [%1+%2];" : "=r"(v) : "l"(base), "n"(ELEMENTS * 4));
  return v;
}
template <typename WT>
__device__ __forceinline__ uint32_t unpack_where(uint32_t raw) {
  return sizeof(WT) == 2 ? (raw & 0xffu) | ((raw >> 8) << 16) : raw;
}
template <typename WT>
__device__ __forceinline__ uint32_t load_where(const void *base, int64_t at) {
  return unpack_where<WT>(stream_raw_where<WT>(base, at));
}

}  // namespace ht
