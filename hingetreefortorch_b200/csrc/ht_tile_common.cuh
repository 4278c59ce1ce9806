// Building blocks shared by the shared-memory tile kernels (forward and backward): the per-tree
// record layout and its repack kernel, mbarrier / bulk-copy (TMA engine) wrappers with bounded
// waits, named barriers and explicit shared-memory loads.
#pragma once

#include "ht_common.cuh"

namespace ht {
namespace tile {

constexpr int kThreads = 1024;
constexpr int kWarps = kThreads / 32;
constexpr size_t kSmemBudget = 227 * 1024;
constexpr int kHeadBytes = 16;  // tree records start with {thr(1), thr(2), thr(3), packed ordinals}
// Limits of a wait on the parameter pipeline: one try may sleep in the hardware for up to kTryNanoseconds
// (no issue slots spent meanwhile), and kMaxSpins tries end the wait: far beyond any real copy latency,
// small enough that a lost copy ends the kernel (with a flag) within about two seconds instead of hanging
// the device.
constexpr uint32_t kTryNanoseconds = 4096;
constexpr uint32_t kMaxSpins = 1u << 19;

__host__ __device__ constexpr uint32_t round16(uint32_t v) { return (v + 15u) & ~15u; }

// Into how many CTAs to split the tree groups of one sample tile (each split stages the tile's
// features again, charged here at 6 % of a whole tile's work — 256 tiles of the 1024-tree benchmark
// forest ran 368 us unsplit, 390 us in 2 and 384 us in 4 splits): the count that minimises the
// number of rounds the 148 SMs need, in units of a whole tile's work.  One split when the tiles
// alone fill the machine evenly enough.
inline int choose_splits(int64_t tiles, int64_t max_splits) {
  constexpr int64_t kSMs = 148;
  int best = 1;
  double best_cost = 0.0;
  for (int64_t s = 1; s <= max_splits && s <= 16; ++s) {
    const double rounds = (double)((tiles * s + kSMs - 1) / kSMs);
    const double cost = rounds * (1.0 / (double)s + 0.06);  // a CTA: its share of the walk + staging
    if (s == 1 || cost < best_cost * 0.999) {
      best = (int)s;
      best_cost = cost;
    }
  }
  return best;
}

// Byte layout of one tree record; the same arithmetic runs on the host (plan) and in the kernel.
struct RecordLayout {
  uint32_t thr, ord, w, bytes;
  bool paired;  // feature indices stored as words {own, left child's, right child's} of the even-level vertices
};

// Trees with one-byte feature indices can store them so that one 4-byte load serves two levels: a
// word per vertex of every even level >= 2 holding {its own index, 0, its left child's, its right child's}
// (levels 0 and 1 come from the record's head, whose last word has the same form).  With the children in
// bytes 2 and 3 the byte-permute selector of a child is its vertex index's low bit OR-ed into a constant.  Word of vertex v (1-based) of even level l: paired_first(l) + v - 2^l.
__host__ __device__ constexpr bool paired_ordinals(int kind, int depth, uint32_t ord_size) {
  return kind == TREE && ord_size == 1 && depth >= 3;
}
__host__ __device__ constexpr uint32_t paired_first(int level) { return ((1u << level) - 4u) / 3u; }
__host__ __device__ constexpr uint32_t paired_words(int depth) {
  const int top = ((depth - 1) / 2) * 2;  // the deepest even level
  return paired_first(top) + (1u << top);
}

// with_weights: the record carries the leaf weights (one output per leaf); with several outputs
// per leaf the weights stay in global memory and the record ends after the feature indices.
__host__ __device__ constexpr RecordLayout record_layout(int kind, int depth, uint32_t ord_size, bool with_weights = true,
                                                        bool paired = false) {
  const uint32_t n = kind == FERN ? (uint32_t)depth : (1u << depth) - 1u;
  const uint32_t thr = kind == FERN ? 0u : (uint32_t)kHeadBytes;
  const uint32_t ord = thr + round16(4u * n);
  const uint32_t w = ord + round16(paired ? 4u * paired_words(depth) : ord_size * n);
  return RecordLayout{thr, ord, w, with_weights ? round16(w + 4u * (1u << depth)) : w, paired};
}

__device__ __forceinline__ uint32_t bit_reverse(uint32_t v, int bits) { return __brev(v) >> (32 - bits); }

// How the repack kernel places things.  Feature index f: stored as is for tabular input; for a
// 2-D convolution window cell f = (row, column) the record holds the offset of that cell inside a
// staged image patch.  Tree t: record t, or, for trees numbered (outer, inner) = t / inner, t % inner,
// record inner * outer_count + outer (the transposed order) when `inner` is set.
struct RecordMap {
  int columns = 0;  // cells per window row; 0: features stored as they are
  int row_step = 0, column_step = 0;
  int64_t inner = 0, outer_count = 0;
  __host__ __device__ uint32_t feature(uint32_t f) const {
    return columns == 0 ? f : (f / (uint32_t)columns) * (uint32_t)row_step + (f % (uint32_t)columns) * (uint32_t)column_step;
  }
  __host__ __device__ int64_t slot(int64_t t) const { return inner == 0 ? t : (t % inner) * outer_count + t / inner; }
};

// One thread per record element.  Leaf weights are permuted so that the path bits in the order
// the traversal collects them (root first, most significant) address them directly.
template <typename OrdT>
__global__ void repack_records_kernel(const float *__restrict__ thr, const int32_t *__restrict__ ord,
                                      const float *__restrict__ w, unsigned char *__restrict__ records, int kind,
                                      int depth, int64_t T, RecordLayout lay, RecordMap map = RecordMap()) {
  const int64_t N = threshold_count(kind, depth);
  const int64_t L = ((int64_t)1) << depth;
  const int64_t per_tree = N + L;
  const int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= T * per_tree) return;
  const int64_t j = e / per_tree;
  const int64_t r = e - j * per_tree;
  unsigned char *rec = records + map.slot(j) * lay.bytes;
  if (r < N) {
    float t = thr[j * N + r];
    t = t == 0.0f ? 0.0f : t;  // -0 becomes +0
    const uint32_t c = map.feature((uint32_t)ord[j * N + r]);
    reinterpret_cast<float *>(rec + lay.thr)[r] = t;
    if (!lay.paired) {
      reinterpret_cast<OrdT *>(rec + lay.ord)[r] = (OrdT)c;
    } else if (r >= 3) {  // vertex v = r + 1 of level >= 2: byte 0 of its own word, or byte 1 / 2 of its parent's
      const uint32_t v = (uint32_t)r + 1u;
      const int level = 31 - __clz((int)v);
      const uint32_t owner = (level & 1) ? v >> 1 : v;
      const int owner_level = level & ~1;
      const uint32_t word = paired_first(owner_level) + owner - (1u << owner_level);
      rec[lay.ord + 4u * word + ((level & 1) ? 2u + (v & 1u) : 0u)] = (unsigned char)c;
      if ((level & 1) == 0) rec[lay.ord + 4u * word + 1u] = 0;
    }
    if (kind == TREE && r < 3) {  // root and its children again, for one broadcast load
      reinterpret_cast<float *>(rec)[r] = t;
      if (sizeof(OrdT) == 1) rec[12 + (r == 0 ? 0 : r + 1)] = (unsigned char)c;  // {root, 0, left, right}
    }
    if (kind == TREE && r == 0 && N < 3) {  // depth 1: no children; keep the head defined
      reinterpret_cast<float *>(rec)[1] = 0.0f;
      reinterpret_cast<float *>(rec)[2] = 0.0f;
      rec[14] = rec[15] = 0;
    }
    if (kind == TREE && r == 0) rec[13] = 0;
  } else if (lay.bytes > lay.w) {  // records that carry the leaf weights
    const int64_t h = r - N;
    reinterpret_cast<float *>(rec + lay.w)[h] = w[j * L + (int64_t)bit_reverse((uint32_t)h, depth)];
  }
}

__device__ __forceinline__ uint32_t smem_addr(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count));
}

__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}

// 1-D bulk copy global -> shared through the TMA engine; completion is counted in bytes on `bar`.
__device__ __forceinline__ void bulk_load(uint32_t dst, const void *src, uint32_t bytes, uint64_t *bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(smem_addr(bar))
               : "memory");
}

// Bounded wait on a phase of the barrier.  Returns false when the limit ran out.
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, uint32_t max_tries = kMaxSpins) {
  for (uint32_t spin = 0; spin < max_tries; ++spin) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(smem_addr(bar)), "r"(parity), "n"(kTryNanoseconds)
        : "memory");
    if (done) return true;
  }
  return false;
}

__device__ __forceinline__ void named_barrier(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

__device__ __forceinline__ float lds_f32(uint32_t addr) {
  float v;
  asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(addr));
  return v;
}

// The same loads with a constant part of the address as an immediate operand of the instruction.
template <uint32_t OFFSET>
__device__ __forceinline__ float lds_f32_at(uint32_t addr) {
  float v;
  asm volatile("ld.shared.f32 %0, [%1+%2];" : "=f"(v) : "r"(addr), "n"(OFFSET));
  return v;
}
template <uint32_t OFFSET>
__device__ __forceinline__ uint32_t lds_b32_at(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1+%2];" : "=r"(v) : "r"(addr), "n"(OFFSET));
  return v;
}
template <uint32_t OFFSET>
__device__ __forceinline__ uint4 lds_b128_at(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4+%5];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "r"(addr), "n"(OFFSET));
  return v;
}

__device__ __forceinline__ void sts_f32(uint32_t addr, float v) {
  asm volatile("st.shared.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}

__device__ __forceinline__ void sts_b128(uint32_t addr, float a, float b, float c, float d) {
  asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

__device__ __forceinline__ uint32_t lds_b32(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}

__device__ __forceinline__ uint4 lds_b128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}

template <typename OrdT>
__device__ __forceinline__ uint32_t lds_ord(uint32_t addr) {
  uint32_t v;
  if (sizeof(OrdT) == 1)
    asm volatile("ld.shared.u8 %0, [%1];" : "=r"(v) : "r"(addr));
  else
    asm volatile("ld.shared.u16 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}

// Minimum of three with one instruction (a NaN operand is ignored, as by fminf).
__device__ __forceinline__ float min3(float a, float b, float c) {
  float r;
  asm("min.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}

// Byte permute as the instruction defines it (the selector is used as given: bit 3 of a nibble would
// replicate the chosen byte's sign, so callers keep it clear).  The intrinsic of the same purpose first
// masks the selector, which costs an instruction.
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t selector) {
  uint32_t r;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(selector));
  return r;
}

__device__ __forceinline__ uint32_t pick(const uint4 &q, int i) {
  return i == 0 ? q.x : i == 1 ? q.y : i == 2 ? q.z : q.w;
}

// Walks NT trees (records at rec[0..NT)) for this lane's sample.  With the leaf weights in the
// records (WREC) result is |min margin| * leaf weight; otherwise result is |min margin| and
// path is 2^DEPTH + the path bits, root first.
// CONSECUTIVE: the NT records follow one another from rec[0] (rec[1..] are not read), so the place of a
// record is a constant that joins the immediate offset of every load and one register addresses all NT.
template <int KIND, int DEPTH, typename OrdT, int NT, bool WREC, bool CONSECUTIVE = false>
__device__ __forceinline__ void walk(const uint32_t (&rec)[NT], uint32_t xl_addr, uint32_t x_stride,
                                     float (&result)[NT], uint32_t (&path)[NT]) {
  constexpr bool kPaired = paired_ordinals(KIND, DEPTH, (uint32_t)sizeof(OrdT));
  constexpr RecordLayout lay = record_layout(KIND, DEPTH, (uint32_t)sizeof(OrdT), WREC, kPaired);
  // scalar copies: constants a lambda may use without capturing the struct
  constexpr uint32_t kRecordBytes = lay.bytes, kThrAt = lay.thr, kOrdAt = lay.ord, kWeightAt = lay.w;
  constexpr uint32_t kLeaves = 1u << DEPTH;
  uint32_t v[NT];
  float best[NT], first[NT], held[NT] = {};
  if constexpr (KIND == FERN) {
    // every lane tests the same decisions: thresholds and feature indices come in 16-byte broadcasts
    constexpr int kPerWord = 4 / (int)sizeof(OrdT);   // feature indices per 32-bit word
    constexpr int kPerQuad = 4 * kPerWord;            // ... per 16-byte load
    uint4 tq[NT], oq[NT];
#pragma unroll
    for (int u = 0; u < NT; ++u) v[u] = 1u;
#pragma unroll
    for (int l = 0; l < DEPTH; ++l) {
#pragma unroll
      for (int u = 0; u < NT; ++u) {
        const uint32_t at = CONSECUTIVE ? rec[0] + (uint32_t)u * lay.bytes : rec[u];
        if (l % 4 == 0) tq[u] = lds_b128(at + lay.thr + 4u * l);
        if (l % kPerQuad == 0) oq[u] = lds_b128(at + lay.ord + (uint32_t)sizeof(OrdT) * l);
        const uint32_t tbits = pick(tq[u], l % 4);
        const uint32_t obits = pick(oq[u], (l % kPerQuad) / kPerWord);
        const uint32_t c = (obits >> (8 * (int)sizeof(OrdT) * (l % kPerWord))) & (sizeof(OrdT) == 1 ? 0xffu : 0xffffu);
        const float nm = __uint_as_float(tbits) - lds_f32(c * x_stride + xl_addr);
        const float am = fabsf(nm);
        if (l == 0) {
          best[u] = am;
          first[u] = am;
        } else {
          best[u] = fminf(best[u], am);
        }
        v[u] = __funnelshift_l(__float_as_uint(nm), v[u], 1);
      }
    }
  } else {
    constexpr bool kHead = sizeof(OrdT) == 1;  // root + children in one 16-byte broadcast
    uint4 head[NT] = {};
    uint32_t family[NT];  // paired form: feature indices of an even-level vertex and its children
    static_for<0, NT>([&](auto tree) {
      constexpr int u = decltype(tree)::value;
      v[u] = 1u;
      family[u] = 0u;
      held[u] = 0.0f;
      if constexpr (kHead) head[u] = lds_b128_at<(CONSECUTIVE ? u * kRecordBytes : 0u)>(rec[CONSECUTIVE ? 0 : u]);
    });
    static_for<0, DEPTH>([&](auto level) {
      constexpr int l = decltype(level)::value;
      static_for<0, NT>([&](auto tree) {
        constexpr int u = decltype(tree)::value;
        [[maybe_unused]] constexpr uint32_t place = CONSECUTIVE ? u * kRecordBytes : 0u;  // of record u, from the base register
        [[maybe_unused]] const uint32_t base = rec[CONSECUTIVE ? 0 : u];
        float thr;
        uint32_t c;
        if constexpr (kHead && l == 0) {
          thr = __uint_as_float(head[u].x);
          c = head[u].w & 0xffu;
        } else if constexpr (kHead && l == 1) {
          thr = __uint_as_float(v[u] == 3u ? head[u].z : head[u].y);
          c = prmt(head[u].w, 0u, v[u] | 0x4440u);  // v is 2 or 3: the left or the right child's byte
        } else {
          const uint32_t at = base + 4u * v[u];  // one address for this vertex's threshold and feature word
          thr = lds_f32_at<place + kThrAt - 4u>(at);
          if constexpr (kPaired) {
            if constexpr (l % 2 == 0) {
              family[u] = lds_b32_at<place + kOrdAt + 4u * paired_first(l) - 4u * (1u << l)>(at);
              c = family[u] & 0xffu;
            } else {
              c = prmt(family[u], 0u, (v[u] & 1u) | 0x4442u);  // byte 2 (left child) or 3 (right child)
            }
          } else {
            c = lds_ord<OrdT>(base + place + (uint32_t)sizeof(OrdT) * v[u] + (kOrdAt - (uint32_t)sizeof(OrdT)));
          }
        }
        const float nm = thr - lds_f32(c * x_stride + xl_addr);
        const float am = fabsf(nm);
        if constexpr (l == 0) {
          best[u] = am;
          first[u] = am;
        } else if constexpr (l % 2 == 1) {
          held[u] = am;  // joins the minimum together with the next level's
        } else {
          best[u] = min3(best[u], held[u], am);
        }
        v[u] = __funnelshift_l(__float_as_uint(nm), v[u], 1);
      });
    });
  }
  static_for<0, NT>([&](auto tree) {
    constexpr int u = decltype(tree)::value;
    [[maybe_unused]] constexpr uint32_t place = CONSECUTIVE ? u * kRecordBytes : 0u;
    [[maybe_unused]] const uint32_t base = rec[CONSECUTIVE ? 0 : u];
    if (DEPTH % 2 == 0 && KIND != FERN) best[u] = fminf(best[u], held[u]);  // the last level was an odd one
    const float am = (first[u] != first[u]) ? first[u] : best[u];
    path[u] = v[u];
    if constexpr (!WREC)
      result[u] = am;
    else if constexpr (kWeightAt >= 4u * kLeaves)
      result[u] = __fmul_rn(am, lds_f32_at<place + kWeightAt - 4u * kLeaves>(base + 4u * v[u]));
    else  // short records (ferns): the constant is negative
      result[u] = __fmul_rn(am, lds_f32(base + place + 4u * v[u] + (kWeightAt - 4u * kLeaves)));
  });
}

// The traversal as the backward needs it: the signed margin and the deciding vertex, with the
// reference's strict `<` so that the shallowest minimum wins.
struct Walked {
  float nm;      // threshold - feature at the deciding vertex (the negated signed margin)
  uint32_t v;    // 1-based index of the deciding vertex (ferns: level + 1); with WITH_FEATURE the feature that
                 // vertex tests (as stored in the record) rides in the high 16 bits: one register, one select
  uint32_t path; // 2^DEPTH + path bits, root first (most significant)
};

// sign(margin) * wg with margin = -nm: wg, -wg, or 0 * wg where the margin is zero or not a number.  Written with
// both values at hand so that it compiles to selects (the nested conditional became a divergent branch per evaluation).
__device__ __forceinline__ float signed_term(float nm, float wg) {
  const float off_zero = nm < 0.0f ? wg : -wg;
  const float at_zero = __fmul_rn(0.0f, wg);
  return (nm < 0.0f || nm > 0.0f) ? off_zero : at_zero;
}

// rec[u] and x_addr[u]: record and feature base (shared-memory addresses) of the u-th walk in flight.
// PAIRED: the records hold the feature indices in the paired form (see paired_ordinals).
template <int KIND, int DEPTH, typename OrdT, int NT, bool PAIRED = false, bool WITH_FEATURE = false>
__device__ __forceinline__ void walk_full(const uint32_t (&rec)[NT], const uint32_t (&x_addr)[NT], uint32_t x_stride,
                                          Walked (&out)[NT]) {
  constexpr RecordLayout lay = record_layout(KIND, DEPTH, (uint32_t)sizeof(OrdT), true, PAIRED);
  uint32_t v[NT];
  uint4 head[NT];
  uint32_t family[NT];
#pragma unroll
  for (int u = 0; u < NT; ++u) {
    v[u] = 1u;
    family[u] = 0u;
    if (PAIRED) head[u] = lds_b128(rec[u]);
  }
#pragma unroll
  for (int l = 0; l < DEPTH; ++l) {
#pragma unroll
    for (int u = 0; u < NT; ++u) {
      const uint32_t at = KIND == FERN ? (uint32_t)(l + 1) : v[u];
      float thr;
      uint32_t c;
      if (PAIRED && l == 0) {
        thr = __uint_as_float(head[u].x);
        c = head[u].w & 0xffu;
      } else if (PAIRED && l == 1) {
        thr = __uint_as_float((at & 1u) ? head[u].z : head[u].y);
        c = prmt(head[u].w, 0u, at | 0x4440u);
      } else if (PAIRED) {
        thr = lds_f32(rec[u] + 4u * at + (lay.thr - 4u));
        if (l % 2 == 0) {
          family[u] = lds_b32(rec[u] + 4u * at + (lay.ord + 4u * paired_first(l) - 4u * (1u << l)));
          c = family[u] & 0xffu;
        } else {
          c = prmt(family[u], 0u, (at & 1u) | 0x4442u);
        }
      } else {
        thr = lds_f32(rec[u] + 4u * at + (lay.thr - 4u));
        c = lds_ord<OrdT>(rec[u] + (uint32_t)sizeof(OrdT) * at + (lay.ord - (uint32_t)sizeof(OrdT)));
      }
      const float nm = thr - lds_f32(c * x_stride + x_addr[u]);
      if (l == 0 || fabsf(nm) < fabsf(out[u].nm)) {
        out[u].nm = nm;
        out[u].v = WITH_FEATURE ? (at | (c << 16)) : at;
      }
      v[u] = __funnelshift_l(__float_as_uint(nm), v[u], 1);
    }
  }
#pragma unroll
  for (int u = 0; u < NT; ++u) out[u].path = v[u];
}

// The same with one feature base for all walks (several trees on one sample or position).
template <int KIND, int DEPTH, typename OrdT, int NT, bool PAIRED = false, bool WITH_FEATURE = false>
__device__ __forceinline__ void walk_full(const uint32_t (&rec)[NT], uint32_t xl_addr, uint32_t x_stride,
                                          Walked (&out)[NT]) {
  uint32_t x_addr[NT];
#pragma unroll
  for (int u = 0; u < NT; ++u) x_addr[u] = xl_addr;
  walk_full<KIND, DEPTH, OrdT, NT, PAIRED, WITH_FEATURE>(rec, x_addr, x_stride, out);
}

// Sum of `val` over the lanes of the warp whose `key` equals this lane's, delivered in the lowest
// of those lanes (`leader`).  All 32 lanes call it.  The lanes of a key form a list (each points to
// the next higher one); pointer jumping doubles the span a lane has summed in every round, so the
// cost grows with the logarithm of the longest list, not its length.  The leaders hold distinct
// keys, so their updates of shared-memory bins do not collide inside the warp.
__device__ __forceinline__ float sum_by_key(uint32_t key, float val, int lane, bool &leader) {
  const uint32_t mask = __match_any_sync(0xffffffffu, key);
  leader = (mask & ((1u << lane) - 1u)) == 0u;
  const uint32_t above = mask & ~((2u << lane) - 1u);
  int next = above != 0u ? __ffs((int)above) - 1 : 32;
  float sum = val;
  const int longest = __reduce_max_sync(0xffffffffu, __popc(mask));
  for (int span = 1; span < longest; span <<= 1) {
    const int src = next < 32 ? next : lane;
    const float v = __shfl_sync(0xffffffffu, sum, src);
    const int after = __shfl_sync(0xffffffffu, next, src);
    if (next < 32) {
      sum = __fadd_rn(sum, v);
      next = after;
    }
  }
  return sum;
}

}  // namespace tile
}  // namespace ht
