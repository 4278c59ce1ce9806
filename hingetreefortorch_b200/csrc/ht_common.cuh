// Shared device code of the sm_100a hinge tree library: the traversal, feature lookups,
// launch helpers and argument checks used by every kernel file.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <type_traits>

#include "hingetree_b200.h"

namespace ht {

// f(std::integral_constant<int, I>) for I = 0 .. N-1, unrolled at compile time (the index can then
// be used where the language wants a constant: template arguments, immediate operands).
template <int I, int N, typename F>
__host__ __device__ __forceinline__ void static_for(F &&f) {
  if constexpr (I < N) {
    f(std::integral_constant<int, I>{});
    static_for<I + 1, N>(f);
  }
}


constexpr int TREE = HT_KIND_TREE;
constexpr int FERN = HT_KIND_FERN;

// Per-thread record of the last failed CUDA runtime call (ht_last_cuda_error()).
extern thread_local int g_last_cuda_error;

inline int cuda_fail(cudaError_t e) {
  g_last_cuda_error = (int)e;
  return HT_ERR_CUDA;
}

#define HT_CUDA_TRY(expr)                                   \
  do {                                                      \
    cudaError_t _e = (expr);                                \
    if (_e != cudaSuccess) return ::ht::cuda_fail(_e);      \
  } while (0)

// Kernel launches issued by this library in this process (ht_launch_count()).
void count_launch();

// Checks the launch that was just issued (never synchronises) and counts it.
#define HT_CHECK_LAUNCH()                    \
  do {                                       \
    ::ht::count_launch();                    \
    HT_CUDA_TRY(cudaPeekAtLastError());      \
  } while (0)

inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

__host__ __device__ inline int64_t threshold_count(int kind, int depth) {
  return kind == FERN ? (int64_t)depth : (((int64_t)1) << depth) - 1;
}

// Result of one traversal: leaf key (bit l = decision at depth l, LSB = root), signed margin
// of the decision with the smallest |margin| (first one wins ties) and its vertex index.
template <typename Real>
struct PathOf {
  uint32_t key;
  Real margin;
  uint32_t vertex;
};
using Path = PathOf<float>;

// Rounded-once arithmetic (no contraction into fused multiply-adds) and |.| for both real types.
// Two or four adjacent floats added to global memory with one reduction (8- / 16-byte aligned address).
__device__ __forceinline__ void red_add_pair(float *p, float a, float b) {
  asm volatile("red.global.add.v2.f32 [%0], {%1, %2};" ::"l"(p), "f"(a), "f"(b) : "memory");
}
__device__ __forceinline__ void red_add_quad(float *p, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

__device__ __forceinline__ float mul_rn(float a, float b) { return __fmul_rn(a, b); }
__device__ __forceinline__ double mul_rn(double a, double b) { return __dmul_rn(a, b); }
__device__ __forceinline__ float add_rn(float a, float b) { return __fadd_rn(a, b); }
__device__ __forceinline__ double add_rn(double a, double b) { return __dadd_rn(a, b); }
__device__ __forceinline__ float abs_of(float a) { return fabsf(a); }
__device__ __forceinline__ double abs_of(double a) { return fabs(a); }

// Feature of one (sample, position): x[i, c, k] with the (i, k) part folded into `base`.
template <typename Real>
struct PlainFeatureOf {
  typedef Real value_type;
  const Real *__restrict__ base;
  int64_t stride;  // K
  __device__ __forceinline__ Real operator()(int c) const { return __ldg(base + (int64_t)c * stride); }
};
using PlainFeature = PlainFeatureOf<float>;

// Image + per-sample vector lookup: features below the image channel count come from the
// image, the rest from the vector (reference semantics: HingeTreeCommon.cuh:81-107, 156-184).
template <typename Real>
struct FusionFeatureOf {
  typedef Real value_type;
  const Real *__restrict__ img;
  int64_t stride;
  const Real *__restrict__ vec;
  int img_channels;
  __device__ __forceinline__ Real operator()(int c) const {
    return c < img_channels ? __ldg(img + (int64_t)c * stride) : __ldg(vec + (c - img_channels));
  }
};
using FusionFeature = FusionFeatureOf<float>;

// The traversal.  One plain fp32 subtract per level; `m > 0` sends NaN and 0 to the left;
// strict `<` keeps the shallowest minimum.  Level 0 seeds the minimum, which is what the
// reference's initialisation from vertex 0 amounts to (also for NaN margins).
template <int KIND, typename OrdT, typename Feature>
__device__ __forceinline__ PathOf<typename Feature::value_type> traverse(const Feature &feat,
                                                                        const typename Feature::value_type *__restrict__ thr,
                                                                        const OrdT *__restrict__ ord, int depth) {
  typedef typename Feature::value_type Real;
  PathOf<Real> p;
  p.key = 0;
  p.vertex = 0;
  p.margin = (Real)0;
  uint32_t v = 0;
  for (int l = 0; l < depth; ++l) {
    const uint32_t at = (KIND == FERN) ? (uint32_t)l : v;
    const Real m = feat((int)ord[at]) - thr[at];
    const uint32_t bit = (m > (Real)0) ? 1u : 0u;
    if (l == 0 || abs_of(m) < abs_of(p.margin)) {
      p.margin = m;
      p.vertex = at;
    }
    p.key |= bit << l;
    v = 2 * v + 1 + bit;
  }
  return p;
}

__device__ __forceinline__ float sign_of(float m) { return (float)((0.0f < m) - (m < 0.0f)); }
__device__ __forceinline__ double sign_of(double m) { return (double)((0.0 < m) - (m < 0.0)); }

// Common argument screening for the forest entry points.
inline int check_forest_problem(const ht_forest_problem *p) {
  if (p == nullptr) return HT_ERR_INVALID_ARGUMENT;
  if (p->kind != TREE && p->kind != FERN) return HT_ERR_INVALID_ARGUMENT;
  if (p->depth < 1 || p->depth > 31) return HT_ERR_DEPTH;
  if (p->B < 0 || p->C < 1 || p->K < 0 || p->T < 0 || p->M < 0) return HT_ERR_INVALID_ARGUMENT;
  if (p->C > 0x7fffffff) return HT_ERR_UNSUPPORTED;
  return HT_OK;
}

// Converts int64 ordinals to int32, clamping out-of-range values to 0 and flagging them.
int pack_ordinals(const int64_t *ord, int64_t n, int64_t C, int32_t *packed, uint32_t *status_word,
                  cudaStream_t stream);

}  // namespace ht
