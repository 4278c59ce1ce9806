// Threshold initialisation and hygiene on the device: the step before the hot path of every training
// script, which the reference runs on the host only (MedianInit.h:133-257, HingeTreeCommon.h:211-287).
//
//  ht_init_medians_f32 / _f64   every threshold becomes the median of its feature over the samples that
//      reach its vertex: the value of rank floor(n / 2) counted from the largest (MedianInit.h:229-235);
//      samples whose feature exceeds it go to the right child, a vertex no sample reaches keeps its
//      threshold, ferns see all samples at every level.  The value at a rank does not depend on how the
//      samples are held, so the result equals the host's bit for bit.
//      Level by level, all trees and all vertices of the level at once: the value of rank k in a vertex's
//      samples is found by radix selection on an order-preserving integer image of the floats, one byte
//      per pass from the top — a histogram pass over all (tree, sample) pairs (256 counters per vertex,
//      integer atomics: exact and order-free), then one warp per vertex picks the byte that holds rank k.
//      After the last byte the prefix IS the median.  A last pass sends every sample to a child.
//  ht_thresholds_f32 / _f64     check (consistent?) or fix (make consistent) the thresholds of trees whose
//      vertices test a feature an ancestor tested already (HingeTreeCommon.h:244-287): one thread per
//      tree, parents first, exactly the host loop.
#include <algorithm>
#include <type_traits>

#include "ht_common.cuh"

namespace ht {
namespace {

inline unsigned blocks_for(int64_t n, int block) { return (unsigned)((n + block - 1) / block); }

template <typename Real>
struct KeyOf;
template <>
struct KeyOf<float> {
  typedef uint32_t type;
};
template <>
struct KeyOf<double> {
  typedef uint64_t type;
};

// Integer image of a float that orders like the float (negative values below positive ones).
__device__ __forceinline__ uint32_t to_key(float v) {
  const uint32_t u = __float_as_uint(v);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ uint64_t to_key(double v) {
  const uint64_t u = (uint64_t)__double_as_longlong(v);
  return (u >> 63) ? ~u : (u | 0x8000000000000000ull);
}
__device__ __forceinline__ float from_key(uint32_t k) { return __uint_as_float((k & 0x80000000u) ? (k ^ 0x80000000u) : ~k); }
__device__ __forceinline__ double from_key(uint64_t k) {
  return __longlong_as_double((long long)((k >> 63) ? (k ^ 0x8000000000000000ull) : ~k));
}

struct MedianShape {
  int64_t samples, C, K, N;  // samples = B * K; N thresholds per tree
  int64_t trees;             // of this chunk
  int kind, level, vertices; // vertices of this level (1 for ferns)
};

// Selection state of one (tree, vertex of the level).
template <typename Key>
struct Selection {
  Key prefix;       // the bytes of the answer found so far (right-aligned)
  int64_t rank;     // rank still to find among the samples that match the prefix, from the largest
  int64_t reached;  // samples at this vertex
};

__device__ __forceinline__ int64_t vertex_of(const MedianShape &s, int local) {
  return s.kind == FERN ? (int64_t)s.level : (((int64_t)1 << s.level) - 1 + local);
}

template <typename Real>
__device__ __forceinline__ Real feature_of(const Real *x, const MedianShape &s, int64_t sample, int64_t feature) {
  const int64_t b = sample / s.K, k = sample - b * s.K;
  return __ldg(x + (b * s.C + feature) * s.K + k);
}

// Pass `byte` (0 = most significant): count, per vertex, the samples whose higher bytes match the prefix by
// the value of this byte.
template <typename Real>
__global__ void __launch_bounds__(256) median_histogram_kernel(MedianShape s, const Real *__restrict__ x,
                                                               const int64_t *__restrict__ ord, const uint32_t *__restrict__ at,
                                                               const Selection<typename KeyOf<Real>::type> *__restrict__ state,
                                                               uint32_t *hist, int byte) {
  typedef typename KeyOf<Real>::type Key;
  const int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= s.trees * s.samples) return;
  const int64_t t = e / s.samples, sample = e - t * s.samples;
  const int local = s.kind == FERN ? 0 : (int)at[e];
  int64_t feature = ord[t * s.N + vertex_of(s, local)];
  feature = feature < 0 || feature >= s.C ? 0 : feature;  // the caller has checked the range; never read outside x
  const Key key = to_key(feature_of(x, s, sample, feature));
  constexpr int kBytes = (int)sizeof(Key);
  const int shift = 8 * (kBytes - 1 - byte);
  const int64_t slot = t * s.vertices + local;
  if (byte > 0 && (key >> (shift + 8)) != state[slot].prefix) return;
  atomicAdd(hist + slot * 256 + (int)((key >> shift) & 0xffu), 1u);
}

// One warp per (tree, vertex): the byte value that holds the wanted rank, scanning from the largest.
template <typename Key>
__global__ void __launch_bounds__(128) median_select_kernel(int64_t slots, Selection<Key> *state, uint32_t *hist, int byte) {
  const int64_t slot = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (slot >= slots) return;
  uint32_t *h = hist + slot * 256;
  // lane l holds the 8 counters of byte values 255 - 8 l ... 248 - 8 l (descending)
  uint32_t c[8];
  uint32_t mine = 0;
#pragma unroll
  for (int q = 0; q < 8; ++q) {
    c[q] = h[255 - 8 * lane - q];
    mine += c[q];
    h[255 - 8 * lane - q] = 0u;  // ready for the next pass
  }
  uint32_t before = mine;  // exclusive prefix sum over the lanes
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const uint32_t up = __shfl_up_sync(0xffffffffu, before, d);
    if (lane >= d) before += up;
  }
  const uint32_t total = __shfl_sync(0xffffffffu, before, 31);
  before -= mine;
  Selection<Key> st = state[slot];
  if (byte == 0) {
    st.prefix = 0;
    st.reached = (int64_t)total;
    st.rank = (int64_t)total / 2;
  }
  if (st.reached == 0) {
    if (lane == 0 && byte == 0) state[slot] = st;
    return;
  }
  const bool holds = (int64_t)before <= st.rank && st.rank < (int64_t)before + (int64_t)mine;
  if (holds) {
    int64_t r = st.rank - (int64_t)before;
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      if (r >= 0 && r < (int64_t)c[q]) {
        st.prefix = (Key)((st.prefix << 8) | (Key)(255 - 8 * lane - q));
        st.rank = r;
        state[slot] = st;
        r = -1;
      } else if (r >= 0) {
        r -= (int64_t)c[q];
      }
    }
  }
}

// The medians are known: write them, and send every sample of a tree to the child its value picks.
template <typename Real>
__global__ void __launch_bounds__(256) median_route_kernel(MedianShape s, const Real *__restrict__ x,
                                                           const int64_t *__restrict__ ord, uint32_t *at,
                                                           const Selection<typename KeyOf<Real>::type> *__restrict__ state,
                                                           Real *thr) {
  const int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (e < s.trees * s.vertices) {  // the first threads also store the thresholds
    const int64_t t = e / s.vertices;
    const int local = (int)(e - t * s.vertices);
    if (state[e].reached > 0) thr[t * s.N + vertex_of(s, local)] = from_key(state[e].prefix);
  }
  if (s.kind == FERN || e >= s.trees * s.samples) return;
  const int64_t t = e / s.samples, sample = e - t * s.samples;
  const int local = (int)at[e];
  int64_t feature = ord[t * s.N + vertex_of(s, local)];
  feature = feature < 0 || feature >= s.C ? 0 : feature;
  const Real median = from_key(state[t * s.vertices + local].prefix);
  at[e] = (uint32_t)(2 * local + (feature_of(x, s, sample, feature) > median ? 1 : 0));
}

size_t per_tree_bytes(int64_t samples, int kind, int depth, size_t key_bytes) {
  const size_t widest = kind == FERN ? 1 : (size_t)1 << (depth - 1);
  return (size_t)samples * 4 + widest * (256 * 4 + 2 * 8 + 8 + key_bytes);
}

template <typename Real>
int init_medians(int kind, const Real *x, Real *thr, const int64_t *ord, int64_t B, int64_t C, int64_t K, int64_t T, int depth,
                 void *workspace, size_t workspace_bytes, cudaStream_t stream) {
  typedef typename KeyOf<Real>::type Key;
  if ((kind != TREE && kind != FERN) || depth < 1 || depth > 20 || B < 0 || C < 1 || K < 1 || T < 0) return HT_ERR_INVALID_ARGUMENT;
  if (B == 0 || T == 0) return HT_OK;
  if (x == nullptr || thr == nullptr || ord == nullptr || workspace == nullptr) return HT_ERR_INVALID_ARGUMENT;
  const int64_t samples = B * K;
  const int64_t N = kind == FERN ? depth : (((int64_t)1) << depth) - 1;
  const size_t widest = kind == FERN ? 1 : (size_t)1 << (depth - 1);
  const size_t per_tree = per_tree_bytes(samples, kind, depth, sizeof(Key)) + 64;
  const int64_t chunk = (int64_t)std::min<size_t>((size_t)T, workspace_bytes / per_tree);
  if (chunk < 1) return HT_ERR_WORKSPACE;
  if ((double)chunk * (double)samples >= 2147483648.0 * 256.0) return HT_ERR_UNSUPPORTED;
  unsigned char *base = static_cast<unsigned char *>(workspace);
  uint32_t *at = reinterpret_cast<uint32_t *>(base);
  size_t offset = (((size_t)chunk * samples * 4) + 15) & ~(size_t)15;
  uint32_t *hist = reinterpret_cast<uint32_t *>(base + offset);
  offset += (size_t)chunk * widest * 256 * 4;
  Selection<Key> *state = reinterpret_cast<Selection<Key> *>(base + offset);

  for (int64_t first = 0; first < T; first += chunk) {
    MedianShape s;
    s.samples = samples;
    s.C = C;
    s.K = K;
    s.N = N;
    s.trees = std::min(chunk, T - first);
    s.kind = kind;
    const int64_t *tree_ord = ord + first * N;
    Real *tree_thr = thr + first * N;
    HT_CUDA_TRY(cudaMemsetAsync(at, 0, (size_t)s.trees * samples * 4, stream));
    HT_CUDA_TRY(cudaMemsetAsync(hist, 0, (size_t)s.trees * widest * 256 * 4, stream));
    const unsigned pair_grid = blocks_for(s.trees * samples, 256);
    for (int level = 0; level < depth; ++level) {
      s.level = level;
      s.vertices = kind == FERN ? 1 : 1 << level;
      const int64_t slots = s.trees * s.vertices;
      for (int byte = 0; byte < (int)sizeof(Key); ++byte) {
        median_histogram_kernel<Real><<<pair_grid, 256, 0, stream>>>(s, x, tree_ord, at, state, hist, byte);
        HT_CHECK_LAUNCH();
        median_select_kernel<Key><<<blocks_for(slots * 32, 128), 128, 0, stream>>>(slots, state, hist, byte);
        HT_CHECK_LAUNCH();
      }
      const unsigned route_grid = kind == FERN ? blocks_for(slots, 256) : pair_grid;
      median_route_kernel<Real><<<std::max(route_grid, blocks_for(slots, 256)), 256, 0, stream>>>(s, x, tree_ord, at, state, tree_thr);
      HT_CHECK_LAUNCH();
    }
  }
  return HT_OK;
}

// ---- threshold hygiene ------------------------------------------------------------------------

template <typename Real>
__device__ void feasible_interval(const Real *thr, const int64_t *ord, int64_t vertex, Real &lo, Real &hi) {
  lo = -INFINITY;
  hi = INFINITY;
  const int64_t feature = ord[vertex];
  for (int64_t child = vertex; child > 0;) {
    const int64_t parent = (child - 1) / 2;
    if (ord[parent] == feature) {
      if (child == 2 * parent + 2)
        lo = thr[parent] > lo ? thr[parent] : lo;  // reached through the right branch: x > thr[parent]
      else
        hi = thr[parent] < hi ? thr[parent] : hi;
    }
    child = parent;
  }
}

// result[j]: check: 1 when tree j is consistent; fix: 1 when a threshold of tree j was moved.
template <typename Real>
__global__ void thresholds_kernel(Real *thr, const int64_t *__restrict__ ord, int64_t T, int64_t N, int fix, unsigned char *result) {
  const int64_t j = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (j >= T) return;
  Real *t = thr + j * N;
  const int64_t *o = ord + j * N;
  Real lo, hi;
  if (!fix) {
    unsigned char ok = 1;
    for (int64_t v = N - 1; v > 0; --v) {
      feasible_interval(t, o, v, lo, hi);
      if (t[v] < lo || t[v] > hi) {
        ok = 0;
        break;
      }
    }
    result[j] = ok;
    return;
  }
  unsigned char changed = 0;
  for (int64_t v = 1; v < N; ++v) {  // parents first: a fixed parent constrains its subtree
    feasible_interval(t, o, v, lo, hi);
    if (t[v] < lo || t[v] > hi) {
      if (isinf(lo))
        t[v] = hi - (Real)1;
      else if (isinf(hi))
        t[v] = lo + (Real)1;
      else
        t[v] = (Real)0.5 * (lo + hi);
      changed = 1;
    }
  }
  result[j] = changed;
}

template <typename Real>
int thresholds(int fix, Real *thr, const int64_t *ord, int64_t T, int depth, unsigned char *result, cudaStream_t stream) {
  if (depth < 1 || depth > 31 || T < 0) return HT_ERR_INVALID_ARGUMENT;
  if (T == 0) return HT_OK;
  if (thr == nullptr || ord == nullptr || result == nullptr) return HT_ERR_INVALID_ARGUMENT;
  const int64_t N = (((int64_t)1) << depth) - 1;
  thresholds_kernel<Real><<<blocks_for(T, 128), 128, 0, stream>>>(thr, ord, T, N, fix, result);
  HT_CHECK_LAUNCH();
  return HT_OK;
}

}  // namespace
}  // namespace ht

using namespace ht;

extern "C" size_t ht_init_medians_workspace_bytes(int kind, int64_t B, int64_t K, int64_t T, int depth, int element_bytes) {
  if (B < 1 || K < 1 || T < 1 || depth < 1 || depth > 20) return 0;
  const size_t per_tree = per_tree_bytes(B * K, kind, depth, (size_t)element_bytes) + 64;
  const size_t cap = (size_t)1 << 30;  // more trees than fit 1 GiB are done in several rounds
  const size_t trees = std::max<size_t>(1, std::min<size_t>((size_t)T, cap / per_tree));
  return trees * per_tree;
}

extern "C" int ht_init_medians_f32(int kind, const float *x, float *thr, const int64_t *ord, int64_t B, int64_t C, int64_t K, int64_t T,
                                   int depth, void *workspace, size_t workspace_bytes, ht_stream_t stream) {
  return init_medians<float>(kind, x, thr, ord, B, C, K, T, depth, workspace, workspace_bytes, reinterpret_cast<cudaStream_t>(stream));
}

extern "C" int ht_init_medians_f64(int kind, const double *x, double *thr, const int64_t *ord, int64_t B, int64_t C, int64_t K,
                                   int64_t T, int depth, void *workspace, size_t workspace_bytes, ht_stream_t stream) {
  return init_medians<double>(kind, x, thr, ord, B, C, K, T, depth, workspace, workspace_bytes, reinterpret_cast<cudaStream_t>(stream));
}

extern "C" int ht_thresholds_f32(int fix, float *thr, const int64_t *ord, int64_t T, int depth, unsigned char *result, ht_stream_t stream) {
  return thresholds<float>(fix, thr, ord, T, depth, result, reinterpret_cast<cudaStream_t>(stream));
}

extern "C" int ht_thresholds_f64(int fix, double *thr, const int64_t *ord, int64_t T, int depth, unsigned char *result, ht_stream_t stream) {
  return thresholds<double>(fix, thr, ord, T, depth, result, reinterpret_cast<cudaStream_t>(stream));
}
