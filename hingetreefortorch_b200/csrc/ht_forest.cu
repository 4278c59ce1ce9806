// Hinge forest / fern evaluation: C-ABI entry points, the any-shape kernels and the backward.
//
// The any-shape kernels run one thread per (sample i, tree j, position k) and read the
// parameters and the input through L1/L2.  They accept every shape the reference accepts
// (any C, K, M, depth up to 31).  Shapes the shared-memory tile kernel (ht_forest_tiled.cu)
// can take are routed there by ht_forest_forward_f32.
#include <atomic>

#include "ht_common.cuh"
#include "ht_forest_tiled.cuh"

namespace ht {

thread_local int g_last_cuda_error = 0;

static std::atomic<uint64_t> g_launches{0};
void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

namespace {

constexpr int kBlock = 256;

__global__ void pack_ordinals_kernel(const int64_t *__restrict__ ord, int64_t n, int64_t C,
                                     int32_t *__restrict__ packed, uint32_t *status_word) {
  const int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= n) return;
  int64_t o = ord[e];
  if (o < 0 || o >= C) {
    o = 0;
    if (status_word != nullptr) atomicOr(status_word, HT_FLAG_ORDINAL_RANGE);
  }
  packed[e] = (int32_t)o;
}

template <typename Real>
struct ForestArgsOf {
  const Real *x;
  const Real *thr;
  const int32_t *ord;
  const Real *w;
  int64_t B, C, K, T, N, L, M;
  int depth;
};
using ForestArgs = ForestArgsOf<float>;

template <typename Real>
__device__ __forceinline__ void split_index(const ForestArgsOf<Real> &a, int64_t e, int64_t &i, int64_t &j, int64_t &k) {
  if (a.K == 1) {
    k = 0;
    i = e / a.T;
    j = e - i * a.T;
  } else {
    const int64_t ij = e / a.K;
    k = e - ij * a.K;
    i = ij / a.T;
    j = ij - i * a.T;
  }
}

enum { MODE_FORWARD = 0, MODE_LEAFMAP = 1, MODE_MARGINMAP = 2, MODE_REACH = 3 };

template <int KIND, int MODE, typename Real>
__global__ void __launch_bounds__(kBlock) forest_any_kernel(ForestArgsOf<Real> a, Real *__restrict__ out_f,
                                                            int64_t *__restrict__ out_i) {
  const int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= a.B * a.T * a.K) return;
  int64_t i, j, k;
  split_index(a, e, i, j, k);
  const PlainFeatureOf<Real> feat{a.x + i * a.C * a.K + k, a.K};
  const PathOf<Real> p = traverse<KIND>(feat, a.thr + j * a.N, a.ord + j * a.N, a.depth);
  if (MODE == MODE_FORWARD) {
    const Real am = abs_of(p.margin);
    const Real *wl = a.w + (j * a.L + p.key) * a.M;
    Real *o = out_f + e * a.M;
    for (int64_t m = 0; m < a.M; ++m) o[m] = am * __ldg(wl + m);
  } else if (MODE == MODE_LEAFMAP) {
    out_i[e] = (int64_t)p.key;
  } else if (MODE == MODE_MARGINMAP) {
    out_f[e] = p.margin;
    out_i[e] = (int64_t)a.ord[j * a.N + p.vertex];
  } else {
    atomicAdd(reinterpret_cast<unsigned long long *>(out_i) + (j * a.L + p.key), 1ull);
  }
}

// One thread per (i, j, k): the three gradient scatters after a single traversal.
template <int KIND, typename Real>
__global__ void __launch_bounds__(kBlock) forest_backward_atomic_kernel(ForestArgsOf<Real> a, const Real *__restrict__ g,
                                                                        Real *gx, Real *gthr, Real *gw) {
  const int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= a.B * a.T * a.K) return;
  int64_t i, j, k;
  split_index(a, e, i, j, k);
  const PlainFeatureOf<Real> feat{a.x + i * a.C * a.K + k, a.K};
  const PathOf<Real> p = traverse<KIND>(feat, a.thr + j * a.N, a.ord + j * a.N, a.depth);
  const Real s = sign_of(p.margin);
  const Real am = abs_of(p.margin);
  const Real *wl = a.w + (j * a.L + p.key) * a.M;
  const Real *gl = g + e * a.M;
  Real acc = (Real)0;
  if constexpr (std::is_same<Real, float>::value) {
    // an even number of outputs per leaf: the rows of g, w and gw start on 8-byte boundaries (given aligned
    // tensors), so they are read two at a time and the leaf-weight gradient takes one reduction per pair
    if ((a.M & 1) == 0 && ((reinterpret_cast<uintptr_t>(g) | reinterpret_cast<uintptr_t>(a.w) | reinterpret_cast<uintptr_t>(gw)) & 7u) == 0) {
      float *gwl = gw != nullptr ? gw + (j * a.L + p.key) * a.M : nullptr;
      // (a row of 8-byte alignment starts with a pair when it is not on a 16-byte boundary, then goes on in fours)
      int64_t m = 0;
      auto pair = [&]() {
        const float2 gm = __ldg(reinterpret_cast<const float2 *>(gl + m));
        const float2 wm = __ldg(reinterpret_cast<const float2 *>(wl + m));
        acc = add_rn(acc, mul_rn(mul_rn(s, wm.x), gm.x));  // the same terms in the same order as one at a time
        acc = add_rn(acc, mul_rn(mul_rn(s, wm.y), gm.y));
        if (gwl != nullptr) red_add_pair(gwl + m, mul_rn(am, gm.x), mul_rn(am, gm.y));
        m += 2;
      };
      if (gwl == nullptr || (reinterpret_cast<uintptr_t>(gwl) & 15u) != 0) pair();
      for (; m + 4 <= a.M; m += 4) {
        const float2 g0 = __ldg(reinterpret_cast<const float2 *>(gl + m)), g1 = __ldg(reinterpret_cast<const float2 *>(gl + m + 2));
        const float2 w0 = __ldg(reinterpret_cast<const float2 *>(wl + m)), w1 = __ldg(reinterpret_cast<const float2 *>(wl + m + 2));
        acc = add_rn(acc, mul_rn(mul_rn(s, w0.x), g0.x));
        acc = add_rn(acc, mul_rn(mul_rn(s, w0.y), g0.y));
        acc = add_rn(acc, mul_rn(mul_rn(s, w1.x), g1.x));
        acc = add_rn(acc, mul_rn(mul_rn(s, w1.y), g1.y));
        if (gwl != nullptr) red_add_quad(gwl + m, mul_rn(am, g0.x), mul_rn(am, g0.y), mul_rn(am, g1.x), mul_rn(am, g1.y));
      }
      while (m < a.M) pair();
      if (gx != nullptr) atomicAdd(gx + (i * a.C + a.ord[j * a.N + p.vertex]) * a.K + k, acc);
      if (gthr != nullptr) atomicAdd(gthr + j * a.N + p.vertex, -acc);
      return;
    }
  }
  for (int64_t m = 0; m < a.M; ++m) {
    const Real gm = __ldg(gl + m);
    acc = add_rn(acc, mul_rn(mul_rn(s, __ldg(wl + m)), gm));
    if (gw != nullptr) atomicAdd(gw + (j * a.L + p.key) * a.M + m, mul_rn(am, gm));
  }
  if (gx != nullptr) atomicAdd(gx + (i * a.C + a.ord[j * a.N + p.vertex]) * a.K + k, acc);
  if (gthr != nullptr) atomicAdd(gthr + j * a.N + p.vertex, -acc);
}

// ---- fixed-order (deterministic) backward ---------------------------------------------
//
// The reference CPU loops add, into every gradient element, one term per (i, j, k, m) in
// the order i, j, k, m.  Floating point addition is not associative, so reproducing those
// sums bit for bit means adding the same terms in the same order per destination element.
// Destinations are independent of one another; the kernels below parallelise over them and
// keep the order inside each.

// Runs f() on the valid lanes of a warp so that lanes sharing `key` execute in lane order
// and lanes with different keys execute concurrently.  Keys must be below 2^31.
template <typename F>
__device__ __forceinline__ void in_lane_order_per_key(bool valid, uint32_t key, F &&f) {
  const unsigned lane = threadIdx.x & 31u;
  const uint32_t tag = valid ? key : (0x80000000u | lane);
  const unsigned peers = __match_any_sync(0xffffffffu, tag);
  const int rank = __popc(peers & ((1u << lane) - 1u));
  const int last = __reduce_max_sync(0xffffffffu, valid ? rank : 0);
  for (int r = 0; r <= last; ++r) {
    if (valid && rank == r) f();
    __syncwarp();
  }
}

// x gradient, one thread per (i, k) walking the trees in ascending order.
template <int KIND, typename Real>
__global__ void __launch_bounds__(128) forest_backward_x_ordered_thread_kernel(ForestArgsOf<Real> a,
                                                                               const Real *__restrict__ g, Real *gx) {
  const int64_t p = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (p >= a.B * a.K) return;
  const int64_t i = p / a.K, k = p - i * a.K;
  const PlainFeatureOf<Real> feat{a.x + i * a.C * a.K + k, a.K};
  for (int64_t j = 0; j < a.T; ++j) {
    const PathOf<Real> path = traverse<KIND>(feat, a.thr + j * a.N, a.ord + j * a.N, a.depth);
    const Real s = sign_of(path.margin);
    const Real *wl = a.w + (j * a.L + path.key) * a.M;
    const Real *gl = g + ((i * a.T + j) * a.K + k) * a.M;
    Real *dst = gx + (i * a.C + a.ord[j * a.N + path.vertex]) * a.K + k;
    Real acc = *dst;
    for (int64_t m = 0; m < a.M; ++m) acc = add_rn(acc, mul_rn(mul_rn(s, __ldg(wl + m)), __ldg(gl + m)));
    *dst = acc;
  }
}

// x gradient, one warp per (i, k): lanes take 32 consecutive trees, traverse concurrently and
// then add into the row in tree order wherever two of them hit the same feature.
template <int KIND, typename Real>
__global__ void __launch_bounds__(128) forest_backward_x_ordered_warp_kernel(ForestArgsOf<Real> a,
                                                                             const Real *__restrict__ g, Real *gx) {
  const int64_t p = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  if (p >= a.B * a.K) return;  // whole warps leave together
  const unsigned lane = threadIdx.x & 31u;
  const int64_t i = p / a.K, k = p - i * a.K;
  const PlainFeatureOf<Real> feat{a.x + i * a.C * a.K + k, a.K};
  for (int64_t j0 = 0; j0 < a.T; j0 += 32) {
    const int64_t j = j0 + lane;
    const bool valid = j < a.T;
    PathOf<Real> path{0u, (Real)0, 0u};
    int c = 0;
    if (valid) {
      path = traverse<KIND>(feat, a.thr + j * a.N, a.ord + j * a.N, a.depth);
      c = a.ord[j * a.N + path.vertex];
    }
    in_lane_order_per_key(valid, (uint32_t)c, [&]() {
      const Real s = sign_of(path.margin);
      const Real *wl = a.w + (j * a.L + path.key) * a.M;
      const Real *gl = g + ((i * a.T + j) * a.K + k) * a.M;
      Real *dst = gx + (i * a.C + c) * a.K + k;
      Real acc = __ldcg(dst);
      for (int64_t m = 0; m < a.M; ++m) acc = add_rn(acc, mul_rn(mul_rn(s, __ldg(wl + m)), __ldg(gl + m)));
      __stcg(dst, acc);
    });
  }
}

// Threshold and leaf-weight gradients, one warp per tree.  Lanes take 32 consecutive (i, k)
// positions, traverse concurrently, then add into the tree's bins in position order wherever
// two of them hit the same bin.  Bins live in shared memory when they fit, else in the
// (already cleared) global outputs, which no other warp touches.
template <int KIND, typename Real>
__global__ void __launch_bounds__(32) forest_backward_params_ordered_kernel(ForestArgsOf<Real> a, const Real *__restrict__ g,
                                                                            Real *gthr, Real *gw, int thr_in_smem,
                                                                            int w_in_smem) {
  extern __shared__ __align__(16) unsigned char bins_raw[];
  Real *bins = reinterpret_cast<Real *>(bins_raw);
  const int64_t j = blockIdx.x;
  const unsigned lane = threadIdx.x;
  const int64_t LM = a.L * a.M;
  Real *thr_bins = nullptr, *w_bins = nullptr;
  if (gthr != nullptr) thr_bins = thr_in_smem ? bins : gthr + j * a.N;
  if (gw != nullptr) w_bins = w_in_smem ? bins + (thr_in_smem ? a.N : 0) : gw + j * LM;
  if (thr_bins != nullptr && thr_in_smem)
    for (int64_t t = lane; t < a.N; t += 32) thr_bins[t] = (Real)0;
  if (w_bins != nullptr && w_in_smem)
    for (int64_t t = lane; t < LM; t += 32) w_bins[t] = (Real)0;
  __syncwarp();

  const Real *thr = a.thr + j * a.N;
  const int32_t *ord = a.ord + j * a.N;
  const int64_t P = a.B * a.K;
  for (int64_t p0 = 0; p0 < P; p0 += 32) {
    const int64_t p = p0 + lane;
    const bool valid = p < P;
    PathOf<Real> path{0u, (Real)0, 0u};
    int64_t i = 0, k = 0;
    if (valid) {
      i = p / a.K;
      k = p - i * a.K;
      const PlainFeatureOf<Real> feat{a.x + i * a.C * a.K + k, a.K};
      path = traverse<KIND>(feat, thr, ord, a.depth);
    }
    const Real *gl = g + ((i * a.T + j) * a.K + k) * a.M;
    const Real *wl = a.w + (j * a.L + path.key) * a.M;
    if (thr_bins != nullptr) {
      in_lane_order_per_key(valid, path.vertex, [&]() {
        const Real ns = -sign_of(path.margin);
        volatile Real *dst = thr_bins + path.vertex;
        Real acc = *dst;
        for (int64_t m = 0; m < a.M; ++m) acc = add_rn(acc, mul_rn(mul_rn(ns, __ldg(wl + m)), __ldg(gl + m)));
        *dst = acc;
      });
    }
    if (w_bins != nullptr) {
      in_lane_order_per_key(valid, path.key, [&]() {
        const Real am = abs_of(path.margin);
        volatile Real *dst = w_bins + (int64_t)path.key * a.M;
        for (int64_t m = 0; m < a.M; ++m) dst[m] = add_rn(dst[m], mul_rn(am, __ldg(gl + m)));
      });
    }
  }
  __syncwarp();
  if (thr_bins != nullptr && thr_in_smem)
    for (int64_t t = lane; t < a.N; t += 32) gthr[j * a.N + t] = thr_bins[t];
  if (w_bins != nullptr && w_in_smem)
    for (int64_t t = lane; t < LM; t += 32) gw[j * LM + t] = w_bins[t];
}

// The workspace starts with the compact int32 ordinals; the tile kernel's records follow.
inline size_t ordinals_bytes(const ht_forest_problem *p) {
  return align_up((size_t)(p->T * threshold_count(p->kind, p->depth)) * sizeof(int32_t), 256);
}

inline unsigned blocks_for(int64_t n, int block) { return (unsigned)((n + block - 1) / block); }

template <typename Real>
struct PreparedOf {
  ForestArgsOf<Real> args;
  cudaStream_t stream;
  int64_t evals;
};
using Prepared = PreparedOf<float>;

// Validates the call, converts the ordinals into the workspace and fills the kernel arguments.
template <typename Real>
int prepare(const ht_forest_problem *p, const Real *x, const Real *thr, const int64_t *ord, const Real *w,
            bool need_w, void *workspace, size_t workspace_bytes, uint32_t *status_word, ht_stream_t stream,
            PreparedOf<Real> &out) {
  const int rc = check_forest_problem(p);
  if (rc != HT_OK) return rc;
  // a null pointer is only acceptable for a tensor without elements
  const int64_t decisions = p->T * threshold_count(p->kind, p->depth);
  if ((x == nullptr && p->B * p->C * p->K > 0) || ((thr == nullptr || ord == nullptr) && decisions > 0) ||
      (need_w && w == nullptr && p->T * p->M > 0))
    return HT_ERR_INVALID_ARGUMENT;
  // the double precision entry points run the any-shape kernels only: compact ordinals are all they keep
  const size_t need = sizeof(Real) == 4 ? ht_forest_workspace_bytes(p) : ordinals_bytes(p) + 256;
  if (workspace == nullptr || workspace_bytes < need || (reinterpret_cast<uintptr_t>(workspace) & 255u) != 0)
    return HT_ERR_WORKSPACE;
  ForestArgsOf<Real> &a = out.args;
  a.x = x;
  a.thr = thr;
  a.ord = static_cast<const int32_t *>(workspace);
  a.w = w;
  a.B = p->B;
  a.C = p->C;
  a.K = p->K;
  a.T = p->T;
  a.M = p->M;
  a.depth = p->depth;
  a.N = threshold_count(p->kind, p->depth);
  a.L = ((int64_t)1) << p->depth;
  out.stream = reinterpret_cast<cudaStream_t>(stream);
  out.evals = p->B * p->T * p->K;
  if (a.T * a.N > 0) {
    const int prc = pack_ordinals(ord, a.T * a.N, a.C, static_cast<int32_t *>(workspace), status_word, out.stream);
    if (prc != HT_OK) return prc;
  }
  return HT_OK;
}

template <int MODE, typename Real>
int launch_any(const ht_forest_problem *p, const PreparedOf<Real> &pr, Real *out_f, int64_t *out_i) {
  if (pr.evals == 0) return HT_OK;
  const unsigned grid = blocks_for(pr.evals, kBlock);
  if (p->kind == TREE)
    forest_any_kernel<TREE, MODE, Real><<<grid, kBlock, 0, pr.stream>>>(pr.args, out_f, out_i);
  else
    forest_any_kernel<FERN, MODE, Real><<<grid, kBlock, 0, pr.stream>>>(pr.args, out_f, out_i);
  HT_CHECK_LAUNCH();
  return HT_OK;
}

// Clears the requested gradients (the entry points' contract).
template <typename Real>
int clear_gradients(const PreparedOf<Real> &pr, Real *gx, Real *gthr, Real *gw) {
  const ForestArgsOf<Real> &a = pr.args;
  if (gx != nullptr && a.B * a.C * a.K > 0)
    HT_CUDA_TRY(cudaMemsetAsync(gx, 0, sizeof(Real) * (size_t)(a.B * a.C * a.K), pr.stream));
  if (gthr != nullptr && a.T * a.N > 0)
    HT_CUDA_TRY(cudaMemsetAsync(gthr, 0, sizeof(Real) * (size_t)(a.T * a.N), pr.stream));
  if (gw != nullptr && a.T * a.L * a.M > 0)
    HT_CUDA_TRY(cudaMemsetAsync(gw, 0, sizeof(Real) * (size_t)(a.T * a.L * a.M), pr.stream));
  return HT_OK;
}

// The backward with the any-shape kernels: one traversal and atomic scatters in default mode; in fixed-order
// mode the x gradient by a thread (or a warp) per (sample, position) in tree order and the parameter gradients
// by a warp per tree in sample order.
template <typename Real>
int backward_any(const ht_forest_problem *p, const PreparedOf<Real> &pr, const Real *g, Real *gx, Real *gthr, Real *gw) {
  const ForestArgsOf<Real> &a = pr.args;
  if ((p->flags & HT_DETERMINISTIC) == 0) {
    const unsigned grid = blocks_for(pr.evals, kBlock);
    if (p->kind == TREE)
      forest_backward_atomic_kernel<TREE, Real><<<grid, kBlock, 0, pr.stream>>>(a, g, gx, gthr, gw);
    else
      forest_backward_atomic_kernel<FERN, Real><<<grid, kBlock, 0, pr.stream>>>(a, g, gx, gthr, gw);
    HT_CHECK_LAUNCH();
    return HT_OK;
  }
  const int64_t P = a.B * a.K;
  if (gx != nullptr) {
    if (P >= 32768) {
      const unsigned grid = blocks_for(P, 128);
      if (p->kind == TREE)
        forest_backward_x_ordered_thread_kernel<TREE, Real><<<grid, 128, 0, pr.stream>>>(a, g, gx);
      else
        forest_backward_x_ordered_thread_kernel<FERN, Real><<<grid, 128, 0, pr.stream>>>(a, g, gx);
    } else {
      const unsigned grid = blocks_for(P * 32, 128);
      if (p->kind == TREE)
        forest_backward_x_ordered_warp_kernel<TREE, Real><<<grid, 128, 0, pr.stream>>>(a, g, gx);
      else
        forest_backward_x_ordered_warp_kernel<FERN, Real><<<grid, 128, 0, pr.stream>>>(a, g, gx);
    }
    HT_CHECK_LAUNCH();
  }
  if (gthr != nullptr || gw != nullptr) {
    const size_t thr_bytes = gthr != nullptr ? sizeof(Real) * (size_t)a.N : 0;
    const size_t w_bytes = gw != nullptr ? sizeof(Real) * (size_t)(a.L * a.M) : 0;
    const size_t limit = 96 * 1024;
    const int thr_in_smem = thr_bytes > 0 && thr_bytes <= 32 * 1024;
    const int w_in_smem = w_bytes > 0 && w_bytes + (thr_in_smem ? thr_bytes : 0) <= limit;
    const size_t smem = (thr_in_smem ? thr_bytes : 0) + (w_in_smem ? w_bytes : 0);
    auto kernel = p->kind == TREE ? forest_backward_params_ordered_kernel<TREE, Real>
                                  : forest_backward_params_ordered_kernel<FERN, Real>;
    if (smem > 48 * 1024)
      HT_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)limit));
    kernel<<<(unsigned)a.T, 32, smem, pr.stream>>>(a, g, gthr, gw, thr_in_smem, w_in_smem);
    HT_CHECK_LAUNCH();
  }
  return HT_OK;
}

}  // namespace

int pack_ordinals(const int64_t *ord, int64_t n, int64_t C, int32_t *packed, uint32_t *status_word,
                  cudaStream_t stream) {
  if (n <= 0) return HT_OK;
  pack_ordinals_kernel<<<blocks_for(n, kBlock), kBlock, 0, stream>>>(ord, n, C, packed, status_word);
  HT_CHECK_LAUNCH();
  return HT_OK;
}

}  // namespace ht

using namespace ht;

extern "C" {

int ht_version(void) { return 100; }

int ht_last_cuda_error(void) { return ht::g_last_cuda_error; }

uint64_t ht_launch_count(void) { return ht::g_launches.load(std::memory_order_relaxed); }

const char *ht_status_string(int status) {
  switch (status) {
    case HT_OK: return "ok";
    case HT_ERR_INVALID_ARGUMENT: return "invalid argument (null pointer, bad kind or negative size)";
    case HT_ERR_DEPTH: return "tree depth outside [1, 31] or threshold count does not match the depth";
    case HT_ERR_CUDA: return "CUDA runtime or launch error";
    case HT_ERR_WORKSPACE: return "workspace missing, not 256-byte aligned or too small";
    case HT_ERR_UNSUPPORTED: return "request not supported by this build";
    default: return "unknown status";
  }
}

int ht_forest_forward_saves(const ht_forest_problem *p) {
  return check_forest_problem(p) == HT_OK && forward_saves(p) ? 1 : 0;
}

size_t ht_forest_workspace_bytes(const ht_forest_problem *p) {
  if (check_forest_problem(p) != HT_OK) return 0;
  const size_t base = ordinals_bytes(p) + forward_tiled_workspace_bytes(p) + 256;
  return (p->flags & HT_WORKSPACE_FOR_BACKWARD) != 0 ? base + backward_records_bytes(p) : base;
}

int ht_forest_forward_f32(const ht_forest_problem *p, const float *x, const float *thr, const int64_t *ord,
                          const float *w, float *out, void *workspace, size_t workspace_bytes,
                          uint32_t *status_word, ht_stream_t stream) {
  Prepared pr;
  const int rc = prepare(p, x, thr, ord, w, true, workspace, workspace_bytes, status_word, stream, pr);
  if (rc != HT_OK) return rc;
  if (pr.evals * p->M == 0) return HT_OK;
  if (out == nullptr) return HT_ERR_INVALID_ARGUMENT;
  // HT_SAVE_FOR_BACKWARD: the traversal goes to the evaluation-record area of the workspace, when it is there
  unsigned char *ws = static_cast<unsigned char *>(workspace);
  void *eval_records = nullptr;
  if ((p->flags & HT_SAVE_FOR_BACKWARD) != 0 && forward_saves(p)) {
    const size_t records_at = ordinals_bytes(p) + forward_tiled_workspace_bytes(p);
    if (workspace_bytes >= records_at + backward_records_bytes(p)) eval_records = ws + records_at;
  }
  const int trc = forward_tiled(p, x, thr, pr.args.ord, w, out, ws + ordinals_bytes(p), eval_records, status_word, pr.stream);
  if (trc != HT_ERR_UNSUPPORTED) return trc;
  return launch_any<MODE_FORWARD>(p, pr, out, nullptr);
}

int ht_forest_leafmap_f32(const ht_forest_problem *p, const float *x, const float *thr, const int64_t *ord,
                          int64_t *leaf, void *workspace, size_t workspace_bytes, uint32_t *status_word,
                          ht_stream_t stream) {
  Prepared pr;
  const int rc = prepare<float>(p, x, thr, ord, nullptr, false, workspace, workspace_bytes, status_word, stream, pr);
  if (rc != HT_OK) return rc;
  if (leaf == nullptr && pr.evals > 0) return HT_ERR_INVALID_ARGUMENT;
  return launch_any<MODE_LEAFMAP, float>(p, pr, nullptr, leaf);
}

int ht_forest_marginmap_f32(const ht_forest_problem *p, const float *x, const float *thr, const int64_t *ord,
                            float *margin, int64_t *margin_ord, void *workspace, size_t workspace_bytes,
                            uint32_t *status_word, ht_stream_t stream) {
  Prepared pr;
  const int rc = prepare<float>(p, x, thr, ord, nullptr, false, workspace, workspace_bytes, status_word, stream, pr);
  if (rc != HT_OK) return rc;
  if ((margin == nullptr || margin_ord == nullptr) && pr.evals > 0) return HT_ERR_INVALID_ARGUMENT;
  return launch_any<MODE_MARGINMAP>(p, pr, margin, margin_ord);
}

int ht_forest_reachability_f32(const ht_forest_problem *p, const float *x, const float *thr, const int64_t *ord,
                               int64_t *counts, void *workspace, size_t workspace_bytes, uint32_t *status_word,
                               ht_stream_t stream) {
  Prepared pr;
  const int rc = prepare<float>(p, x, thr, ord, nullptr, false, workspace, workspace_bytes, status_word, stream, pr);
  if (rc != HT_OK) return rc;
  if (counts == nullptr && pr.args.T > 0) return HT_ERR_INVALID_ARGUMENT;
  if (pr.args.T * pr.args.L > 0)
    HT_CUDA_TRY(cudaMemsetAsync(counts, 0, sizeof(int64_t) * (size_t)(pr.args.T * pr.args.L), pr.stream));
  return launch_any<MODE_REACH, float>(p, pr, nullptr, counts);
}

int ht_forest_backward_f32(const ht_forest_problem *p, const float *x, const float *thr, const int64_t *ord,
                           const float *w, const float *g, float *gx, float *gthr, float *gw, void *workspace,
                           size_t workspace_bytes, uint32_t *status_word, ht_stream_t stream) {
  Prepared pr;
  const int rc = prepare(p, x, thr, ord, w, true, workspace, workspace_bytes, status_word, stream, pr);
  if (rc != HT_OK) return rc;
  if (g == nullptr && pr.evals * p->M > 0) return HT_ERR_INVALID_ARGUMENT;
  const ForestArgs &a = pr.args;
  // The parameter gradients are sums into cleared memory on every path.  The x gradient is cleared only for the
  // paths that add into it: from a kept traversal it is written tile by tile, every element once.
  int crc = clear_gradients(pr, static_cast<float *>(nullptr), gthr, gw);
  if (crc != HT_OK) return crc;
  if (pr.evals * a.M == 0 || (gx == nullptr && gthr == nullptr && gw == nullptr))
    return clear_gradients(pr, gx, static_cast<float *>(nullptr), static_cast<float *>(nullptr));

  {
    // Tile kernels when the shape qualifies; with room for the evaluation records in the workspace
    // they serve both modes (that path is fixed-order), without it only the default mode.
    unsigned char *ws = static_cast<unsigned char *>(workspace);
    const size_t records_at = ordinals_bytes(p) + forward_tiled_workspace_bytes(p);
    const size_t eval_bytes = backward_records_bytes(p);
    void *eval_records = eval_bytes > 0 && workspace_bytes >= records_at + eval_bytes ? ws + records_at : nullptr;
    if ((p->flags & HT_SAVED_FORWARD) != 0 && eval_records != nullptr) {
      // the records of the forward that ran on these inputs are still there: no tree is walked again
      const int src = backward_saved(p, a.ord, w, g, gx, gthr, gw, eval_records, pr.stream);
      if (src != HT_ERR_UNSUPPORTED) return src;
    }
    crc = clear_gradients(pr, gx, static_cast<float *>(nullptr), static_cast<float *>(nullptr));
    if (crc != HT_OK) return crc;
    const int trc = backward_tiled(p, x, thr, a.ord, w, g, gx, gthr, gw, ws + ordinals_bytes(p), eval_records,
                                   status_word, pr.stream);
    if (trc != HT_ERR_UNSUPPORTED) return trc;
    const int mrc = backward_tiled_multi(p, x, thr, a.ord, w, g, gx, gthr, gw, ws + ordinals_bytes(p),
                                         forward_tiled_workspace_bytes(p), status_word, pr.stream);
    if (mrc != HT_ERR_UNSUPPORTED) return mrc;
  }
  return backward_any(p, pr, g, gx, gthr, gw);
}

/* ---- double precision: the any-shape kernels instantiated for double ---------------------------------------- */

int ht_forest_forward_f64(const ht_forest_problem *p, const double *x, const double *thr, const int64_t *ord,
                          const double *w, double *out, void *workspace, size_t workspace_bytes, uint32_t *status_word,
                          ht_stream_t stream) {
  PreparedOf<double> pr;
  const int rc = prepare(p, x, thr, ord, w, true, workspace, workspace_bytes, status_word, stream, pr);
  if (rc != HT_OK) return rc;
  if (pr.evals * p->M == 0) return HT_OK;
  if (out == nullptr) return HT_ERR_INVALID_ARGUMENT;
  return launch_any<MODE_FORWARD>(p, pr, out, nullptr);
}

int ht_forest_leafmap_f64(const ht_forest_problem *p, const double *x, const double *thr, const int64_t *ord, int64_t *leaf,
                          void *workspace, size_t workspace_bytes, uint32_t *status_word, ht_stream_t stream) {
  PreparedOf<double> pr;
  const int rc = prepare<double>(p, x, thr, ord, nullptr, false, workspace, workspace_bytes, status_word, stream, pr);
  if (rc != HT_OK) return rc;
  if (leaf == nullptr && pr.evals > 0) return HT_ERR_INVALID_ARGUMENT;
  return launch_any<MODE_LEAFMAP, double>(p, pr, nullptr, leaf);
}

int ht_forest_marginmap_f64(const ht_forest_problem *p, const double *x, const double *thr, const int64_t *ord,
                            double *margin, int64_t *margin_ord, void *workspace, size_t workspace_bytes,
                            uint32_t *status_word, ht_stream_t stream) {
  PreparedOf<double> pr;
  const int rc = prepare<double>(p, x, thr, ord, nullptr, false, workspace, workspace_bytes, status_word, stream, pr);
  if (rc != HT_OK) return rc;
  if ((margin == nullptr || margin_ord == nullptr) && pr.evals > 0) return HT_ERR_INVALID_ARGUMENT;
  return launch_any<MODE_MARGINMAP>(p, pr, margin, margin_ord);
}

int ht_forest_reachability_f64(const ht_forest_problem *p, const double *x, const double *thr, const int64_t *ord,
                               int64_t *counts, void *workspace, size_t workspace_bytes, uint32_t *status_word,
                               ht_stream_t stream) {
  PreparedOf<double> pr;
  const int rc = prepare<double>(p, x, thr, ord, nullptr, false, workspace, workspace_bytes, status_word, stream, pr);
  if (rc != HT_OK) return rc;
  if (counts == nullptr && pr.args.T > 0) return HT_ERR_INVALID_ARGUMENT;
  if (pr.args.T * pr.args.L > 0)
    HT_CUDA_TRY(cudaMemsetAsync(counts, 0, sizeof(int64_t) * (size_t)(pr.args.T * pr.args.L), pr.stream));
  return launch_any<MODE_REACH, double>(p, pr, nullptr, counts);
}

int ht_forest_backward_f64(const ht_forest_problem *p, const double *x, const double *thr, const int64_t *ord,
                           const double *w, const double *g, double *gx, double *gthr, double *gw, void *workspace,
                           size_t workspace_bytes, uint32_t *status_word, ht_stream_t stream) {
  PreparedOf<double> pr;
  const int rc = prepare(p, x, thr, ord, w, true, workspace, workspace_bytes, status_word, stream, pr);
  if (rc != HT_OK) return rc;
  if (g == nullptr && pr.evals * p->M > 0) return HT_ERR_INVALID_ARGUMENT;
  const int crc = clear_gradients(pr, gx, gthr, gw);
  if (crc != HT_OK) return crc;
  if (pr.evals * p->M == 0 || (gx == nullptr && gthr == nullptr && gw == nullptr)) return HT_OK;
  return backward_any(p, pr, g, gx, gthr, gw);
}

}  // extern "C"
