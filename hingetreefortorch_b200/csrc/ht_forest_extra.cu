// Hinge tries, and the "touched" masks behind the sparse-gradient operators.
//
// Trie: every decision on the root-to-leaf path contributes, with one weight row per internal
// vertex: out[i,j,k,m] = sum over depth d ascending of |margin_d| * w[j, vertex_d, m].  The
// reference evaluates tries on the CPU only (hingetrie.cpp:33-267; a CUDA tensor gets an empty
// result, :286-288); this is the same arithmetic on the GPU, forward in the same order.
//
// Sparse gradients: the reference's sparse backward returns COO tensors holding exactly the
// gradient elements some (sample, tree, position) contributed to, found with a device hash table
// (hingetree_sparse_gpu.cu:61-101).  Here the dense backward computes the values and the kernel
// below marks the contributed-to elements in byte masks; the host binding compacts mask and
// values into the (sorted, duplicate-free) COO form.  No hash table, no overflow case.
#include "ht_common.cuh"

namespace ht {

namespace {

constexpr int kBlock = 256;

template <typename Real>
struct ExtraArgsOf {
  const Real *x;
  const Real *thr;
  const int32_t *ord;
  const Real *w;
  int64_t B, C, K, T, N, L, M;
  int depth;
};

template <typename Real>
__device__ __forceinline__ void split3(const ExtraArgsOf<Real> &a, int64_t e, int64_t &i, int64_t &j, int64_t &k) {
  const int64_t ij = e / a.K;
  k = e - ij * a.K;
  i = ij / a.T;
  j = ij - i * a.T;
}

template <typename Real>
__global__ void __launch_bounds__(kBlock) trie_forward_kernel(ExtraArgsOf<Real> a, Real *__restrict__ out) {
  const int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= a.B * a.T * a.K) return;
  int64_t i, j, k;
  split3(a, e, i, j, k);
  const Real *xb = a.x + i * a.C * a.K + k;
  const Real *thr = a.thr + j * a.N;
  const int32_t *ord = a.ord + j * a.N;
  for (int64_t m = 0; m < a.M; ++m) {
    Real acc = (Real)0;
    uint32_t v = 0;
    for (int d = 0; d < a.depth; ++d) {  // the walk is repeated per output: depth is small, M usually 1
      const Real margin = __ldg(xb + (int64_t)ord[v] * a.K) - thr[v];
      acc = add_rn(acc, mul_rn(abs_of(margin), __ldg(a.w + (j * a.N + v) * a.M + m)));
      v = 2 * v + 1 + (margin > (Real)0 ? 1u : 0u);
    }
    out[e * a.M + m] = acc;
  }
}

template <typename Real>
__global__ void __launch_bounds__(kBlock) trie_backward_kernel(ExtraArgsOf<Real> a, const Real *__restrict__ g, Real *gx,
                                                               Real *gthr, Real *gw) {
  const int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= a.B * a.T * a.K) return;
  int64_t i, j, k;
  split3(a, e, i, j, k);
  const Real *xb = a.x + i * a.C * a.K + k;
  const Real *thr = a.thr + j * a.N;
  const int32_t *ord = a.ord + j * a.N;
  uint32_t v = 0;
  for (int d = 0; d < a.depth; ++d) {
    const int c = ord[v];
    const Real margin = __ldg(xb + (int64_t)c * a.K) - thr[v];
    const Real s = sign_of(margin), am = abs_of(margin);
    Real acc = (Real)0;
    for (int64_t m = 0; m < a.M; ++m) {
      const Real gm = __ldg(g + e * a.M + m);
      acc = add_rn(acc, mul_rn(mul_rn(s, __ldg(a.w + (j * a.N + v) * a.M + m)), gm));
      if (gw != nullptr) atomicAdd(gw + (j * a.N + v) * a.M + m, mul_rn(am, gm));
    }
    if (gx != nullptr) atomicAdd(gx + (i * a.C + c) * a.K + k, acc);
    if (gthr != nullptr) atomicAdd(gthr + j * a.N + v, -acc);
    v = 2 * v + 1 + (margin > (Real)0 ? 1u : 0u);
  }
}

// Marks the elements of the x, threshold and leaf-weight gradients that receive a contribution.
template <int KIND, typename Real>
__global__ void __launch_bounds__(kBlock) touched_kernel(ExtraArgsOf<Real> a, uint8_t *tx, uint8_t *tthr, uint8_t *tw) {
  const int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= a.B * a.T * a.K) return;
  int64_t i, j, k;
  split3(a, e, i, j, k);
  const PlainFeatureOf<Real> feat{a.x + i * a.C * a.K + k, a.K};
  const PathOf<Real> p = traverse<KIND>(feat, a.thr + j * a.N, a.ord + j * a.N, a.depth);
  if (tx != nullptr) tx[(i * a.C + a.ord[j * a.N + p.vertex]) * a.K + k] = 1;
  if (tthr != nullptr) tthr[j * a.N + p.vertex] = 1;
  if (tw != nullptr)
    for (int64_t m = 0; m < a.M; ++m) tw[(j * a.L + p.key) * a.M + m] = 1;
}

inline unsigned blocks_for(int64_t n) { return (unsigned)((n + kBlock - 1) / kBlock); }

template <typename Real>
int prepare(const ht_forest_problem *p, bool trie, const Real *x, const Real *thr, const int64_t *ord, const Real *w,
            void *workspace, size_t workspace_bytes, uint32_t *status_word, cudaStream_t stream, ExtraArgsOf<Real> &a) {
  const int rc = check_forest_problem(p);
  if (rc != HT_OK) return rc;
  if (trie && p->kind != TREE) return HT_ERR_INVALID_ARGUMENT;
  a.N = threshold_count(p->kind, p->depth);
  a.L = trie ? a.N : ((int64_t)1) << p->depth;  // rows of w: internal vertices for a trie, leaves otherwise
  const int64_t decisions = p->T * a.N;
  if ((x == nullptr && p->B * p->C * p->K > 0) || ((thr == nullptr || ord == nullptr) && decisions > 0))
    return HT_ERR_INVALID_ARGUMENT;
  const size_t need = align_up((size_t)decisions * sizeof(int32_t), 256) + 256;
  if (workspace == nullptr || workspace_bytes < need || (reinterpret_cast<uintptr_t>(workspace) & 255u) != 0)
    return HT_ERR_WORKSPACE;
  a.x = x;
  a.thr = thr;
  a.w = w;
  a.ord = static_cast<const int32_t *>(workspace);
  a.B = p->B;
  a.C = p->C;
  a.K = p->K;
  a.T = p->T;
  a.M = p->M;
  a.depth = p->depth;
  return pack_ordinals(ord, decisions, p->C, static_cast<int32_t *>(workspace), status_word, stream);
}

int clear_bytes(void *ptr, int64_t bytes, cudaStream_t stream) {
  if (ptr != nullptr && bytes > 0) HT_CUDA_TRY(cudaMemsetAsync(ptr, 0, (size_t)bytes, stream));
  return HT_OK;
}

}  // namespace
}  // namespace ht

using namespace ht;

namespace ht {
namespace {

template <typename Real>
int trie_forward(const ht_forest_problem *p, const Real *x, const Real *thr, const int64_t *ord, const Real *w, Real *out,
                 void *workspace, size_t workspace_bytes, uint32_t *status_word, ht_stream_t stream) {
  ExtraArgsOf<Real> a;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const int rc = prepare<Real>(p, true, x, thr, ord, w, workspace, workspace_bytes, status_word, s, a);
  if (rc != HT_OK) return rc;
  const int64_t evals = a.B * a.T * a.K;
  if (evals * a.M == 0) return HT_OK;
  if (out == nullptr || w == nullptr) return HT_ERR_INVALID_ARGUMENT;
  trie_forward_kernel<Real><<<blocks_for(evals), kBlock, 0, s>>>(a, out);
  HT_CHECK_LAUNCH();
  return HT_OK;
}

template <typename Real>
int trie_backward(const ht_forest_problem *p, const Real *x, const Real *thr, const int64_t *ord, const Real *w, const Real *g,
                  Real *gx, Real *gthr, Real *gw, void *workspace, size_t workspace_bytes, uint32_t *status_word,
                  ht_stream_t stream) {
  ExtraArgsOf<Real> a;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const int rc = prepare<Real>(p, true, x, thr, ord, w, workspace, workspace_bytes, status_word, s, a);
  if (rc != HT_OK) return rc;
  const int64_t size = (int64_t)sizeof(Real);
  int crc;
  if ((crc = clear_bytes(gx, size * a.B * a.C * a.K, s)) != HT_OK) return crc;
  if ((crc = clear_bytes(gthr, size * a.T * a.N, s)) != HT_OK) return crc;
  if ((crc = clear_bytes(gw, size * a.T * a.N * a.M, s)) != HT_OK) return crc;
  const int64_t evals = a.B * a.T * a.K;
  if (evals * a.M == 0 || (gx == nullptr && gthr == nullptr && gw == nullptr)) return HT_OK;
  if (g == nullptr || w == nullptr) return HT_ERR_INVALID_ARGUMENT;
  trie_backward_kernel<Real><<<blocks_for(evals), kBlock, 0, s>>>(a, g, gx, gthr, gw);
  HT_CHECK_LAUNCH();
  return HT_OK;
}

template <typename Real>
int touched(const ht_forest_problem *p, const Real *x, const Real *thr, const int64_t *ord, uint8_t *touched_x,
            uint8_t *touched_thr, uint8_t *touched_w, void *workspace, size_t workspace_bytes, uint32_t *status_word,
            ht_stream_t stream) {
  ExtraArgsOf<Real> a;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const int rc = prepare<Real>(p, false, x, thr, ord, nullptr, workspace, workspace_bytes, status_word, s, a);
  if (rc != HT_OK) return rc;
  int crc;
  if ((crc = clear_bytes(touched_x, a.B * a.C * a.K, s)) != HT_OK) return crc;
  if ((crc = clear_bytes(touched_thr, a.T * a.N, s)) != HT_OK) return crc;
  if ((crc = clear_bytes(touched_w, a.T * a.L * a.M, s)) != HT_OK) return crc;
  const int64_t evals = a.B * a.T * a.K;
  if (evals == 0) return HT_OK;
  if (p->kind == TREE)
    touched_kernel<TREE, Real><<<blocks_for(evals), kBlock, 0, s>>>(a, touched_x, touched_thr, touched_w);
  else
    touched_kernel<FERN, Real><<<blocks_for(evals), kBlock, 0, s>>>(a, touched_x, touched_thr, touched_w);
  HT_CHECK_LAUNCH();
  return HT_OK;
}

}  // namespace
}  // namespace ht

extern "C" {

int ht_trie_forward_f32(const ht_forest_problem *p, const float *x, const float *thr, const int64_t *ord, const float *w,
                        float *out, void *workspace, size_t workspace_bytes, uint32_t *status_word, ht_stream_t stream) {
  return trie_forward<float>(p, x, thr, ord, w, out, workspace, workspace_bytes, status_word, stream);
}
int ht_trie_forward_f64(const ht_forest_problem *p, const double *x, const double *thr, const int64_t *ord, const double *w,
                        double *out, void *workspace, size_t workspace_bytes, uint32_t *status_word, ht_stream_t stream) {
  return trie_forward<double>(p, x, thr, ord, w, out, workspace, workspace_bytes, status_word, stream);
}

int ht_trie_backward_f32(const ht_forest_problem *p, const float *x, const float *thr, const int64_t *ord, const float *w,
                         const float *g, float *gx, float *gthr, float *gw, void *workspace, size_t workspace_bytes,
                         uint32_t *status_word, ht_stream_t stream) {
  return trie_backward<float>(p, x, thr, ord, w, g, gx, gthr, gw, workspace, workspace_bytes, status_word, stream);
}
int ht_trie_backward_f64(const ht_forest_problem *p, const double *x, const double *thr, const int64_t *ord, const double *w,
                         const double *g, double *gx, double *gthr, double *gw, void *workspace, size_t workspace_bytes,
                         uint32_t *status_word, ht_stream_t stream) {
  return trie_backward<double>(p, x, thr, ord, w, g, gx, gthr, gw, workspace, workspace_bytes, status_word, stream);
}

int ht_forest_touched_f32(const ht_forest_problem *p, const float *x, const float *thr, const int64_t *ord,
                          uint8_t *touched_x, uint8_t *touched_thr, uint8_t *touched_w, void *workspace,
                          size_t workspace_bytes, uint32_t *status_word, ht_stream_t stream) {
  return touched<float>(p, x, thr, ord, touched_x, touched_thr, touched_w, workspace, workspace_bytes, status_word, stream);
}
int ht_forest_touched_f64(const ht_forest_problem *p, const double *x, const double *thr, const int64_t *ord,
                          uint8_t *touched_x, uint8_t *touched_thr, uint8_t *touched_w, void *workspace,
                          size_t workspace_bytes, uint32_t *status_word, ht_stream_t stream) {
  return touched<double>(p, x, thr, ord, touched_x, touched_thr, touched_w, workspace, workspace_bytes, status_word, stream);
}

}  // extern "C"
