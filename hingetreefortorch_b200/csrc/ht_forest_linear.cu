// Image + vector "fusion" forests and forests followed by a linear layer over the tree dimension.
//
// Both families share one scheme: a `paths` kernel walks every (sample, tree, position) once and
// stores the signed margin, leaf key and deciding vertex; forward and backward kernels consume
// those records.  The fused-linear forward then adds, per output element, the bias and the terms
// (|margin| * L[o,j]) * w[j,leaf,m] for j ascending -- the reference CPU order
// (hingetree_fused_linear.cpp:154-181), so the result is deterministic and equal to it bit for
// bit (the reference GPU kernel scatters the same terms with atomics in arbitrary order).
#include <algorithm>

#include "ht_common.cuh"

namespace ht {

namespace {

constexpr int kBlock = 256;

template <typename Real>
struct FusionArgsOf {
  const Real *img;   // [B, C, K]
  const Real *vec;   // [B, Cv] or null
  const Real *thr;
  const int32_t *ord;
  const Real *w;
  int64_t B, C, Cv, K, T, N, L, M;
  int depth;
};

template <typename Real>
struct PathRecordsOf {
  Real *margin;    // signed
  int32_t *leaf;
  int32_t *vertex;
};

template <typename Real>
__device__ __forceinline__ void split3(const FusionArgsOf<Real> &a, int64_t e, int64_t &i, int64_t &j, int64_t &k) {
  const int64_t ij = e / a.K;
  k = e - ij * a.K;
  i = ij / a.T;
  j = ij - i * a.T;
}

template <int KIND, typename Real>
__device__ __forceinline__ PathOf<Real> walk(const FusionArgsOf<Real> &a, int64_t i, int64_t j, int64_t k) {
  if (a.vec != nullptr) {
    const FusionFeatureOf<Real> feat{a.img + i * a.C * a.K + k, a.K, a.vec + i * a.Cv, (int)a.C};
    return traverse<KIND>(feat, a.thr + j * a.N, a.ord + j * a.N, a.depth);
  }
  const PlainFeatureOf<Real> feat{a.img + i * a.C * a.K + k, a.K};
  return traverse<KIND>(feat, a.thr + j * a.N, a.ord + j * a.N, a.depth);
}

// Destination of the data gradient of feature c of sample i at position k: image or vector.
template <typename Real>
__device__ __forceinline__ Real *data_grad_slot(const FusionArgsOf<Real> &a, Real *gimg, Real *gvec, int64_t i, int c,
                                                 int64_t k) {
  if (a.vec == nullptr || c < a.C) return gimg == nullptr ? nullptr : gimg + (i * a.C + c) * a.K + k;
  return gvec == nullptr ? nullptr : gvec + i * a.Cv + (c - a.C);
}

template <int KIND, typename Real>
__global__ void __launch_bounds__(kBlock) fusion_forward_kernel(FusionArgsOf<Real> a, Real *__restrict__ out) {
  const int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= a.B * a.T * a.K) return;
  int64_t i, j, k;
  split3(a, e, i, j, k);
  const PathOf<Real> p = walk<KIND>(a, i, j, k);
  const Real am = abs_of(p.margin);
  const Real *wl = a.w + (j * a.L + p.key) * a.M;
  for (int64_t m = 0; m < a.M; ++m) out[e * a.M + m] = am * __ldg(wl + m);
}

template <int KIND, typename Real>
__global__ void __launch_bounds__(kBlock) fusion_backward_kernel(FusionArgsOf<Real> a, const Real *__restrict__ g, Real *gimg,
                                                                 Real *gvec, Real *gthr, Real *gw) {
  const int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= a.B * a.T * a.K) return;
  int64_t i, j, k;
  split3(a, e, i, j, k);
  const PathOf<Real> p = walk<KIND>(a, i, j, k);
  const Real s = sign_of(p.margin), am = abs_of(p.margin);
  const Real *wl = a.w + (j * a.L + p.key) * a.M;
  const Real *gl = g + e * a.M;
  Real acc = (Real)0;
  for (int64_t m = 0; m < a.M; ++m) {
    const Real gm = __ldg(gl + m);
    acc = add_rn(acc, mul_rn(mul_rn(s, __ldg(wl + m)), gm));
    if (gw != nullptr) atomicAdd(gw + (j * a.L + p.key) * a.M + m, mul_rn(am, gm));
  }
  Real *slot = data_grad_slot(a, gimg, gvec, i, a.ord[j * a.N + p.vertex], k);
  if (slot != nullptr) atomicAdd(slot, acc);
  if (gthr != nullptr) atomicAdd(gthr + j * a.N + p.vertex, -acc);
}

template <int KIND, typename Real>
__global__ void __launch_bounds__(kBlock) paths_kernel(FusionArgsOf<Real> a, PathRecordsOf<Real> r) {
  const int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= a.B * a.T * a.K) return;
  int64_t i, j, k;
  split3(a, e, i, j, k);
  const PathOf<Real> p = walk<KIND>(a, i, j, k);
  r.margin[e] = p.margin;
  r.leaf[e] = (int32_t)p.key;
  r.vertex[e] = (int32_t)p.vertex;
}

// out[i,o,k,m] = bias[o] + sum over j ascending of (|margin| * L[o,j]) * w[j,leaf,m]; one thread per element.
template <typename Real>
__global__ void __launch_bounds__(kBlock) linear_forward_kernel(FusionArgsOf<Real> a, PathRecordsOf<Real> r, const Real *__restrict__ lin,
                                                                const Real *__restrict__ bias, int64_t O,
                                                                Real *__restrict__ out) {
  const int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= a.B * O * a.K * a.M) return;
  const int64_t m = e % a.M;
  const int64_t k = (e / a.M) % a.K;
  const int64_t o = (e / (a.M * a.K)) % O;
  const int64_t i = e / (a.M * a.K * O);
  Real acc = __ldg(bias + o);
  for (int64_t j = 0; j < a.T; ++j) {
    const int64_t p = (i * a.T + j) * a.K + k;
    const Real scale = mul_rn(abs_of(r.margin[p]), __ldg(lin + o * a.T + j));
    acc = add_rn(acc, mul_rn(scale, __ldg(a.w + (j * a.L + r.leaf[p]) * a.M + m)));
  }
  out[e] = acc;
}

// Data, threshold and leaf-weight gradients through the linear layer; one thread per (i, j, k).
template <typename Real>
__global__ void __launch_bounds__(kBlock) linear_backward_kernel(FusionArgsOf<Real> a, PathRecordsOf<Real> r, const Real *__restrict__ lin,
                                                                 const Real *__restrict__ g, int64_t O, Real *gimg,
                                                                 Real *gvec, Real *gthr, Real *gw) {
  const int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= a.B * a.T * a.K) return;
  int64_t i, j, k;
  split3(a, e, i, j, k);
  const Real margin = r.margin[e];
  const int64_t leaf = r.leaf[e], vertex = r.vertex[e];
  const Real s = sign_of(margin), am = abs_of(margin);
  const Real *wl = a.w + (j * a.L + leaf) * a.M;
  // the gradient arriving at this tree's output m: the upstream gradients of all linear outputs, weighted; then the
  // tree's own backward with it (one reduction per leaf-weight element, not one per linear output)
  Real acc = (Real)0;
  for (int64_t m = 0; m < a.M; ++m) {
    Real through = (Real)0;
    for (int64_t o = 0; o < O; ++o)
      through = add_rn(through, mul_rn(__ldg(lin + o * a.T + j), __ldg(g + ((i * O + o) * a.K + k) * a.M + m)));
    acc = add_rn(acc, mul_rn(mul_rn(s, __ldg(wl + m)), through));
    if (gw != nullptr) atomicAdd(gw + (j * a.L + leaf) * a.M + m, mul_rn(am, through));
  }
  Real *slot = data_grad_slot(a, gimg, gvec, i, a.ord[j * a.N + vertex], k);
  if (slot != nullptr) atomicAdd(slot, acc);
  if (gthr != nullptr) atomicAdd(gthr + j * a.N + vertex, -acc);
}

// Gradient of the linear weights: gL[o,j] = sum over (i,k,m) of (|margin| * w[j,leaf,m]) * g[i,o,k,m].
// CTA = (tree j, a slice of the positions): its threads walk the slice ONCE, keeping the sums of up to kLinearOutputs
// linear outputs in registers, reduce them over the CTA and add the result to glin (cleared by the caller) with one
// reduction per output.
constexpr int kLinearOutputs = 16;

template <typename Real>
__global__ void __launch_bounds__(kBlock) linear_weight_grad_kernel(FusionArgsOf<Real> a, PathRecordsOf<Real> r, const Real *__restrict__ g,
                                                                    int64_t O, Real *glin) {
  __shared__ Real partial[kBlock / 32][kLinearOutputs];
  const int64_t j = blockIdx.x;
  const int64_t P = a.B * a.K;
  const int64_t per_slice = (P + gridDim.y - 1) / gridDim.y;
  const int64_t first = (int64_t)blockIdx.y * per_slice, last = min(P, first + per_slice);
  for (int64_t o0 = 0; o0 < O; o0 += kLinearOutputs) {
    const int outputs = (int)min((int64_t)kLinearOutputs, O - o0);
    Real sum[kLinearOutputs];
#pragma unroll
    for (int u = 0; u < kLinearOutputs; ++u) sum[u] = (Real)0;
    for (int64_t p = first + threadIdx.x; p < last; p += kBlock) {
      const int64_t i = p / a.K, k = p - i * a.K;
      const int64_t e = (i * a.T + j) * a.K + k;
      const Real am = abs_of(r.margin[e]);
      const Real *wl = a.w + (j * a.L + r.leaf[e]) * a.M;
      for (int64_t m = 0; m < a.M; ++m) {
        const Real scaled = mul_rn(am, __ldg(wl + m));
#pragma unroll
        for (int u = 0; u < kLinearOutputs; ++u)
          if (u < outputs) sum[u] = add_rn(sum[u], mul_rn(scaled, __ldg(g + ((i * O + o0 + u) * a.K + k) * a.M + m)));
      }
    }
#pragma unroll
    for (int u = 0; u < kLinearOutputs; ++u) {
      Real v = sum[u];
      for (int off = 16; off > 0; off >>= 1) v += __shfl_down_sync(0xffffffffu, v, off);
      if ((threadIdx.x & 31) == 0) partial[threadIdx.x >> 5][u] = v;
    }
    __syncthreads();
    if ((int)threadIdx.x < outputs) {
      Real total = (Real)0;
      for (int wi = 0; wi < kBlock / 32; ++wi) total += partial[wi][threadIdx.x];
      atomicAdd(glin + (o0 + threadIdx.x) * a.T + j, total);
    }
    __syncthreads();
  }
}

inline unsigned blocks_for(int64_t n) { return (unsigned)((n + kBlock - 1) / kBlock); }

template <typename Real>
struct PreparedOf {
  FusionArgsOf<Real> args;
  PathRecordsOf<Real> records;
  cudaStream_t stream;
  int64_t evals;
};

size_t ordinal_bytes(const ht_forest_problem *p) {
  return align_up((size_t)(p->T * threshold_count(p->kind, p->depth)) * sizeof(int32_t), 256);
}

size_t record_bytes(const ht_forest_problem *p, size_t real_bytes) { return align_up((size_t)(p->B * p->T * p->K) * real_bytes, 256); }

template <typename Real>
int prepare(const ht_forest_problem *p, const Real *img, const Real *vec, int64_t Cv, const Real *thr,
            const int64_t *ord, const Real *w, bool with_records, void *workspace, size_t workspace_bytes,
            uint32_t *status_word, ht_stream_t stream, PreparedOf<Real> &out) {
  const int rc = check_forest_problem(p);
  if (rc != HT_OK) return rc;
  if (Cv < 0 || (vec == nullptr && p->B * Cv > 0)) return HT_ERR_INVALID_ARGUMENT;
  if (p->C + Cv > 0x7fffffff) return HT_ERR_UNSUPPORTED;
  const int64_t decisions = p->T * threshold_count(p->kind, p->depth);
  if ((img == nullptr && p->B * p->C * p->K > 0) || ((thr == nullptr || ord == nullptr) && decisions > 0) ||
      (w == nullptr && p->T * p->M > 0))
    return HT_ERR_INVALID_ARGUMENT;
  const size_t need = ordinal_bytes(p) + (with_records ? record_bytes(p, sizeof(Real)) + 2 * record_bytes(p, 4) : 0) + 256;
  if (workspace == nullptr || workspace_bytes < need || (reinterpret_cast<uintptr_t>(workspace) & 255u) != 0)
    return HT_ERR_WORKSPACE;
  unsigned char *ws = static_cast<unsigned char *>(workspace);
  FusionArgsOf<Real> &a = out.args;
  a.img = img;
  a.vec = Cv > 0 ? vec : nullptr;
  a.thr = thr;
  a.ord = reinterpret_cast<const int32_t *>(ws);
  a.w = w;
  a.B = p->B;
  a.C = p->C;
  a.Cv = Cv;
  a.K = p->K;
  a.T = p->T;
  a.M = p->M;
  a.depth = p->depth;
  a.N = threshold_count(p->kind, p->depth);
  a.L = ((int64_t)1) << p->depth;
  out.stream = reinterpret_cast<cudaStream_t>(stream);
  out.evals = p->B * p->T * p->K;
  if (with_records) {
    out.records.margin = reinterpret_cast<Real *>(ws + ordinal_bytes(p));
    out.records.leaf = reinterpret_cast<int32_t *>(ws + ordinal_bytes(p) + record_bytes(p, sizeof(Real)));
    out.records.vertex = reinterpret_cast<int32_t *>(ws + ordinal_bytes(p) + record_bytes(p, sizeof(Real)) + record_bytes(p, 4));
  }
  return pack_ordinals(ord, decisions, p->C + Cv, reinterpret_cast<int32_t *>(ws), status_word, out.stream);
}

template <typename Real>
int run_paths(const ht_forest_problem *p, const PreparedOf<Real> &pr) {
  if (pr.evals == 0) return HT_OK;
  if (p->kind == TREE)
    paths_kernel<TREE, Real><<<blocks_for(pr.evals), kBlock, 0, pr.stream>>>(pr.args, pr.records);
  else
    paths_kernel<FERN, Real><<<blocks_for(pr.evals), kBlock, 0, pr.stream>>>(pr.args, pr.records);
  HT_CHECK_LAUNCH();
  return HT_OK;
}

template <typename Real>
int clear(Real *ptr, int64_t count, cudaStream_t stream) {
  if (ptr != nullptr && count > 0) HT_CUDA_TRY(cudaMemsetAsync(ptr, 0, sizeof(Real) * (size_t)count, stream));
  return HT_OK;
}

}  // namespace
}  // namespace ht

namespace ht {
namespace {

template <typename Real>
int fusion_forward(const ht_forest_problem *p, const Real *img, const Real *vec, int64_t vec_channels, const Real *thr,
                   const int64_t *ord, const Real *w, Real *out, void *workspace, size_t workspace_bytes, uint32_t *status_word,
                   ht_stream_t stream) {
  PreparedOf<Real> pr;
  const int rc = prepare<Real>(p, img, vec, vec_channels, thr, ord, w, false, workspace, workspace_bytes, status_word, stream, pr);
  if (rc != HT_OK) return rc;
  if (pr.evals * p->M == 0) return HT_OK;
  if (out == nullptr) return HT_ERR_INVALID_ARGUMENT;
  if (p->kind == TREE)
    fusion_forward_kernel<TREE, Real><<<blocks_for(pr.evals), kBlock, 0, pr.stream>>>(pr.args, out);
  else
    fusion_forward_kernel<FERN, Real><<<blocks_for(pr.evals), kBlock, 0, pr.stream>>>(pr.args, out);
  HT_CHECK_LAUNCH();
  return HT_OK;
}

template <typename Real>
int fusion_backward(const ht_forest_problem *p, const Real *img, const Real *vec, int64_t vec_channels, const Real *thr,
                    const int64_t *ord, const Real *w, const Real *g, Real *gimg, Real *gvec, Real *gthr, Real *gw,
                    void *workspace, size_t workspace_bytes, uint32_t *status_word, ht_stream_t stream) {
  PreparedOf<Real> pr;
  const int rc = prepare<Real>(p, img, vec, vec_channels, thr, ord, w, false, workspace, workspace_bytes, status_word, stream, pr);
  if (rc != HT_OK) return rc;
  const FusionArgsOf<Real> &a = pr.args;
  int crc;
  if ((crc = clear(gimg, a.B * a.C * a.K, pr.stream)) != HT_OK) return crc;
  if ((crc = clear(gvec, a.B * a.Cv, pr.stream)) != HT_OK) return crc;
  if ((crc = clear(gthr, a.T * a.N, pr.stream)) != HT_OK) return crc;
  if ((crc = clear(gw, a.T * a.L * a.M, pr.stream)) != HT_OK) return crc;
  if (pr.evals * a.M == 0) return HT_OK;
  if (g == nullptr) return HT_ERR_INVALID_ARGUMENT;
  if (p->kind == TREE)
    fusion_backward_kernel<TREE, Real><<<blocks_for(pr.evals), kBlock, 0, pr.stream>>>(a, g, gimg, gvec, gthr, gw);
  else
    fusion_backward_kernel<FERN, Real><<<blocks_for(pr.evals), kBlock, 0, pr.stream>>>(a, g, gimg, gvec, gthr, gw);
  HT_CHECK_LAUNCH();
  return HT_OK;
}

template <typename Real>
int linear_forward(const ht_forest_problem *p, int64_t out_channels, const Real *img, const Real *vec, int64_t vec_channels,
                   const Real *thr, const int64_t *ord, const Real *w, const Real *lin, const Real *bias, Real *out,
                   void *workspace, size_t workspace_bytes, uint32_t *status_word, ht_stream_t stream) {
  PreparedOf<Real> pr;
  const int rc = prepare<Real>(p, img, vec, vec_channels, thr, ord, w, true, workspace, workspace_bytes, status_word, stream, pr);
  if (rc != HT_OK) return rc;
  if (out_channels < 0) return HT_ERR_INVALID_ARGUMENT;
  const int64_t elements = p->B * out_channels * p->K * p->M;
  if (elements == 0) return HT_OK;
  if (out == nullptr || bias == nullptr || (lin == nullptr && p->T > 0)) return HT_ERR_INVALID_ARGUMENT;
  const int prc = run_paths<Real>(p, pr);
  if (prc != HT_OK) return prc;
  linear_forward_kernel<Real><<<blocks_for(elements), kBlock, 0, pr.stream>>>(pr.args, pr.records, lin, bias, out_channels, out);
  HT_CHECK_LAUNCH();
  return HT_OK;
}

template <typename Real>
int linear_backward(const ht_forest_problem *p, int64_t out_channels, const Real *img, const Real *vec, int64_t vec_channels,
                    const Real *thr, const int64_t *ord, const Real *w, const Real *lin, const Real *g, Real *gimg, Real *gvec,
                    Real *gthr, Real *gw, Real *glin, void *workspace, size_t workspace_bytes, uint32_t *status_word,
                    ht_stream_t stream) {
  PreparedOf<Real> pr;
  const int rc = prepare<Real>(p, img, vec, vec_channels, thr, ord, w, true, workspace, workspace_bytes, status_word, stream, pr);
  if (rc != HT_OK) return rc;
  if (out_channels < 0) return HT_ERR_INVALID_ARGUMENT;
  const FusionArgsOf<Real> &a = pr.args;
  int crc;
  if ((crc = clear(gimg, a.B * a.C * a.K, pr.stream)) != HT_OK) return crc;
  if ((crc = clear(gvec, a.B * a.Cv, pr.stream)) != HT_OK) return crc;
  if ((crc = clear(gthr, a.T * a.N, pr.stream)) != HT_OK) return crc;
  if ((crc = clear(gw, a.T * a.L * a.M, pr.stream)) != HT_OK) return crc;
  if ((crc = clear(glin, out_channels * a.T, pr.stream)) != HT_OK) return crc;
  if (pr.evals * a.M * out_channels == 0) return HT_OK;
  if (g == nullptr || lin == nullptr) return HT_ERR_INVALID_ARGUMENT;
  const int prc = run_paths<Real>(p, pr);
  if (prc != HT_OK) return prc;
  if (gimg != nullptr || gvec != nullptr || gthr != nullptr || gw != nullptr) {
    linear_backward_kernel<Real><<<blocks_for(pr.evals), kBlock, 0, pr.stream>>>(a, pr.records, lin, g, out_channels, gimg, gvec,
                                                                                gthr, gw);
    HT_CHECK_LAUNCH();
  }
  if (glin != nullptr) {
    // enough CTAs to fill the machine: the positions of a tree are split when there are few trees
    const int64_t positions = a.B * a.K;
    const unsigned slices = (unsigned)std::max<int64_t>(1, std::min<int64_t>(std::min<int64_t>((148 * 8 + a.T - 1) / a.T, 65535),
                                                                             (positions + 4 * kBlock - 1) / (4 * kBlock)));
    linear_weight_grad_kernel<Real><<<dim3((unsigned)a.T, slices), kBlock, 0, pr.stream>>>(a, pr.records, g, out_channels, glin);
    HT_CHECK_LAUNCH();
  }
  return HT_OK;
}

size_t linear_workspace(const ht_forest_problem *p, size_t real_bytes) {
  if (check_forest_problem(p) != HT_OK) return 0;
  return ordinal_bytes(p) + record_bytes(p, real_bytes) + 2 * record_bytes(p, 4) + 256;
}

}  // namespace
}  // namespace ht

using namespace ht;

extern "C" {

size_t ht_forest_fusion_workspace_bytes(const ht_forest_problem *p) {
  if (check_forest_problem(p) != HT_OK) return 0;
  return ordinal_bytes(p) + 256;
}

size_t ht_forest_linear_workspace_bytes(const ht_forest_problem *p) { return linear_workspace(p, 4); }
size_t ht_forest_linear_workspace_bytes_f64(const ht_forest_problem *p) { return linear_workspace(p, 8); }

#define HT_FUSION_ENTRIES(SUFFIX, REAL)                                                                                          \
  int ht_forest_fusion_forward_##SUFFIX(const ht_forest_problem *p, const REAL *img, const REAL *vec, int64_t vec_channels,      \
                                        const REAL *thr, const int64_t *ord, const REAL *w, REAL *out, void *workspace,          \
                                        size_t workspace_bytes, uint32_t *status_word, ht_stream_t stream) {                    \
    return fusion_forward<REAL>(p, img, vec, vec_channels, thr, ord, w, out, workspace, workspace_bytes, status_word, stream);   \
  }                                                                                                                              \
  int ht_forest_fusion_backward_##SUFFIX(const ht_forest_problem *p, const REAL *img, const REAL *vec, int64_t vec_channels,     \
                                         const REAL *thr, const int64_t *ord, const REAL *w, const REAL *g, REAL *gimg,          \
                                         REAL *gvec, REAL *gthr, REAL *gw, void *workspace, size_t workspace_bytes,              \
                                         uint32_t *status_word, ht_stream_t stream) {                                            \
    return fusion_backward<REAL>(p, img, vec, vec_channels, thr, ord, w, g, gimg, gvec, gthr, gw, workspace, workspace_bytes,    \
                                 status_word, stream);                                                                           \
  }                                                                                                                              \
  int ht_forest_linear_forward_##SUFFIX(const ht_forest_problem *p, int64_t out_channels, const REAL *img, const REAL *vec,      \
                                        int64_t vec_channels, const REAL *thr, const int64_t *ord, const REAL *w,                \
                                        const REAL *lin, const REAL *bias, REAL *out, void *workspace, size_t workspace_bytes,   \
                                        uint32_t *status_word, ht_stream_t stream) {                                             \
    return linear_forward<REAL>(p, out_channels, img, vec, vec_channels, thr, ord, w, lin, bias, out, workspace,                 \
                                workspace_bytes, status_word, stream);                                                           \
  }                                                                                                                              \
  int ht_forest_linear_backward_##SUFFIX(const ht_forest_problem *p, int64_t out_channels, const REAL *img, const REAL *vec,     \
                                         int64_t vec_channels, const REAL *thr, const int64_t *ord, const REAL *w,               \
                                         const REAL *lin, const REAL *g, REAL *gimg, REAL *gvec, REAL *gthr, REAL *gw,           \
                                         REAL *glin, void *workspace, size_t workspace_bytes, uint32_t *status_word,             \
                                         ht_stream_t stream) {                                                                   \
    return linear_backward<REAL>(p, out_channels, img, vec, vec_channels, thr, ord, w, lin, g, gimg, gvec, gthr, gw, glin,       \
                                 workspace, workspace_bytes, status_word, stream);                                               \
  }

HT_FUSION_ENTRIES(f32, float)
HT_FUSION_ENTRIES(f64, double)
#undef HT_FUSION_ENTRIES

}  // extern "C"
