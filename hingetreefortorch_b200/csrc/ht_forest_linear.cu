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

struct FusionArgs {
  const float *img;   // [B, C, K]
  const float *vec;   // [B, Cv] or null
  const float *thr;
  const int32_t *ord;
  const float *w;
  int64_t B, C, Cv, K, T, N, L, M;
  int depth;
};

struct PathRecords {
  float *margin;    // signed
  int32_t *leaf;
  int32_t *vertex;
};

__device__ __forceinline__ void split3(const FusionArgs &a, int64_t e, int64_t &i, int64_t &j, int64_t &k) {
  const int64_t ij = e / a.K;
  k = e - ij * a.K;
  i = ij / a.T;
  j = ij - i * a.T;
}

template <int KIND>
__device__ __forceinline__ Path walk(const FusionArgs &a, int64_t i, int64_t j, int64_t k) {
  if (a.vec != nullptr) {
    const FusionFeature feat{a.img + i * a.C * a.K + k, a.K, a.vec + i * a.Cv, (int)a.C};
    return traverse<KIND>(feat, a.thr + j * a.N, a.ord + j * a.N, a.depth);
  }
  const PlainFeature feat{a.img + i * a.C * a.K + k, a.K};
  return traverse<KIND>(feat, a.thr + j * a.N, a.ord + j * a.N, a.depth);
}

// Destination of the data gradient of feature c of sample i at position k: image or vector.
__device__ __forceinline__ float *data_grad_slot(const FusionArgs &a, float *gimg, float *gvec, int64_t i, int c,
                                                 int64_t k) {
  if (a.vec == nullptr || c < a.C) return gimg == nullptr ? nullptr : gimg + (i * a.C + c) * a.K + k;
  return gvec == nullptr ? nullptr : gvec + i * a.Cv + (c - a.C);
}

template <int KIND>
__global__ void __launch_bounds__(kBlock) fusion_forward_kernel(FusionArgs a, float *__restrict__ out) {
  const int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= a.B * a.T * a.K) return;
  int64_t i, j, k;
  split3(a, e, i, j, k);
  const Path p = walk<KIND>(a, i, j, k);
  const float am = fabsf(p.margin);
  const float *wl = a.w + (j * a.L + p.key) * a.M;
  for (int64_t m = 0; m < a.M; ++m) out[e * a.M + m] = am * __ldg(wl + m);
}

template <int KIND>
__global__ void __launch_bounds__(kBlock) fusion_backward_kernel(FusionArgs a, const float *__restrict__ g, float *gimg,
                                                                 float *gvec, float *gthr, float *gw) {
  const int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= a.B * a.T * a.K) return;
  int64_t i, j, k;
  split3(a, e, i, j, k);
  const Path p = walk<KIND>(a, i, j, k);
  const float s = sign_of(p.margin), am = fabsf(p.margin);
  const float *wl = a.w + (j * a.L + p.key) * a.M;
  const float *gl = g + e * a.M;
  float acc = 0.0f;
  for (int64_t m = 0; m < a.M; ++m) {
    const float gm = __ldg(gl + m);
    acc = __fadd_rn(acc, __fmul_rn(__fmul_rn(s, __ldg(wl + m)), gm));
    if (gw != nullptr) atomicAdd(gw + (j * a.L + p.key) * a.M + m, __fmul_rn(am, gm));
  }
  float *slot = data_grad_slot(a, gimg, gvec, i, a.ord[j * a.N + p.vertex], k);
  if (slot != nullptr) atomicAdd(slot, acc);
  if (gthr != nullptr) atomicAdd(gthr + j * a.N + p.vertex, -acc);
}

template <int KIND>
__global__ void __launch_bounds__(kBlock) paths_kernel(FusionArgs a, PathRecords r) {
  const int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= a.B * a.T * a.K) return;
  int64_t i, j, k;
  split3(a, e, i, j, k);
  const Path p = walk<KIND>(a, i, j, k);
  r.margin[e] = p.margin;
  r.leaf[e] = (int32_t)p.key;
  r.vertex[e] = (int32_t)p.vertex;
}

// out[i,o,k,m] = bias[o] + sum over j ascending of (|margin| * L[o,j]) * w[j,leaf,m]; one thread per element.
__global__ void __launch_bounds__(kBlock) linear_forward_kernel(FusionArgs a, PathRecords r, const float *__restrict__ lin,
                                                                const float *__restrict__ bias, int64_t O,
                                                                float *__restrict__ out) {
  const int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= a.B * O * a.K * a.M) return;
  const int64_t m = e % a.M;
  const int64_t k = (e / a.M) % a.K;
  const int64_t o = (e / (a.M * a.K)) % O;
  const int64_t i = e / (a.M * a.K * O);
  float acc = __ldg(bias + o);
  for (int64_t j = 0; j < a.T; ++j) {
    const int64_t p = (i * a.T + j) * a.K + k;
    const float scale = __fmul_rn(fabsf(r.margin[p]), __ldg(lin + o * a.T + j));
    acc = __fadd_rn(acc, __fmul_rn(scale, __ldg(a.w + (j * a.L + r.leaf[p]) * a.M + m)));
  }
  out[e] = acc;
}

// Data, threshold and leaf-weight gradients through the linear layer; one thread per (i, j, k).
__global__ void __launch_bounds__(kBlock) linear_backward_kernel(FusionArgs a, PathRecords r, const float *__restrict__ lin,
                                                                 const float *__restrict__ g, int64_t O, float *gimg,
                                                                 float *gvec, float *gthr, float *gw) {
  const int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= a.B * a.T * a.K) return;
  int64_t i, j, k;
  split3(a, e, i, j, k);
  const float margin = r.margin[e];
  const int64_t leaf = r.leaf[e], vertex = r.vertex[e];
  const float s = sign_of(margin), am = fabsf(margin);
  const float *wl = a.w + (j * a.L + leaf) * a.M;
  // the gradient arriving at this tree's output m: the upstream gradients of all linear outputs, weighted; then the
  // tree's own backward with it (one reduction per leaf-weight element, not one per linear output)
  float acc = 0.0f;
  for (int64_t m = 0; m < a.M; ++m) {
    float through = 0.0f;
    for (int64_t o = 0; o < O; ++o)
      through = __fadd_rn(through, __fmul_rn(__ldg(lin + o * a.T + j), __ldg(g + ((i * O + o) * a.K + k) * a.M + m)));
    acc = __fadd_rn(acc, __fmul_rn(__fmul_rn(s, __ldg(wl + m)), through));
    if (gw != nullptr) atomicAdd(gw + (j * a.L + leaf) * a.M + m, __fmul_rn(am, through));
  }
  float *slot = data_grad_slot(a, gimg, gvec, i, a.ord[j * a.N + vertex], k);
  if (slot != nullptr) atomicAdd(slot, acc);
  if (gthr != nullptr) atomicAdd(gthr + j * a.N + vertex, -acc);
}

// Gradient of the linear weights: gL[o,j] = sum over (i,k,m) of (|margin| * w[j,leaf,m]) * g[i,o,k,m].
// CTA = (tree j, a slice of the positions): its threads walk the slice ONCE, keeping the sums of up to kLinearOutputs
// linear outputs in registers, reduce them over the CTA and add the result to glin (cleared by the caller) with one
// reduction per output.
constexpr int kLinearOutputs = 16;

__global__ void __launch_bounds__(kBlock) linear_weight_grad_kernel(FusionArgs a, PathRecords r, const float *__restrict__ g,
                                                                    int64_t O, float *glin) {
  __shared__ float partial[kBlock / 32][kLinearOutputs];
  const int64_t j = blockIdx.x;
  const int64_t P = a.B * a.K;
  const int64_t per_slice = (P + gridDim.y - 1) / gridDim.y;
  const int64_t first = (int64_t)blockIdx.y * per_slice, last = min(P, first + per_slice);
  for (int64_t o0 = 0; o0 < O; o0 += kLinearOutputs) {
    const int outputs = (int)min((int64_t)kLinearOutputs, O - o0);
    float sum[kLinearOutputs];
#pragma unroll
    for (int u = 0; u < kLinearOutputs; ++u) sum[u] = 0.0f;
    for (int64_t p = first + threadIdx.x; p < last; p += kBlock) {
      const int64_t i = p / a.K, k = p - i * a.K;
      const int64_t e = (i * a.T + j) * a.K + k;
      const float am = fabsf(r.margin[e]);
      const float *wl = a.w + (j * a.L + r.leaf[e]) * a.M;
      for (int64_t m = 0; m < a.M; ++m) {
        const float scaled = __fmul_rn(am, __ldg(wl + m));
#pragma unroll
        for (int u = 0; u < kLinearOutputs; ++u)
          if (u < outputs) sum[u] = __fadd_rn(sum[u], __fmul_rn(scaled, __ldg(g + ((i * O + o0 + u) * a.K + k) * a.M + m)));
      }
    }
#pragma unroll
    for (int u = 0; u < kLinearOutputs; ++u) {
      float v = sum[u];
      for (int off = 16; off > 0; off >>= 1) v += __shfl_down_sync(0xffffffffu, v, off);
      if ((threadIdx.x & 31) == 0) partial[threadIdx.x >> 5][u] = v;
    }
    __syncthreads();
    if ((int)threadIdx.x < outputs) {
      float total = 0.0f;
      for (int wi = 0; wi < kBlock / 32; ++wi) total += partial[wi][threadIdx.x];
      atomicAdd(glin + (o0 + threadIdx.x) * a.T + j, total);
    }
    __syncthreads();
  }
}

inline unsigned blocks_for(int64_t n) { return (unsigned)((n + kBlock - 1) / kBlock); }

struct Prepared {
  FusionArgs args;
  PathRecords records;
  cudaStream_t stream;
  int64_t evals;
};

size_t ordinal_bytes(const ht_forest_problem *p) {
  return align_up((size_t)(p->T * threshold_count(p->kind, p->depth)) * sizeof(int32_t), 256);
}

size_t record_bytes(const ht_forest_problem *p) { return align_up((size_t)(p->B * p->T * p->K) * 4, 256); }

int prepare(const ht_forest_problem *p, const float *img, const float *vec, int64_t Cv, const float *thr,
            const int64_t *ord, const float *w, bool with_records, void *workspace, size_t workspace_bytes,
            uint32_t *status_word, ht_stream_t stream, Prepared &out) {
  const int rc = check_forest_problem(p);
  if (rc != HT_OK) return rc;
  if (Cv < 0 || (vec == nullptr && p->B * Cv > 0)) return HT_ERR_INVALID_ARGUMENT;
  if (p->C + Cv > 0x7fffffff) return HT_ERR_UNSUPPORTED;
  const int64_t decisions = p->T * threshold_count(p->kind, p->depth);
  if ((img == nullptr && p->B * p->C * p->K > 0) || ((thr == nullptr || ord == nullptr) && decisions > 0) ||
      (w == nullptr && p->T * p->M > 0))
    return HT_ERR_INVALID_ARGUMENT;
  const size_t need = ordinal_bytes(p) + (with_records ? 3 * record_bytes(p) : 0) + 256;
  if (workspace == nullptr || workspace_bytes < need || (reinterpret_cast<uintptr_t>(workspace) & 255u) != 0)
    return HT_ERR_WORKSPACE;
  unsigned char *ws = static_cast<unsigned char *>(workspace);
  FusionArgs &a = out.args;
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
    out.records.margin = reinterpret_cast<float *>(ws + ordinal_bytes(p));
    out.records.leaf = reinterpret_cast<int32_t *>(ws + ordinal_bytes(p) + record_bytes(p));
    out.records.vertex = reinterpret_cast<int32_t *>(ws + ordinal_bytes(p) + 2 * record_bytes(p));
  }
  return pack_ordinals(ord, decisions, p->C + Cv, reinterpret_cast<int32_t *>(ws), status_word, out.stream);
}

int run_paths(const ht_forest_problem *p, const Prepared &pr) {
  if (pr.evals == 0) return HT_OK;
  if (p->kind == TREE)
    paths_kernel<TREE><<<blocks_for(pr.evals), kBlock, 0, pr.stream>>>(pr.args, pr.records);
  else
    paths_kernel<FERN><<<blocks_for(pr.evals), kBlock, 0, pr.stream>>>(pr.args, pr.records);
  HT_CHECK_LAUNCH();
  return HT_OK;
}

int clear(float *ptr, int64_t count, cudaStream_t stream) {
  if (ptr != nullptr && count > 0) HT_CUDA_TRY(cudaMemsetAsync(ptr, 0, sizeof(float) * (size_t)count, stream));
  return HT_OK;
}

}  // namespace
}  // namespace ht

using namespace ht;

extern "C" {

size_t ht_forest_fusion_workspace_bytes(const ht_forest_problem *p) {
  if (check_forest_problem(p) != HT_OK) return 0;
  return ordinal_bytes(p) + 256;
}

size_t ht_forest_linear_workspace_bytes(const ht_forest_problem *p) {
  if (check_forest_problem(p) != HT_OK) return 0;
  return ordinal_bytes(p) + 3 * record_bytes(p) + 256;
}

int ht_forest_fusion_forward_f32(const ht_forest_problem *p, const float *img, const float *vec, int64_t vec_channels,
                                 const float *thr, const int64_t *ord, const float *w, float *out, void *workspace,
                                 size_t workspace_bytes, uint32_t *status_word, ht_stream_t stream) {
  Prepared pr;
  const int rc = prepare(p, img, vec, vec_channels, thr, ord, w, false, workspace, workspace_bytes, status_word, stream, pr);
  if (rc != HT_OK) return rc;
  if (pr.evals * p->M == 0) return HT_OK;
  if (out == nullptr) return HT_ERR_INVALID_ARGUMENT;
  if (p->kind == TREE)
    fusion_forward_kernel<TREE><<<blocks_for(pr.evals), kBlock, 0, pr.stream>>>(pr.args, out);
  else
    fusion_forward_kernel<FERN><<<blocks_for(pr.evals), kBlock, 0, pr.stream>>>(pr.args, out);
  HT_CHECK_LAUNCH();
  return HT_OK;
}

int ht_forest_fusion_backward_f32(const ht_forest_problem *p, const float *img, const float *vec, int64_t vec_channels,
                                  const float *thr, const int64_t *ord, const float *w, const float *g, float *gimg,
                                  float *gvec, float *gthr, float *gw, void *workspace, size_t workspace_bytes,
                                  uint32_t *status_word, ht_stream_t stream) {
  Prepared pr;
  const int rc = prepare(p, img, vec, vec_channels, thr, ord, w, false, workspace, workspace_bytes, status_word, stream, pr);
  if (rc != HT_OK) return rc;
  const FusionArgs &a = pr.args;
  int crc;
  if ((crc = clear(gimg, a.B * a.C * a.K, pr.stream)) != HT_OK) return crc;
  if ((crc = clear(gvec, a.B * a.Cv, pr.stream)) != HT_OK) return crc;
  if ((crc = clear(gthr, a.T * a.N, pr.stream)) != HT_OK) return crc;
  if ((crc = clear(gw, a.T * a.L * a.M, pr.stream)) != HT_OK) return crc;
  if (pr.evals * a.M == 0) return HT_OK;
  if (g == nullptr) return HT_ERR_INVALID_ARGUMENT;
  if (p->kind == TREE)
    fusion_backward_kernel<TREE><<<blocks_for(pr.evals), kBlock, 0, pr.stream>>>(a, g, gimg, gvec, gthr, gw);
  else
    fusion_backward_kernel<FERN><<<blocks_for(pr.evals), kBlock, 0, pr.stream>>>(a, g, gimg, gvec, gthr, gw);
  HT_CHECK_LAUNCH();
  return HT_OK;
}

int ht_forest_linear_forward_f32(const ht_forest_problem *p, int64_t out_channels, const float *img, const float *vec,
                                 int64_t vec_channels, const float *thr, const int64_t *ord, const float *w,
                                 const float *lin, const float *bias, float *out, void *workspace,
                                 size_t workspace_bytes, uint32_t *status_word, ht_stream_t stream) {
  Prepared pr;
  const int rc = prepare(p, img, vec, vec_channels, thr, ord, w, true, workspace, workspace_bytes, status_word, stream, pr);
  if (rc != HT_OK) return rc;
  if (out_channels < 0) return HT_ERR_INVALID_ARGUMENT;
  const int64_t elements = p->B * out_channels * p->K * p->M;
  if (elements == 0) return HT_OK;
  if (out == nullptr || bias == nullptr || (lin == nullptr && p->T > 0)) return HT_ERR_INVALID_ARGUMENT;
  const int prc = run_paths(p, pr);
  if (prc != HT_OK) return prc;
  linear_forward_kernel<<<blocks_for(elements), kBlock, 0, pr.stream>>>(pr.args, pr.records, lin, bias, out_channels, out);
  HT_CHECK_LAUNCH();
  return HT_OK;
}

int ht_forest_linear_backward_f32(const ht_forest_problem *p, int64_t out_channels, const float *img, const float *vec,
                                  int64_t vec_channels, const float *thr, const int64_t *ord, const float *w,
                                  const float *lin, const float *g, float *gimg, float *gvec, float *gthr, float *gw,
                                  float *glin, void *workspace, size_t workspace_bytes, uint32_t *status_word,
                                  ht_stream_t stream) {
  Prepared pr;
  const int rc = prepare(p, img, vec, vec_channels, thr, ord, w, true, workspace, workspace_bytes, status_word, stream, pr);
  if (rc != HT_OK) return rc;
  if (out_channels < 0) return HT_ERR_INVALID_ARGUMENT;
  const FusionArgs &a = pr.args;
  int crc;
  if ((crc = clear(gimg, a.B * a.C * a.K, pr.stream)) != HT_OK) return crc;
  if ((crc = clear(gvec, a.B * a.Cv, pr.stream)) != HT_OK) return crc;
  if ((crc = clear(gthr, a.T * a.N, pr.stream)) != HT_OK) return crc;
  if ((crc = clear(gw, a.T * a.L * a.M, pr.stream)) != HT_OK) return crc;
  if ((crc = clear(glin, out_channels * a.T, pr.stream)) != HT_OK) return crc;
  if (pr.evals * a.M * out_channels == 0) return HT_OK;
  if (g == nullptr || lin == nullptr) return HT_ERR_INVALID_ARGUMENT;
  const int prc = run_paths(p, pr);
  if (prc != HT_OK) return prc;
  if (gimg != nullptr || gvec != nullptr || gthr != nullptr || gw != nullptr) {
    linear_backward_kernel<<<blocks_for(pr.evals), kBlock, 0, pr.stream>>>(a, pr.records, lin, g, out_channels, gimg, gvec,
                                                                          gthr, gw);
    HT_CHECK_LAUNCH();
  }
  if (glin != nullptr) {
    // enough CTAs to fill the machine: the positions of a tree are split when there are few trees
    const int64_t positions = a.B * a.K;
    const unsigned slices = (unsigned)std::max<int64_t>(1, std::min<int64_t>(std::min<int64_t>((148 * 8 + a.T - 1) / a.T, 65535),
                                                                             (positions + 4 * kBlock - 1) / (4 * kBlock)));
    linear_weight_grad_kernel<<<dim3((unsigned)a.T, slices), kBlock, 0, pr.stream>>>(a, pr.records, g, out_channels, glin);
    HT_CHECK_LAUNCH();
  }
  return HT_OK;
}

}  // extern "C"
