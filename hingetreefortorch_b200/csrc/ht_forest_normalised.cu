// Hinge forest behind a batch normalisation that is never materialised.
//
// The reference's sequential-initialisation pipeline is Linear -> BatchNorm1d(affine=False) -> forest
// (README.md:110-129, _RandomHingeForest.py:56-59).  A forest reads only the few features on each
// sample's paths (depth of them per tree), while the normalisation writes every activation again and
// its backward reads all of them twice more.  Here the forest normalises the features it visits on the
// fly, from the raw activations z [B, C] and the per-column mean and 1/std, exactly as ATen's
// batch_norm_elemt rounds them ((z - mean) rounded, times invstd rounded), so its results equal those of
// the forest behind a materialised normalisation bit for bit; and its backward leaves the gradient with
// respect to the normalised activations as what it is — one value per (sample, tree) — together with the
// two column sums the normalisation's backward needs, so that the gradient with respect to z,
//     dz[i, c] = invstd[c] * ( gy[i, c] - mean_i(gy[., c]) - y[i, c] * mean_i(gy[., c] * y[., c]) ),
// is formed in one pass over z (ht_batchnorm_input_grad_f32) instead of a zero-fill, a scatter, a
// reduction pass and an element-wise pass.
//
// Tabular inputs only (K = 1); default-mode sums (atomics), no fixed-order variant.
#include "ht_common.cuh"

namespace ht {
namespace {

constexpr int kNormBlock = 256;
inline unsigned norm_blocks(int64_t n) { return (unsigned)((n + kNormBlock - 1) / kNormBlock); }

struct NormalisedFeature {
  typedef float value_type;
  const float *__restrict__ row;     // z[i, :]
  const float *__restrict__ mean;    // [C]
  const float *__restrict__ invstd;  // [C]
  __device__ __forceinline__ float operator()(int c) const {
    return __fmul_rn(__fsub_rn(__ldg(row + c), __ldg(mean + c)), __ldg(invstd + c));
  }
};

struct NormalisedArgs {
  const float *z, *mean, *invstd, *thr, *w;
  const int32_t *ord;  // compact, clamped into [0, C)
  int64_t B, C, T, N, L, M;
  int depth;
};

__global__ void __launch_bounds__(kNormBlock) compact_ordinals_kernel(const int64_t *__restrict__ ord, int64_t n, int64_t C,
                                                                     int32_t *__restrict__ packed, uint32_t *status_word) {
  const int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= n) return;
  int64_t c = ord[e];
  if (c < 0 || c >= C) {
    if (status_word != nullptr) atomicOr(status_word, HT_FLAG_ORDINAL_RANGE);
    c = 0;
  }
  packed[e] = (int32_t)c;
}

// save_margin / save_where (both or neither): the signed margin and the pair (deciding vertex, leaf key) of every
// (sample, tree), 12 bytes, so that the backward need not read z and walk again.
template <int KIND>
__global__ void __launch_bounds__(kNormBlock) normalised_forward_kernel(NormalisedArgs a, float *__restrict__ out,
                                                                       float *__restrict__ save_margin,
                                                                       uint2 *__restrict__ save_where) {
  const int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= a.B * a.T) return;
  const int64_t i = e / a.T, j = e - i * a.T;
  const NormalisedFeature feat{a.z + i * a.C, a.mean, a.invstd};
  const Path p = traverse<KIND>(feat, a.thr + j * a.N, a.ord + j * a.N, a.depth);
  if (save_margin != nullptr) {
    save_margin[e] = p.margin;
    save_where[e] = make_uint2(p.vertex, p.key);
  }
  const float am = fabsf(p.margin);
  const float *wl = a.w + (j * a.L + p.key) * a.M;
  float *o = out + e * a.M;
  for (int64_t m = 0; m < a.M; ++m) o[m] = __fmul_rn(__ldg(wl + m), am);
}

// One thread per (sample, tree): the threshold and leaf-weight gradients as in the plain backward, and the
// gradient with respect to the normalised feature of the deciding vertex as a record (column, value), plus its
// contribution to the two column sums of the normalisation's backward.
template <int KIND>
__global__ void __launch_bounds__(kNormBlock) normalised_backward_kernel(NormalisedArgs a, const float *__restrict__ g, float *gthr,
                                                                        float *gw, int32_t *__restrict__ column,
                                                                        float *__restrict__ value, float *sum_g, float *sum_gy,
                                                                        const float *__restrict__ saved_margin,
                                                                        const uint2 *__restrict__ saved_where) {
  const int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= a.B * a.T) return;
  const int64_t i = e / a.T, j = e - i * a.T;
  const NormalisedFeature feat{a.z + i * a.C, a.mean, a.invstd};
  Path p;
  if (saved_margin != nullptr) {  // the forward kept its traversal
    const uint2 where = saved_where[e];
    p.margin = saved_margin[e];
    p.vertex = where.x;
    p.key = where.y;
  } else {
    p = traverse<KIND>(feat, a.thr + j * a.N, a.ord + j * a.N, a.depth);
  }
  const float s = sign_of(p.margin), am = fabsf(p.margin);
  const float *wl = a.w + (j * a.L + p.key) * a.M;
  const float *gl = g + e * a.M;
  float acc = 0.0f;
  for (int64_t m = 0; m < a.M; ++m) {
    const float gm = __ldg(gl + m);
    acc = __fadd_rn(acc, __fmul_rn(__fmul_rn(s, __ldg(wl + m)), gm));
    if (gw != nullptr) atomicAdd(gw + (j * a.L + p.key) * a.M + m, __fmul_rn(am, gm));
  }
  if (gthr != nullptr) atomicAdd(gthr + j * a.N + p.vertex, -acc);
  const int c = a.ord[j * a.N + p.vertex];
  column[e] = c;
  value[e] = acc;
  if (acc != 0.0f) {
    atomicAdd(sum_g + c, acc);
    // the normalised feature at the deciding vertex: read again, or margin + threshold (a rounding apart)
    const float y = saved_margin != nullptr ? __fadd_rn(p.margin, __ldg(a.thr + j * a.N + p.vertex)) : feat(c);
    atomicAdd(sum_gy + c, __fmul_rn(acc, y));
  }
}

// dz = invstd * (-mean(gy) - y * mean(gy y)) for every element: the part of the normalisation's backward that
// does not depend on where gy is non-zero.  Four columns per thread.
__global__ void __launch_bounds__(kNormBlock) input_grad_dense_kernel(const float *__restrict__ z, const float *__restrict__ mean,
                                                                     const float *__restrict__ invstd,
                                                                     const float *__restrict__ sum_g,
                                                                     const float *__restrict__ sum_gy, float *__restrict__ dz,
                                                                     int64_t B, int64_t C, float inv_rows) {
  const int64_t quads = C >> 2;
  const int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= B * quads) return;
  const int64_t i = e / quads, q = e - i * quads;
  const float4 zv = __ldg(reinterpret_cast<const float4 *>(z + i * C) + q);
  const float4 mu = __ldg(reinterpret_cast<const float4 *>(mean) + q);
  const float4 is = __ldg(reinterpret_cast<const float4 *>(invstd) + q);
  const float4 sg = __ldg(reinterpret_cast<const float4 *>(sum_g) + q);
  const float4 sy = __ldg(reinterpret_cast<const float4 *>(sum_gy) + q);
  float4 r;
  r.x = is.x * (-sg.x * inv_rows - ((zv.x - mu.x) * is.x) * (sy.x * inv_rows));
  r.y = is.y * (-sg.y * inv_rows - ((zv.y - mu.y) * is.y) * (sy.y * inv_rows));
  r.z = is.z * (-sg.z * inv_rows - ((zv.z - mu.z) * is.z) * (sy.z * inv_rows));
  r.w = is.w * (-sg.w * inv_rows - ((zv.w - mu.w) * is.w) * (sy.w * inv_rows));
  reinterpret_cast<float4 *>(dz + i * C)[q] = r;
}

__global__ void __launch_bounds__(kNormBlock) input_grad_dense_tail_kernel(const float *__restrict__ z, const float *__restrict__ mean,
                                                                          const float *__restrict__ invstd,
                                                                          const float *__restrict__ sum_g,
                                                                          const float *__restrict__ sum_gy,
                                                                          float *__restrict__ dz, int64_t B, int64_t C,
                                                                          int64_t first, float inv_rows) {
  const int64_t width = C - first;
  const int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= B * width) return;
  const int64_t i = e / width, c = first + (e - i * width);
  const float is = invstd[c];
  dz[i * C + c] = is * (-sum_g[c] * inv_rows - ((z[i * C + c] - mean[c]) * is) * (sum_gy[c] * inv_rows));
}

// ... and the part that does: invstd * gy at the recorded places (several trees of a sample may meet in a column).
__global__ void __launch_bounds__(kNormBlock) input_grad_sparse_kernel(const int32_t *__restrict__ column,
                                                                      const float *__restrict__ value,
                                                                      const float *__restrict__ invstd, float *dz, int64_t B,
                                                                      int64_t C, int64_t T) {
  const int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= B * T) return;
  const float v = value[e];
  if (v == 0.0f) return;
  const int64_t i = e / T;
  const int c = column[e];
  atomicAdd(dz + i * C + c, __ldg(invstd + c) * v);
}

// mean, biased variance and 1 / sqrt(variance + eps) of every column from its sum and sum of squares.
__global__ void __launch_bounds__(kNormBlock) statistics_kernel(const float *__restrict__ sum, const float *__restrict__ sumsq,
                                                               int64_t C, float inv_rows, float eps, float *__restrict__ mean,
                                                               float *__restrict__ var, float *__restrict__ invstd) {
  const int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const float m = __fmul_rn(sum[c], inv_rows);
  const float v = fmaxf(__fsub_rn(__fmul_rn(sumsq[c], inv_rows), __fmul_rn(m, m)), 0.0f);
  mean[c] = m;
  var[c] = v;
  invstd[c] = rsqrtf(__fadd_rn(v, eps));
}

int check(const ht_forest_problem *p, NormalisedArgs &a) {
  if (p == nullptr) return HT_ERR_INVALID_ARGUMENT;
  if (p->kind != TREE && p->kind != FERN) return HT_ERR_INVALID_ARGUMENT;
  if (p->depth < 1 || p->depth > 31) return HT_ERR_DEPTH;
  if (p->K != 1 || p->B < 0 || p->C < 1 || p->T < 0 || p->M < 1) return HT_ERR_INVALID_ARGUMENT;
  if (p->C > 0x7fffffff) return HT_ERR_UNSUPPORTED;
  a.B = p->B;
  a.C = p->C;
  a.T = p->T;
  a.M = p->M;
  a.depth = p->depth;
  a.N = threshold_count(p->kind, p->depth);
  a.L = ((int64_t)1) << p->depth;
  return HT_OK;
}

}  // namespace
}  // namespace ht

using namespace ht;

extern "C" size_t ht_forest_normalised_workspace_bytes(const ht_forest_problem *p) {
  if (p == nullptr || p->depth < 1 || p->depth > 31 || p->T < 0) return 0;
  return (size_t)p->T * (size_t)threshold_count(p->kind, p->depth) * sizeof(int32_t) + 16;
}

extern "C" int ht_forest_normalised_forward_f32(const ht_forest_problem *p, const float *z, const float *mean, const float *invstd,
                                                const float *thr, const int64_t *ord, const float *w, float *out,
                                                float *save_margin, void *save_where, void *workspace, size_t workspace_bytes,
                                                uint32_t *status_word, ht_stream_t stream_) {
  NormalisedArgs a = {};
  if ((save_margin == nullptr) != (save_where == nullptr)) return HT_ERR_INVALID_ARGUMENT;
  const int rc = check(p, a);
  if (rc != HT_OK) return rc;
  if (a.B == 0 || a.T == 0) return HT_OK;
  if (z == nullptr || mean == nullptr || invstd == nullptr || thr == nullptr || ord == nullptr || w == nullptr || out == nullptr)
    return HT_ERR_INVALID_ARGUMENT;
  if (workspace == nullptr || workspace_bytes < ht_forest_normalised_workspace_bytes(p)) return HT_ERR_WORKSPACE;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  int32_t *packed = static_cast<int32_t *>(workspace);
  compact_ordinals_kernel<<<norm_blocks(a.T * a.N), kNormBlock, 0, stream>>>(ord, a.T * a.N, a.C, packed, status_word);
  HT_CHECK_LAUNCH();
  a.z = z;
  a.mean = mean;
  a.invstd = invstd;
  a.thr = thr;
  a.w = w;
  a.ord = packed;
  if (p->kind == TREE)
    normalised_forward_kernel<TREE><<<norm_blocks(a.B * a.T), kNormBlock, 0, stream>>>(a, out, save_margin, static_cast<uint2 *>(save_where));
  else
    normalised_forward_kernel<FERN><<<norm_blocks(a.B * a.T), kNormBlock, 0, stream>>>(a, out, save_margin, static_cast<uint2 *>(save_where));
  HT_CHECK_LAUNCH();
  return HT_OK;
}

extern "C" int ht_forest_normalised_backward_f32(const ht_forest_problem *p, const float *z, const float *mean, const float *invstd,
                                                 const float *thr, const int64_t *ord, const float *w, const float *g, float *gthr,
                                                 float *gw, int32_t *column, float *value, float *sum_g, float *sum_gy,
                                                 const float *saved_margin, const void *saved_where, void *workspace,
                                                 size_t workspace_bytes, uint32_t *status_word, ht_stream_t stream_) {
  NormalisedArgs a = {};
  if ((saved_margin == nullptr) != (saved_where == nullptr)) return HT_ERR_INVALID_ARGUMENT;
  const int rc = check(p, a);
  if (rc != HT_OK) return rc;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (sum_g == nullptr || sum_gy == nullptr) return HT_ERR_INVALID_ARGUMENT;
  HT_CUDA_TRY(cudaMemsetAsync(sum_g, 0, sizeof(float) * (size_t)a.C, stream));
  HT_CUDA_TRY(cudaMemsetAsync(sum_gy, 0, sizeof(float) * (size_t)a.C, stream));
  if (gthr != nullptr) HT_CUDA_TRY(cudaMemsetAsync(gthr, 0, sizeof(float) * (size_t)(a.T * a.N), stream));
  if (gw != nullptr) HT_CUDA_TRY(cudaMemsetAsync(gw, 0, sizeof(float) * (size_t)(a.T * a.L * a.M), stream));
  if (a.B == 0 || a.T == 0) return HT_OK;
  if (z == nullptr || mean == nullptr || invstd == nullptr || thr == nullptr || ord == nullptr || w == nullptr || g == nullptr ||
      column == nullptr || value == nullptr)
    return HT_ERR_INVALID_ARGUMENT;
  if (workspace == nullptr || workspace_bytes < ht_forest_normalised_workspace_bytes(p)) return HT_ERR_WORKSPACE;
  int32_t *packed = static_cast<int32_t *>(workspace);
  compact_ordinals_kernel<<<norm_blocks(a.T * a.N), kNormBlock, 0, stream>>>(ord, a.T * a.N, a.C, packed, status_word);
  HT_CHECK_LAUNCH();
  a.z = z;
  a.mean = mean;
  a.invstd = invstd;
  a.thr = thr;
  a.w = w;
  a.ord = packed;
  if (p->kind == TREE)
    normalised_backward_kernel<TREE><<<norm_blocks(a.B * a.T), kNormBlock, 0, stream>>>(
        a, g, gthr, gw, column, value, sum_g, sum_gy, saved_margin, static_cast<const uint2 *>(saved_where));
  else
    normalised_backward_kernel<FERN><<<norm_blocks(a.B * a.T), kNormBlock, 0, stream>>>(
        a, g, gthr, gw, column, value, sum_g, sum_gy, saved_margin, static_cast<const uint2 *>(saved_where));
  HT_CHECK_LAUNCH();
  return HT_OK;
}

extern "C" int ht_batchnorm_input_grad_f32(const float *z, const float *mean, const float *invstd, const float *sum_g,
                                           const float *sum_gy, const int32_t *column, const float *value, float *dz, int64_t B,
                                           int64_t C, int64_t T, ht_stream_t stream_) {
  if (B < 0 || C < 1 || T < 0) return HT_ERR_INVALID_ARGUMENT;
  if (B == 0) return HT_OK;
  if (z == nullptr || mean == nullptr || invstd == nullptr || sum_g == nullptr || sum_gy == nullptr || dz == nullptr)
    return HT_ERR_INVALID_ARGUMENT;
  if (T > 0 && (column == nullptr || value == nullptr)) return HT_ERR_INVALID_ARGUMENT;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  const float inv_rows = 1.0f / (float)B;
  const bool aligned = ((reinterpret_cast<uintptr_t>(z) | reinterpret_cast<uintptr_t>(dz) | reinterpret_cast<uintptr_t>(mean) |
                         reinterpret_cast<uintptr_t>(invstd) | reinterpret_cast<uintptr_t>(sum_g) |
                         reinterpret_cast<uintptr_t>(sum_gy)) & 15u) == 0 && (C & 3) == 0;
  if (aligned) {
    input_grad_dense_kernel<<<norm_blocks(B * (C >> 2)), kNormBlock, 0, stream>>>(z, mean, invstd, sum_g, sum_gy, dz, B, C, inv_rows);
    HT_CHECK_LAUNCH();
  } else {
    input_grad_dense_tail_kernel<<<norm_blocks(B * C), kNormBlock, 0, stream>>>(z, mean, invstd, sum_g, sum_gy, dz, B, C, 0, inv_rows);
    HT_CHECK_LAUNCH();
  }
  if (T > 0) {
    input_grad_sparse_kernel<<<norm_blocks(B * T), kNormBlock, 0, stream>>>(column, value, invstd, dz, B, C, T);
    HT_CHECK_LAUNCH();
  }
  return HT_OK;
}

extern "C" int ht_batchnorm_statistics_f32(const float *sum, const float *sumsq, int64_t rows, int64_t C, float eps, float *mean,
                                           float *var, float *invstd, ht_stream_t stream_) {
  if (rows < 1 || C < 0) return HT_ERR_INVALID_ARGUMENT;
  if (C == 0) return HT_OK;
  if (sum == nullptr || sumsq == nullptr || mean == nullptr || var == nullptr || invstd == nullptr) return HT_ERR_INVALID_ARGUMENT;
  statistics_kernel<<<norm_blocks(C), kNormBlock, 0, reinterpret_cast<cudaStream_t>(stream_)>>>(sum, sumsq, C, 1.0f / (float)rows, eps,
                                                                                              mean, var, invstd);
  HT_CHECK_LAUNCH();
  return HT_OK;
}
