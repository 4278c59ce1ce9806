// Operators of `hingetree_cpp` beyond the plain forest: image+vector fusion, fused linear,
// convolution, sparse gradients, trie and contract/expand.  Same conventions as
// hingetree_cpp.cpp: validate like the reference (ValueError for argument problems,
// RuntimeError for depth / ordinal range), allocate, call the C ABI on the current stream.
#include <c10/core/DeviceGuard.h>

#include <sstream>

#include "hingetree_cpp_ops.h"

namespace htx {

namespace {

void require_real(const torch::Tensor &t) {
  if (t.scalar_type() != torch::kFloat32 && t.scalar_type() != torch::kFloat64)
    bad_argument("Error: Unsupported data type. Only torch.float32 and torch.float64 are supported.");
}

// Shared validation of the fusion / fused-linear families (reference: hingetree_fusion.cpp:41-75,
// 306-366; hingetree_fused_linear.cpp:75-100, 414-440, 769-860, 956-1050).
struct FamilyCall {
  ht_forest_problem problem;
  int64_t vec_channels = 0;
  int64_t out_channels = 0;
  std::vector<int64_t> out_sizes;

  FamilyCall(int kind, const torch::Tensor &data, const torch::Tensor *vec, const torch::Tensor &thr,
             const torch::Tensor &ord, const torch::Tensor &w, const torch::Tensor *lin, const torch::Tensor *bias,
             const torch::Tensor *g) {
    std::vector<const torch::Tensor *> reals = {&data, &thr, &w};
    for (const torch::Tensor *t : {vec, lin, bias, g})
      if (t != nullptr) reals.push_back(t);
    for (const torch::Tensor *t : reals)
      if (t->dtype() != data.dtype())
        bad_argument("Error: all real-valued tensors are expected to share the same torch real number data type. "
                     "inOrdinals is expected to be type torch.int64.");
    if (ord.scalar_type() != torch::kInt64)
      bad_argument("Error: all real-valued tensors are expected to share the same torch real number data type. "
                   "inOrdinals is expected to be type torch.int64.");
    for (const torch::Tensor *t : reals)
      if (t->device() != data.device()) bad_argument("Error: All tensors are expected to be on the same device.");
    if (ord.device() != data.device()) bad_argument("Error: All tensors are expected to be on the same device.");
    for (const torch::Tensor *t : reals)
      if (!t->is_contiguous()) bad_argument("Error: All tensors are expected to be contiguous.");
    if (!ord.is_contiguous()) bad_argument("Error: All tensors are expected to be contiguous.");
    require_real(data);
    require_cuda(data);
    if (data.dim() < 2 || (vec != nullptr && vec->dim() != 2) || thr.dim() != 2 || ord.dim() != 2 || w.dim() < 2 ||
        (lin != nullptr && lin->dim() != 2) || (bias != nullptr && bias->dim() != 1))
      bad_argument("Error: the data and inWeights must have at least 2 dimensions. inVec, inThresholds, inOrdinals and "
                   "inLinearWeights must have 2 dimensions. inLinearBias must have 1 dimension.");
    if (thr.sizes() != ord.sizes() || w.size(0) != thr.size(0) || (vec != nullptr && vec->size(0) != data.size(0)) ||
        (lin != nullptr && lin->size(1) != w.size(0)) || (lin != nullptr && bias != nullptr && lin->size(0) != bias->size(0)))
      bad_argument("Error: inThresholds and inOrdinals must be the same shape. inWeights.shape[0] must be the same as "
                   "inThresholds.shape[0] (and as inLinearWeights.shape[1]). inImg.shape[0] must be the same as "
                   "inVec.shape[0]. inLinearWeights.shape[0] must be the same as inLinearBias.shape[0].");
    const int depth = depth_of(w.size(1));
    if (depth > 31 || depth < 1 || thr.size(1) != threshold_count(kind, depth)) {
      std::ostringstream ss;
      ss << "Error: The tree depth exceeds compile-time constraints or the number of thresholds is incorrect for the "
            "tree depth (tree depth = "
         << depth << ").";
      bad_runtime(ss.str());
    }
    problem.kind = kind;
    problem.depth = depth;
    problem.B = data.size(0);
    problem.C = data.size(1);
    problem.K = inner_count(data, 2);
    problem.T = w.size(0);
    problem.M = inner_count(w, 2);
    problem.flags = 0;
    problem.reserved = 0;
    vec_channels = vec != nullptr ? vec->size(1) : 0;
    out_channels = lin != nullptr ? lin->size(0) : 0;
    out_sizes = {data.size(0), lin != nullptr ? lin->size(0) : w.size(0)};
    for (int64_t d = 2; d < data.dim(); ++d) out_sizes.push_back(data.size(d));
    for (int64_t d = 2; d < w.dim(); ++d) out_sizes.push_back(w.size(d));
    if (g != nullptr && g->sizes() != c10::IntArrayRef(out_sizes)) {
      std::ostringstream ss;
      ss << "Error: outDataGrad.shape does not match the expected shape (" << g->sizes() << " != "
         << c10::IntArrayRef(out_sizes) << ").";
      bad_argument(ss.str());
    }
  }
};

template <typename Real>
Real *ptr_or_null(torch::Tensor &t) {
  return t.defined() ? t.data_ptr<Real>() : nullptr;
}

// f(float()) or f(double()) by the tensor's type (the operators of this file take both precisions).
template <typename F>
void dispatch_real(const torch::Tensor &t, F &&f) {
  if (t.scalar_type() == torch::kFloat64)
    f(double());
  else
    f(float());
}

// The C ABI's single and double precision entries under one name each.
namespace abi {
#define HT_BOTH(NAME, PARAMS_F, PARAMS_D, ARGS)                               \
  inline int NAME PARAMS_F { return ht_##NAME##_f32 ARGS; }                   \
  inline int NAME PARAMS_D { return ht_##NAME##_f64 ARGS; }
#define HT_P const ht_forest_problem *p
#define HT_TAIL void *ws, size_t wsb, uint32_t *st, ht_stream_t s
HT_BOTH(forest_fusion_forward,
        (HT_P, const float *img, const float *vec, int64_t cv, const float *thr, const int64_t *ord, const float *w, float *out, HT_TAIL),
        (HT_P, const double *img, const double *vec, int64_t cv, const double *thr, const int64_t *ord, const double *w, double *out, HT_TAIL),
        (p, img, vec, cv, thr, ord, w, out, ws, wsb, st, s))
HT_BOTH(forest_fusion_backward,
        (HT_P, const float *img, const float *vec, int64_t cv, const float *thr, const int64_t *ord, const float *w, const float *g,
         float *gi, float *gv, float *gt, float *gw, HT_TAIL),
        (HT_P, const double *img, const double *vec, int64_t cv, const double *thr, const int64_t *ord, const double *w, const double *g,
         double *gi, double *gv, double *gt, double *gw, HT_TAIL),
        (p, img, vec, cv, thr, ord, w, g, gi, gv, gt, gw, ws, wsb, st, s))
HT_BOTH(forest_linear_forward,
        (HT_P, int64_t o, const float *img, const float *vec, int64_t cv, const float *thr, const int64_t *ord, const float *w,
         const float *lin, const float *bias, float *out, HT_TAIL),
        (HT_P, int64_t o, const double *img, const double *vec, int64_t cv, const double *thr, const int64_t *ord, const double *w,
         const double *lin, const double *bias, double *out, HT_TAIL),
        (p, o, img, vec, cv, thr, ord, w, lin, bias, out, ws, wsb, st, s))
HT_BOTH(forest_linear_backward,
        (HT_P, int64_t o, const float *img, const float *vec, int64_t cv, const float *thr, const int64_t *ord, const float *w,
         const float *lin, const float *g, float *gi, float *gv, float *gt, float *gw, float *gl, HT_TAIL),
        (HT_P, int64_t o, const double *img, const double *vec, int64_t cv, const double *thr, const int64_t *ord, const double *w,
         const double *lin, const double *g, double *gi, double *gv, double *gt, double *gw, double *gl, HT_TAIL),
        (p, o, img, vec, cv, thr, ord, w, lin, g, gi, gv, gt, gw, gl, ws, wsb, st, s))
HT_BOTH(forest_touched,
        (HT_P, const float *x, const float *thr, const int64_t *ord, uint8_t *tx, uint8_t *tt, uint8_t *tw, HT_TAIL),
        (HT_P, const double *x, const double *thr, const int64_t *ord, uint8_t *tx, uint8_t *tt, uint8_t *tw, HT_TAIL),
        (p, x, thr, ord, tx, tt, tw, ws, wsb, st, s))
HT_BOTH(forest_backward,
        (HT_P, const float *x, const float *thr, const int64_t *ord, const float *w, const float *g, float *gx, float *gt, float *gw, HT_TAIL),
        (HT_P, const double *x, const double *thr, const int64_t *ord, const double *w, const double *g, double *gx, double *gt, double *gw, HT_TAIL),
        (p, x, thr, ord, w, g, gx, gt, gw, ws, wsb, st, s))
HT_BOTH(trie_forward,
        (HT_P, const float *x, const float *thr, const int64_t *ord, const float *w, float *out, HT_TAIL),
        (HT_P, const double *x, const double *thr, const int64_t *ord, const double *w, double *out, HT_TAIL),
        (p, x, thr, ord, w, out, ws, wsb, st, s))
HT_BOTH(trie_backward,
        (HT_P, const float *x, const float *thr, const int64_t *ord, const float *w, const float *g, float *gx, float *gt, float *gw, HT_TAIL),
        (HT_P, const double *x, const double *thr, const int64_t *ord, const double *w, const double *g, double *gx, double *gt, double *gw, HT_TAIL),
        (p, x, thr, ord, w, g, gx, gt, gw, ws, wsb, st, s))
#undef HT_P
#define HT_P const ht_conv_problem *p
HT_BOTH(conv_forward,
        (HT_P, const float *x, const float *thr, const int64_t *ord, const float *w, float *out, HT_TAIL),
        (HT_P, const double *x, const double *thr, const int64_t *ord, const double *w, double *out, HT_TAIL),
        (p, x, thr, ord, w, out, ws, wsb, st, s))
HT_BOTH(conv_backward,
        (HT_P, const float *x, const float *thr, const int64_t *ord, const float *w, const float *g, float *gx, float *gt, float *gw, HT_TAIL),
        (HT_P, const double *x, const double *thr, const int64_t *ord, const double *w, const double *g, double *gx, double *gt, double *gw, HT_TAIL),
        (p, x, thr, ord, w, g, gx, gt, gw, ws, wsb, st, s))
#undef HT_P
#undef HT_TAIL
#undef HT_BOTH
}  // namespace abi

// ---- fusion --------------------------------------------------------------------------------

torch::Tensor fusion_forward(int kind, torch::Tensor img, torch::Tensor vec, torch::Tensor thr, torch::Tensor ord,
                             torch::Tensor w) {
  FamilyCall call(kind, img, &vec, thr, ord, w, nullptr, nullptr, nullptr);
  c10::DeviceGuard guard(img.device());
  torch::Tensor out = torch::empty(call.out_sizes, img.options());
  torch::Tensor ws = make_workspace(ht_forest_fusion_workspace_bytes(&call.problem), img);
  OrdinalGuard og(ord, call.problem.C + call.vec_channels);
  dispatch_real(img, [&](auto real) {
    using Real = decltype(real);
    raise_status(abi::forest_fusion_forward(&call.problem, img.data_ptr<Real>(), vec.data_ptr<Real>(), call.vec_channels,
                                              thr.data_ptr<Real>(), ord.data_ptr<int64_t>(), w.data_ptr<Real>(),
                                              out.data_ptr<Real>(), ws.data_ptr(), ws.numel(), og.word(),
                                              current_stream(img)),
                 "fusion forward");
  });
  og.finish();
  return out;
}

std::vector<torch::Tensor> fusion_backward(int kind, torch::Tensor img, bool need_img, torch::Tensor vec, bool need_vec,
                                           torch::Tensor thr, bool need_thr, torch::Tensor ord, bool need_ord,
                                           torch::Tensor w, bool need_w, torch::Tensor g) {
  if (need_ord) bad_runtime("Error: Gradient on inOrdinals is requested, but inOrdinals never has a gradient.");
  FamilyCall call(kind, img, &vec, thr, ord, w, nullptr, nullptr, &g);
  c10::DeviceGuard guard(img.device());
  std::vector<torch::Tensor> grads(5);
  if (!need_img && !need_vec && !need_thr && !need_w) return grads;
  if (need_img || need_vec) {  // the reference returns both when either is requested
    grads[0] = torch::empty_like(img);
    grads[1] = torch::empty_like(vec);
  }
  if (need_thr) grads[2] = torch::empty_like(thr);
  if (need_w) grads[4] = torch::empty_like(w);
  torch::Tensor ws = make_workspace(ht_forest_fusion_workspace_bytes(&call.problem), img);
  OrdinalGuard og(ord, call.problem.C + call.vec_channels);
  dispatch_real(img, [&](auto real) {
    using Real = decltype(real);
    raise_status(abi::forest_fusion_backward(&call.problem, img.data_ptr<Real>(), vec.data_ptr<Real>(),
                                               call.vec_channels, thr.data_ptr<Real>(), ord.data_ptr<int64_t>(),
                                               w.data_ptr<Real>(), g.data_ptr<Real>(), ptr_or_null<Real>(grads[0]),
                                               ptr_or_null<Real>(grads[1]), ptr_or_null<Real>(grads[2]), ptr_or_null<Real>(grads[4]),
                                               ws.data_ptr(), ws.numel(), og.word(), current_stream(img)),
                 "fusion backward");
  });
  og.finish();
  return grads;
}

// ---- fused linear (plain and fusion) -------------------------------------------------------

torch::Tensor linear_forward(int kind, torch::Tensor data, const torch::Tensor *vec, torch::Tensor thr, torch::Tensor ord,
                             torch::Tensor w, torch::Tensor lin, torch::Tensor bias) {
  FamilyCall call(kind, data, vec, thr, ord, w, &lin, &bias, nullptr);
  c10::DeviceGuard guard(data.device());
  torch::Tensor out = torch::empty(call.out_sizes, data.options());
  torch::Tensor ws = make_workspace(data.scalar_type() == torch::kFloat64 ? ht_forest_linear_workspace_bytes_f64(&call.problem)
                                                                                  : ht_forest_linear_workspace_bytes(&call.problem),
                                     data);
  OrdinalGuard og(ord, call.problem.C + call.vec_channels);
  dispatch_real(data, [&](auto real) {
    using Real = decltype(real);
    raise_status(abi::forest_linear_forward(&call.problem, call.out_channels, data.data_ptr<Real>(),
                                              vec != nullptr ? vec->data_ptr<Real>() : nullptr, call.vec_channels,
                                              thr.data_ptr<Real>(), ord.data_ptr<int64_t>(), w.data_ptr<Real>(),
                                              lin.data_ptr<Real>(), bias.data_ptr<Real>(), out.data_ptr<Real>(),
                                              ws.data_ptr(), ws.numel(), og.word(), current_stream(data)),
                 "fused linear forward");
  });
  og.finish();
  return out;
}

// Returns [gdata, (gvec,) gthr, None, gw, glin, gbias] in the reference's slot order.
std::vector<torch::Tensor> linear_backward(int kind, torch::Tensor data, bool need_data, const torch::Tensor *vec,
                                           bool need_vec, torch::Tensor thr, bool need_thr, torch::Tensor ord,
                                           bool need_ord, torch::Tensor w, bool need_w, torch::Tensor lin, bool need_lin,
                                           torch::Tensor bias, bool need_bias, torch::Tensor g) {
  if (need_ord) bad_runtime("Error: Gradient on inOrdinals is requested, but inOrdinals never has a gradient.");
  FamilyCall call(kind, data, vec, thr, ord, w, &lin, &bias, &g);
  c10::DeviceGuard guard(data.device());
  const bool fusion = vec != nullptr;
  torch::Tensor gdata, gvec, gthr, gw, glin, gbias;
  if (fusion ? (need_data || need_vec) : need_data) {
    gdata = torch::empty_like(data);
    if (fusion) gvec = torch::empty_like(*vec);
  }
  if (need_thr) gthr = torch::empty_like(thr);
  if (need_w) gw = torch::empty_like(w);
  if (need_lin) glin = torch::empty_like(lin);
  if (gdata.defined() || gthr.defined() || gw.defined() || glin.defined()) {
    torch::Tensor ws = make_workspace(data.scalar_type() == torch::kFloat64 ? ht_forest_linear_workspace_bytes_f64(&call.problem)
                                                                                  : ht_forest_linear_workspace_bytes(&call.problem),
                                     data);
    OrdinalGuard og(ord, call.problem.C + call.vec_channels);
    dispatch_real(data, [&](auto real) {
      using Real = decltype(real);
      raise_status(abi::forest_linear_backward(&call.problem, call.out_channels, data.data_ptr<Real>(),
                                                 fusion ? vec->data_ptr<Real>() : nullptr, call.vec_channels,
                                                 thr.data_ptr<Real>(), ord.data_ptr<int64_t>(), w.data_ptr<Real>(),
                                                 lin.data_ptr<Real>(), g.data_ptr<Real>(), ptr_or_null<Real>(gdata),
                                                 ptr_or_null<Real>(gvec), ptr_or_null<Real>(gthr), ptr_or_null<Real>(gw), ptr_or_null<Real>(glin),
                                                 ws.data_ptr(), ws.numel(), og.word(), current_stream(data)),
                   "fused linear backward");
    });
    og.finish();
  }
  if (need_bias) {  // sum over every dimension but the output channel, as the reference does with Tensor::sum
    std::vector<int64_t> dims = {0};
    for (int64_t d = 2; d < g.dim(); ++d) dims.push_back(d);
    gbias = g.sum(dims);
  }
  if (fusion) return {gdata, gvec, gthr, torch::Tensor(), gw, glin, gbias};
  return {gdata, gthr, torch::Tensor(), gw, glin, gbias};
}

// ---- sparse gradients ----------------------------------------------------------------------------
// The dense backward gives the values, ht_forest_touched_f32 the elements that were contributed
// to; both are compacted into a coalesced COO tensor of the full shape, which is what the
// reference's sparse operators return (hingetree_sparse_gpu.cu:422-457).

torch::Tensor to_sparse(const torch::Tensor &dense, const torch::Tensor &mask_bytes) {
  torch::Tensor mask = mask_bytes.view(dense.sizes()).to(torch::kBool);
  torch::Tensor indices = mask.nonzero().t().contiguous();  // row-major order: sorted, unique
  torch::Tensor values = dense.masked_select(mask);
  torch::Tensor sparse = torch::sparse_coo_tensor(indices, values, dense.sizes(), dense.options().layout(torch::kSparse));
  return sparse._coalesced_(true);
}

struct TouchedMasks {
  torch::Tensor x, thr, w;
};

TouchedMasks touched_masks(const ht_forest_problem &problem, const torch::Tensor &x, bool need_x, const torch::Tensor &thr,
                           bool need_thr, const torch::Tensor &ord, const torch::Tensor &w, bool need_w) {
  TouchedMasks masks;
  auto bytes = x.options().dtype(torch::kUInt8);
  if (need_x) masks.x = torch::empty({x.numel()}, bytes);
  if (need_thr) masks.thr = torch::empty({thr.numel()}, bytes);
  if (need_w) masks.w = torch::empty({w.numel()}, bytes);
  torch::Tensor ws = make_workspace(ht_forest_workspace_bytes(&problem), x);
  dispatch_real(x, [&](auto real) {
    using Real = decltype(real);
    raise_status(abi::forest_touched(&problem, x.data_ptr<Real>(), thr.data_ptr<Real>(), ord.data_ptr<int64_t>(),
                                       need_x ? masks.x.data_ptr<uint8_t>() : nullptr,
                                       need_thr ? masks.thr.data_ptr<uint8_t>() : nullptr,
                                       need_w ? masks.w.data_ptr<uint8_t>() : nullptr, ws.data_ptr(), ws.numel(), nullptr,
                                       current_stream(x)),
                 "touched masks");
  });
  return masks;
}

std::vector<torch::Tensor> sparse_backward(int kind, torch::Tensor x, bool need_x, torch::Tensor thr, bool need_thr,
                                           torch::Tensor ord, bool need_ord, torch::Tensor w, bool need_w, torch::Tensor g) {
  if (need_ord) bad_runtime("Error: Gradient on inOrdinals is requested, but inOrdinals never has a gradient.");
  ForestCall call(kind, x, thr, ord, w, &g, true);
  c10::DeviceGuard guard(x.device());
  std::vector<torch::Tensor> grads(4);
  if (!need_x && !need_thr && !need_w) return grads;
  torch::Tensor gx, gthr, gw;
  if (need_x) gx = torch::empty_like(x);
  if (need_thr) gthr = torch::empty_like(thr);
  if (need_w) gw = torch::empty_like(w);
  torch::Tensor ws = make_workspace(ht_forest_workspace_bytes(&call.problem), x);
  OrdinalGuard og(ord, call.problem.C);
  dispatch_real(x, [&](auto real) {
    using Real = decltype(real);
    raise_status(abi::forest_backward(&call.problem, x.data_ptr<Real>(), thr.data_ptr<Real>(), ord.data_ptr<int64_t>(),
                                        w.data_ptr<Real>(), g.data_ptr<Real>(), ptr_or_null<Real>(gx), ptr_or_null<Real>(gthr),
                                        ptr_or_null<Real>(gw), ws.data_ptr(), ws.numel(), og.word(), current_stream(x)),
                 "sparse forest backward");
  });
  og.finish();
  TouchedMasks masks = touched_masks(call.problem, x, need_x, thr, need_thr, ord, w, need_w);
  if (need_x) grads[0] = to_sparse(gx, masks.x);
  if (need_thr) grads[1] = to_sparse(gthr, masks.thr);
  if (need_w) grads[3] = to_sparse(gw, masks.w);
  return grads;
}

std::vector<torch::Tensor> linear_backward(int kind, torch::Tensor data, bool need_data, const torch::Tensor *vec,
                                           bool need_vec, torch::Tensor thr, bool need_thr, torch::Tensor ord,
                                           bool need_ord, torch::Tensor w, bool need_w, torch::Tensor lin, bool need_lin,
                                           torch::Tensor bias, bool need_bias, torch::Tensor g);

// Sparse data / threshold / leaf-weight gradients; the linear layer's gradients stay dense
// (hingetree_sparse_gpu.cu:743-761).
std::vector<torch::Tensor> sparse_linear_backward(int kind, torch::Tensor x, bool need_x, torch::Tensor thr, bool need_thr,
                                                  torch::Tensor ord, bool need_ord, torch::Tensor w, bool need_w,
                                                  torch::Tensor lin, bool need_lin, torch::Tensor bias, bool need_bias,
                                                  torch::Tensor g) {
  std::vector<torch::Tensor> grads =
      linear_backward(kind, x, need_x, nullptr, false, thr, need_thr, ord, need_ord, w, need_w, lin, need_lin, bias,
                      need_bias, g);
  if (!need_x && !need_thr && !need_w) return grads;
  FamilyCall call(kind, x, nullptr, thr, ord, w, &lin, &bias, &g);
  c10::DeviceGuard guard(x.device());
  TouchedMasks masks = touched_masks(call.problem, x, need_x, thr, need_thr, ord, w, need_w);
  if (need_x) grads[0] = to_sparse(grads[0], masks.x);
  if (need_thr) grads[1] = to_sparse(grads[1], masks.thr);
  if (need_w) grads[3] = to_sparse(grads[3], masks.w);
  return grads;
}

// ---- trie ------------------------------------------------------------------------------------------
// Weights are [T, 2^depth - 1, ...]: one row per internal vertex (hingetrie.cpp:43-49).

struct TrieCall {
  ht_forest_problem problem;
  std::vector<int64_t> out_sizes;
  TrieCall(const torch::Tensor &x, const torch::Tensor &thr, const torch::Tensor &ord, const torch::Tensor &w,
           const torch::Tensor *g) {
    if (x.dtype() != thr.dtype() || torch::kInt64 != ord.scalar_type() || x.dtype() != w.dtype() ||
        (g != nullptr && x.dtype() != g->dtype()))
      bad_argument("Error: inData, inThresholds, inWeights (and outDataGrad) are expected to share the same torch real "
                   "number data type. inOrdinals is expected to be type torch.int64.");
    if (x.device() != thr.device() || x.device() != ord.device() || x.device() != w.device() ||
        (g != nullptr && x.device() != g->device()))
      bad_argument("Error: All tensors are expected to be on the same device.");
    if (!x.is_contiguous() || !thr.is_contiguous() || !ord.is_contiguous() || !w.is_contiguous() ||
        (g != nullptr && !g->is_contiguous()))
      bad_argument("Error: All tensors are expected to be contiguous.");
    require_real(x);
    require_cuda(x);
    if (x.dim() < 2 || thr.dim() != 2 || ord.dim() != 2 || w.dim() < 2)
      bad_argument("Error: inData, inWeights must have at least 2 dimensions. inThresholds and inOrdinals must have 2 "
                   "dimensions.");
    if (thr.sizes() != ord.sizes() || w.size(0) != thr.size(0) || w.size(1) != thr.size(1))
      bad_argument("Error: inThresholds and inOrdinals must be the same shape, and inWeights.shape[:2] must equal it.");
    const int depth = depth_of(w.size(1) + 1);
    if (depth > 31 || depth < 1) {
      std::ostringstream ss;
      ss << "Error: The tree depth exceeds compile-time constraints or the number of thresholds is incorrect for the "
            "tree depth (tree depth = "
         << depth << ").";
      bad_runtime(ss.str());
    }
    problem = {HT_KIND_TREE, depth, x.size(0), x.size(1), inner_count(x, 2), w.size(0), inner_count(w, 2), 0, 0};
    out_sizes = {x.size(0), w.size(0)};
    for (int64_t d = 2; d < x.dim(); ++d) out_sizes.push_back(x.size(d));
    for (int64_t d = 2; d < w.dim(); ++d) out_sizes.push_back(w.size(d));
    if (g != nullptr && g->sizes() != c10::IntArrayRef(out_sizes))
      bad_argument("Error: outDataGrad.shape does not match the expected shape.");
  }
};

torch::Tensor trie_forward(torch::Tensor x, torch::Tensor thr, torch::Tensor ord, torch::Tensor w) {
  TrieCall call(x, thr, ord, w, nullptr);
  c10::DeviceGuard guard(x.device());
  torch::Tensor out = torch::empty(call.out_sizes, x.options());
  torch::Tensor ws = make_workspace(ht_forest_workspace_bytes(&call.problem), x);
  OrdinalGuard og(ord, call.problem.C);
  dispatch_real(x, [&](auto real) {
    using Real = decltype(real);
    raise_status(abi::trie_forward(&call.problem, x.data_ptr<Real>(), thr.data_ptr<Real>(), ord.data_ptr<int64_t>(),
                                     w.data_ptr<Real>(), out.data_ptr<Real>(), ws.data_ptr(), ws.numel(), og.word(),
                                     current_stream(x)),
                 "trie forward");
  });
  og.finish();
  return out;
}

std::vector<torch::Tensor> trie_backward(torch::Tensor x, bool need_x, torch::Tensor thr, bool need_thr, torch::Tensor ord,
                                         bool need_ord, torch::Tensor w, bool need_w, torch::Tensor g) {
  if (need_ord) bad_runtime("Error: Gradient on inOrdinals is requested, but inOrdinals never has a gradient.");
  TrieCall call(x, thr, ord, w, &g);
  c10::DeviceGuard guard(x.device());
  std::vector<torch::Tensor> grads(4);
  if (!need_x && !need_thr && !need_w) return grads;
  if (need_x) grads[0] = torch::empty_like(x);
  if (need_thr) grads[1] = torch::empty_like(thr);
  if (need_w) grads[3] = torch::empty_like(w);
  torch::Tensor ws = make_workspace(ht_forest_workspace_bytes(&call.problem), x);
  OrdinalGuard og(ord, call.problem.C);
  dispatch_real(x, [&](auto real) {
    using Real = decltype(real);
    raise_status(abi::trie_backward(&call.problem, x.data_ptr<Real>(), thr.data_ptr<Real>(), ord.data_ptr<int64_t>(),
                                      w.data_ptr<Real>(), g.data_ptr<Real>(), ptr_or_null<Real>(grads[0]),
                                      ptr_or_null<Real>(grads[1]), ptr_or_null<Real>(grads[3]), ws.data_ptr(), ws.numel(), og.word(),
                                      current_stream(x)),
                 "trie backward");
  });
  og.finish();
  return grads;
}

// ---- convolution -------------------------------------------------------------------------------
// Checks follow hingetree_conv.cpp:51-130 (argument problems -> ValueError; geometry, ordinal
// range and depth -> RuntimeError).

struct ConvCall {
  ht_conv_problem problem;
  std::vector<int64_t> out_sizes;
  int64_t window_cells = 1;

  ConvCall(int kind, int dims, const torch::Tensor &x, const torch::Tensor &thr, const torch::Tensor &ord,
           const torch::Tensor &w, const torch::Tensor *g, const std::vector<int64_t> &kernel,
           const std::vector<int64_t> &stride, const std::vector<int64_t> &padding, const std::vector<int64_t> &dilation) {
    if (x.dtype() != thr.dtype() || torch::kInt64 != ord.scalar_type() || x.dtype() != w.dtype() ||
        (g != nullptr && x.dtype() != g->dtype()))
      bad_argument("Error: inData, inThresholds, inWeights (and outDataGrad) are expected to share the same torch real "
                   "number data type. inOrdinals is expected to be type torch.int64.");
    if (x.device() != thr.device() || x.device() != ord.device() || x.device() != w.device() ||
        (g != nullptr && x.device() != g->device()))
      bad_argument("Error: All tensors are expected to be on the same device.");
    if (!x.is_contiguous() || !thr.is_contiguous() || !ord.is_contiguous() || !w.is_contiguous() ||
        (g != nullptr && !g->is_contiguous()))
      bad_argument("Error: All tensors are expected to be contiguous.");
    require_real(x);
    require_cuda(x);
    if ((int)kernel.size() != dims || (int)stride.size() != dims || (int)padding.size() != dims ||
        (int)dilation.size() != dims) {
      std::ostringstream ss;
      ss << "Error: kernel, stride, padding, dilation all expected to have " << dims << " dimensions.";
      bad_argument(ss.str());
    }
    if (x.dim() != dims + 2 || thr.dim() != 3 || ord.dim() != 3 || w.dim() < 3) {
      std::ostringstream ss;
      ss << "Error: inData expected to have " << dims + 2
         << " dimensions. inThresholds, inOrdinals expected to have 3 dimensions. inWeights expected to have at least 3 "
            "dimensions.";
      bad_argument(ss.str());
    }
    if (thr.sizes() != ord.sizes() || w.size(0) != thr.size(0) || w.size(1) != thr.size(1))
      bad_argument("Error: inThresholds and inOrdinals must be the same shape. inWeights.shape[0] and shape[1] must be "
                   "the same as inThresholds.shape[0] and shape[1].");
    if (w.size(1) != x.size(1))
      bad_argument("Error: inWeights.shape[1] must equal inData.shape[1]: only one channel group is supported.");
    const int depth = depth_of(w.size(2));
    problem.kind = kind;
    problem.depth = depth;
    problem.dims = dims;
    problem.reserved = 0;
    problem.B = x.size(0);
    problem.Ci = x.size(1);
    problem.Co = w.size(0);
    problem.M = inner_count(w, 3);
    for (int d = 0; d < 3; ++d) {
      problem.size[d] = d < dims ? x.size(2 + d) : 1;
      problem.kernel[d] = d < dims ? kernel[d] : 1;
      problem.stride[d] = d < dims ? stride[d] : 1;
      problem.padding[d] = d < dims ? padding[d] : 0;
      problem.dilation[d] = d < dims ? dilation[d] : 1;
      if (d < dims) window_cells *= kernel[d];
    }
    if (depth > 31 || depth < 1 || thr.size(2) != threshold_count(kind, depth)) {
      std::ostringstream ss;
      ss << "Error: The tree depth exceeds compile-time constraints or the number of thresholds is incorrect for the "
            "tree depth (tree depth = "
         << depth << ").";
      bad_runtime(ss.str());
    }
    int64_t osize[3] = {1, 1, 1};
    const int rc = ht_conv_output_size(&problem, osize);
    if (rc == HT_ERR_INVALID_ARGUMENT) bad_runtime("Error: Unable to convert image patches to matrix.");
    raise_status(rc, "convolution geometry");
    out_sizes = {x.size(0), w.size(0)};
    for (int d = 0; d < dims; ++d) out_sizes.push_back(osize[d]);
    for (int64_t d = 3; d < w.dim(); ++d) out_sizes.push_back(w.size(d));
    if (g != nullptr && g->sizes() != c10::IntArrayRef(out_sizes)) {
      std::ostringstream ss;
      ss << "Error: outDataGrad.shape does not match the expected shape (" << g->sizes() << " != "
         << c10::IntArrayRef(out_sizes) << ").";
      bad_argument(ss.str());
    }
  }
};

torch::Tensor conv_forward(int kind, int dims, torch::Tensor x, torch::Tensor thr, torch::Tensor ord, torch::Tensor w,
                           std::vector<int64_t> kernel, std::vector<int64_t> stride, std::vector<int64_t> padding,
                           std::vector<int64_t> dilation) {
  ConvCall call(kind, dims, x, thr, ord, w, nullptr, kernel, stride, padding, dilation);
  c10::DeviceGuard guard(x.device());
  torch::Tensor out = torch::empty(call.out_sizes, x.options());
  torch::Tensor ws = make_workspace(ht_conv_workspace_bytes(&call.problem), x);
  OrdinalGuard og(ord, call.window_cells);
  dispatch_real(x, [&](auto real) {
    using Real = decltype(real);
    raise_status(abi::conv_forward(&call.problem, x.data_ptr<Real>(), thr.data_ptr<Real>(), ord.data_ptr<int64_t>(),
                                     w.data_ptr<Real>(), out.data_ptr<Real>(), ws.data_ptr(), ws.numel(), og.word(),
                                     current_stream(x)),
                 "convolution forward");
  });
  og.finish();
  return out;
}

std::vector<torch::Tensor> conv_backward(int kind, int dims, torch::Tensor x, bool need_x, torch::Tensor thr, bool need_thr,
                                         torch::Tensor ord, bool need_ord, torch::Tensor w, bool need_w, torch::Tensor g,
                                         std::vector<int64_t> kernel, std::vector<int64_t> stride,
                                         std::vector<int64_t> padding, std::vector<int64_t> dilation) {
  if (need_ord) bad_runtime("Error: Gradient on inOrdinals is requested, but inOrdinals never has a gradient.");
  ConvCall call(kind, dims, x, thr, ord, w, &g, kernel, stride, padding, dilation);
  c10::DeviceGuard guard(x.device());
  std::vector<torch::Tensor> grads(4);
  if (!need_x && !need_thr && !need_w) return grads;
  if (need_x) grads[0] = torch::empty_like(x);
  if (need_thr) grads[1] = torch::empty_like(thr);
  if (need_w) grads[3] = torch::empty_like(w);
  torch::Tensor ws = make_workspace(ht_conv_workspace_bytes(&call.problem), x);
  OrdinalGuard og(ord, call.window_cells);
  dispatch_real(x, [&](auto real) {
    using Real = decltype(real);
    raise_status(abi::conv_backward(&call.problem, x.data_ptr<Real>(), thr.data_ptr<Real>(), ord.data_ptr<int64_t>(),
                                      w.data_ptr<Real>(), g.data_ptr<Real>(), ptr_or_null<Real>(grads[0]),
                                      ptr_or_null<Real>(grads[1]), ptr_or_null<Real>(grads[3]), ws.data_ptr(), ws.numel(), og.word(),
                                      current_stream(x)),
                 "convolution backward");
  });
  og.finish();
  return grads;
}

// ---- contract / expand (expand.cpp:353-457, 475-577) ---------------------------------------

int element_bytes_of(const torch::Tensor &t) {
  switch (t.scalar_type()) {
    case torch::kUInt8:
    case torch::kInt8:
    case torch::kInt16:
    case torch::kInt32:
    case torch::kInt64:
    case torch::kFloat32:
    case torch::kFloat64:
      return (int)t.element_size();
    default:
      bad_argument("Error: Unsupported data type. Only torch.uint8, int8, int16, int32, int64, float32 and float64 are "
                   "supported.");
  }
}

torch::Tensor contract_op(torch::Tensor x, std::vector<int64_t> window, std::vector<int64_t> padding) {
  if (window.empty() || window.size() != padding.size())
    bad_argument("Error: window and padding must be non-empty and the same size.");
  if (!x.is_contiguous()) bad_argument("Error: All tensors are expected to be contiguous.");
  const int elem = element_bytes_of(x);
  const int dims = (int)window.size();
  if (dims != 2 && dims != 3) bad_argument("Error: Only 2D and 3D window sizes are supported.");
  require_cuda(x);
  if (x.dim() != dims + 2) {
    std::ostringstream ss;
    ss << "Error: inData must have " << dims + 2 << " dimensions. Padding must be non-negative.";
    bad_argument(ss.str());
  }
  std::vector<int64_t> sizes = {x.size(0), x.size(1)}, size(dims);
  for (int d = 0; d < dims; ++d) {
    size[d] = x.size(2 + d);
    if (padding[d] < 0) bad_argument("Error: Padding must be non-negative.");
    if (window[d] < 1 || window[d] > size[d] + 2 * padding[d])
      bad_argument("Error: Window dimensions must be at least 1 but no greater than the size of the padded image.");
    sizes.push_back((size[d] + 2 * padding[d] - window[d]) / window[d] + 1);
  }
  sizes.insert(sizes.end(), window.begin(), window.end());
  c10::DeviceGuard guard(x.device());
  torch::Tensor out = torch::empty(sizes, x.options());
  raise_status(ht_contract(dims, elem, x.data_ptr(), out.data_ptr(), x.size(0) * x.size(1), size.data(), window.data(),
                           padding.data(), current_stream(x)),
               "contract");
  return out;
}

torch::Tensor expand_op(torch::Tensor x, std::vector<int64_t> padding) {
  if (padding.empty()) bad_argument("Error: padding must be non-empty.");
  if (!x.is_contiguous()) bad_argument("Error: All tensors are expected to be contiguous.");
  const int elem = element_bytes_of(x);
  const int dims = (int)padding.size();
  if (dims != 2 && dims != 3) bad_argument("Error: Only 2D and 3D padding sizes are supported.");
  require_cuda(x);
  if (x.dim() != 2 * dims + 2) {
    std::ostringstream ss;
    ss << "Error: inData must have " << 2 * dims + 2 << " dimensions. Padding must be non-negative.";
    bad_argument(ss.str());
  }
  std::vector<int64_t> sizes = {x.size(0), x.size(1)}, osize(dims), window(dims);
  for (int d = 0; d < dims; ++d) {
    osize[d] = x.size(2 + d);
    window[d] = x.size(2 + dims + d);
    if (padding[d] < 0) bad_argument("Error: Padding must be non-negative.");
    const int64_t extent = window[d] > 0 ? osize[d] * window[d] - ((2 * padding[d]) / window[d]) * window[d] : 0;
    if (extent < 1) bad_argument("Error: The expanded size of the image must be non-empty.");
    sizes.push_back(extent);
  }
  c10::DeviceGuard guard(x.device());
  torch::Tensor out = torch::empty(sizes, x.options());
  raise_status(ht_expand(dims, elem, x.data_ptr(), out.data_ptr(), x.size(0) * x.size(1), osize.data(), window.data(),
                         padding.data(), current_stream(x)),
               "expand");
  return out;
}

}  // namespace

#define HT_BIND_CONV(prefix, KIND, D)                                                                                \
  m.def(prefix "_conv" #D "d_forward",                                                                               \
        [](torch::Tensor x, torch::Tensor t, torch::Tensor o, torch::Tensor w, std::vector<int64_t> k,                \
           std::vector<int64_t> s, std::vector<int64_t> p, std::vector<int64_t> d) {                                  \
          return conv_forward(KIND, D, x, t, o, w, k, s, p, d);                                                       \
        });                                                                                                          \
  m.def(prefix "_conv" #D "d_backward",                                                                              \
        [](torch::Tensor x, bool nx, torch::Tensor t, bool nt, torch::Tensor o, bool no, torch::Tensor w, bool nw,    \
           torch::Tensor g, std::vector<int64_t> k, std::vector<int64_t> s, std::vector<int64_t> p,                   \
           std::vector<int64_t> d) { return conv_backward(KIND, D, x, nx, t, nt, o, no, w, nw, g, k, s, p, d); });

#define HT_BIND_FAMILY(prefix, KIND)                                                                                 \
  m.def(prefix "_fusion_forward", [](torch::Tensor img, torch::Tensor vec, torch::Tensor t, torch::Tensor o,          \
                                     torch::Tensor w) { return fusion_forward(KIND, img, vec, t, o, w); });           \
  m.def(prefix "_fusion_backward",                                                                                    \
        [](torch::Tensor img, bool ni, torch::Tensor vec, bool nv, torch::Tensor t, bool nt, torch::Tensor o, bool no, \
           torch::Tensor w, bool nw, torch::Tensor g) {                                                               \
          return fusion_backward(KIND, img, ni, vec, nv, t, nt, o, no, w, nw, g);                                      \
        });                                                                                                           \
  m.def(prefix "_fused_linear_forward", [](torch::Tensor x, torch::Tensor t, torch::Tensor o, torch::Tensor w,        \
                                           torch::Tensor l, torch::Tensor b) {                                        \
    return linear_forward(KIND, x, nullptr, t, o, w, l, b);                                                           \
  });                                                                                                                 \
  m.def(prefix "_fused_linear_backward",                                                                              \
        [](torch::Tensor x, bool nx, torch::Tensor t, bool nt, torch::Tensor o, bool no, torch::Tensor w, bool nw,     \
           torch::Tensor l, bool nl, torch::Tensor b, bool nb, torch::Tensor g) {                                      \
          return linear_backward(KIND, x, nx, nullptr, false, t, nt, o, no, w, nw, l, nl, b, nb, g);                   \
        });                                                                                                           \
  m.def(prefix "_fusion_fused_linear_forward", [](torch::Tensor img, torch::Tensor vec, torch::Tensor t,              \
                                                  torch::Tensor o, torch::Tensor w, torch::Tensor l, torch::Tensor b) { \
    return linear_forward(KIND, img, &vec, t, o, w, l, b);                                                            \
  });                                                                                                                 \
  m.def(prefix "_fusion_fused_linear_backward",                                                                       \
        [](torch::Tensor img, bool ni, torch::Tensor vec, bool nv, torch::Tensor t, bool nt, torch::Tensor o, bool no, \
           torch::Tensor w, bool nw, torch::Tensor l, bool nl, torch::Tensor b, bool nb, torch::Tensor g) {            \
          return linear_backward(KIND, img, ni, &vec, nv, t, nt, o, no, w, nw, l, nl, b, nb, g);                       \
        });

void bind_more_ops(pybind11::module_ &m) {
  HT_BIND_FAMILY("tree", HT_KIND_TREE)
  HT_BIND_FAMILY("fern", HT_KIND_FERN)
  HT_BIND_CONV("tree", HT_KIND_TREE, 1)
  HT_BIND_CONV("tree", HT_KIND_TREE, 2)
  HT_BIND_CONV("tree", HT_KIND_TREE, 3)
  HT_BIND_CONV("fern", HT_KIND_FERN, 1)
  HT_BIND_CONV("fern", HT_KIND_FERN, 2)
  HT_BIND_CONV("fern", HT_KIND_FERN, 3)
  m.def("contract", &contract_op, "Collapse batched 2D or 3D image to 2D or 3D images of patches.");
  m.def("expand", &expand_op, "Expand batched 2D or 3D images of patches to 2D or 3D images.");
  m.def("sparse_tree_backward", [](torch::Tensor x, bool nx, torch::Tensor t, bool nt, torch::Tensor o, bool no,
                                   torch::Tensor w, bool nw, torch::Tensor g) {
    return sparse_backward(HT_KIND_TREE, x, nx, t, nt, o, no, w, nw, g);
  });
  m.def("sparse_fern_backward", [](torch::Tensor x, bool nx, torch::Tensor t, bool nt, torch::Tensor o, bool no,
                                   torch::Tensor w, bool nw, torch::Tensor g) {
    return sparse_backward(HT_KIND_FERN, x, nx, t, nt, o, no, w, nw, g);
  });
  m.def("sparse_tree_fused_linear_backward",
        [](torch::Tensor x, bool nx, torch::Tensor t, bool nt, torch::Tensor o, bool no, torch::Tensor w, bool nw,
           torch::Tensor l, bool nl, torch::Tensor b, bool nb, torch::Tensor g) {
          return sparse_linear_backward(HT_KIND_TREE, x, nx, t, nt, o, no, w, nw, l, nl, b, nb, g);
        });
  m.def("sparse_fern_fused_linear_backward",
        [](torch::Tensor x, bool nx, torch::Tensor t, bool nt, torch::Tensor o, bool no, torch::Tensor w, bool nw,
           torch::Tensor l, bool nl, torch::Tensor b, bool nb, torch::Tensor g) {
          return sparse_linear_backward(HT_KIND_FERN, x, nx, t, nt, o, no, w, nw, l, nl, b, nb, g);
        });
  m.def("trie_forward", &trie_forward, "Hinge trie forward.");
  m.def("trie_backward", &trie_backward, "Hinge trie backward.");
  m.def("trie_init_medians", [](torch::Tensor x, torch::Tensor t, torch::Tensor o, torch::Tensor w) {
    return init_medians(InitFamily::Trie, x, t, o, w);
  });
}

}  // namespace htx
