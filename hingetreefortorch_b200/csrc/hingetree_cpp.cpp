// torch extension `hingetree_cpp`: the host side of the drop-in.  It presents the operator
// names, argument order, checks and exception types of the reference's pybind module
// (hingetree.cpp:1962-2031) and does nothing but validate, allocate and forward to the C ABI
// in hingetree_b200.h on the caller's current CUDA stream.  There is no CPU evaluation path:
// CPU tensors are refused, except by the threshold-hygiene utilities, which the reference
// itself only runs on CPU tensors (module constructors call them before .to(device)).
#include <torch/extension.h>

#include <c10/core/DeviceGuard.h>
#include <c10/cuda/CUDAFunctions.h>
#include <c10/cuda/CUDAStream.h>

#include <algorithm>
#include <cmath>
#include <limits>
#include <mutex>
#include <numeric>
#include <sstream>
#include <stdexcept>
#include <string>
#include <vector>

#include "hingetree_b200.h"
#include "hingetree_cpp_ops.h"

namespace htx {

[[noreturn]] void bad_argument(const std::string &what) { throw std::invalid_argument(what); }
[[noreturn]] void bad_runtime(const std::string &what) { throw std::runtime_error(what); }

ht_stream_t current_stream(const torch::Tensor &t) {
  return reinterpret_cast<ht_stream_t>(c10::cuda::getCurrentCUDAStream(t.device().index()).stream());
}

void raise_status(int rc, const char *op) {
  if (rc == HT_OK) return;
  std::ostringstream ss;
  ss << "Error: " << op << ": " << ht_status_string(rc);
  if (rc == HT_ERR_CUDA) ss << " (cudaError " << ht_last_cuda_error() << ")";
  ss << ".";
  if (rc == HT_ERR_INVALID_ARGUMENT) bad_argument(ss.str());
  bad_runtime(ss.str());
}

int64_t inner_count(const torch::Tensor &t, int64_t from) {
  int64_t n = 1;
  for (int64_t d = from; d < t.dim(); ++d) n *= t.size(d);
  return n;
}

// -1 unless the leaf count is a power of two (the reference's ComputeDepth).
int depth_of(int64_t leaves) {
  if (leaves <= 0 || (leaves & (leaves - 1)) != 0) return -1;
  int d = 0;
  while (leaves > 1) {
    leaves >>= 1;
    ++d;
  }
  return d;
}

int64_t threshold_count(int kind, int depth) { return kind == HT_KIND_FERN ? depth : (int64_t(1) << depth) - 1; }

void require_cuda(const torch::Tensor &t) {
  if (!t.is_cuda())
    bad_runtime("Error: this build of hingetree_cpp evaluates on CUDA devices only (no CPU path); move the tensors "
                "to a CUDA device.");
}

void require_float32(const torch::Tensor &t) {
  if (t.scalar_type() == torch::kFloat32) return;
  if (t.scalar_type() == torch::kFloat64)
    bad_argument("Error: this operator takes torch.float32 only (the reference's operators take torch.float64 as well and so "
                 "do their counterparts here; the additions to the reference's surface are single precision).");
  bad_argument("Error: Unsupported data type. Only torch.float32 and torch.float64 are supported.");
}

// ---- ordinal validation ----------------------------------------------------------------
// The reference reads min/max of the ordinals back to the host on every call
// (hingetree_gpu.cu:445).  Here the kernels flag out-of-range ordinals in a device word;
// the word is read back (one small blocking copy) unless this exact ordinals storage at
// this exact version has already been seen valid for this channel count.
namespace {

enum class OrdinalCheck { Cached, Always, Never };
OrdinalCheck g_ordinal_check = OrdinalCheck::Cached;

struct SeenOrdinals {
  c10::weak_intrusive_ptr<c10::StorageImpl> storage;
  const void *data;
  int64_t version;
  int64_t numel;
  int64_t channels;
};
std::mutex g_seen_mutex;
std::vector<SeenOrdinals> g_seen;

bool seen_valid(const torch::Tensor &ord, int64_t channels) {
  if (g_ordinal_check != OrdinalCheck::Cached || ord.is_inference()) return false;
  std::lock_guard<std::mutex> lock(g_seen_mutex);
  for (auto it = g_seen.begin(); it != g_seen.end();) {
    if (it->storage.expired()) {
      it = g_seen.erase(it);
      continue;
    }
    if (it->data == ord.const_data_ptr() && it->version == ord._version() && it->numel == ord.numel() &&
        it->channels == channels && it->storage._unsafe_get_target() == ord.storage().unsafeGetStorageImpl())
      return true;
    ++it;
  }
  return false;
}

void remember_valid(const torch::Tensor &ord, int64_t channels) {
  if (g_ordinal_check != OrdinalCheck::Cached || ord.is_inference()) return;
  std::lock_guard<std::mutex> lock(g_seen_mutex);
  if (g_seen.size() >= 256) g_seen.erase(g_seen.begin());
  auto strong = c10::intrusive_ptr<c10::StorageImpl>::reclaim_copy(ord.storage().unsafeGetStorageImpl());
  g_seen.push_back({c10::weak_intrusive_ptr<c10::StorageImpl>(strong), ord.const_data_ptr(), ord._version(),
                    ord.numel(), channels});
}

}  // namespace

// Calls whose ordinals are already known to be valid do not read anything back (no synchronisation), but their
// kernels still get a status word: one long-lived word per device that collects HT_FLAG_PIPELINE_TIMEOUT (a
// bounded wait inside a kernel ran out: outputs incomplete).  It is read together with the next call that
// synchronises anyway, and by pipeline_status().
namespace {
std::mutex g_sticky_mutex;
std::vector<torch::Tensor> g_sticky_words;

torch::Tensor sticky_word(const c10::Device &device, bool create) {
  std::lock_guard<std::mutex> lock(g_sticky_mutex);
  const size_t index = device.has_index() ? (size_t)device.index() : (size_t)c10::cuda::current_device();
  if (g_sticky_words.size() <= index) g_sticky_words.resize(index + 1);
  if (!g_sticky_words[index].defined() && create)
    g_sticky_words[index] = torch::zeros({1}, torch::TensorOptions().dtype(torch::kInt32).device(device));
  return g_sticky_words[index];
}

[[noreturn]] void raise_pipeline_timeout() {
  bad_runtime("Error: a bounded wait inside a hinge tree kernel ran out (a parameter or gradient copy never arrived); "
              "the results of the calls since the last check are incomplete.");
}
}  // namespace

OrdinalGuard::OrdinalGuard(const torch::Tensor &ord, int64_t channels) : ord_(ord), channels_(channels) {
  check_ = g_ordinal_check != OrdinalCheck::Never && !seen_valid(ord, channels);
  // a checked call synchronises and is never part of a stream capture: the place to create the device's word
  if (check_) {
    word_ = torch::zeros({1}, torch::TensorOptions().dtype(torch::kInt32).device(ord.device()));
    sticky_ = sticky_word(ord.device(), true);
  } else {
    sticky_ = sticky_word(ord.device(), false);
  }
}

uint32_t *OrdinalGuard::word() {
  if (check_) return reinterpret_cast<uint32_t *>(word_.data_ptr<int32_t>());
  return sticky_.defined() ? reinterpret_cast<uint32_t *>(sticky_.data_ptr<int32_t>()) : nullptr;
}

void OrdinalGuard::finish() {
  if (!check_) return;
  const torch::Tensor both = torch::cat({word_, sticky_}).cpu();  // one blocking copy for both words
  const int32_t flags = both.data_ptr<int32_t>()[0], earlier = both.data_ptr<int32_t>()[1];
  if (earlier != 0) sticky_.zero_();
  if (((uint32_t)flags | (uint32_t)earlier) & HT_FLAG_PIPELINE_TIMEOUT) raise_pipeline_timeout();
  if (flags & (int32_t)HT_FLAG_ORDINAL_RANGE)
    bad_runtime("Error: An ordinal value is either negative or larger than or equal to the number of channels.");
  remember_valid(ord_, channels_);
}

// Reads (and clears) the long-lived status word of the current device; raises when a kernel reported a timeout.
int64_t pipeline_status() {
  torch::Tensor word = sticky_word(c10::Device(c10::kCUDA, c10::cuda::current_device()), false);
  if (!word.defined()) return 0;
  const int32_t flags = word.item<int32_t>();
  if (flags != 0) word.zero_();
  if ((uint32_t)flags & HT_FLAG_PIPELINE_TIMEOUT) raise_pipeline_timeout();
  return flags;
}

// The library's self test of a bounded wait, reporting into the current device's long-lived status word exactly
// as a tile kernel would: the next pipeline_status() (or checked call) raises.
void selftest_bounded_wait() {
  const c10::Device device(c10::kCUDA, c10::cuda::current_device());
  torch::Tensor word = sticky_word(device, true);
  raise_status(ht_selftest_bounded_wait(reinterpret_cast<uint32_t *>(word.data_ptr<int32_t>()),
                                        (ht_stream_t)c10::cuda::getCurrentCUDAStream().stream()),
               "selftest_bounded_wait");
}

// Most scratch a backward call may take for its per-evaluation records (12 bytes per tree
// evaluation).  Beyond it the call runs without them: atomic scatters instead of ordered sums.
// Default: whatever fits (an allocation that fails falls back to the path without records); a caller may
// set a smaller figure.
static int64_t g_backward_scratch_limit = INT64_MAX;

void set_backward_scratch_limit(int64_t bytes) {
  if (bytes < 0) bad_argument("Error: the scratch limit is a number of bytes >= 0.");
  g_backward_scratch_limit = bytes;
}

void set_ordinal_check(const std::string &mode) {
  if (mode == "cached")
    g_ordinal_check = OrdinalCheck::Cached;
  else if (mode == "always")
    g_ordinal_check = OrdinalCheck::Always;
  else if (mode == "never")
    g_ordinal_check = OrdinalCheck::Never;
  else
    bad_argument("Error: ordinal check mode must be 'cached', 'always' or 'never'.");
}

torch::Tensor make_workspace(size_t bytes, const torch::Tensor &like) {
  return torch::empty({(int64_t)std::max<size_t>(bytes, 256)}, torch::TensorOptions().dtype(torch::kUInt8).device(like.device()));
}

// ---- plain forest ------------------------------------------------------------------------

ForestCall::ForestCall(int kind, const torch::Tensor &x, const torch::Tensor &thr, const torch::Tensor &ord,
                       const torch::Tensor &w, const torch::Tensor *g, bool allow_double) {
  // same order of checks as the reference dispatcher and GPU host function
  // (hingetree.cpp:648-664, hingetree_gpu.cu:420-447)
  if (x.dtype() != thr.dtype() || torch::kInt64 != ord.scalar_type() || x.dtype() != w.dtype() ||
      (g != nullptr && x.dtype() != g->dtype()))
    bad_argument(g == nullptr
                     ? "Error: inData, inThresholds, inWeights are expected to share the same torch real number data "
                       "type. inOrdinals is expected to be type torch.int64."
                     : "Error: inData, inThresholds, inWeights, outDataGrad are expected to share the same torch real "
                       "number data type. inOrdinals is expected to be type torch.int64.");
  if (x.device() != thr.device() || x.device() != ord.device() || x.device() != w.device() ||
      (g != nullptr && x.device() != g->device()))
    bad_argument("Error: All tensors are expected to be on the same device.");
  if (!x.is_contiguous() || !thr.is_contiguous() || !ord.is_contiguous() || !w.is_contiguous() ||
      (g != nullptr && !g->is_contiguous()))
    bad_argument("Error: All tensors are expected to be contiguous.");
  is_double = allow_double && x.scalar_type() == torch::kFloat64;
  if (!is_double) require_float32(x);
  require_cuda(x);
  if (x.dim() < 2 || thr.dim() != 2 || ord.dim() != 2 || w.dim() < 2)
    bad_argument("Error: inData, inWeights must have at least 2 dimensions. inThresholds and inOrdinals must have 2 "
                 "dimensions.");
  if (thr.sizes() != ord.sizes() || w.size(0) != thr.size(0))
    bad_argument("Error: inThresholds and inOrdinals must be the same shape. inWeights.shape[0] must be the same as "
                 "inThresholds.shape[0].");
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
  problem.B = x.size(0);
  problem.C = x.size(1);
  problem.K = inner_count(x, 2);
  problem.T = w.size(0);
  problem.M = inner_count(w, 2);
  problem.flags = 0;
  problem.reserved = 0;
  out_sizes = {x.size(0), w.size(0)};
  for (int64_t d = 2; d < x.dim(); ++d) out_sizes.push_back(x.size(d));
  map_sizes = out_sizes;
  for (int64_t d = 2; d < w.dim(); ++d) out_sizes.push_back(w.size(d));
  if (g != nullptr && g->sizes() != c10::IntArrayRef(out_sizes)) {
    std::ostringstream ss;
    ss << "Error: outDataGrad.shape does not match the expected shape (" << g->sizes() << " != "
       << c10::IntArrayRef(out_sizes) << ").";
    bad_argument(ss.str());
  }
}

namespace {

torch::Tensor forest_forward(int kind, torch::Tensor x, torch::Tensor thr, torch::Tensor ord, torch::Tensor w) {
  ForestCall call(kind, x, thr, ord, w, nullptr, true);
  c10::DeviceGuard guard(x.device());
  torch::Tensor out = torch::empty(call.out_sizes, x.options());
  torch::Tensor ws = make_workspace(ht_forest_workspace_bytes(&call.problem), x);
  OrdinalGuard og(ord, call.problem.C);
  if (call.is_double) {
    raise_status(ht_forest_forward_f64(&call.problem, x.data_ptr<double>(), thr.data_ptr<double>(), ord.data_ptr<int64_t>(),
                                       w.data_ptr<double>(), out.data_ptr<double>(), ws.data_ptr(), ws.numel(), og.word(),
                                       current_stream(x)),
                 "forest forward");
    og.finish();
    return out;
  }
  raise_status(ht_forest_forward_f32(&call.problem, x.data_ptr<float>(), thr.data_ptr<float>(), ord.data_ptr<int64_t>(),
                                     w.data_ptr<float>(), out.data_ptr<float>(), ws.data_ptr(), ws.numel(), og.word(),
                                     current_stream(x)),
               "forest forward");
  og.finish();
  return out;
}

std::vector<torch::Tensor> forest_backward(int kind, bool deterministic, torch::Tensor x, bool need_x, torch::Tensor thr,
                                           bool need_thr, torch::Tensor ord, bool need_ord, torch::Tensor w, bool need_w,
                                           torch::Tensor g) {
  if (need_ord) bad_runtime("Error: Gradient on inOrdinals is requested, but inOrdinals never has a gradient.");
  ForestCall call(kind, x, thr, ord, w, &g, true);
  c10::DeviceGuard guard(x.device());
  std::vector<torch::Tensor> grads(4);
  if (!need_x && !need_thr && !need_w) return grads;
  if (deterministic) call.problem.flags |= HT_DETERMINISTIC;
  if (need_x) grads[0] = torch::empty_like(x);
  if (need_thr) grads[1] = torch::empty_like(thr);
  if (need_w) grads[3] = torch::empty_like(w);
  if (call.is_double) {
    torch::Tensor ws = make_workspace(ht_forest_workspace_bytes(&call.problem), x);
    OrdinalGuard og(ord, call.problem.C);
    raise_status(
        ht_forest_backward_f64(&call.problem, x.data_ptr<double>(), thr.data_ptr<double>(), ord.data_ptr<int64_t>(),
                               w.data_ptr<double>(), g.data_ptr<double>(), need_x ? grads[0].data_ptr<double>() : nullptr,
                               need_thr ? grads[1].data_ptr<double>() : nullptr,
                               need_w ? grads[3].data_ptr<double>() : nullptr, ws.data_ptr(), ws.numel(), og.word(),
                               current_stream(x)),
        "forest backward");
    og.finish();
    return grads;
  }
  call.problem.flags |= HT_WORKSPACE_FOR_BACKWARD;
  if ((int64_t)ht_forest_workspace_bytes(&call.problem) > g_backward_scratch_limit && !deterministic)
    call.problem.flags &= ~HT_WORKSPACE_FOR_BACKWARD;
  torch::Tensor ws;
  try {
    ws = make_workspace(ht_forest_workspace_bytes(&call.problem), x);
  } catch (const c10::OutOfMemoryError &) {
    // no room for the evaluation records (10 to 12 bytes per tree evaluation): the default mode can do
    // without them (the reference allocates nothing for its backward either); the fixed-order mode cannot
    if (deterministic || (call.problem.flags & HT_WORKSPACE_FOR_BACKWARD) == 0) throw;
    call.problem.flags &= ~HT_WORKSPACE_FOR_BACKWARD;
    ws = make_workspace(ht_forest_workspace_bytes(&call.problem), x);
  }
  OrdinalGuard og(ord, call.problem.C);
  raise_status(
      ht_forest_backward_f32(&call.problem, x.data_ptr<float>(), thr.data_ptr<float>(), ord.data_ptr<int64_t>(),
                             w.data_ptr<float>(), g.data_ptr<float>(), need_x ? grads[0].data_ptr<float>() : nullptr,
                             need_thr ? grads[1].data_ptr<float>() : nullptr,
                             need_w ? grads[3].data_ptr<float>() : nullptr, ws.data_ptr(), ws.numel(), og.word(),
                             current_stream(x)),
      "forest backward");
  og.finish();
  return grads;
}

// ---- forward that keeps its traversal for the backward -----------------------------------------------------
// Not part of the reference's operator set: the reference's backward walks every tree again (three times).  These
// two let the autograd layer walk them once per training step.  `saved` is the call's scratch, which holds the
// traversal; it is empty when the library does not save for this problem (the caller then uses the plain backward).
static bool g_save_forward = true;

std::vector<torch::Tensor> forest_forward_saving(int kind, torch::Tensor x, torch::Tensor thr, torch::Tensor ord,
                                                 torch::Tensor w) {
  if (x.scalar_type() == torch::kFloat64)  // no kept traversal in double precision: the plain forward
    return {forest_forward(kind, x, thr, ord, w), torch::empty({0}, x.options().dtype(torch::kUInt8))};
  ForestCall call(kind, x, thr, ord, w, nullptr);
  c10::DeviceGuard guard(x.device());
  const bool saves = g_save_forward && ht_forest_forward_saves(&call.problem) != 0;
  if (saves) call.problem.flags |= HT_WORKSPACE_FOR_BACKWARD | HT_SAVE_FOR_BACKWARD;
  if (saves && (int64_t)ht_forest_workspace_bytes(&call.problem) > g_backward_scratch_limit)
    call.problem.flags &= ~(HT_WORKSPACE_FOR_BACKWARD | HT_SAVE_FOR_BACKWARD);
  torch::Tensor out = torch::empty(call.out_sizes, x.options());
  torch::Tensor ws;
  try {
    ws = make_workspace(ht_forest_workspace_bytes(&call.problem), x);
  } catch (const c10::OutOfMemoryError &) {
    if ((call.problem.flags & HT_SAVE_FOR_BACKWARD) == 0) throw;
    call.problem.flags &= ~(HT_WORKSPACE_FOR_BACKWARD | HT_SAVE_FOR_BACKWARD);  // no room: a plain forward
    ws = make_workspace(ht_forest_workspace_bytes(&call.problem), x);
  }
  OrdinalGuard og(ord, call.problem.C);
  raise_status(ht_forest_forward_f32(&call.problem, x.data_ptr<float>(), thr.data_ptr<float>(), ord.data_ptr<int64_t>(),
                                     w.data_ptr<float>(), out.data_ptr<float>(), ws.data_ptr(), ws.numel(), og.word(),
                                     current_stream(x)),
               "forest forward");
  og.finish();
  const bool saved = (call.problem.flags & HT_SAVE_FOR_BACKWARD) != 0;
  return {out, saved ? ws : torch::empty({0}, ws.options())};
}

std::vector<torch::Tensor> forest_backward_saved(int kind, bool deterministic, torch::Tensor x, bool need_x,
                                                 torch::Tensor thr, bool need_thr, torch::Tensor ord, bool need_ord,
                                                 torch::Tensor w, bool need_w, torch::Tensor g, torch::Tensor saved) {
  if (need_ord) bad_runtime("Error: Gradient on inOrdinals is requested, but inOrdinals never has a gradient.");
  ForestCall call(kind, x, thr, ord, w, &g);
  c10::DeviceGuard guard(x.device());
  std::vector<torch::Tensor> grads(4);
  if (!need_x && !need_thr && !need_w) return grads;
  if (deterministic) call.problem.flags |= HT_DETERMINISTIC;
  call.problem.flags |= HT_WORKSPACE_FOR_BACKWARD | HT_SAVED_FORWARD;
  if (!saved.defined() || saved.device() != x.device() || saved.scalar_type() != torch::kUInt8 ||
      (size_t)saved.numel() < ht_forest_workspace_bytes(&call.problem) || ht_forest_forward_saves(&call.problem) == 0)
    bad_argument("Error: `saved` is not the scratch a saving forward returned for these tensors.");
  if (need_x) grads[0] = torch::empty_like(x);
  if (need_thr) grads[1] = torch::empty_like(thr);
  if (need_w) grads[3] = torch::empty_like(w);
  OrdinalGuard og(ord, call.problem.C);
  raise_status(
      ht_forest_backward_f32(&call.problem, x.data_ptr<float>(), thr.data_ptr<float>(), ord.data_ptr<int64_t>(),
                             w.data_ptr<float>(), g.data_ptr<float>(), need_x ? grads[0].data_ptr<float>() : nullptr,
                             need_thr ? grads[1].data_ptr<float>() : nullptr,
                             need_w ? grads[3].data_ptr<float>() : nullptr, saved.data_ptr(), saved.numel(), og.word(),
                             current_stream(x)),
      "forest backward");
  og.finish();
  return grads;
}

// ---- dense projection with batch-normalisation statistics on the tensor cores --------------------------------
// Not part of the reference's operator set (its pipelines call torch.nn.Linear and torch.nn.BatchNorm1d,
// README.md:110-129).  Returns {z = x w^T (TF32 products, fp32 accumulation), column sums of z, column sums of z^2}.
std::vector<torch::Tensor> linear_tf32_stats(torch::Tensor x, torch::Tensor w) {
  if (x.scalar_type() != torch::kFloat32 || w.scalar_type() != torch::kFloat32)
    bad_argument("Error: x and w are expected to be torch.float32.");
  if (x.device() != w.device()) bad_argument("Error: All tensors are expected to be on the same device.");
  require_cuda(x);
  if (x.dim() != 2 || w.dim() != 2 || x.size(1) != w.size(1))
    bad_argument("Error: x must be [M, K] and w [N, K].");
  if (!x.is_contiguous() || !w.is_contiguous()) bad_argument("Error: All tensors are expected to be contiguous.");
  c10::DeviceGuard guard(x.device());
  const int64_t M = x.size(0), K = x.size(1), N = w.size(0);
  torch::Tensor z = torch::empty({M, N}, x.options());
  torch::Tensor sum = torch::empty({N}, x.options()), sumsq = torch::empty({N}, x.options());
  torch::Tensor status = sticky_word(x.device(), true);
  raise_status(ht_linear_tf32_stats_f32(x.data_ptr<float>(), w.data_ptr<float>(), z.data_ptr<float>(), sum.data_ptr<float>(),
                                        sumsq.data_ptr<float>(), M, N, K,
                                        reinterpret_cast<uint32_t *>(status.data_ptr<int32_t>()), current_stream(x)),
               "linear (tf32) with column statistics");
  return {z, sum, sumsq};
}

// The forest of a Linear -> BatchNorm1d(affine=False) -> forest pipeline on the raw activations z [B, C] with the
// normalisation's mean and 1/std per column (no reference operator: its pipeline materialises the normalisation).
namespace {
void check_statistics(const torch::Tensor &z, const torch::Tensor &mean, const torch::Tensor &invstd) {
  if (z.dim() != 2) bad_argument("Error: the activations are expected to be [batch, channels].");
  if (mean.scalar_type() != torch::kFloat32 || invstd.scalar_type() != torch::kFloat32 || mean.device() != z.device() ||
      invstd.device() != z.device() || mean.dim() != 1 || invstd.dim() != 1 || mean.size(0) != z.size(1) ||
      invstd.size(0) != z.size(1) || !mean.is_contiguous() || !invstd.is_contiguous())
    bad_argument("Error: mean and invstd are expected to be contiguous torch.float32 vectors of one entry per channel, "
                 "on the device of the activations.");
}
}  // namespace

// {mean, biased variance, 1 / sqrt(variance + eps)} of the columns from their sums and sums of squares over `rows` rows.
std::vector<torch::Tensor> batchnorm_statistics(torch::Tensor sum, torch::Tensor sumsq, int64_t rows, double eps) {
  if (sum.scalar_type() != torch::kFloat32 || sumsq.scalar_type() != torch::kFloat32 || sum.dim() != 1 ||
      sumsq.sizes() != sum.sizes() || sum.device() != sumsq.device() || !sum.is_contiguous() || !sumsq.is_contiguous())
    bad_argument("Error: sum and sumsq are expected to be contiguous torch.float32 vectors of the same length on one device.");
  require_cuda(sum);
  if (rows < 1) bad_argument("Error: rows must be positive.");
  c10::DeviceGuard guard(sum.device());
  torch::Tensor out = torch::empty({3, sum.size(0)}, sum.options());
  const int64_t C = sum.size(0);
  raise_status(ht_batchnorm_statistics_f32(sum.data_ptr<float>(), sumsq.data_ptr<float>(), rows, C, (float)eps,
                                           out.data_ptr<float>(), out.data_ptr<float>() + C, out.data_ptr<float>() + 2 * C,
                                           current_stream(sum)),
               "batch normalisation statistics");
  return {out[0], out[1], out[2]};
}

// Returns {out, margin, where}: with `keep` the forward leaves its traversal (signed margin; deciding vertex and leaf
// key) for forest_normalised_backward, else the two are empty tensors.
std::vector<torch::Tensor> forest_normalised_forward(int kind, torch::Tensor z, torch::Tensor mean, torch::Tensor invstd,
                                                     torch::Tensor thr, torch::Tensor ord, torch::Tensor w, bool keep) {
  ForestCall call(kind, z, thr, ord, w, nullptr);
  check_statistics(z, mean, invstd);
  c10::DeviceGuard guard(z.device());
  const int64_t B = call.problem.B, T = call.problem.T;
  torch::Tensor out = torch::empty(call.out_sizes, z.options());
  torch::Tensor margin = torch::empty({keep ? B : 0, T}, z.options());
  torch::Tensor where = torch::empty({keep ? B : 0, T, 2}, z.options().dtype(torch::kInt32));
  torch::Tensor ws = make_workspace(ht_forest_normalised_workspace_bytes(&call.problem), z);
  OrdinalGuard og(ord, call.problem.C);
  raise_status(ht_forest_normalised_forward_f32(&call.problem, z.data_ptr<float>(), mean.data_ptr<float>(),
                                                invstd.data_ptr<float>(), thr.data_ptr<float>(), ord.data_ptr<int64_t>(),
                                                w.data_ptr<float>(), out.data_ptr<float>(),
                                                keep && B * T > 0 ? margin.data_ptr<float>() : nullptr,
                                                keep && B * T > 0 ? where.data_ptr() : nullptr, ws.data_ptr(), ws.numel(),
                                                og.word(), current_stream(z)),
               "forest forward on normalised activations");
  og.finish();
  return {out, margin, where};
}

// Returns {dz, gthr or None, gw or None}: the gradient with respect to the RAW activations (through the
// normalisation with batch statistics) and the forest's parameter gradients.  margin / where: what the forward kept
// (empty tensors: the trees are walked again).
std::vector<torch::Tensor> forest_normalised_backward(int kind, torch::Tensor z, torch::Tensor mean, torch::Tensor invstd,
                                                      torch::Tensor thr, bool need_thr, torch::Tensor ord, torch::Tensor w,
                                                      bool need_w, torch::Tensor g, torch::Tensor margin, torch::Tensor where) {
  ForestCall call(kind, z, thr, ord, w, &g);
  check_statistics(z, mean, invstd);
  c10::DeviceGuard guard(z.device());
  const int64_t B = call.problem.B, C = call.problem.C, T = call.problem.T;
  const bool kept = margin.defined() && margin.numel() > 0;
  if (kept && (margin.scalar_type() != torch::kFloat32 || where.scalar_type() != torch::kInt32 || margin.numel() != B * T ||
               where.numel() != 2 * B * T || margin.device() != z.device() || where.device() != z.device() ||
               !margin.is_contiguous() || !where.is_contiguous()))
    bad_argument("Error: margin / where are not what the forward of this call kept.");
  torch::Tensor gthr = need_thr ? torch::empty_like(thr) : torch::Tensor();
  torch::Tensor gw = need_w ? torch::empty_like(w) : torch::Tensor();
  torch::Tensor column = torch::empty({B, T}, z.options().dtype(torch::kInt32));
  torch::Tensor value = torch::empty({B, T}, z.options());
  torch::Tensor sums = torch::empty({2, C}, z.options());
  torch::Tensor dz = torch::empty_like(z);
  torch::Tensor ws = make_workspace(ht_forest_normalised_workspace_bytes(&call.problem), z);
  OrdinalGuard og(ord, C);
  raise_status(ht_forest_normalised_backward_f32(
                   &call.problem, z.data_ptr<float>(), mean.data_ptr<float>(), invstd.data_ptr<float>(), thr.data_ptr<float>(),
                   ord.data_ptr<int64_t>(), w.data_ptr<float>(), g.data_ptr<float>(), need_thr ? gthr.data_ptr<float>() : nullptr,
                   need_w ? gw.data_ptr<float>() : nullptr, column.data_ptr<int32_t>(), value.data_ptr<float>(),
                   sums.data_ptr<float>(), sums.data_ptr<float>() + C, kept ? margin.data_ptr<float>() : nullptr,
                   kept ? where.data_ptr() : nullptr, ws.data_ptr(), ws.numel(), og.word(), current_stream(z)),
               "forest backward on normalised activations");
  raise_status(ht_batchnorm_input_grad_f32(z.data_ptr<float>(), mean.data_ptr<float>(), invstd.data_ptr<float>(),
                                           sums.data_ptr<float>(), sums.data_ptr<float>() + C, column.data_ptr<int32_t>(),
                                           value.data_ptr<float>(), dz.data_ptr<float>(), B, C, T, current_stream(z)),
               "batch normalisation input gradient");
  og.finish();
  return {dz, gthr, gw};
}

torch::Tensor forest_leafmap(int kind, torch::Tensor x, torch::Tensor thr, torch::Tensor ord, torch::Tensor w) {
  ForestCall call(kind, x, thr, ord, w, nullptr, true);
  c10::DeviceGuard guard(x.device());
  torch::Tensor leaf = torch::empty(call.map_sizes, x.options().dtype(torch::kInt64));
  torch::Tensor ws = make_workspace(ht_forest_workspace_bytes(&call.problem), x);
  OrdinalGuard og(ord, call.problem.C);
  if (call.is_double) {
    raise_status(ht_forest_leafmap_f64(&call.problem, x.data_ptr<double>(), thr.data_ptr<double>(), ord.data_ptr<int64_t>(),
                                       leaf.data_ptr<int64_t>(), ws.data_ptr(), ws.numel(), og.word(), current_stream(x)),
                 "forest leafmap");
    og.finish();
    return leaf;
  }
  raise_status(ht_forest_leafmap_f32(&call.problem, x.data_ptr<float>(), thr.data_ptr<float>(), ord.data_ptr<int64_t>(),
                                     leaf.data_ptr<int64_t>(), ws.data_ptr(), ws.numel(), og.word(), current_stream(x)),
               "forest leafmap");
  og.finish();
  return leaf;
}

std::vector<torch::Tensor> forest_marginmap(int kind, torch::Tensor x, torch::Tensor thr, torch::Tensor ord,
                                            torch::Tensor w) {
  ForestCall call(kind, x, thr, ord, w, nullptr, true);
  c10::DeviceGuard guard(x.device());
  torch::Tensor margins = torch::empty(call.map_sizes, x.options());
  torch::Tensor ords = torch::empty(call.map_sizes, x.options().dtype(torch::kInt64));
  torch::Tensor ws = make_workspace(ht_forest_workspace_bytes(&call.problem), x);
  OrdinalGuard og(ord, call.problem.C);
  if (call.is_double) {
    raise_status(
        ht_forest_marginmap_f64(&call.problem, x.data_ptr<double>(), thr.data_ptr<double>(), ord.data_ptr<int64_t>(),
                                margins.data_ptr<double>(), ords.data_ptr<int64_t>(), ws.data_ptr(), ws.numel(), og.word(),
                                current_stream(x)),
        "forest marginmap");
    og.finish();
    return {margins, ords};
  }
  raise_status(
      ht_forest_marginmap_f32(&call.problem, x.data_ptr<float>(), thr.data_ptr<float>(), ord.data_ptr<int64_t>(),
                              margins.data_ptr<float>(), ords.data_ptr<int64_t>(), ws.data_ptr(), ws.numel(), og.word(),
                              current_stream(x)),
      "forest marginmap");
  og.finish();
  return {margins, ords};
}

torch::Tensor forest_reachability(int kind, torch::Tensor x, torch::Tensor thr, torch::Tensor ord, torch::Tensor w) {
  ForestCall call(kind, x, thr, ord, w, nullptr, true);
  c10::DeviceGuard guard(x.device());
  torch::Tensor counts = torch::empty({w.size(0), w.size(1)}, x.options().dtype(torch::kInt64));
  torch::Tensor ws = make_workspace(ht_forest_workspace_bytes(&call.problem), x);
  OrdinalGuard og(ord, call.problem.C);
  if (call.is_double) {
    raise_status(ht_forest_reachability_f64(&call.problem, x.data_ptr<double>(), thr.data_ptr<double>(),
                                            ord.data_ptr<int64_t>(), counts.data_ptr<int64_t>(), ws.data_ptr(), ws.numel(),
                                            og.word(), current_stream(x)),
                 "forest reachability");
    og.finish();
    return counts;
  }
  raise_status(ht_forest_reachability_f32(&call.problem, x.data_ptr<float>(), thr.data_ptr<float>(),
                                          ord.data_ptr<int64_t>(), counts.data_ptr<int64_t>(), ws.data_ptr(),
                                          ws.numel(), og.word(), current_stream(x)),
               "forest reachability");
  og.finish();
  return counts;
}

// ---- threshold hygiene (host utilities on CPU tensors) -----------------------------------
// A vertex that tests the same feature as one of its ancestors is only reachable when its
// threshold lies on the side of the ancestor's threshold that the path took.  check reports
// trees that violate this; fix moves offending thresholds inside the feasible interval
// (semantics of HingeTreeCommon.h:211-287; ferns have nothing to check, :122-126).

template <typename Real>
struct FeasibleInterval {
  Real lo = -std::numeric_limits<Real>::infinity();
  Real hi = std::numeric_limits<Real>::infinity();
};

template <typename Real>
FeasibleInterval<Real> feasible_interval(const Real *thr, const int64_t *ord, int64_t vertex) {
  FeasibleInterval<Real> iv;
  const int64_t feature = ord[vertex];
  for (int64_t child = vertex; child > 0;) {
    const int64_t parent = (child - 1) / 2;
    if (ord[parent] == feature) {
      if (child == 2 * parent + 2)
        iv.lo = std::max(iv.lo, thr[parent]);  // reached through the right branch: x > thr[parent]
      else
        iv.hi = std::min(iv.hi, thr[parent]);
    }
    child = parent;
  }
  return iv;
}

template <typename Real>
bool tree_is_consistent(const Real *thr, const int64_t *ord, int64_t count) {
  // The reference compares against every same-feature ancestor separately, which is the same
  // as comparing against the tightest bounds.
  for (int64_t v = count - 1; v > 0; --v) {
    const FeasibleInterval<Real> iv = feasible_interval(thr, ord, v);
    if (thr[v] < iv.lo || thr[v] > iv.hi) return false;
  }
  return true;
}

template <typename Real>
bool tree_make_consistent(Real *thr, const int64_t *ord, int64_t count) {
  bool changed = false;
  for (int64_t v = 1; v < count; ++v) {  // parents first: a fixed parent constrains its subtree
    const FeasibleInterval<Real> iv = feasible_interval(thr, ord, v);
    if (thr[v] < iv.lo || thr[v] > iv.hi) {
      if (!std::isfinite(iv.lo))
        thr[v] = iv.hi - Real(1);
      else if (!std::isfinite(iv.hi))
        thr[v] = iv.lo + Real(1);
      else
        thr[v] = Real(0.5) * (iv.lo + iv.hi);
      changed = true;
    }
  }
  return changed;
}

std::vector<bool> thresholds_utility(int kind, bool fix, torch::Tensor thr, torch::Tensor ord, torch::Tensor w) {
  if (thr.dtype() != w.dtype() || torch::kInt64 != ord.scalar_type())
    bad_argument("Error: inThresholds and inWeights are expected to share the same torch real number data type. "
                 "inOrdinals is expected to be type torch.int64.");
  if (thr.device() != ord.device() || thr.device() != w.device())
    bad_argument("Error: All tensors are expected to be on the same device.");
  if (!thr.is_contiguous() || !ord.is_contiguous() || !w.is_contiguous())
    bad_argument("Error: All tensors are expected to be contiguous.");
  if (thr.dim() != 2 || ord.dim() != 2 || w.dim() < 2)
    bad_argument("Error: inWeights must have at least 2 dimensions. inThresholds and inOrdinals must have 2 dimensions.");
  if (thr.sizes() != ord.sizes() || w.size(0) != thr.size(0))
    bad_argument("Error: inThresholds and inOrdinals must be the same shape. inWeights.shape[0] must be the same as "
                 "inThresholds.shape[0].");
  const int depth = depth_of(w.size(1));
  if (depth > 31 || depth < 0 || thr.size(1) != threshold_count(kind, depth)) {
    std::ostringstream ss;
    ss << "Error: The tree depth exceeds compile-time constraints or the number of thresholds is incorrect for the "
          "tree depth (tree depth = "
       << depth << ").";
    bad_runtime(ss.str());
  }
  const int64_t trees = thr.size(0), count = thr.size(1);
  std::vector<bool> result(trees, kind == HT_KIND_FERN ? !fix : false);
  if (kind == HT_KIND_FERN) return result;  // decision order is irrelevant for ferns
  if (thr.scalar_type() != torch::kFloat32 && thr.scalar_type() != torch::kFloat64)
    bad_argument("Error: Unsupported data type. Only torch.float32 and torch.float64 are supported.");
  if (thr.device().is_cuda()) {
    // the reference refuses anything but CPU tensors; parameters that live on a device are handled there
    c10::DeviceGuard guard(thr.device());
    torch::Tensor flags = torch::zeros({trees}, torch::TensorOptions().dtype(torch::kUInt8).device(thr.device()));
    const int rc = thr.scalar_type() == torch::kFloat32
                       ? ht_thresholds_f32(fix ? 1 : 0, thr.data_ptr<float>(), ord.data_ptr<int64_t>(), trees, depth,
                                           flags.data_ptr<uint8_t>(), current_stream(thr))
                       : ht_thresholds_f64(fix ? 1 : 0, thr.data_ptr<double>(), ord.data_ptr<int64_t>(), trees, depth,
                                           flags.data_ptr<uint8_t>(), current_stream(thr));
    raise_status(rc, "thresholds");
    const torch::Tensor host = flags.cpu();
    for (int64_t j = 0; j < trees; ++j) result[j] = host.data_ptr<uint8_t>()[j] != 0;
    return result;
  }
  if (!thr.device().is_cpu()) bad_argument("Error: This operation is only supported on CPU and CUDA tensors.");
  const int64_t *po = ord.data_ptr<int64_t>();
  auto run = [&](auto *pt) {
    for (int64_t j = 0; j < trees; ++j)
      result[j] = fix ? tree_make_consistent(pt + j * count, po + j * count, count)
                      : tree_is_consistent(pt + j * count, po + j * count, count);
  };
  if (thr.scalar_type() == torch::kFloat32)
    run(thr.data_ptr<float>());
  else if (thr.scalar_type() == torch::kFloat64)
    run(thr.data_ptr<double>());
  else
    bad_argument("Error: Unsupported data type. Only torch.float32 and torch.float64 are supported.");
  return result;
}

// ---- speedtest ---------------------------------------------------------------------------
// Same sweep and result layout as the reference (hingetree.cpp:1361-1438): trees 1..512 in
// powers of two, depth 1..12, 100 forwards and 100 backwards each; rows of the result are
// trees, depth, forward ms, backward ms.  Timed with CUDA events on the current stream.
torch::Tensor forest_speedtest(int kind, torch::Tensor x, bool deterministic) {
  constexpr int64_t kBatches = 100, kTreeSteps = 10, kMaxDepth = 12;
  if (x.dim() < 2)
    bad_argument("Error: inData tensor expected to have at least 2 dimensions (i.e. [batch_size, num_channels, ...]).");
  require_cuda(x);
  require_float32(x);
  c10::DeviceGuard guard(x.device());
  cudaStream_t stream = c10::cuda::getCurrentCUDAStream(x.device().index()).stream();
  cudaEvent_t start, stop;
  cudaEventCreate(&start);
  cudaEventCreate(&stop);
  torch::Tensor timings = torch::zeros({4, kTreeSteps * kMaxDepth}, torch::kFloat32);
  float *row = timings.data_ptr<float>();
  const int64_t cols = kTreeSteps * kMaxDepth;
  const char *name = kind == HT_KIND_TREE ? "hingetree" : "hingefern";
  int64_t t = 0;
  for (int64_t s = 0; s < kTreeSteps; ++s) {
    const int64_t trees = int64_t(1) << s;
    for (int64_t depth = 1; depth <= kMaxDepth; ++depth, ++t) {
      torch::Tensor thr = torch::rand({trees, threshold_count(kind, (int)depth)}, x.options()) * 6.0f - 3.0f;
      torch::Tensor w = torch::randn({trees, int64_t(1) << depth}, x.options());
      torch::Tensor ord = torch::randint(0, x.size(1), {trees, threshold_count(kind, (int)depth)},
                                         x.options().dtype(torch::kInt64));
      row[t] = (float)trees;
      row[cols + t] = (float)depth;
      torch::Tensor out;
      float ms = 0.0f;
      cudaEventRecord(start, stream);
      for (int64_t b = 0; b < kBatches; ++b) out = forest_forward(kind, x, thr, ord, w);
      cudaEventRecord(stop, stream);
      cudaEventSynchronize(stop);
      cudaEventElapsedTime(&ms, start, stop);
      row[2 * cols + t] = ms / kBatches;
      std::cout << name << "_forward: numBatches = " << kBatches << ", numTrees = " << trees << ", depth = " << depth
                << ": " << ms / kBatches << " ms per batch." << std::endl;
      torch::Tensor g = torch::ones_like(out);
      cudaEventRecord(start, stream);
      for (int64_t b = 0; b < kBatches; ++b) forest_backward(kind, deterministic, x, true, thr, true, ord, false, w, true, g);
      cudaEventRecord(stop, stream);
      cudaEventSynchronize(stop);
      cudaEventElapsedTime(&ms, start, stop);
      row[3 * cols + t] = ms / kBatches;
      std::cout << name << (deterministic ? "_backward_deterministic" : "_backward") << ": numBatches = " << kBatches
                << ", numTrees = " << trees << ", depth = " << depth << ": " << ms / kBatches << " ms per batch."
                << std::endl;
    }
  }
  cudaEventDestroy(start);
  cudaEventDestroy(stop);
  return timings;
}

}  // namespace
}  // namespace htx

using namespace htx;

#define HT_BIND_KIND(prefix, KIND)                                                                                  \
  m.def(prefix "_forward", [](torch::Tensor x, torch::Tensor t, torch::Tensor o, torch::Tensor w) {                  \
    return forest_forward(KIND, x, t, o, w);                                                                        \
  });                                                                                                               \
  m.def(prefix "_backward", [](torch::Tensor x, bool nx, torch::Tensor t, bool nt, torch::Tensor o, bool no,        \
                               torch::Tensor w, bool nw, torch::Tensor g) {                                         \
    return forest_backward(KIND, false, x, nx, t, nt, o, no, w, nw, g);                                             \
  });                                                                                                               \
  m.def(prefix "_backward_deterministic", [](torch::Tensor x, bool nx, torch::Tensor t, bool nt, torch::Tensor o,   \
                                             bool no, torch::Tensor w, bool nw, torch::Tensor g) {                  \
    return forest_backward(KIND, true, x, nx, t, nt, o, no, w, nw, g);                                              \
  });                                                                                                               \
  m.def(prefix "_forward_saving", [](torch::Tensor x, torch::Tensor t, torch::Tensor o, torch::Tensor w) {           \
    return forest_forward_saving(KIND, x, t, o, w);                                                                 \
  });                                                                                                               \
  m.def(prefix "_backward_saved", [](torch::Tensor x, bool nx, torch::Tensor t, bool nt, torch::Tensor o, bool no,  \
                                     torch::Tensor w, bool nw, torch::Tensor g, torch::Tensor saved, bool det) {    \
    return forest_backward_saved(KIND, det, x, nx, t, nt, o, no, w, nw, g, saved);                                  \
  });                                                                                                               \
  m.def(prefix "_normalised_forward", [](torch::Tensor z, torch::Tensor mean, torch::Tensor invstd, torch::Tensor t,  \
                                         torch::Tensor o, torch::Tensor w, bool keep) {                             \
    return forest_normalised_forward(KIND, z, mean, invstd, t, o, w, keep);                                         \
  }, pybind11::arg("z"), pybind11::arg("mean"), pybind11::arg("invstd"), pybind11::arg("thresholds"),              \
     pybind11::arg("ordinals"), pybind11::arg("weights"), pybind11::arg("keep") = false);                         \
  m.def(prefix "_normalised_backward", [](torch::Tensor z, torch::Tensor mean, torch::Tensor invstd, torch::Tensor t, \
                                          bool nt, torch::Tensor o, torch::Tensor w, bool nw, torch::Tensor g,       \
                                          c10::optional<torch::Tensor> margin, c10::optional<torch::Tensor> where) { \
    return forest_normalised_backward(KIND, z, mean, invstd, t, nt, o, w, nw, g,                                    \
                                      margin.has_value() ? *margin : torch::Tensor(),                              \
                                      where.has_value() ? *where : torch::Tensor());                               \
  }, pybind11::arg("z"), pybind11::arg("mean"), pybind11::arg("invstd"), pybind11::arg("thresholds"),              \
     pybind11::arg("need_thresholds"), pybind11::arg("ordinals"), pybind11::arg("weights"),                       \
     pybind11::arg("need_weights"), pybind11::arg("grad"), pybind11::arg("margin") = pybind11::none(),            \
     pybind11::arg("where") = pybind11::none());                                                                  \
  m.def(prefix "_check_thresholds", [](torch::Tensor t, torch::Tensor o, torch::Tensor w) {                         \
    return thresholds_utility(KIND, false, t, o, w);                                                                \
  });                                                                                                               \
  m.def(prefix "_fix_thresholds", [](torch::Tensor t, torch::Tensor o, torch::Tensor w) {                           \
    return thresholds_utility(KIND, true, t, o, w);                                                                 \
  });                                                                                                               \
  m.def(prefix "_reachability", [](torch::Tensor x, torch::Tensor t, torch::Tensor o, torch::Tensor w) {             \
    return forest_reachability(KIND, x, t, o, w);                                                                   \
  });                                                                                                               \
  m.def(prefix "_leafmap", [](torch::Tensor x, torch::Tensor t, torch::Tensor o, torch::Tensor w) {                  \
    return forest_leafmap(KIND, x, t, o, w);                                                                        \
  });                                                                                                               \
  m.def(prefix "_marginmap", [](torch::Tensor x, torch::Tensor t, torch::Tensor o, torch::Tensor w) {                \
    return forest_marginmap(KIND, x, t, o, w);                                                                      \
  });                                                                                                               \
  m.def(prefix "_speedtest", [](torch::Tensor x, bool det) { return forest_speedtest(KIND, x, det); });             \
  m.def(prefix "_init_medians", [](torch::Tensor x, torch::Tensor t, torch::Tensor o, torch::Tensor w) {            \
    return init_medians(KIND == HT_KIND_FERN ? InitFamily::Fern : InitFamily::Tree, x, t, o, w);                    \
  });

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.doc() = "sm_100a drop-in for HingeTreeForTorch's hingetree_cpp (CUDA tensors only)";
  HT_BIND_KIND("tree", HT_KIND_TREE)
  HT_BIND_KIND("fern", HT_KIND_FERN)
  m.def("tree_init_greedy", &init_greedy,
        "Initialize thresholds and ordinals by random decision tree learning on class labels (CPU only).");
  m.def("seed_init", &seed_init, "Seed the generator tree_init_greedy draws from.");
  m.def("set_backward_scratch_limit", &set_backward_scratch_limit,
        "Upper bound in bytes on the scratch a default-mode backward call allocates for its per-evaluation records "
        "(12 bytes per tree evaluation); above it the gradients are scattered with atomics instead. Default: no bound.");
  m.def("batchnorm_statistics", &batchnorm_statistics,
        "[mean, biased variance, 1 / sqrt(variance + eps)] per column from the columns' sums and sums of squares over `rows` rows.");
  m.def("linear_tf32_stats", &linear_tf32_stats,
        "z = x @ w.T on the tensor cores (TF32 products, fp32 accumulation) and the column sums of z and z*z: "
        "[z, sum, sumsq]. K and N must be multiples of 4.");
  m.def("set_save_forward", [](bool on) { g_save_forward = on; },
        "Whether tree_/fern_forward_saving keep the traversal for the backward (default) or act as the plain forward.");
  m.def("selftest_bounded_wait", &selftest_bounded_wait,
        "Runs a one-warp kernel whose bounded wait has to run out (nothing faults): the next pipeline_status() raises.");
  m.def("pipeline_status", &pipeline_status,
        "Reads and clears the current device's long-lived kernel status word (calls on ordinals already known to be "
        "valid do not synchronise; a kernel that gave up on a bounded wait leaves its flag there). Raises RuntimeError "
        "when a timeout was flagged; returns the other flag bits.");
  m.def("set_ordinal_check", &set_ordinal_check,
        "When to read the ordinal range flag back from the device: 'cached' (default: once per ordinals tensor "
        "version), 'always' (every call, like the reference) or 'never'.");
  m.def("abi_version", []() { return ht_version(); });
  htx::bind_more_ops(m);
}
