// `*_init_medians` for trees, ferns and tries: host C++ on CPU tensors.  The reference's operators
// are CPU-only too and refuse anything else (hingetree.cpp:1519-1533); its modules call them once,
// before training, on data that still lives on the host (_RandomHingeForest.py:132-133).
//
// Every threshold becomes the median of its feature over the samples that reach its vertex — the
// value of rank floor(n / 2) counted from the largest (MedianInit.h:229-235).  Samples whose feature
// exceeds the threshold go on to the right child (heap index 2v + 2), the others to the left
// (2v + 1), and a vertex no sample reaches keeps its threshold (MedianInit.h:224-227,239-252).
// Ferns see all samples at every level (MedianInit.h:204-219).  The value at a rank and a split by
// value do not depend on the order the samples are held in, so the thresholds are a function of the
// data alone and can be compared with the reference bit for bit.
//
// `tree_init_greedy` (classification labels): every tree is grown vertex by vertex like a randomised
// decision tree (GreedyInit.h:54-170,172-313).  A vertex looks at up to 1000 of its samples drawn at
// random and at floor(sqrt(C)) features drawn at random; for each feature the candidate thresholds are
// the midpoints between consecutive distinct values (more than 1e-5 apart), and the split with the
// largest drop of the normalised Gini impurity k/(k-1) * (1 - sum p^2) wins.  Samples above the
// threshold go right.  A vertex that cannot be split (fewer than 2 samples, one class, no candidate)
// copies its parent's feature and gets the largest finite threshold, so everything goes left.  Both
// thresholds and feature indices are written, and only when every tree could be grown.  The draws
// come from a process-wide generator, as in the reference (GreedyInit.h:35-38), so two runs agree
// only after seed_init(); the reference's own results depend on its generator's history in the same
// way, and there is nothing to pin this operator against bit for bit.  One deliberate difference:
// the class counts of a vertex are taken on the drawn samples throughout, where the reference mixes
// counts over all samples of the vertex with counts over the drawn ones (GreedyInit.h:68-76,148-158).
#include "hingetree_cpp_ops.h"

#include <c10/core/DeviceGuard.h>

#include <algorithm>
#include <cmath>
#include <limits>
#include <numeric>
#include <random>

namespace htx {
namespace {

struct InitShape {
  int64_t trees, decisions, depth, rows, channels, inner;
};

// The reference returns false (it does not raise) when the shapes do not describe a forest.
bool read_shape(InitFamily family, const torch::Tensor &x, const torch::Tensor &thr, const torch::Tensor &ord,
                const torch::Tensor &w, InitShape &s) {
  if (thr.dim() != 2 || ord.dim() != 2 || w.dim() < 2 || x.dim() < 2) return false;
  if (thr.sizes() != ord.sizes() || w.size(0) != thr.size(0)) return false;
  // a trie has one weight row per internal vertex, trees and ferns one per leaf
  const int64_t leaves = family == InitFamily::Trie ? w.size(1) + 1 : w.size(1);
  const int depth = depth_of(leaves);
  if (depth < 0 || depth > 31) return false;
  s.trees = w.size(0);
  s.depth = depth;
  s.decisions = family == InitFamily::Fern ? depth : (int64_t(1) << depth) - 1;
  if (thr.size(1) != s.decisions || s.trees == 0 || s.decisions == 0) return false;
  s.rows = x.size(0);
  s.channels = x.size(1);
  s.inner = inner_count(x, 2);
  return true;
}

template <typename Real>
bool median_splits(InitFamily family, const InitShape &s, const Real *x, Real *thr, const int64_t *ord) {
  for (int64_t e = 0; e < s.trees * s.decisions; ++e)
    if (ord[e] < 0 || ord[e] >= s.channels) return false;

  // sample r = (b, k) has feature f at x[(b * channels + f) * inner + k]
  const int64_t samples = s.rows * s.inner;
  std::vector<int64_t> base(samples);
  for (int64_t b = 0; b < s.rows; ++b)
    for (int64_t k = 0; k < s.inner; ++k) base[b * s.inner + k] = b * s.channels * s.inner + k;

  std::vector<int64_t> held(samples);                        // sample offsets, regrouped vertex by vertex
  std::vector<int64_t> first(s.decisions), last(s.decisions);  // the stretch of `held` that reaches a vertex
  for (int64_t j = 0; j < s.trees; ++j) {
    Real *tree_thr = thr + j * s.decisions;
    const int64_t *tree_ord = ord + j * s.decisions;
    held = base;
    std::fill(first.begin(), first.end(), 0);
    std::fill(last.begin(), last.end(), 0);
    first[0] = 0;
    last[0] = samples;
    for (int64_t v = 0; v < s.decisions; ++v) {
      if (family == InitFamily::Fern) {
        first[v] = 0;
        last[v] = samples;
      }
      const int64_t n = last[v] - first[v];
      if (n == 0) continue;
      const int64_t shift = tree_ord[v] * s.inner;
      auto value = [&](int64_t at) { return x[at + shift]; };
      auto lo = held.begin() + first[v], hi = held.begin() + last[v], mid = lo + n / 2;
      std::nth_element(lo, mid, hi, [&](int64_t a, int64_t b) { return value(a) > value(b); });
      const Real median = value(*mid);
      tree_thr[v] = median;
      if (family != InitFamily::Fern && 2 * v + 2 < s.decisions) {
        auto split = std::partition(lo, hi, [&](int64_t a) { return value(a) > median; });
        first[2 * v + 2] = first[v];  // larger values: right child
        last[2 * v + 2] = split - held.begin();
        first[2 * v + 1] = split - held.begin();  // the rest: left child
        last[2 * v + 1] = last[v];
      }
    }
  }
  return true;
}

std::mt19937_64 g_draws;  // process-wide, default-seeded: the reference's arrangement

double gini(const std::vector<int64_t> &counts, int64_t total) {
  if (counts.size() < 2 || total == 0) return -1.0;
  double squares = 0.0;
  for (int64_t n : counts) squares += (double(n) / double(total)) * (double(n) / double(total));
  return double(counts.size()) * (1.0 - squares) / double(counts.size() - 1);
}

template <typename Real>
struct Split {
  double gain = -1.0;
  int64_t feature = 0;
  Real threshold = Real();
};

// Best split of the samples held[first, last) (offsets of the samples' first feature; labels at label_of).
template <typename Real, typename LabelOf>
Split<Real> best_split(std::vector<int64_t> &held, int64_t first, int64_t last, const Real *x, int64_t inner,
                       int64_t channels, int64_t classes, LabelOf label_of) {
  Split<Real> best;
  const int64_t n = last - first;
  if (n < 2 || classes < 2) return best;
  std::shuffle(held.begin() + first, held.begin() + last, g_draws);
  const int64_t drawn = std::min<int64_t>(1000, n);
  std::vector<int64_t> all(classes, 0);
  for (int64_t r = first; r < first + drawn; ++r) {
    const int64_t label = label_of(held[r]);
    if (label < 0 || label >= classes) return best;
    ++all[label];
  }
  if (std::count_if(all.begin(), all.end(), [](int64_t c) { return c > 0; }) < 2) return best;
  const double impurity = gini(all, drawn);

  std::vector<int64_t> features(channels);
  std::iota(features.begin(), features.end(), int64_t(0));
  std::shuffle(features.begin(), features.end(), g_draws);
  features.resize(std::max<int64_t>(1, (int64_t)std::sqrt((double)channels)));
  best.feature = features[0];

  std::vector<std::pair<Real, int64_t>> values(drawn);
  std::vector<int64_t> right(classes), left(classes);
  for (int64_t f : features) {
    for (int64_t r = 0; r < drawn; ++r) values[r] = {x[held[first + r] + f * inner], label_of(held[first + r])};
    std::sort(values.begin(), values.end(), [](const auto &a, const auto &b) { return a.first < b.first; });
    // sweep the cut from the top: samples above it are on the right
    std::fill(right.begin(), right.end(), 0);
    for (int64_t r = drawn - 1; r >= 1; --r) {
      ++right[values[r].second];
      if (!(values[r].first - values[r - 1].first > Real(1e-5))) continue;
      const int64_t on_right = drawn - r;
      for (int64_t c = 0; c < classes; ++c) left[c] = all[c] - right[c];
      double gain = impurity - double(on_right) * gini(right, on_right) / double(drawn) -
                    double(drawn - on_right) * gini(left, drawn - on_right) / double(drawn);
      gain = std::max(0.0, gain);
      if (gain > best.gain) {
        best.gain = gain;
        best.feature = f;
        best.threshold = (values[r].first + values[r - 1].first) / 2;
      }
    }
  }
  return best;
}

template <typename Real>
bool greedy_splits(const InitShape &s, const Real *x, const int64_t *labels, Real *thr, int64_t *ord) {
  for (int64_t e = 0; e < s.trees * s.decisions; ++e)
    if (ord[e] < 0 || ord[e] >= s.channels) return false;
  const int64_t samples = s.rows * s.inner;
  if (samples == 0) return false;
  const int64_t classes = *std::max_element(labels, labels + samples) + 1;
  if (*std::min_element(labels, labels + samples) < 0 || classes < 2) return false;

  // sample (b, k): features at x[(b * channels + f) * inner + k], label at labels[b * inner + k]
  std::vector<int64_t> base(samples);
  for (int64_t b = 0; b < s.rows; ++b)
    for (int64_t k = 0; k < s.inner; ++k) base[b * s.inner + k] = b * s.channels * s.inner + k;
  const int64_t row_span = s.channels * s.inner;
  auto label_of = [&](int64_t at) { return labels[(at / row_span) * s.inner + at % s.inner]; };

  std::vector<Real> new_thr(thr, thr + s.trees * s.decisions);
  std::vector<int64_t> new_ord(ord, ord + s.trees * s.decisions);
  std::vector<int64_t> held, first(s.decisions), last(s.decisions);
  for (int64_t j = 0; j < s.trees; ++j) {
    Real *tree_thr = new_thr.data() + j * s.decisions;
    int64_t *tree_ord = new_ord.data() + j * s.decisions;
    held = base;
    std::fill(first.begin(), first.end(), 0);
    std::fill(last.begin(), last.end(), 0);
    last[0] = samples;
    for (int64_t v = 0; v < s.decisions; ++v) {
      const Split<Real> split = best_split<Real>(held, first[v], last[v], x, s.inner, s.channels, classes, label_of);
      if (split.gain < 0.0) {
        if (v == 0) return false;  // the root must split
        tree_ord[v] = tree_ord[(v - 1) / 2];
        tree_thr[v] = std::numeric_limits<Real>::max();
        continue;
      }
      tree_ord[v] = split.feature;
      tree_thr[v] = split.threshold;
      if (2 * v + 2 < s.decisions) {
        const int64_t shift = split.feature * s.inner;
        auto lo = held.begin() + first[v], hi = held.begin() + last[v];
        auto cut = std::partition(lo, hi, [&](int64_t at) { return x[at + shift] > split.threshold; });
        first[2 * v + 2] = first[v];  // larger values: right child
        last[2 * v + 2] = cut - held.begin();
        first[2 * v + 1] = cut - held.begin();
        last[2 * v + 1] = last[v];
      }
    }
  }
  std::copy(new_thr.begin(), new_thr.end(), thr);
  std::copy(new_ord.begin(), new_ord.end(), ord);
  return true;
}

}  // namespace

void seed_init(uint64_t seed) { g_draws.seed(seed); }

bool init_greedy(torch::Tensor x, torch::Tensor labels, torch::Tensor thr, torch::Tensor ord, torch::Tensor w) {
  if (x.dtype() != thr.dtype() || ord.scalar_type() != torch::kInt64 || x.dtype() != w.dtype())
    bad_argument(
        "Error: inData, inThresholds, inWeights are expected to share the same torch real number data type. "
        "inOrdinals is expected to be type torch.int64.");
  if (labels.scalar_type() != torch::kInt64 && labels.dtype() != x.dtype())
    bad_argument(
        "Error: inLabels expected to be of type torch.int64 (classification) or share the same torch real number "
        "data type (regression).");
  if (!x.device().is_cpu() || !labels.device().is_cpu() || !thr.device().is_cpu() || !ord.device().is_cpu() ||
      !w.device().is_cpu())
    bad_argument("Error: All tensors are expected to be on the CPU.");
  if (!x.is_contiguous() || !labels.is_contiguous() || !thr.is_contiguous() || !ord.is_contiguous() || !w.is_contiguous())
    bad_argument("Error: All tensors are expected to be contiguous.");
  if (x.scalar_type() != torch::kFloat32 && x.scalar_type() != torch::kFloat64)
    bad_argument("Error: Unsupported data type. Only torch.float32 and torch.float64 are supported.");
  InitShape s;
  if (!read_shape(InitFamily::Tree, x, thr, ord, w, s)) return false;
  if (labels.scalar_type() != torch::kInt64) return false;  // regression labels: not implemented in the reference either
  if (labels.dim() < 1 || labels.dim() + 1 != x.dim() || labels.size(0) != x.size(0)) return false;
  for (int64_t d = 1; d < labels.dim(); ++d)
    if (labels.size(d) != x.size(d + 1)) return false;
  if (x.scalar_type() == torch::kFloat32)
    return greedy_splits<float>(s, x.data_ptr<float>(), labels.data_ptr<int64_t>(), thr.data_ptr<float>(),
                                ord.data_ptr<int64_t>());
  return greedy_splits<double>(s, x.data_ptr<double>(), labels.data_ptr<int64_t>(), thr.data_ptr<double>(),
                               ord.data_ptr<int64_t>());
}

bool init_medians(InitFamily family, torch::Tensor x, torch::Tensor thr, torch::Tensor ord, torch::Tensor w) {
  if (x.dtype() != thr.dtype() || ord.scalar_type() != torch::kInt64 || x.dtype() != w.dtype())
    bad_argument(
        "Error: inData, inThresholds, inWeights are expected to share the same torch real number data type. "
        "inOrdinals is expected to be type torch.int64.");
  // The reference takes CPU tensors only; here tensors that all live on one CUDA device are taken as well
  // and the medians are found there (ht_init_medians_*), with the same result.
  const bool on_device = x.device().is_cuda();
  if (on_device) {
    if (thr.device() != x.device() || ord.device() != x.device() || w.device() != x.device())
      bad_argument("Error: All tensors are expected to be on the same device.");
  } else if (!x.device().is_cpu() || !thr.device().is_cpu() || !ord.device().is_cpu() || !w.device().is_cpu()) {
    bad_argument("Error: All tensors are expected to be on the CPU.");
  }
  if (!x.is_contiguous() || !thr.is_contiguous() || !ord.is_contiguous() || !w.is_contiguous())
    bad_argument("Error: All tensors are expected to be contiguous.");
  if (x.scalar_type() != torch::kFloat32 && x.scalar_type() != torch::kFloat64)
    bad_argument("Error: Unsupported data type. Only torch.float32 and torch.float64 are supported.");
  InitShape s;
  if (!read_shape(family, x, thr, ord, w, s)) return false;
  if (on_device) {
    if (s.depth > 20) return false;
    if (s.rows == 0) return true;
    if (ord.min().item<int64_t>() < 0 || ord.max().item<int64_t>() >= s.channels) return false;  // as the host path
    c10::DeviceGuard guard(x.device());
    const int kind = family == InitFamily::Fern ? HT_KIND_FERN : HT_KIND_TREE;
    const size_t need = ht_init_medians_workspace_bytes(kind, s.rows, s.inner, s.trees, (int)s.depth, (int)x.element_size());
    torch::Tensor ws = torch::empty({(int64_t)std::max<size_t>(need, 1)}, torch::TensorOptions().dtype(torch::kUInt8).device(x.device()));
    ht_stream_t stream = current_stream(x);
    const int rc = x.scalar_type() == torch::kFloat32
                       ? ht_init_medians_f32(kind, x.data_ptr<float>(), thr.data_ptr<float>(), ord.data_ptr<int64_t>(), s.rows,
                                             s.channels, s.inner, s.trees, (int)s.depth, ws.data_ptr(), (size_t)ws.numel(), stream)
                       : ht_init_medians_f64(kind, x.data_ptr<double>(), thr.data_ptr<double>(), ord.data_ptr<int64_t>(), s.rows,
                                             s.channels, s.inner, s.trees, (int)s.depth, ws.data_ptr(), (size_t)ws.numel(), stream);
    raise_status(rc, "init_medians");
    return true;
  }
  if (x.scalar_type() == torch::kFloat32)
    return median_splits<float>(family, s, x.data_ptr<float>(), thr.data_ptr<float>(), ord.data_ptr<int64_t>());
  return median_splits<double>(family, s, x.data_ptr<double>(), thr.data_ptr<double>(), ord.data_ptr<int64_t>());
}

}  // namespace htx
