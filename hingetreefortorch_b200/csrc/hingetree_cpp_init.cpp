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
#include "hingetree_cpp_ops.h"

#include <algorithm>
#include <numeric>

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

}  // namespace

bool init_medians(InitFamily family, torch::Tensor x, torch::Tensor thr, torch::Tensor ord, torch::Tensor w) {
  if (x.dtype() != thr.dtype() || ord.scalar_type() != torch::kInt64 || x.dtype() != w.dtype())
    bad_argument(
        "Error: inData, inThresholds, inWeights are expected to share the same torch real number data type. "
        "inOrdinals is expected to be type torch.int64.");
  if (!x.device().is_cpu() || !thr.device().is_cpu() || !ord.device().is_cpu() || !w.device().is_cpu())
    bad_argument("Error: All tensors are expected to be on the CPU.");
  if (!x.is_contiguous() || !thr.is_contiguous() || !ord.is_contiguous() || !w.is_contiguous())
    bad_argument("Error: All tensors are expected to be contiguous.");
  if (x.scalar_type() != torch::kFloat32 && x.scalar_type() != torch::kFloat64)
    bad_argument("Error: Unsupported data type. Only torch.float32 and torch.float64 are supported.");
  InitShape s;
  if (!read_shape(family, x, thr, ord, w, s)) return false;
  if (x.scalar_type() == torch::kFloat32)
    return median_splits<float>(family, s, x.data_ptr<float>(), thr.data_ptr<float>(), ord.data_ptr<int64_t>());
  return median_splits<double>(family, s, x.data_ptr<double>(), thr.data_ptr<double>(), ord.data_ptr<int64_t>());
}

}  // namespace htx
