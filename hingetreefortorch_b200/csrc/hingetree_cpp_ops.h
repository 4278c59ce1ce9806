// Helpers shared by the translation units of the `hingetree_cpp` torch extension.
#pragma once

#include <torch/extension.h>

#include <string>
#include <vector>

#include "hingetree_b200.h"

namespace htx {

[[noreturn]] void bad_argument(const std::string &what);  // std::invalid_argument -> ValueError
[[noreturn]] void bad_runtime(const std::string &what);   // std::runtime_error -> RuntimeError
void raise_status(int rc, const char *op);

ht_stream_t current_stream(const torch::Tensor &t);
int64_t inner_count(const torch::Tensor &t, int64_t from);
int depth_of(int64_t leaves);
int64_t threshold_count(int kind, int depth);
void require_cuda(const torch::Tensor &t);
void require_float32(const torch::Tensor &t);
torch::Tensor make_workspace(size_t bytes, const torch::Tensor &like);
void set_ordinal_check(const std::string &mode);
int64_t pipeline_status();

// Owns the device status word of one call and turns a flagged ordinal into the reference's
// RuntimeError.  When this ordinals tensor is already known to be valid nothing is read back and word() is the
// device's long-lived status word, which keeps a kernel's timeout flag for the next call that synchronises.
class OrdinalGuard {
 public:
  OrdinalGuard(const torch::Tensor &ord, int64_t channels);
  uint32_t *word();
  void finish();

 private:
  torch::Tensor ord_, word_, sticky_;
  int64_t channels_;
  bool check_;
};

// Argument checks and shape bookkeeping of the plain forest operators.
struct ForestCall {
  // allow_double: torch.float64 tensors are taken too (the plain operators have double precision kernels)
  ForestCall(int kind, const torch::Tensor &x, const torch::Tensor &thr, const torch::Tensor &ord,
             const torch::Tensor &w, const torch::Tensor *g, bool allow_double = false);
  ht_forest_problem problem;
  bool is_double = false;
  std::vector<int64_t> out_sizes;  // [B, T, inner data dims..., inner weight dims...]
  std::vector<int64_t> map_sizes;  // [B, T, inner data dims...]
};

// Registers the convolution, fused-linear, fusion, sparse, trie and contract/expand operators.
void bind_more_ops(pybind11::module_ &m);

// Median initialisation of the thresholds (CPU tensors, in place); false when the shapes or the
// feature indices do not describe a forest over the data.
enum class InitFamily { Tree, Fern, Trie };
bool init_medians(InitFamily family, torch::Tensor x, torch::Tensor thr, torch::Tensor ord, torch::Tensor w);

// Greedy initialisation of a forest's thresholds and feature indices from class labels (CPU tensors, in
// place), drawing from a process-wide generator that seed_init() resets.
bool init_greedy(torch::Tensor x, torch::Tensor labels, torch::Tensor thr, torch::Tensor ord, torch::Tensor w);
void seed_init(uint64_t seed);

}  // namespace htx
