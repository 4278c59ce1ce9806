// Operators of `hingetree_cpp` beyond the plain forest: convolution, fused linear, image+vector
// fusion, sparse gradients, trie and contract/expand.
#include "hingetree_cpp_ops.h"

namespace htx {

namespace {

[[noreturn]] void pending(const char *name) {
  bad_runtime(std::string("Error: ") + name + " is not implemented in this build yet.");
}

}  // namespace

void bind_more_ops(pybind11::module_ &m) {
  static const char *const names[] = {
      "sparse_tree_backward", "sparse_fern_backward", "tree_conv1d_forward", "tree_conv2d_forward",
      "tree_conv3d_forward", "tree_conv1d_backward", "tree_conv2d_backward", "tree_conv3d_backward",
      "fern_conv1d_forward", "fern_conv2d_forward", "fern_conv3d_forward", "fern_conv1d_backward",
      "fern_conv2d_backward", "fern_conv3d_backward", "trie_forward", "trie_backward", "trie_init_medians",
      "tree_fused_linear_forward", "tree_fused_linear_backward", "sparse_tree_fused_linear_backward",
      "fern_fused_linear_forward", "fern_fused_linear_backward", "sparse_fern_fused_linear_backward",
      "tree_fusion_forward", "tree_fusion_backward", "fern_fusion_forward", "fern_fusion_backward",
      "tree_fusion_fused_linear_forward", "tree_fusion_fused_linear_backward", "fern_fusion_fused_linear_forward",
      "fern_fusion_fused_linear_backward", "contract", "expand"};
  for (const char *name : names)
    m.def(name, [name](pybind11::args, pybind11::kwargs) -> pybind11::object { pending(name); });
}

}  // namespace htx
