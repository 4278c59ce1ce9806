// Shared-memory tile kernels for 1-D / 2-D convolutional hinge trees and ferns (one output per leaf).
#pragma once

#include "ht_common.cuh"

namespace ht {

// A 1-D convolution is passed as a 2-D one with a single row.
struct ConvTileProblem {
  int kind, depth;
  int64_t B, Ci, Co;
  int H, W, Ho, Wo;
  int kh, kw, sy, sx, py, px, dy, dx;
};

// Bytes of per-call scratch (tree records) the tile kernels need; 0 when they do not take the problem.
size_t conv_tiled_workspace_bytes(const ConvTileProblem &p);

// HT_ERR_UNSUPPORTED when the tile kernel does not take the problem (the caller falls back to the
// thread-per-output kernel).  `ord` holds validated window-cell indices, `records` is scratch of
// conv_tiled_workspace_bytes.
int conv_forward_tiled(const ConvTileProblem &p, const float *x, const float *thr, const int32_t *ord, const float *w,
                       float *out, void *records, uint32_t *status_word, cudaStream_t stream);

}  // namespace ht
