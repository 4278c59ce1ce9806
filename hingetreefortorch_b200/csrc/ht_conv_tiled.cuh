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

// Bytes of per-call scratch (tree records) the forward / backward tile kernel needs; 0 when it does not
// take the problem.
size_t conv_tiled_workspace_bytes(const ConvTileProblem &p);
size_t conv_backward_tiled_workspace_bytes(const ConvTileProblem &p);

// HT_ERR_UNSUPPORTED when the tile kernel does not take the problem (the caller falls back to the
// thread-per-output kernel).  `ord` holds validated window-cell indices, `records` is scratch of
// conv_tiled_workspace_bytes.
int conv_forward_tiled(const ConvTileProblem &p, const float *x, const float *thr, const int32_t *ord, const float *w,
                       float *out, void *records, uint32_t *status_word, cudaStream_t stream);

// Gradients are ADDED to gx, gthr, gw (the caller clears them); any of the three may be null.
int conv_backward_tiled(const ConvTileProblem &p, const float *x, const float *thr, const int32_t *ord, const float *w,
                        const float *g, float *gx, float *gthr, float *gw, void *records, uint32_t *status_word,
                        cudaStream_t stream);

namespace conv_tile {

constexpr int kTileColumns = 32;  // a warp's lanes are 32 consecutive output positions of one row

// Image patch under a tile of TY x 32 output positions: extent, and the largest offset of a window
// cell from the window origin.
struct PatchShape {
  int h, w;
  int64_t far;
};

inline PatchShape patch_shape(const ConvTileProblem &p, int TY) {
  PatchShape s;
  s.h = (TY - 1) * p.sy + (p.kh - 1) * p.dy + 1;
  s.w = (kTileColumns - 1) * p.sx + (p.kw - 1) * p.dx + 1;
  s.far = (int64_t)(p.kh - 1) * p.dy * s.w + (int64_t)(p.kw - 1) * p.dx;
  return s;
}

#ifdef __CUDACC__
// Copies the patches of all input channels of sample image `image` ([Ci, H, W]) whose top-left
// corner is image pixel (iy0, ix0) into shared memory, [Ci][patch_h][patch_w]; cells outside the
// image read as 0, the reference's padding value (ImageToMatrix.h:138).
__device__ __forceinline__ void stage_patches(float *patches, const float *__restrict__ image, int Ci, int H, int W,
                                              int iy0, int ix0, int patch_h, int patch_w) {
  const int patch_elems = patch_h * patch_w;
  const int total = Ci * patch_elems;
  for (int idx = threadIdx.x; idx < total; idx += blockDim.x) {
    const int c = idx / patch_elems, r = idx - c * patch_elems;
    const int yy = r / patch_w, xx = r - yy * patch_w;
    const int iy = iy0 + yy, ix = ix0 + xx;
    float v = 0.0f;
    if (iy >= 0 && iy < H && ix >= 0 && ix < W) v = __ldg(image + ((int64_t)c * H + iy) * W + ix);
    patches[idx] = v;
  }
}
#endif

}  // namespace conv_tile
}  // namespace ht
