/*
 * CPU restatement of the convolutional hinge trees and of contract / expand (second part of
 * the oracle; see hinge_oracle.c for the rules: test infrastructure only, never shipped).
 *
 * Convolution (hingetree_conv.cpp:199-225 forward, :388-497 backward; geometry from
 * ImageToMatrix.h:189-221,304-347): output channel j sums, over the input channels c in
 * ascending order, the value of tree (j,c) evaluated on the kernel window of channel c at
 * every output position p.  A window cell q (row-major over the kernel dims) reads the input at
 * out*stride - padding + q*dilation per dimension, or the pad value 0 outside the image.  The
 * data gradient of a decision that looked at a padding cell is dropped.
 *
 * Layouts: x [B, Ci, size...]; thr, ord [Co, Ci, N]; w [Co, Ci, L, M]; out [B, Co, osize..., M].
 */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <math.h>

#include "hinge_oracle_terms.h"

#define HO_FERN 1
#define HO_MAX_DIMS 3

typedef struct {
  int dims;
  int64_t size[HO_MAX_DIMS], kernel[HO_MAX_DIMS], stride[HO_MAX_DIMS], pad[HO_MAX_DIMS], dil[HO_MAX_DIMS];
  int64_t osize[HO_MAX_DIMS];
  int64_t in_count, out_count, cells;
} ho_geometry;

static int ho_make_geometry(ho_geometry *g, int dims, const int64_t *size, const int64_t *kernel, const int64_t *stride,
                            const int64_t *pad, const int64_t *dil) {
  if (dims < 1 || dims > HO_MAX_DIMS) return -1;
  g->dims = dims;
  g->in_count = g->out_count = g->cells = 1;
  for (int d = 0; d < dims; ++d) {
    if (kernel[d] <= 0 || stride[d] <= 0 || pad[d] < 0 || dil[d] <= 0 || size[d] < 1) return -1;
    const int64_t window = kernel[d] + (kernel[d] - 1) * (dil[d] - 1); /* ImageToMatrix.h:189-197 */
    if (size[d] + 2 * pad[d] < window) return -1;
    g->size[d] = size[d]; g->kernel[d] = kernel[d]; g->stride[d] = stride[d]; g->pad[d] = pad[d]; g->dil[d] = dil[d];
    g->osize[d] = (size[d] + 2 * pad[d] - window) / stride[d] + 1;      /* ImageToMatrix.h:201-209 */
    g->in_count *= size[d];
    g->out_count *= g->osize[d];
    g->cells *= kernel[d];
  }
  return 0;
}

/* Flat input index of window cell q at output position p, or -1 for padding (ImageToMatrix.h:304-347). */
static int64_t ho_cell_index(const ho_geometry *g, int64_t p, int64_t q) {
  int64_t index = 0, scale = 1;
  for (int d = g->dims - 1; d >= 0; --d) {
    const int64_t od = p % g->osize[d], qd = q % g->kernel[d];
    p /= g->osize[d];
    q /= g->kernel[d];
    const int64_t at = od * g->stride[d] - g->pad[d] + qd * g->dil[d];
    if (at < 0 || at >= g->size[d]) return -1;
    index += at * scale;
    scale *= g->size[d];
  }
  return index;
}

typedef struct { uint32_t key; float margin; uint32_t vertex; } ho_cpath;

/* Traversal on one window: HingeTreeCommon.h:157-178 (tree), :72-91 (fern). */
static ho_cpath ho_conv_traverse(int kind, const ho_geometry *g, const float *chan, int64_t p, const float *thr,
                                 const int64_t *ord, int depth) {
  ho_cpath r = {0u, 0.0f, 0u};
  uint32_t v = 0;
  for (int l = 0; l < depth; ++l) {
    const uint32_t at = kind == HO_FERN ? (uint32_t)l : v;
    const int64_t idx = ho_cell_index(g, p, ord[at]);
    const float m = (idx < 0 ? 0.0f : chan[idx]) - thr[at];
    const uint32_t bit = m > 0.0f;
    if (l == 0 || fabsf(m) < fabsf(r.margin)) { r.margin = m; r.vertex = at; }
    r.key |= bit << l;
    v = 2 * v + 1 + bit;
  }
  return r;
}

static int ho_conv_depth(int64_t L) {
  if (L <= 0 || (L & (L - 1)) != 0) return -1;
  int d = 0;
  while (L > 1) { L >>= 1; ++d; }
  return d;
}

int64_t ho_conv_output_size(int dims, const int64_t *size, const int64_t *kernel, const int64_t *stride,
                            const int64_t *pad, const int64_t *dil, int64_t *osize) {
  ho_geometry g;
  if (ho_make_geometry(&g, dims, size, kernel, stride, pad, dil) != 0) return -1;
  for (int d = 0; d < dims; ++d) osize[d] = g.osize[d];
  return g.out_count;
}

int ho_conv_forward(int kind, int dims, const float *x, const float *thr, const int64_t *ord, const float *w, float *out,
                    int64_t B, int64_t Ci, int64_t Co, int64_t L, int64_t M, const int64_t *size, const int64_t *kernel,
                    const int64_t *stride, const int64_t *pad, const int64_t *dil) {
  ho_geometry g;
  const int depth = ho_conv_depth(L);
  if (depth < 0 || ho_make_geometry(&g, dims, size, kernel, stride, pad, dil) != 0) return -1;
  const int64_t N = kind == HO_FERN ? depth : (((int64_t)1) << depth) - 1;
  memset(out, 0, sizeof(float) * (size_t)(B * Co * g.out_count * M));
  for (int64_t i = 0; i < B; ++i)
    for (int64_t c = 0; c < Ci; ++c) {
      const float *chan = x + (i * Ci + c) * g.in_count;
      for (int64_t j = 0; j < Co; ++j)
        for (int64_t p = 0; p < g.out_count; ++p) {
          const ho_cpath r = ho_conv_traverse(kind, &g, chan, p, thr + (j * Ci + c) * N, ord + (j * Ci + c) * N, depth);
          const float am = fabsf(r.margin);
          const float *wl = w + ((j * Ci + c) * L + r.key) * M;
          for (int64_t m = 0; m < M; ++m) out[((i * Co + j) * g.out_count + p) * M + m] += wl[m] * am;
        }
    }
  return 0;
}

int ho_conv_backward(int kind, int dims, const float *x, const float *thr, const int64_t *ord, const float *w,
                     const float *gout, float *gx, float *gthr, float *gw, int64_t B, int64_t Ci, int64_t Co, int64_t L,
                     int64_t M, const int64_t *size, const int64_t *kernel, const int64_t *stride, const int64_t *pad,
                     const int64_t *dil) {
  ho_geometry g;
  const int depth = ho_conv_depth(L);
  if (depth < 0 || ho_make_geometry(&g, dims, size, kernel, stride, pad, dil) != 0) return -1;
  const int64_t N = kind == HO_FERN ? depth : (((int64_t)1) << depth) - 1;
  for (int64_t i = 0; i < B; ++i)
    for (int64_t c = 0; c < Ci; ++c) {
      const float *chan = x + (i * Ci + c) * g.in_count;
      for (int64_t j = 0; j < Co; ++j) {
        const int64_t tree = j * Ci + c;
        for (int64_t p = 0; p < g.out_count; ++p) {
          const ho_cpath r = ho_conv_traverse(kind, &g, chan, p, thr + tree * N, ord + tree * N, depth);
          const float sign = (float)((0.0f < r.margin) - (r.margin < 0.0f));
          const float am = fabsf(r.margin);
          const float *wl = w + (tree * L + r.key) * M;
          const float *gl = gout + ((i * Co + j) * g.out_count + p) * M;
          const int64_t idx = ho_cell_index(&g, p, ord[tree * N + r.vertex]);
          for (int64_t m = 0; m < M; ++m) {
            if (gx && idx >= 0) gx[(i * Ci + c) * g.in_count + idx] += ho_term(sign * wl[m] * gl[m]);
            if (gthr) gthr[tree * N + r.vertex] += ho_term(-sign * wl[m] * gl[m]);
            if (gw) gw[(tree * L + r.key) * M + m] += ho_term(am * gl[m]);
          }
        }
      }
    }
  return 0;
}

/* ---- contract / expand (expand.cpp:70-92 and :202-224 for 2-D, the 3-D forms alike) -----------
 * contract: image [BC, size...] -> non-overlapping windows [BC, osize..., win...], zero padded,
 *           osize = (size + 2*pad - win) / win + 1.
 * expand:   the inverse; image size = osize*win - (2*pad / win)*win; cells in the padding are dropped.
 * Element type is opaque: `elem` bytes are moved. */
int ho_contract(int dims, int elem, const void *in, void *out, int64_t BC, const int64_t *size, const int64_t *win,
                const int64_t *pad) {
  if (dims < 2 || dims > 3) return -1;
  int64_t osize[3], in_count = 1, out_count = 1, cells = 1;
  for (int d = 0; d < dims; ++d) {
    if (pad[d] < 0 || win[d] < 1 || win[d] > size[d] + 2 * pad[d]) return -1;
    osize[d] = (size[d] + 2 * pad[d] - win[d]) / win[d] + 1;
    in_count *= size[d]; out_count *= osize[d]; cells *= win[d];
  }
  memset(out, 0, (size_t)(BC * out_count * cells * elem));
  for (int64_t b = 0; b < BC; ++b)
    for (int64_t p = 0; p < out_count; ++p)
      for (int64_t q = 0; q < cells; ++q) {
        int64_t pp = p, qq = q, index = 0, scale = 1, inside = 1;
        for (int d = dims - 1; d >= 0; --d) {
          const int64_t at = (pp % osize[d]) * win[d] - pad[d] + (qq % win[d]);
          pp /= osize[d]; qq /= win[d];
          if (at < 0 || at >= size[d]) inside = 0;
          index += at * scale; scale *= size[d];
        }
        if (inside)
          memcpy((char *)out + ((b * out_count + p) * cells + q) * elem, (const char *)in + (b * in_count + index) * elem,
                 (size_t)elem);
      }
  return 0;
}

int ho_expand(int dims, int elem, const void *in, void *out, int64_t BC, const int64_t *osize, const int64_t *win,
              const int64_t *pad, int64_t *size) {
  if (dims < 2 || dims > 3) return -1;
  int64_t in_count = 1, out_count = 1, cells = 1;
  for (int d = 0; d < dims; ++d) {
    if (pad[d] < 0) return -1;
    size[d] = osize[d] * win[d] - ((2 * pad[d]) / win[d]) * win[d];
    if (size[d] < 1) return -1;
    in_count *= size[d]; out_count *= osize[d]; cells *= win[d];
  }
  if (out == NULL) return 0; /* size query */
  memset(out, 0, (size_t)(BC * in_count * elem));
  for (int64_t b = 0; b < BC; ++b)
    for (int64_t p = 0; p < out_count; ++p)
      for (int64_t q = 0; q < cells; ++q) {
        int64_t pp = p, qq = q, index = 0, scale = 1, inside = 1;
        for (int d = dims - 1; d >= 0; --d) {
          const int64_t at = (pp % osize[d]) * win[d] - pad[d] + (qq % win[d]);
          pp /= osize[d]; qq /= win[d];
          if (at < 0 || at >= size[d]) inside = 0;
          index += at * scale; scale *= size[d];
        }
        if (inside)
          memcpy((char *)out + (b * in_count + index) * elem, (const char *)in + ((b * out_count + p) * cells + q) * elem,
                 (size_t)elem);
      }
  return 0;
}
