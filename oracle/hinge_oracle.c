/*
 * CPU restatement of the hinge tree / hinge fern evaluation path of HingeTreeForTorch.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker for the CUDA path: only the tests,
 * the smoke check and the CPU-baseline legs of the benchmark may build, load or call it.
 * The product never does, and has no CPU fallback.
 *
 * Parity pinning: the reference ships no tests or golden vectors for this path.  This
 * restatement is pinned instead against outputs of the unmodified reference CPU build
 * (oracle/build_ref.py -> oracle/_ref) on seeded inputs, committed as fixtures under
 * tests/golden/ together with the script that generated them, and against the
 * hand-checkable known-answer cases in tests/test_oracle.py.
 *
 * Every function cites the reference file:line whose arithmetic and accumulation order it
 * follows.  Floating point is plain single precision with no fused multiply-add
 * (build with -ffp-contract=off), matching the reference's x86-64 -O2 build.
 *
 * Layouts (all row-major, contiguous):
 *   x   [B, C, K]        K = product of the inner data dims (1 for tabular input)
 *   thr [T, N]           N = 2^d - 1 (tree) or d (fern)
 *   ord [T, N] int64     feature index of each decision, in [0, C)
 *   w   [T, L, M]        L = 2^d leaves, M = product of the inner weight dims
 *   out [B, T, K, M]
 */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <math.h>

#include "hinge_oracle_terms.h"

int ho_magnitude_mode = 0;
void ho_set_magnitude_mode(int on) { ho_magnitude_mode = on; }

#define HO_TREE 0
#define HO_FERN 1

typedef struct {
  uint32_t key;     /* leaf key: bit l is the decision taken at depth l (LSB = root) */
  float margin;     /* signed margin of the decision with the smallest |margin| */
  uint32_t vertex;  /* index (into thr/ord of this tree) of that decision */
} ho_path;

/* Feature lookup for the plain and the image+vector "fusion" forms.
 * Fusion: HingeTreeCommon.h:95-100 (fern) and :182-187 (tree): ordinals below the image
 * channel count address the image (strided by K), the rest address the per-sample vector. */
typedef struct {
  const float *img;   /* points at x[i, 0, k] */
  int64_t stride;     /* K */
  const float *vec;   /* points at vec[i, 0], or NULL for the plain form */
  int64_t img_channels;
} ho_feat;

static inline float ho_get(const ho_feat *f, int64_t j) {
  if (f->vec == NULL || j < f->img_channels) return f->img[f->stride * j];
  return f->vec[j - f->img_channels];
}

/* Tree traversal: HingeTreeCommon.h:157-178.  Fern: HingeTreeCommon.h:72-91.
 * Strict '<' keeps the first (shallowest) minimum; margin == 0 or NaN goes left. */
static ho_path ho_traverse(int kind, const ho_feat *f, const float *thr, const int64_t *ord, int depth) {
  ho_path p;
  p.key = 0;
  p.margin = ho_get(f, ord[0]) - thr[0];
  p.vertex = 0;
  uint32_t v = 0;
  for (int l = 0; l < depth; ++l) {
    const uint32_t at = (kind == HO_FERN) ? (uint32_t)l : v;
    const float m = ho_get(f, ord[at]) - thr[at];
    const uint32_t bit = (m > 0.0f);
    if (fabsf(m) < fabsf(p.margin)) { p.margin = m; p.vertex = at; }
    p.key |= (bit << l);
    v = 2 * v + 1 + bit;
  }
  return p;
}

static int ho_depth_of(int64_t leaves) {
  /* HingeTreeCommon.h:141-152: -1 unless the leaf count is a power of two */
  if (leaves <= 0 || (leaves & (leaves - 1)) != 0) return -1;
  int d = 0;
  while (leaves > 1) { leaves >>= 1; ++d; }
  return d;
}

int64_t ho_threshold_count(int kind, int depth) {
  /* HingeTreeCommon.h:69 (fern) and :154 (tree) */
  return kind == HO_FERN ? depth : (((int64_t)1) << depth) - 1;
}

/* hingetree.cpp:137-150 (forward), with the fusion feature lookup of
 * hingetree_fusion.cpp:120-133 when vec != NULL.  C is the image channel count. */
int ho_forward(int kind, const float *x, const float *vec, int64_t Cv, const float *thr, const int64_t *ord,
               const float *w, float *out, int64_t B, int64_t C, int64_t K, int64_t T, int64_t L, int64_t M) {
  const int d = ho_depth_of(L);
  if (d < 0) return -1;
  const int64_t N = ho_threshold_count(kind, d);
  for (int64_t i = 0; i < B; ++i)
    for (int64_t j = 0; j < T; ++j)
      for (int64_t k = 0; k < K; ++k) {
        ho_feat f = { x + (i * C) * K + k, K, vec ? vec + i * Cv : NULL, C };
        const ho_path p = ho_traverse(kind, &f, thr + j * N, ord + j * N, d);
        for (int64_t m = 0; m < M; ++m)
          out[((i * T + j) * K + k) * M + m] = fabsf(p.margin) * w[(j * L + p.key) * M + m];
      }
  return 0;
}

/* hingetree.cpp:313-389 (leaf map; int64 here, as the reference's GPU path returns,
 * hingetree_gpu.cu:842), :391-472 (margin map) and :583-646 (reachability). */
int ho_maps(int kind, const float *x, const float *thr, const int64_t *ord, int64_t *leaf, float *margin,
            int64_t *margin_ord, int64_t *reach, int64_t B, int64_t C, int64_t K, int64_t T, int64_t L) {
  const int d = ho_depth_of(L);
  if (d < 0) return -1;
  const int64_t N = ho_threshold_count(kind, d);
  if (reach) memset(reach, 0, sizeof(int64_t) * (size_t)(T * L));
  for (int64_t i = 0; i < B; ++i)
    for (int64_t j = 0; j < T; ++j)
      for (int64_t k = 0; k < K; ++k) {
        ho_feat f = { x + (i * C) * K + k, K, NULL, C };
        const ho_path p = ho_traverse(kind, &f, thr + j * N, ord + j * N, d);
        const int64_t o = (i * T + j) * K + k;
        if (leaf) leaf[o] = (int64_t)p.key;
        if (margin) margin[o] = p.margin;
        if (margin_ord) margin_ord[o] = ord[j * N + p.vertex];
        if (reach) reach[j * L + p.key] += 1;
      }
  return 0;
}

/* hingetree.cpp:232-308 (backward), fusion form hingetree_fusion.cpp:225-301.
 * Accumulation order is the reference's: i outer, then j, k, and m innermost, every term
 * ((+-sign)*w)*g added on its own.  Any of gx/gvec/gthr/gw may be NULL (not requested);
 * the ones given must be zero-filled by the caller.  With vec != NULL, gx and gvec are the
 * image and vector gradients (the vector gradient sums over k). */
int ho_backward(int kind, const float *x, const float *vec, int64_t Cv, const float *thr, const int64_t *ord,
                const float *w, const float *g, float *gx, float *gvec, float *gthr, float *gw,
                int64_t B, int64_t C, int64_t K, int64_t T, int64_t L, int64_t M) {
  const int d = ho_depth_of(L);
  if (d < 0) return -1;
  const int64_t N = ho_threshold_count(kind, d);
  for (int64_t i = 0; i < B; ++i)
    for (int64_t j = 0; j < T; ++j)
      for (int64_t k = 0; k < K; ++k) {
        ho_feat f = { x + (i * C) * K + k, K, vec ? vec + i * Cv : NULL, C };
        const ho_path p = ho_traverse(kind, &f, thr + j * N, ord + j * N, d);
        const float sign = (float)((0.0f < p.margin) - (p.margin < 0.0f));
        const float *wl = w + (j * L + p.key) * M;
        const float *gl = g + ((i * T + j) * K + k) * M;
        const int64_t c = ord[j * N + p.vertex];
        for (int64_t m = 0; m < M; ++m) {
          if (gx || gvec) {
            const float t = ho_term(sign * wl[m] * gl[m]);
            if (vec == NULL || c < C) { if (gx) gx[(i * C + c) * K + k] += t; }
            else if (gvec) gvec[i * Cv + (c - C)] += t;
          }
          if (gthr) gthr[j * N + p.vertex] += ho_term(-sign * wl[m] * gl[m]);
          if (gw) gw[(j * L + p.key) * M + m] += ho_term(fabsf(p.margin) * gl[m]);
        }
      }
  return 0;
}

/* Test helper (no counterpart in the reference): the sum of |term| that ho_backward adds into
 * every gradient element, in double precision.  Tests scale their floating point tolerance
 * for the non-deterministic backward with it. */
int ho_backward_magnitudes(int kind, const float *x, const float *thr, const int64_t *ord, const float *w,
                           const float *g, double *ax, double *athr, double *aw,
                           int64_t B, int64_t C, int64_t K, int64_t T, int64_t L, int64_t M) {
  const int d = ho_depth_of(L);
  if (d < 0) return -1;
  const int64_t N = ho_threshold_count(kind, d);
  for (int64_t i = 0; i < B; ++i)
    for (int64_t j = 0; j < T; ++j)
      for (int64_t k = 0; k < K; ++k) {
        ho_feat f = { x + (i * C) * K + k, K, NULL, C };
        const ho_path p = ho_traverse(kind, &f, thr + j * N, ord + j * N, d);
        const double sign = (double)((0.0f < p.margin) - (p.margin < 0.0f));
        const float *wl = w + (j * L + p.key) * M;
        const float *gl = g + ((i * T + j) * K + k) * M;
        const int64_t c = ord[j * N + p.vertex];
        for (int64_t m = 0; m < M; ++m) {
          const double t = fabs(sign * (double)wl[m] * (double)gl[m]);
          ax[(i * C + c) * K + k] += t;
          athr[j * N + p.vertex] += t;
          aw[(j * L + p.key) * M + m] += fabs((double)p.margin * (double)gl[m]);
        }
      }
  return 0;
}

/* ---- trees followed by a linear layer over the tree dimension ("fused linear") --------------
 * hingetree_fused_linear.cpp:154-181 (forward): out starts as the bias and receives, for j
 * ascending, (|margin| * L[o,j]) * w[j,leaf,m].  With vec != NULL the feature lookup is the
 * image+vector one (hingetree_fused_linear.cpp:414-767).  out is [B, O, K, M]. */
int ho_linear_forward(int kind, const float *x, const float *vec, int64_t Cv, const float *thr, const int64_t *ord,
                      const float *w, const float *lin, const float *bias, float *out,
                      int64_t B, int64_t C, int64_t K, int64_t T, int64_t L, int64_t M, int64_t O) {
  const int d = ho_depth_of(L);
  if (d < 0) return -1;
  const int64_t N = ho_threshold_count(kind, d);
  for (int64_t o = 0; o < O; ++o)
    for (int64_t i = 0; i < B; ++i)
      for (int64_t k = 0; k < K; ++k)
        for (int64_t m = 0; m < M; ++m) out[((i * O + o) * K + k) * M + m] = bias[o];
  for (int64_t i = 0; i < B; ++i)
    for (int64_t j = 0; j < T; ++j)
      for (int64_t k = 0; k < K; ++k) {
        ho_feat f = { x + (i * C) * K + k, K, vec ? vec + i * Cv : NULL, C };
        const ho_path p = ho_traverse(kind, &f, thr + j * N, ord + j * N, d);
        const float am = fabsf(p.margin);
        for (int64_t o = 0; o < O; ++o) {
          const float scale = am * lin[o * T + j];
          for (int64_t m = 0; m < M; ++m)
            out[((i * O + o) * K + k) * M + m] += scale * w[(j * L + p.key) * M + m];
        }
      }
  return 0;
}

/* hingetree_fused_linear.cpp:267-409 (backward); g is [B, O, K, M].  Loop order i, j, k, o, m.
 * The bias gradient is the plain sum of g over every dimension but O (the reference calls
 * Tensor::sum, :385-390); it is accumulated in double here and rounded once. */
int ho_linear_backward(int kind, const float *x, const float *vec, int64_t Cv, const float *thr, const int64_t *ord,
                       const float *w, const float *lin, const float *g, float *gx, float *gvec, float *gthr,
                       float *gw, float *glin, float *gbias,
                       int64_t B, int64_t C, int64_t K, int64_t T, int64_t L, int64_t M, int64_t O) {
  const int d = ho_depth_of(L);
  if (d < 0) return -1;
  const int64_t N = ho_threshold_count(kind, d);
  for (int64_t i = 0; i < B; ++i)
    for (int64_t j = 0; j < T; ++j)
      for (int64_t k = 0; k < K; ++k) {
        ho_feat f = { x + (i * C) * K + k, K, vec ? vec + i * Cv : NULL, C };
        const ho_path p = ho_traverse(kind, &f, thr + j * N, ord + j * N, d);
        const float sign = (float)((0.0f < p.margin) - (p.margin < 0.0f));
        const float am = fabsf(p.margin);
        const float *wl = w + (j * L + p.key) * M;
        const int64_t c = ord[j * N + p.vertex];
        for (int64_t o = 0; o < O; ++o) {
          const float *gl = g + ((i * O + o) * K + k) * M;
          const float lw = lin[o * T + j];
          for (int64_t m = 0; m < M; ++m) {
            if (gx || gvec) {
              const float t = ho_term((sign * lw) * wl[m] * gl[m]);
              if (vec == NULL || c < C) { if (gx) gx[(i * C + c) * K + k] += t; }
              else if (gvec) gvec[i * Cv + (c - C)] += t;
            }
            if (gthr) gthr[j * N + p.vertex] += ho_term((-sign * lw) * wl[m] * gl[m]);
            if (gw) gw[(j * L + p.key) * M + m] += ho_term((am * lw) * gl[m]);
            if (glin) glin[o * T + j] += ho_term(am * wl[m] * gl[m]);
          }
        }
      }
  if (gbias)
    for (int64_t o = 0; o < O; ++o) {
      double s = 0.0;
      for (int64_t i = 0; i < B; ++i)
        for (int64_t k = 0; k < K; ++k)
          for (int64_t m = 0; m < M; ++m) s += (double)ho_term(g[((i * O + o) * K + k) * M + m]);
      gbias[o] = (float)s;
    }
  return 0;
}
