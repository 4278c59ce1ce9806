/*
 * CPU restatement of the hinge trie (third part of the oracle; test infrastructure only).
 *
 * A trie walks a tree like a hinge tree does, but every decision on the path contributes:
 *   out[i,j,k,m] = sum over depth d (ascending) of |margin_d| * w[j, vertex_d, m]
 * with one weight row per INTERNAL vertex, w [T, 2^depth - 1, M] (HingeTrieCommon.h:71-85,
 * hingetrie.cpp:100-118 forward, :160-264 backward).  Backward order: i, j, k, then m, then d.
 */
#include <stdint.h>
#include <math.h>

#include "hinge_oracle_terms.h"

static int ho_trie_depth(int64_t N) {
  const int64_t leaves = N + 1; /* HingeTrieCommon.h:51-64 */
  if (leaves <= 0 || (leaves & (leaves - 1)) != 0) return -1;
  int d = 0;
  for (int64_t l = leaves; l > 1; l >>= 1) ++d;
  return d;
}

static void ho_trie_path(const float *x, int64_t stride, const float *thr, const int64_t *ord, int depth, float *margin,
                         uint32_t *vertex) {
  uint32_t v = 0;
  for (int d = 0; d < depth; ++d) {
    const float m = x[ord[v] * stride] - thr[v];
    margin[d] = m;
    vertex[d] = v;
    v = 2 * v + 1 + (m > 0.0f);
  }
}

int ho_trie_forward(const float *x, const float *thr, const int64_t *ord, const float *w, float *out, int64_t B,
                    int64_t C, int64_t K, int64_t T, int64_t N, int64_t M) {
  const int depth = ho_trie_depth(N);
  if (depth < 0 || depth > 31) return -1;
  float margin[32];
  uint32_t vertex[32];
  for (int64_t i = 0; i < B; ++i)
    for (int64_t j = 0; j < T; ++j)
      for (int64_t k = 0; k < K; ++k) {
        ho_trie_path(x + i * C * K + k, K, thr + j * N, ord + j * N, depth, margin, vertex);
        for (int64_t m = 0; m < M; ++m) {
          float acc = 0.0f;
          for (int d = 0; d < depth; ++d) acc += fabsf(margin[d]) * w[(j * N + vertex[d]) * M + m];
          out[((i * T + j) * K + k) * M + m] = acc;
        }
      }
  return 0;
}

int ho_trie_backward(const float *x, const float *thr, const int64_t *ord, const float *w, const float *g, float *gx,
                     float *gthr, float *gw, int64_t B, int64_t C, int64_t K, int64_t T, int64_t N, int64_t M) {
  const int depth = ho_trie_depth(N);
  if (depth < 0 || depth > 31) return -1;
  float margin[32];
  uint32_t vertex[32];
  for (int64_t i = 0; i < B; ++i)
    for (int64_t j = 0; j < T; ++j)
      for (int64_t k = 0; k < K; ++k) {
        ho_trie_path(x + i * C * K + k, K, thr + j * N, ord + j * N, depth, margin, vertex);
        for (int64_t m = 0; m < M; ++m) {
          const float gm = g[((i * T + j) * K + k) * M + m];
          for (int d = 0; d < depth; ++d) {
            const float sign = (float)((0.0f < margin[d]) - (margin[d] < 0.0f));
            const float wv = w[(j * N + vertex[d]) * M + m];
            if (gx) gx[(i * C + ord[j * N + vertex[d]]) * K + k] += ho_term(sign * wv * gm);
            if (gthr) gthr[j * N + vertex[d]] += ho_term(-sign * wv * gm);
            if (gw) gw[(j * N + vertex[d]) * M + m] += ho_term(fabsf(margin[d]) * gm);
          }
        }
      }
  return 0;
}
