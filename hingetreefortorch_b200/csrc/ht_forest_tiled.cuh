// Shared-memory tile kernel for the forest forward (see ht_forest_tiled.cu).
#pragma once

#include "ht_common.cuh"

namespace ht {

// Bytes of per-tree records the tile kernel needs in the workspace (0 when the shape does not qualify).
size_t forward_tiled_workspace_bytes(const ht_forest_problem *p);

// Runs the forward with the tile kernel when the shape qualifies; returns HT_ERR_UNSUPPORTED
// (and launches nothing) when it does not, so that the caller can use the any-shape kernel.
// `ord` are the compact (validated, clamped) int32 ordinals; `records` is 256-byte aligned
// scratch of forward_tiled_workspace_bytes() bytes.
// With `eval_records` (backward_records_bytes() bytes) and a problem for which forward_saves() holds, the forward
// also leaves its traversal there: the signed margin and the deciding vertex / leaf of every evaluation, from which
// backward_saved() computes the gradients without walking the trees again.
bool forward_saves(const ht_forest_problem *p);
int saved_samples_per_cta(const ht_forest_problem *p);  // 0: the backward from saved records does not take the shape
int forward_tiled(const ht_forest_problem *p, const float *x, const float *thr, const int32_t *ord, const float *w,
                  float *out, void *records, void *eval_records, uint32_t *status_word, cudaStream_t stream);

// The backward from the records a saving forward left (default mode; forward_saves(p) must hold and the inputs must
// be the forward's).  `ord` are the compact ordinals.  Any of gx / gthr / gw may be null; the others must have been
// cleared.
int backward_saved(const ht_forest_problem *p, const int32_t *ord, const float *w, const float *g, float *gx, float *gthr,
                   float *gw, void *eval_records, cudaStream_t stream);

// Backward with the tile kernels of ht_forest_tiled_bwd.cu; same contract as forward_tiled.  With
// `eval_records` (backward_records_bytes() bytes of 256-byte aligned scratch; 0 = shape not
// supported) the traversal kernel writes per-evaluation records and two reduction kernels add
// them in the reference's order: deterministic, and the only tile path taken in HT_DETERMINISTIC
// mode.  Without it the traversal kernel scatters with global reductions (default mode only).
// Any of gx / gthr / gw may be null; the others must have been cleared.
size_t backward_records_bytes(const ht_forest_problem *p);
int backward_tiled(const ht_forest_problem *p, const float *x, const float *thr, const int32_t *ord, const float *w,
                   const float *g, float *gx, float *gthr, float *gw, void *records, void *eval_records,
                   uint32_t *status_word, cudaStream_t stream);

// Backward for several outputs per leaf (default mode, tabular input) with the tile kernel of
// ht_forest_tiled_bwd_multi.cu; same contract as backward_tiled without evaluation records.
// `records` is scratch of `records_bytes` bytes (the forward's record area is large enough).
int backward_tiled_multi(const ht_forest_problem *p, const float *x, const float *thr, const int32_t *ord, const float *w,
                         const float *g, float *gx, float *gthr, float *gw, void *records, size_t records_bytes,
                         uint32_t *status_word, cudaStream_t stream);

}  // namespace ht
