/*
 * hingetree_b200 -- C ABI of the sm_100a hinge tree / hinge fern evaluation library.
 *
 * This is the boundary a binding of HingeTreeForTorch's `hingetree_cpp` extension links
 * against: plain pointers and sizes, no torch types.  Every entry point
 *   - works on DEVICE pointers of the current CUDA device,
 *   - enqueues its kernels on the stream it is given and returns without synchronising,
 *   - allocates nothing (scratch comes from the caller, sized by the *_workspace_bytes query),
 *   - never throws: it returns HT_OK or a negative ht_status.
 *
 * Tensor layouts are the reference's (row-major, contiguous, fp32 data, int64 ordinals):
 *   x   [B, C, K]     K = product of the inner data dimensions (1 for tabular input)
 *   thr [T, N]        N = 2^depth - 1 for trees, depth for ferns
 *   ord [T, N]        int64 feature index of each decision, in [0, C)
 *   w   [T, L, M]     L = 2^depth leaves, M = product of the inner weight dimensions
 *   out [B, T, K, M]
 *
 * Ordinal validation: the reference raises when an ordinal is outside [0, C)
 * (hingetree_gpu.cu:445).  Here the kernels clamp such an ordinal to 0, so that no access
 * ever leaves the input, and OR the bit HT_FLAG_ORDINAL_RANGE into the caller's device
 * status word; the host binding reads the word and raises.  The status word is never
 * cleared by the library.
 */
#ifndef HINGETREE_B200_H
#define HINGETREE_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct CUstream_st *ht_stream_t; /* a cudaStream_t */

typedef enum ht_status {
  HT_OK = 0,
  HT_ERR_INVALID_ARGUMENT = -1, /* shapes / null pointers: the reference's std::invalid_argument (ValueError) */
  HT_ERR_DEPTH = -2,            /* depth outside [1, 31] or N does not match: the reference's std::runtime_error */
  HT_ERR_CUDA = -3,             /* a launch or runtime call failed; ht_last_cuda_error() has the code */
  HT_ERR_WORKSPACE = -4,        /* workspace missing, misaligned or too small */
  HT_ERR_UNSUPPORTED = -5       /* valid request that this build does not implement */
} ht_status;

/* bits OR-ed into the device status word */
#define HT_FLAG_ORDINAL_RANGE 1u /* an ordinal was < 0 or >= C (reference: RuntimeError) */
#define HT_FLAG_PIPELINE_TIMEOUT 0x80000000u /* a bounded wait inside a kernel ran out; outputs are incomplete */

#define HT_KIND_TREE 0 /* complete binary tree: HingeTreeCommon<>  (HingeTreeCommon.h:129) */
#define HT_KIND_FERN 1 /* oblivious fern:       HingeFernCommon<>  (HingeTreeCommon.h:42)  */

/* ht_forest_problem.flags */
#define HT_DETERMINISTIC 1u /* backward: fixed summation order equal to the reference CPU loops */
#define HT_WORKSPACE_FOR_BACKWARD 2u /* ht_forest_workspace_bytes: include the backward's evaluation records */
#define HT_SAVE_FOR_BACKWARD 4u /* ht_forest_forward_f32: also leave the traversal in the workspace (see below) */
#define HT_SAVED_FORWARD 8u     /* ht_forest_backward_f32: the workspace still holds that traversal */

typedef struct ht_forest_problem {
  int32_t kind;   /* HT_KIND_TREE or HT_KIND_FERN */
  int32_t depth;  /* 1..31 (HingeTreeCommon.h:51,138: uint32 leaf keys) */
  int64_t B;      /* batch */
  int64_t C;      /* channels (features) of x */
  int64_t K;      /* inner data positions per sample */
  int64_t T;      /* trees */
  int64_t M;      /* outputs per leaf */
  uint32_t flags;
  uint32_t reserved;
} ht_forest_problem;

int ht_version(void);
const char *ht_status_string(int status);
int ht_last_cuda_error(void); /* cudaError_t of the last failed runtime call on this thread */
uint64_t ht_launch_count(void); /* kernels this library has launched in this process (diagnostics; no reference counterpart) */
/* Self test of the tile kernels' bounded waits: a one-warp kernel waits, with a limit of a few tries, on a barrier
 * that nothing arrives on, and reports the way a tile kernel reports a copy that never came: it ORs
 * HT_FLAG_PIPELINE_TIMEOUT into *status_word and returns.  Nothing faults or hangs.  (No reference counterpart.) */
int ht_selftest_bounded_wait(uint32_t *status_word, ht_stream_t stream);

/* Scratch bytes ht_forest_* calls need for this problem: compact ordinals and the tile kernel's
 * per-tree records.  With HT_WORKSPACE_FOR_BACKWARD in p->flags the figure also covers 12 bytes
 * per (sample, tree) of evaluation records (10 up to depth 8), which let ht_forest_backward_f32 run its fastest,
 * fixed-order path on tabular one-output-per-leaf problems (up to 32 GiB; beyond that, and
 * whenever the workspace passed is smaller, the backward uses its other paths).  The workspace
 * must be 256-byte aligned device memory. */
size_t ht_forest_workspace_bytes(const ht_forest_problem *p);

/* Saving the forward's traversal for the backward.  The reference's backward walks every tree again, three
 * times (hingetree_gpu.cu:699-727); here a training step can walk them once: ht_forest_forward_f32 called with
 * HT_SAVE_FOR_BACKWARD and a workspace sized with HT_WORKSPACE_FOR_BACKWARD leaves, per (sample, tree), the
 * signed margin and the deciding vertex / leaf in the workspace (6 or 8 bytes), and ht_forest_backward_f32
 * called with HT_SAVED_FORWARD on the SAME x, thr, ord, w and workspace — nothing else having used the
 * workspace in between — computes the gradients from them.  ht_forest_forward_saves() tells whether the
 * forward does so for a problem (tabular input, one output per leaf, shapes the tile kernel takes with whole
 * tree groups); where it returns 0 both flags are ignored.  Both modes: with HT_DETERMINISTIC the sums are
 * the reference's, bit for bit, as without saving. */
int ht_forest_forward_saves(const ht_forest_problem *p);

/* out[i,j,k,m] = |margin(i,j,k)| * w[j, leaf(i,j,k), m]
 * Replaces hingetree_gpu_forward / ForwardKernel (hingetree_gpu.cu:416-498, 58-87) and the
 * traversal templates it instantiates (HingeTreeCommon.cuh:60-79 fern, 133-154 tree). */
int ht_forest_forward_f32(const ht_forest_problem *p, const float *x, const float *thr, const int64_t *ord,
                          const float *w, float *out, void *workspace, size_t workspace_bytes,
                          uint32_t *status_word, ht_stream_t stream);

/* The same forward for callers that cannot supply a workspace.  It has no counterpart in the
 * reference.  It is meant for code that may not allocate device memory at the point of the
 * call -- a serving loop running against a frozen memory pool, a plugin host that hands a
 * binding nothing but its input and output buffers, a runtime whose allocator is out of the
 * binding's reach -- and that therefore has no buffer to pass as `workspace`.  The scratch
 * lives in a fixed array inside the library image (ht_forest_static_scratch_bytes() bytes,
 * currently 16 MiB, resident on every device that loads the library until the process exits).
 *   - Nothing is allocated or freed, here or in anything this calls.
 *   - A problem whose ht_forest_workspace_bytes() exceeds the array is refused with
 *     HT_ERR_WORKSPACE; use ht_forest_forward_f32 with your own workspace for those.
 *   - The first call on a device looks up the array's device address (once per device, with
 *     that device current); make that first call outside any stream capture.  The address is
 *     kept for the life of the device's primary context: after cudaDeviceReset() this entry
 *     point must not be used again in the process.
 *   - HT_WORKSPACE_FOR_BACKWARD in p->flags is ignored: only the forward's scratch counts.
 *   - All calls on a device share the one array, which simply keeps what the last call wrote;
 *     every byte that is read is rewritten first, so nothing needs clearing.  Two calls that
 *     overlap on the GPU (different streams, or different host threads) race on it: serialise
 *     them.  x, thr, ord, w, out and status_word are as for ht_forest_forward_f32. */
size_t ht_forest_static_scratch_bytes(void);
int ht_forest_forward_static_f32(const ht_forest_problem *p, const float *x, const float *thr, const int64_t *ord,
                                 const float *w, float *out, uint32_t *status_word, ht_stream_t stream);

/* leaf[i,j,k] = leaf key (bit l = decision at depth l), int64.
 * Replaces hingetree_gpu_leafmap / LeafMapKernel (hingetree_gpu.cu:791-860, 116-139). */
int ht_forest_leafmap_f32(const ht_forest_problem *p, const float *x, const float *thr, const int64_t *ord,
                          int64_t *leaf, void *workspace, size_t workspace_bytes, uint32_t *status_word,
                          ht_stream_t stream);

/* margin[i,j,k] = signed margin of the closest decision, margin_ord[i,j,k] = its feature index.
 * Replaces hingetree_gpu_marginmap / MarginMapKernel (hingetree_gpu.cu:862-933, 141-166). */
int ht_forest_marginmap_f32(const ht_forest_problem *p, const float *x, const float *thr, const int64_t *ord,
                            float *margin, int64_t *margin_ord, void *workspace, size_t workspace_bytes,
                            uint32_t *status_word, ht_stream_t stream);

/* counts[j, leaf] = number of (i,k) positions reaching that leaf, int64 [T, L]; cleared here.
 * Replaces hingetree_gpu_reachability / ReachabilityKernel (hingetree_gpu.cu:732-789, 89-114). */
int ht_forest_reachability_f32(const ht_forest_problem *p, const float *x, const float *thr, const int64_t *ord,
                               int64_t *counts, void *workspace, size_t workspace_bytes, uint32_t *status_word,
                               ht_stream_t stream);

/* Gradients of the forward with respect to x, thr and w given g = d loss / d out [B,T,K,M]:
 *   gx  [i, ord[j,v*], k] += sign * w[j,leaf,m] * g[i,j,k,m]
 *   gthr[j, v*]           += -sign * w[j,leaf,m] * g[i,j,k,m]
 *   gw  [j, leaf, m]      += |margin| * g[i,j,k,m]
 * Any of gx / gthr / gw may be NULL (not requested); the others are cleared here first.
 * Without HT_DETERMINISTIC this replaces hingetree_gpu_backward and its three atomic kernels
 * (hingetree_gpu.cu:619-730, 212-253, 293-325, 370-410).  With HT_DETERMINISTIC it replaces
 * hingetree_gpu_backward_deterministic (hingetree_gpu.cu:500-617, 170-210, 257-291, 328-368):
 * every gradient element is then summed in exactly the order of the reference CPU loops
 * (hingetree.cpp:232-308: i, then j, then k, then m), so results are reproducible and equal
 * to the reference CPU build bit for bit. */
int ht_forest_backward_f32(const ht_forest_problem *p, const float *x, const float *thr, const int64_t *ord,
                           const float *w, const float *g, float *gx, float *gthr, float *gw,
                           void *workspace, size_t workspace_bytes, uint32_t *status_word, ht_stream_t stream);

/* ---- double precision ---------------------------------------------------------------------------
 * The plain forest operators for fp64 tensors, as the reference instantiates them (dispatch hingetree.cpp:666-689,
 * instantiations hingetree_gpu.cu:935-969): same contracts as their _f32 counterparts, every tensor double.  They
 * run the any-shape kernels (a thread per (sample, tree, position)); the shared-memory tile kernels are fp32 only.
 * Workspace: ht_forest_workspace_bytes(p) is enough (only the compact ordinals are kept there). */
int ht_forest_forward_f64(const ht_forest_problem *p, const double *x, const double *thr, const int64_t *ord,
                          const double *w, double *out, void *workspace, size_t workspace_bytes,
                          uint32_t *status_word, ht_stream_t stream);
int ht_forest_leafmap_f64(const ht_forest_problem *p, const double *x, const double *thr, const int64_t *ord,
                          int64_t *leaf, void *workspace, size_t workspace_bytes, uint32_t *status_word,
                          ht_stream_t stream);
int ht_forest_marginmap_f64(const ht_forest_problem *p, const double *x, const double *thr, const int64_t *ord,
                            double *margin, int64_t *margin_ord, void *workspace, size_t workspace_bytes,
                            uint32_t *status_word, ht_stream_t stream);
int ht_forest_reachability_f64(const ht_forest_problem *p, const double *x, const double *thr, const int64_t *ord,
                               int64_t *counts, void *workspace, size_t workspace_bytes, uint32_t *status_word,
                               ht_stream_t stream);
int ht_forest_backward_f64(const ht_forest_problem *p, const double *x, const double *thr, const int64_t *ord,
                           const double *w, const double *g, double *gx, double *gthr, double *gw,
                           void *workspace, size_t workspace_bytes, uint32_t *status_word, ht_stream_t stream);

/* ---- image + per-sample vector ("fusion") forests ------------------------------------------
 * Feature f of sample i at position k is img[i,f,k] for f < C (p->C = image channels) and
 * vec[i, f - C] otherwise, without materialising the concatenation; ordinals range over
 * [0, C + vec_channels).  Replaces hingetree_fusion_gpu_forward / _backward and their kernels
 * (hingetree_fusion_gpu.cu:352-558, 58-88, 135-177, 218-251, 304-346).  The vector gradient
 * sums over k.  gimg / gvec / gthr / gw may each be NULL; the others are cleared here. */
size_t ht_forest_fusion_workspace_bytes(const ht_forest_problem *p);
int ht_forest_fusion_forward_f32(const ht_forest_problem *p, const float *img, const float *vec, int64_t vec_channels,
                                 const float *thr, const int64_t *ord, const float *w, float *out, void *workspace,
                                 size_t workspace_bytes, uint32_t *status_word, ht_stream_t stream);
int ht_forest_fusion_backward_f32(const ht_forest_problem *p, const float *img, const float *vec, int64_t vec_channels,
                                  const float *thr, const int64_t *ord, const float *w, const float *g, float *gimg,
                                  float *gvec, float *gthr, float *gw, void *workspace, size_t workspace_bytes,
                                  uint32_t *status_word, ht_stream_t stream);

/* ---- forest followed by a linear layer over the tree dimension ("fused linear") -------------
 *   out[i,o,k,m] = bias[o] + sum_j lin[o,j] * |margin(i,j,k)| * w[j,leaf,m]        out [B,O,K,M]
 * lin is [O, T], bias [O].  With vec != NULL the features are the fusion ones above.
 * Replaces hingetree_fused_linear_gpu_forward / _backward and hingetree_fusion_fused_linear_gpu_*
 * (hingetree_fused_linear_gpu.cu:509-603, 605-703, 705-839, 841-982 and kernels 58-503).  The
 * forward adds the terms for j ascending, as the reference CPU loop does
 * (hingetree_fused_linear.cpp:154-181): it is deterministic and equal to that loop bit for bit.
 * The backward returns gimg, gvec, gthr, gw and glin (any may be NULL); the bias gradient is
 * the plain sum of g over every dimension but O and is left to the caller, as the reference
 * leaves it to Tensor::sum (hingetree_fused_linear_gpu.cu:828-836). */
size_t ht_forest_linear_workspace_bytes(const ht_forest_problem *p);
int ht_forest_linear_forward_f32(const ht_forest_problem *p, int64_t out_channels, const float *img, const float *vec,
                                 int64_t vec_channels, const float *thr, const int64_t *ord, const float *w,
                                 const float *lin, const float *bias, float *out, void *workspace,
                                 size_t workspace_bytes, uint32_t *status_word, ht_stream_t stream);
int ht_forest_linear_backward_f32(const ht_forest_problem *p, int64_t out_channels, const float *img, const float *vec,
                                  int64_t vec_channels, const float *thr, const int64_t *ord, const float *w,
                                  const float *lin, const float *g, float *gimg, float *gvec, float *gthr, float *gw,
                                  float *glin, void *workspace, size_t workspace_bytes, uint32_t *status_word,
                                  ht_stream_t stream);

/* ---- dense projection with batch-normalisation statistics, on the tensor cores -------------------
 *   z[M,N] = x[M,K] * w[N,K]^T        colsum[n] = sum_m z[m,n]        colsumsq[n] = sum_m z[m,n]^2
 * x, w, z row-major fp32; the products are taken in TF32 (tcgen05.mma.kind::tf32: the operands' upper 19 bits),
 * accumulated in fp32; z differs from an fp32 product by about 1e-3 relative to sum_k |x||w|.  colsum / colsumsq
 * [N] are cleared here.  K and N must be multiples of 4 and x, w, z 16-byte aligned (HT_ERR_UNSUPPORTED otherwise).
 * No workspace.  This is the front of the reference's sequential-initialisation pipeline, Linear ->
 * BatchNorm1d(affine=False) -> RandomHingeForest(init_type="sequential") (README.md:110-129,
 * RandomHingeForest/_RandomHingeForest.py:56-59), where the reference calls torch.nn.Linear and lets BatchNorm
 * read the activations again for its statistics; the reference has no operator of its own for it. */
int ht_linear_tf32_stats_f32(const float *x, const float *w, float *z, float *colsum, float *colsumsq, int64_t M,
                             int64_t N, int64_t K, uint32_t *status_word, ht_stream_t stream);

/* ---- hinge trie ---------------------------------------------------------------------------------
 *   out[i,j,k,m] = sum over depth d (ascending) of |margin_d| * w[j, vertex_d, m]
 * every decision on the path contributes; w is [T, 2^depth - 1, M], one row per internal vertex
 * (p->kind must be HT_KIND_TREE).  The reference implements tries on the CPU only
 * (hingetrie.cpp:33-267, traversal HingeTrieCommon.h:71-85; CUDA tensors get an empty result,
 * hingetrie.cpp:286-288); these entries evaluate the same arithmetic on the GPU, the forward in
 * the same order.  Workspace: ht_forest_workspace_bytes(p). */
int ht_trie_forward_f32(const ht_forest_problem *p, const float *x, const float *thr, const int64_t *ord, const float *w,
                        float *out, void *workspace, size_t workspace_bytes, uint32_t *status_word, ht_stream_t stream);
int ht_trie_backward_f32(const ht_forest_problem *p, const float *x, const float *thr, const int64_t *ord, const float *w,
                         const float *g, float *gx, float *gthr, float *gw, void *workspace, size_t workspace_bytes,
                         uint32_t *status_word, ht_stream_t stream);

/* ---- which gradient elements receive a contribution --------------------------------------------
 * Byte masks (1 = some (i,j,k) contributes) shaped like x, thr and w; any may be NULL; cleared
 * here.  Together with ht_forest_backward_f32 / ht_forest_linear_backward_f32 this replaces the
 * hash-table construction of sparse gradients in sparse_hingetree_gpu_backward and
 * sparse_hingetree_fused_linear_gpu_backward (hingetree_sparse_gpu.cu:461-764, IndexMap 61-101):
 * the binding compacts (mask, dense values) into a coalesced COO tensor.
 * Workspace: ht_forest_workspace_bytes(p). */
int ht_forest_touched_f32(const ht_forest_problem *p, const float *x, const float *thr, const int64_t *ord,
                          uint8_t *touched_x, uint8_t *touched_thr, uint8_t *touched_w, void *workspace,
                          size_t workspace_bytes, uint32_t *status_word, ht_stream_t stream);

/* ---- convolutional hinge trees / ferns, 1-D / 2-D / 3-D -------------------------------------
 *   out[i,j,p,m] = sum over input channels c (ascending) of |margin(i,c,j,p)| * w[j,c,leaf,m]
 * where tree (j,c) is evaluated on the kernel window of input channel c at output position p;
 * ordinals index the window cells in row-major kernel order, cells in the padding read 0, and
 * the output size per dimension is (size + 2*padding - (kernel + (kernel-1)*(dilation-1))) / stride + 1.
 *   x [B, Ci, size...]   thr, ord [Co, Ci, N]   w [Co, Ci, L, M]   out [B, Co, osize..., M]
 * Replaces hingetree_conv_gpu_forward / _backward with their per-(sample, channel) launches
 * (hingetree_conv_gpu.cu:214-618, kernels 64-210) and the im2col helpers they call
 * (ImageToMatrix_gpu.cu:132-239; geometry ImageToMatrix.h:189-221, 304-347).  One group only
 * (w.shape[1] == x.shape[1]), which is all the reference's modules ever build.  The forward adds the
 * input channels in ascending order and equals the reference CPU loop bit for bit; the
 * backward scatters with atomics.  A decision that looked at a padding cell has no data gradient. */
typedef struct ht_conv_problem {
  int32_t kind;   /* HT_KIND_TREE or HT_KIND_FERN */
  int32_t depth;  /* 1..31 */
  int32_t dims;   /* 1, 2 or 3 spatial dimensions */
  int32_t reserved;
  int64_t B, Ci, Co, M;
  int64_t size[3], kernel[3], stride[3], padding[3], dilation[3]; /* first `dims` entries are used */
} ht_conv_problem;

int ht_conv_output_size(const ht_conv_problem *p, int64_t *osize /* [dims] */);
size_t ht_conv_workspace_bytes(const ht_conv_problem *p);
int ht_conv_forward_f32(const ht_conv_problem *p, const float *x, const float *thr, const int64_t *ord, const float *w,
                        float *out, void *workspace, size_t workspace_bytes, uint32_t *status_word, ht_stream_t stream);
int ht_conv_backward_f32(const ht_conv_problem *p, const float *x, const float *thr, const int64_t *ord, const float *w,
                         const float *g, float *gx, float *gthr, float *gw, void *workspace, size_t workspace_bytes,
                         uint32_t *status_word, ht_stream_t stream);

/* ---- contract / expand -------------------------------------------------------------------------
 * contract: image [BC, size...] -> non-overlapping windows [BC, osize..., window...], zero padded,
 *           osize = (size + 2*padding - window) / window + 1 per dimension.
 * expand:   the inverse, image size = osize*window - (2*padding / window)*window; pixels no window
 *           reaches are 0.  dims is 2 or 3; elements are moved as opaque 1, 2, 4 or 8 byte words.
 * Replaces contract2d/3d_gpu and expand2d/3d_gpu (expand_gpu.cu:198-396, kernels 110-194). */
int ht_contract(int dims, int elem_bytes, const void *image, void *patches, int64_t batch_times_channels,
                const int64_t *size, const int64_t *window, const int64_t *padding, ht_stream_t stream);
int ht_expand(int dims, int elem_bytes, const void *patches, void *image, int64_t batch_times_channels,
              const int64_t *osize, const int64_t *window, const int64_t *padding, ht_stream_t stream);

/* ---- double precision forms of the other operator families -------------------------------------------
 * The reference instantiates every operator for float and double (hingetree.cpp:666-689 and the like in
 * hingetree_conv.cpp, hingetree_fused_linear.cpp, hingetree_fusion.cpp, hingetree_sparse.cpp, hingetrie.cpp).  Same
 * arguments and semantics as the _f32 entries above with double in place of float; the any-shape kernels are used
 * (the shared-memory tile kernels are single precision).  ht_forest_linear_workspace_bytes_f64 sizes the workspace of
 * the two linear entries; the other workspaces are those of the _f32 forms. */
size_t ht_forest_linear_workspace_bytes_f64(const ht_forest_problem *p);
int ht_forest_fusion_forward_f64(const ht_forest_problem *p, const double *img, const double *vec, int64_t vec_channels,
                                 const double *thr, const int64_t *ord, const double *w, double *out, void *workspace,
                                 size_t workspace_bytes, uint32_t *status_word, ht_stream_t stream);
int ht_forest_fusion_backward_f64(const ht_forest_problem *p, const double *img, const double *vec, int64_t vec_channels,
                                  const double *thr, const int64_t *ord, const double *w, const double *g, double *gimg,
                                  double *gvec, double *gthr, double *gw, void *workspace, size_t workspace_bytes,
                                  uint32_t *status_word, ht_stream_t stream);
int ht_forest_linear_forward_f64(const ht_forest_problem *p, int64_t out_channels, const double *img, const double *vec,
                                 int64_t vec_channels, const double *thr, const int64_t *ord, const double *w,
                                 const double *lin, const double *bias, double *out, void *workspace, size_t workspace_bytes,
                                 uint32_t *status_word, ht_stream_t stream);
int ht_forest_linear_backward_f64(const ht_forest_problem *p, int64_t out_channels, const double *img, const double *vec,
                                  int64_t vec_channels, const double *thr, const int64_t *ord, const double *w,
                                  const double *lin, const double *g, double *gimg, double *gvec, double *gthr, double *gw,
                                  double *glin, void *workspace, size_t workspace_bytes, uint32_t *status_word,
                                  ht_stream_t stream);
int ht_conv_forward_f64(const ht_conv_problem *p, const double *x, const double *thr, const int64_t *ord, const double *w,
                        double *out, void *workspace, size_t workspace_bytes, uint32_t *status_word, ht_stream_t stream);
int ht_conv_backward_f64(const ht_conv_problem *p, const double *x, const double *thr, const int64_t *ord, const double *w,
                         const double *g, double *gx, double *gthr, double *gw, void *workspace, size_t workspace_bytes,
                         uint32_t *status_word, ht_stream_t stream);
int ht_trie_forward_f64(const ht_forest_problem *p, const double *x, const double *thr, const int64_t *ord, const double *w,
                        double *out, void *workspace, size_t workspace_bytes, uint32_t *status_word, ht_stream_t stream);
int ht_trie_backward_f64(const ht_forest_problem *p, const double *x, const double *thr, const int64_t *ord, const double *w,
                         const double *g, double *gx, double *gthr, double *gw, void *workspace, size_t workspace_bytes,
                         uint32_t *status_word, ht_stream_t stream);
int ht_forest_touched_f64(const ht_forest_problem *p, const double *x, const double *thr, const int64_t *ord,
                          uint8_t *touched_x, uint8_t *touched_thr, uint8_t *touched_w, void *workspace,
                          size_t workspace_bytes, uint32_t *status_word, ht_stream_t stream);

/* ---- forest behind a batch normalisation that is not materialised ---------------------------------------
 * The reference's sequential-initialisation pipeline is torch.nn.Linear -> torch.nn.BatchNorm1d(affine=False) ->
 * RandomHingeForest (README.md:110-129).  These entries are the forest of that pipeline reading the RAW
 * activations z [B, C] (K = 1) with the per-column mean and 1/std: a visited feature is (z - mean) * invstd,
 * rounded as ATen's batch_norm_elemt rounds it, so the forward equals hingetree_gpu_forward (hingetree_gpu.cu:416)
 * on the materialised normalisation bit for bit.  No reference counterpart.
 * workspace: ht_forest_normalised_workspace_bytes(p) bytes. */
size_t ht_forest_normalised_workspace_bytes(const ht_forest_problem *p);
/* save_margin [B, T] floats and save_where [B, T] pairs of uint32 (both or neither): where the forward leaves the signed
 * margin and (deciding vertex, leaf key) of every evaluation for the backward below, which then does not walk again. */
int ht_forest_normalised_forward_f32(const ht_forest_problem *p, const float *z, const float *mean, const float *invstd,
                                     const float *thr, const int64_t *ord, const float *w, float *out, float *save_margin,
                                     void *save_where, void *workspace, size_t workspace_bytes, uint32_t *status_word,
                                     ht_stream_t stream);
/* Backward of the same: gthr [T, N] and gw [T, L, M] (either may be NULL) as ht_forest_backward_f32 gives them
 * (default mode: atomics), and the gradient with respect to the normalised activations y in the form it has —
 * one entry per (sample, tree): column[B, T] (the feature the deciding vertex tests) and value[B, T] — with the two
 * column sums the normalisation's backward needs: sum_g[c] = sum_i gy[i, c], sum_gy[c] = sum_i gy[i, c] * y[i, c]. */
int ht_forest_normalised_backward_f32(const ht_forest_problem *p, const float *z, const float *mean, const float *invstd,
                                      const float *thr, const int64_t *ord, const float *w, const float *g, float *gthr,
                                      float *gw, int32_t *column, float *value, float *sum_g, float *sum_gy,
                                      const float *saved_margin, const void *saved_where, void *workspace,
                                      size_t workspace_bytes, uint32_t *status_word, ht_stream_t stream);
/* mean[c] = sum[c] / rows, var[c] = max(sumsq[c] / rows - mean[c]^2, 0) (the biased variance batch normalisation
 * normalises with), invstd[c] = 1 / sqrt(var[c] + eps): the step between ht_linear_tf32_stats_f32 and the entries above,
 * as one launch. */
int ht_batchnorm_statistics_f32(const float *sum, const float *sumsq, int64_t rows, int64_t C, float eps, float *mean,
                                float *var, float *invstd, ht_stream_t stream);
/* Gradient with respect to z of y = (z - mean) * invstd with batch statistics (training mode, no affine part):
 * dz[i, c] = invstd[c] * (gy[i, c] - sum_g[c] / B - y[i, c] * sum_gy[c] / B), gy given by the records above: one pass
 * over z for the dense part, one over the records (the formula of torch's batch-norm backward,
 * aten/src/ATen/native/cuda/Normalization.cuh, batch_norm_backward_elemt). */
int ht_batchnorm_input_grad_f32(const float *z, const float *mean, const float *invstd, const float *sum_g, const float *sum_gy,
                                const int32_t *column, const float *value, float *dz, int64_t B, int64_t C, int64_t T,
                                ht_stream_t stream);

/* ---- threshold initialisation and hygiene on the device -------------------------------------------------
 * The reference runs these on the host only (tree_/fern_/trie_init_medians: hingetree.cpp:1519-1533,
 * MedianInit.h:133-257; tree_check_thresholds / tree_fix_thresholds: hingetree.cpp:936,1010,
 * HingeTreeCommon.h:244-287); here the data may stay in device memory.
 *
 * ht_init_medians_*: thr [T, N] <- for every vertex the median (rank floor(n / 2) from the largest) of feature
 * ord[t, v] over the samples of x [B, C, K] that reach it; samples with a larger value go to the right child; a
 * vertex no sample reaches keeps its threshold; ferns (kind HT_KIND_FERN, N = depth) see all samples at every
 * level; tries are trees.  Equal to the host operator bit for bit (except for the sign of a zero median when the
 * samples hold both zeros, which the host leaves to its partition order).  The ordinals must be in [0, C).
 * workspace: ht_init_medians_workspace_bytes(...) bytes (at most about 1 GiB: more trees go in several rounds). */
size_t ht_init_medians_workspace_bytes(int kind, int64_t B, int64_t K, int64_t T, int depth, int element_bytes);
int ht_init_medians_f32(int kind, const float *x, float *thr, const int64_t *ord, int64_t B, int64_t C, int64_t K, int64_t T,
                        int depth, void *workspace, size_t workspace_bytes, ht_stream_t stream);
int ht_init_medians_f64(int kind, const double *x, double *thr, const int64_t *ord, int64_t B, int64_t C, int64_t K, int64_t T,
                        int depth, void *workspace, size_t workspace_bytes, ht_stream_t stream);
/* ht_thresholds_*: trees only (thr, ord [T, 2^depth - 1]).  fix == 0: result[t] = 1 when no vertex of tree t has
 * a threshold outside the interval its same-feature ancestors leave reachable; fix != 0: such thresholds are moved
 * inside (parents first; to the middle of a bounded interval, 1 inside an unbounded one) and result[t] = 1 when
 * tree t was changed.  result: T bytes in device memory. */
int ht_thresholds_f32(int fix, float *thr, const int64_t *ord, int64_t T, int depth, unsigned char *result, ht_stream_t stream);
int ht_thresholds_f64(int fix, double *thr, const int64_t *ord, int64_t T, int depth, unsigned char *result, ht_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* HINGETREE_B200_H */
