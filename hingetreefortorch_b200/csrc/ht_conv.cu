// Convolutional hinge trees / ferns (1-D, 2-D, 3-D) and contract / expand.
//
// Output channel j sums, over the input channels c in ascending order, the value of the
// single-channel tree (j, c) evaluated on the kernel window of channel c at every output
// position.  The reference launches one im2col gather and one tree kernel per (sample, input
// channel) and materialises index and feature matrices (hingetree_conv_gpu.cu:368-380);
// here one launch covers the whole call: a thread owns one output position of one (sample,
// output channel), reads window cells straight from the image (padding cells read as 0) and
// walks the input channels itself, adding in the reference's order, so the forward is
// deterministic and equal to the reference CPU loop bit for bit.
#include "ht_common.cuh"
#include "ht_conv_tiled.cuh"

#include <algorithm>

namespace ht {

namespace {

constexpr int kBlock = 256;
constexpr int kMaxCells = 2048;  // window cells whose offsets are tabulated in shared memory

struct ConvShape {
  int64_t B, Ci, Co, M, N, L;
  int64_t in_count, out_count;
  int dims, depth, cells;
  int size[3], osize[3], kernel[3], stride[3], pad[3], dil[3];
};

template <typename Real>
struct ConvArgsOf : ConvShape {
  const Real *x;
  const Real *thr;
  const int32_t *ord;
  const Real *w;
};
using ConvArgs = ConvArgsOf<float>;

// Offsets (in elements along z, y, x; dilation applied) of every window cell, 10 bits each.
__device__ __forceinline__ void fill_cell_table(const ConvShape &a, uint32_t *table) {
  for (int q = threadIdx.x; q < a.cells; q += blockDim.x) {
    int rest = q;
    uint32_t packed = 0;
    for (int d = a.dims - 1; d >= 0; --d) {
      const int qd = rest % a.kernel[d];
      rest /= a.kernel[d];
      packed |= (uint32_t)(qd * a.dil[d]) << (10 * (a.dims - 1 - d));
    }
    table[q] = packed;
  }
}

// Image coordinates of the first window cell of output position p (may be negative: padding).
__device__ __forceinline__ void window_origin(const ConvShape &a, int64_t p, int (&origin)[3]) {
#pragma unroll
  for (int d = 2; d >= 0; --d) {
    if (d < a.dims) {
      const int od = (int)(p % a.osize[d]);
      p /= a.osize[d];
      origin[d] = od * a.stride[d] - a.pad[d];
    } else {
      origin[d] = 0;
    }
  }
}

// Flat index of window cell `packed` inside one channel image, or -1 when it lies in the padding.
__device__ __forceinline__ int cell_index(const ConvShape &a, const int (&origin)[3], uint32_t packed) {
  int index = 0;
  bool inside = true;
#pragma unroll
  for (int d = 0; d < 3; ++d) {
    if (d < a.dims) {
      const int at = origin[d] + (int)((packed >> (10 * (a.dims - 1 - d))) & 1023u);
      inside = inside && at >= 0 && at < a.size[d];
      index = index * a.size[d] + at;
    }
  }
  return inside ? index : -1;
}

template <typename Real>
struct WindowFeatureOf {
  typedef Real value_type;
  const ConvShape &a;
  const Real *chan;
  const int (&origin)[3];
  const uint32_t *table;
  __device__ __forceinline__ Real operator()(int q) const {
    const int idx = cell_index(a, origin, table[q]);
    return idx < 0 ? (Real)0 : __ldg(chan + idx);
  }
};

template <int KIND, typename Real>
__global__ void __launch_bounds__(kBlock) conv_forward_kernel(ConvArgsOf<Real> a, Real *__restrict__ out) {
  __shared__ uint32_t table[kMaxCells];
  fill_cell_table(a, table);
  __syncthreads();
  const int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;  // (i, j, p), p fastest
  if (e >= a.B * a.Co * a.out_count) return;
  const int64_t p = e % a.out_count;
  const int64_t j = (e / a.out_count) % a.Co;
  const int64_t i = e / (a.out_count * a.Co);
  int origin[3];
  window_origin(a, p, origin);
  Real *o = out + e * a.M;
  Real acc[8] = {};
  const bool in_registers = a.M <= 8;
  if (!in_registers)
    for (int64_t m = 0; m < a.M; ++m) o[m] = (Real)0;
  for (int64_t c = 0; c < a.Ci; ++c) {
    const int64_t tree = j * a.Ci + c;
    const WindowFeatureOf<Real> feat{a, a.x + (i * a.Ci + c) * a.in_count, origin, table};
    const PathOf<Real> path = traverse<KIND>(feat, a.thr + tree * a.N, a.ord + tree * a.N, a.depth);
    const Real am = abs_of(path.margin);
    const Real *wl = a.w + (tree * a.L + path.key) * a.M;
    if (in_registers) {
#pragma unroll
      for (int m = 0; m < 8; ++m)
        if (m < a.M) acc[m] = add_rn(acc[m], mul_rn(__ldg(wl + m), am));
    } else {
      for (int64_t m = 0; m < a.M; ++m) o[m] = add_rn(o[m], mul_rn(__ldg(wl + m), am));
    }
  }
  if (in_registers) {
#pragma unroll
    for (int m = 0; m < 8; ++m)
      if (m < a.M) o[m] = acc[m];
  }
}

// One thread per (i, j, p) walking the input channels; the three gradients are scattered with atomics.
template <int KIND, typename Real>
__global__ void __launch_bounds__(kBlock) conv_backward_kernel(ConvArgsOf<Real> a, const Real *__restrict__ g, Real *gx,
                                                               Real *gthr, Real *gw) {
  __shared__ uint32_t table[kMaxCells];
  fill_cell_table(a, table);
  __syncthreads();
  const int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= a.B * a.Co * a.out_count) return;
  const int64_t p = e % a.out_count;
  const int64_t j = (e / a.out_count) % a.Co;
  const int64_t i = e / (a.out_count * a.Co);
  int origin[3];
  window_origin(a, p, origin);
  const Real *gl = g + e * a.M;
  for (int64_t c = 0; c < a.Ci; ++c) {
    const int64_t tree = j * a.Ci + c;
    const WindowFeatureOf<Real> feat{a, a.x + (i * a.Ci + c) * a.in_count, origin, table};
    const PathOf<Real> path = traverse<KIND>(feat, a.thr + tree * a.N, a.ord + tree * a.N, a.depth);
    const Real s = sign_of(path.margin), am = abs_of(path.margin);
    const Real *wl = a.w + (tree * a.L + path.key) * a.M;
    Real acc = (Real)0;
    for (int64_t m = 0; m < a.M; ++m) {
      const Real gm = __ldg(gl + m);
      acc = add_rn(acc, mul_rn(mul_rn(s, __ldg(wl + m)), gm));
      if (gw != nullptr) atomicAdd(gw + (tree * a.L + path.key) * a.M + m, mul_rn(am, gm));
    }
    if (gx != nullptr) {
      const int idx = cell_index(a, origin, table[a.ord[tree * a.N + path.vertex]]);
      if (idx >= 0) atomicAdd(gx + (i * a.Ci + c) * a.in_count + idx, acc);  // a padding cell has no gradient
    }
    if (gthr != nullptr) atomicAdd(gthr + tree * a.N + path.vertex, -acc);
  }
}

// ---- contract / expand: non-overlapping windows <-> image, any element size ----------------

struct PatchArgs {
  int dims;
  int64_t BC, image_count, window_count, cells;
  int64_t size[3], osize[3], win[3], pad[3];
};

// One thread per patch element (b, window p, cell q): its image coordinate, or -1 outside.
__device__ __forceinline__ int64_t patch_image_index(const PatchArgs &a, int64_t p, int64_t q) {
  int64_t index = 0, scale = 1;
  for (int d = a.dims - 1; d >= 0; --d) {
    const int64_t at = (p % a.osize[d]) * a.win[d] - a.pad[d] + (q % a.win[d]);
    p /= a.osize[d];
    q /= a.win[d];
    if (at < 0 || at >= a.size[d]) return -1;
    index += at * scale;
    scale *= a.size[d];
  }
  return index;
}

template <typename Word>
__global__ void __launch_bounds__(kBlock) contract_kernel(PatchArgs a, const Word *__restrict__ image,
                                                          Word *__restrict__ patches) {
  const int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t per_image = a.window_count * a.cells;
  if (e >= a.BC * per_image) return;
  const int64_t b = e / per_image, r = e - b * per_image;
  const int64_t idx = patch_image_index(a, r / a.cells, r % a.cells);
  patches[e] = idx < 0 ? Word(0) : image[b * a.image_count + idx];
}

// One thread per image element: every pixel belongs to exactly one window cell (or to none, when
// the windows do not reach it), so expand is a gather as well and needs no clearing pass.
template <typename Word>
__global__ void __launch_bounds__(kBlock) expand_kernel(PatchArgs a, const Word *__restrict__ patches,
                                                        Word *__restrict__ image) {
  const int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= a.BC * a.image_count) return;
  const int64_t b = e / a.image_count;
  int64_t rest = e - b * a.image_count;
  int64_t p = 0, q = 0, pscale = 1, qscale = 1;
  bool covered = true;
  for (int d = a.dims - 1; d >= 0; --d) {
    const int64_t at = rest % a.size[d] + a.pad[d];
    rest /= a.size[d];
    const int64_t od = at / a.win[d];
    covered = covered && od < a.osize[d];
    p += od * pscale;
    q += (at % a.win[d]) * qscale;
    pscale *= a.osize[d];
    qscale *= a.win[d];
  }
  image[e] = covered ? patches[(b * a.window_count + p) * a.cells + q] : Word(0);
}

// The same two gathers with 32-bit index arithmetic and divisions by multiplication (every divisor is a
// launch constant), for images and patch sets of fewer than 2^31 elements each: the 64-bit division chains
// above cost several hundred instructions per element and kept these pure copies at an eighth of the
// memory bandwidth.  blockIdx.y walks the (batch x channel) images.
struct FastDivisor {
  uint32_t divisor, multiplier, shift;
  __device__ __forceinline__ uint32_t quotient(uint32_t n) const {  // n < 2^31
    return divisor == 1u ? n : __umulhi(n, multiplier) >> shift;
  }
  __device__ __forceinline__ void split(uint32_t n, uint32_t &q, uint32_t &r) const {  // q may be the variable n came from
    const uint32_t whole = quotient(n);
    r = n - whole * divisor;
    q = whole;
  }
};

inline FastDivisor make_divisor(int64_t d) {
  FastDivisor f;
  f.divisor = (uint32_t)d;
  f.multiplier = 0;
  f.shift = 0;
  if (d > 1) {
    uint32_t log2 = 0;
    while ((((uint64_t)1) << log2) < (uint64_t)d) ++log2;  // ceil(log2 d)
    const uint32_t p = 31 + log2;
    f.multiplier = (uint32_t)(((((uint64_t)1) << p) + (uint64_t)d - 1) / (uint64_t)d);
    f.shift = p - 32;
  }
  return f;
}

struct PatchArgs32 {
  int dims;
  uint32_t image_count, per_image;  // elements of one image, of one image's patches
  int64_t BC;
  FastDivisor cells, osize[3], win[3], size[3];
  uint32_t pad[3], window_count;
};

template <typename Word>
__global__ void __launch_bounds__(kBlock) contract32_kernel(PatchArgs32 a, const Word *__restrict__ image,
                                                            Word *__restrict__ patches) {
  const uint32_t r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= a.per_image) return;
  uint32_t p, q;
  a.cells.split(r, p, q);
  uint32_t index = 0, scale = 1;
  bool inside = true;
  for (int d = a.dims - 1; d >= 0; --d) {
    uint32_t pd, qd;
    a.osize[d].split(p, p, pd);
    a.win[d].split(q, q, qd);
    const uint32_t at = pd * a.win[d].divisor + qd - a.pad[d];  // wraps below zero: caught by the comparison
    inside = inside && at < a.size[d].divisor;
    index += at * scale;
    scale *= a.size[d].divisor;
  }
  // the same place in every image: the index arithmetic above is paid once per thread, four copies in flight
  const int64_t step = gridDim.y;
  int64_t b = blockIdx.y;
  for (; b + 3 * step < a.BC; b += 4 * step) {
    Word v[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) v[u] = inside ? image[(b + u * step) * a.image_count + index] : Word(0);
#pragma unroll
    for (int u = 0; u < 4; ++u) patches[(b + u * step) * a.per_image + r] = v[u];
  }
  for (; b < a.BC; b += step) patches[b * a.per_image + r] = inside ? image[b * a.image_count + index] : Word(0);
}

template <typename Word>
__global__ void __launch_bounds__(kBlock) expand32_kernel(PatchArgs32 a, const Word *__restrict__ patches,
                                                          Word *__restrict__ image) {
  const uint32_t e = blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= a.image_count) return;
  uint32_t rest = e, p = 0, q = 0, pscale = 1, qscale = 1;
  bool covered = true;
  for (int d = a.dims - 1; d >= 0; --d) {
    uint32_t at, od, cell;
    a.size[d].split(rest, rest, at);
    at += a.pad[d];
    a.win[d].split(at, od, cell);
    covered = covered && od < a.osize[d].divisor;
    p += od * pscale;
    q += cell * qscale;
    pscale *= a.osize[d].divisor;
    qscale *= a.win[d].divisor;
  }
  const uint32_t from = p * a.cells.divisor + q;
  const int64_t step = gridDim.y;
  int64_t b = blockIdx.y;
  for (; b + 3 * step < a.BC; b += 4 * step) {
    Word v[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) v[u] = covered ? patches[(b + u * step) * a.per_image + from] : Word(0);
#pragma unroll
    for (int u = 0; u < 4; ++u) image[(b + u * step) * a.image_count + e] = v[u];
  }
  for (; b < a.BC; b += step) image[b * a.image_count + e] = covered ? patches[b * a.per_image + from] : Word(0);
}

inline unsigned blocks_for(int64_t n) { return (unsigned)((n + kBlock - 1) / kBlock); }

int check_conv(const ht_conv_problem *p, ConvShape &a) {
  if (p == nullptr) return HT_ERR_INVALID_ARGUMENT;
  if (p->kind != TREE && p->kind != FERN) return HT_ERR_INVALID_ARGUMENT;
  if (p->depth < 1 || p->depth > 31) return HT_ERR_DEPTH;
  if (p->dims < 1 || p->dims > 3 || p->B < 0 || p->Ci < 1 || p->Co < 0 || p->M < 0) return HT_ERR_INVALID_ARGUMENT;
  a.dims = p->dims;
  a.depth = p->depth;
  a.B = p->B;
  a.Ci = p->Ci;
  a.Co = p->Co;
  a.M = p->M;
  a.N = threshold_count(p->kind, p->depth);
  a.L = ((int64_t)1) << p->depth;
  a.in_count = a.out_count = 1;
  int64_t cells = 1;
  for (int d = 0; d < 3; ++d) {
    a.size[d] = a.osize[d] = a.kernel[d] = a.stride[d] = a.dil[d] = 1;
    a.pad[d] = 0;
  }
  for (int d = 0; d < p->dims; ++d) {
    if (p->kernel[d] <= 0 || p->stride[d] <= 0 || p->padding[d] < 0 || p->dilation[d] <= 0 || p->size[d] < 1)
      return HT_ERR_INVALID_ARGUMENT;
    const int64_t window = p->kernel[d] + (p->kernel[d] - 1) * (p->dilation[d] - 1);
    if (p->size[d] + 2 * p->padding[d] < window) return HT_ERR_INVALID_ARGUMENT;
    if ((p->kernel[d] - 1) * p->dilation[d] >= 1024 || p->size[d] > 0x3fffffff) return HT_ERR_UNSUPPORTED;
    a.size[d] = (int)p->size[d];
    a.kernel[d] = (int)p->kernel[d];
    a.stride[d] = (int)p->stride[d];
    a.pad[d] = (int)p->padding[d];
    a.dil[d] = (int)p->dilation[d];
    a.osize[d] = (int)((p->size[d] + 2 * p->padding[d] - window) / p->stride[d] + 1);
    a.in_count *= p->size[d];
    a.out_count *= a.osize[d];
    cells *= p->kernel[d];
  }
  if (cells > kMaxCells || a.in_count > 0x7fffffff) return HT_ERR_UNSUPPORTED;
  a.cells = (int)cells;
  return HT_OK;
}

size_t conv_ordinal_bytes(const ConvShape &a) { return align_up((size_t)(a.Co * a.Ci * a.N) * sizeof(int32_t), 256); }

// The problem as the shared-memory tile kernels see it (1-D and 2-D, one output per leaf).
bool tile_problem(const ht_conv_problem *p, const ConvShape &a, ConvTileProblem &t) {
  if (p->dims > 2 || a.M != 1) return false;
  const int row = p->dims == 2 ? 0 : -1, col = p->dims - 1;  // a 1-D signal is one image row
  t.kind = p->kind;
  t.depth = p->depth;
  t.B = a.B;
  t.Ci = a.Ci;
  t.Co = a.Co;
  t.H = row < 0 ? 1 : a.size[row];
  t.W = a.size[col];
  t.Ho = row < 0 ? 1 : a.osize[row];
  t.Wo = a.osize[col];
  t.kh = row < 0 ? 1 : a.kernel[row];
  t.kw = a.kernel[col];
  t.sy = row < 0 ? 1 : a.stride[row];
  t.sx = a.stride[col];
  t.py = row < 0 ? 0 : a.pad[row];
  t.px = a.pad[col];
  t.dy = row < 0 ? 1 : a.dil[row];
  t.dx = a.dil[col];
  return true;
}

size_t conv_records_bytes(const ht_conv_problem *p, const ConvShape &a) {
  ConvTileProblem t;
  if (!tile_problem(p, a, t)) return 0;
  return std::max(conv_tiled_workspace_bytes(t), conv_backward_tiled_workspace_bytes(t));
}

template <typename Real>
int prepare_conv(const ht_conv_problem *p, const Real *x, const Real *thr, const int64_t *ord, const Real *w,
                 void *workspace, size_t workspace_bytes, uint32_t *status_word, cudaStream_t stream, ConvArgsOf<Real> &a) {
  const int rc = check_conv(p, a);
  if (rc != HT_OK) return rc;
  const int64_t decisions = a.Co * a.Ci * a.N;
  if ((x == nullptr && a.B * a.Ci * a.in_count > 0) || ((thr == nullptr || ord == nullptr) && decisions > 0) ||
      (w == nullptr && a.Co * a.M > 0))
    return HT_ERR_INVALID_ARGUMENT;
  if (workspace == nullptr || workspace_bytes < conv_ordinal_bytes(a) + 256 ||
      (reinterpret_cast<uintptr_t>(workspace) & 255u) != 0)
    return HT_ERR_WORKSPACE;
  a.x = x;
  a.thr = thr;
  a.w = w;
  a.ord = static_cast<const int32_t *>(workspace);
  return pack_ordinals(ord, decisions, a.cells, static_cast<int32_t *>(workspace), status_word, stream);
}

template <typename Word>
int launch_patches(bool contract, const PatchArgs &a, const void *in, void *out, cudaStream_t stream) {
  const int64_t per_image = a.window_count * a.cells;
  bool narrow = a.image_count < 0x40000000 && per_image < 0x40000000 && a.BC > 0;
  for (int d = 0; d < a.dims; ++d) narrow = narrow && a.pad[d] < 0x40000000 && a.size[d] + a.pad[d] < 0x40000000;
  if (narrow) {
    PatchArgs32 n;
    n.dims = a.dims;
    n.image_count = (uint32_t)a.image_count;
    n.per_image = (uint32_t)per_image;
    n.window_count = (uint32_t)a.window_count;
    n.BC = a.BC;
    n.cells = make_divisor(a.cells);
    for (int d = 0; d < 3; ++d) {
      n.osize[d] = make_divisor(d < a.dims ? a.osize[d] : 1);
      n.win[d] = make_divisor(d < a.dims ? a.win[d] : 1);
      n.size[d] = make_divisor(d < a.dims ? a.size[d] : 1);
      n.pad[d] = d < a.dims ? (uint32_t)a.pad[d] : 0u;
    }
    // enough blocks to fill the machine several times over, and as many images per thread as that leaves
    const unsigned across = blocks_for(contract ? per_image : a.image_count);
    const int64_t wanted = std::max<int64_t>(1, (148 * 32 + across - 1) / across);
    const dim3 grid(across, (unsigned)std::min<int64_t>(std::min<int64_t>(a.BC, wanted), 65535));
    if (contract)
      contract32_kernel<Word><<<grid, kBlock, 0, stream>>>(n, static_cast<const Word *>(in), static_cast<Word *>(out));
    else
      expand32_kernel<Word><<<grid, kBlock, 0, stream>>>(n, static_cast<const Word *>(in), static_cast<Word *>(out));
    HT_CHECK_LAUNCH();
    return HT_OK;
  }
  if (contract) {
    const int64_t n = a.BC * a.window_count * a.cells;
    if (n > 0) contract_kernel<Word><<<blocks_for(n), kBlock, 0, stream>>>(a, static_cast<const Word *>(in), static_cast<Word *>(out));
  } else {
    const int64_t n = a.BC * a.image_count;
    if (n > 0) expand_kernel<Word><<<blocks_for(n), kBlock, 0, stream>>>(a, static_cast<const Word *>(in), static_cast<Word *>(out));
  }
  HT_CHECK_LAUNCH();
  return HT_OK;
}

int run_patches(bool contract, int dims, int elem_bytes, const void *in, void *out, int64_t BC, const int64_t *size,
                const int64_t *osize, const int64_t *window, const int64_t *padding, cudaStream_t stream) {
  if (dims < 2 || dims > 3 || BC < 0 || size == nullptr || osize == nullptr || window == nullptr || padding == nullptr)
    return HT_ERR_INVALID_ARGUMENT;
  PatchArgs a;
  a.dims = dims;
  a.BC = BC;
  a.image_count = a.window_count = a.cells = 1;
  for (int d = 0; d < dims; ++d) {
    if (size[d] < 1 || osize[d] < 1 || window[d] < 1 || padding[d] < 0) return HT_ERR_INVALID_ARGUMENT;
    a.size[d] = size[d];
    a.osize[d] = osize[d];
    a.win[d] = window[d];
    a.pad[d] = padding[d];
    a.image_count *= size[d];
    a.window_count *= osize[d];
    a.cells *= window[d];
  }
  if ((in == nullptr || out == nullptr) && BC > 0) return HT_ERR_INVALID_ARGUMENT;
  switch (elem_bytes) {
    case 1: return launch_patches<uint8_t>(contract, a, in, out, stream);
    case 2: return launch_patches<uint16_t>(contract, a, in, out, stream);
    case 4: return launch_patches<uint32_t>(contract, a, in, out, stream);
    case 8: return launch_patches<uint64_t>(contract, a, in, out, stream);
    default: return HT_ERR_UNSUPPORTED;
  }
}

// Forward / backward for either precision; the shared-memory tile kernels are single precision only.
template <typename Real>
int conv_forward(const ht_conv_problem *p, const Real *x, const Real *thr, const int64_t *ord, const Real *w, Real *out,
                 void *workspace, size_t workspace_bytes, uint32_t *status_word, ht_stream_t stream) {
  ConvArgsOf<Real> a;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const int rc = prepare_conv<Real>(p, x, thr, ord, w, workspace, workspace_bytes, status_word, s, a);
  if (rc != HT_OK) return rc;
  const int64_t threads = a.B * a.Co * a.out_count;
  if (threads * a.M == 0) return HT_OK;
  if (out == nullptr) return HT_ERR_INVALID_ARGUMENT;
  if constexpr (std::is_same<Real, float>::value) {
    ConvTileProblem t;
    if (tile_problem(p, a, t)) {
      const size_t records = conv_tiled_workspace_bytes(t);
      if (records != 0 && workspace_bytes >= conv_ordinal_bytes(a) + records + 256) {
        const int tiled = conv_forward_tiled(t, x, thr, a.ord, w, out,
                                             static_cast<unsigned char *>(workspace) + conv_ordinal_bytes(a), status_word, s);
        if (tiled != HT_ERR_UNSUPPORTED) return tiled;
      }
    }
  }
  if (p->kind == TREE)
    conv_forward_kernel<TREE, Real><<<blocks_for(threads), kBlock, 0, s>>>(a, out);
  else
    conv_forward_kernel<FERN, Real><<<blocks_for(threads), kBlock, 0, s>>>(a, out);
  HT_CHECK_LAUNCH();
  return HT_OK;
}

template <typename Real>
int conv_backward(const ht_conv_problem *p, const Real *x, const Real *thr, const int64_t *ord, const Real *w, const Real *g,
                  Real *gx, Real *gthr, Real *gw, void *workspace, size_t workspace_bytes, uint32_t *status_word,
                  ht_stream_t stream) {
  ConvArgsOf<Real> a;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const int rc = prepare_conv<Real>(p, x, thr, ord, w, workspace, workspace_bytes, status_word, s, a);
  if (rc != HT_OK) return rc;
  if (gx != nullptr && a.B * a.Ci * a.in_count > 0)
    HT_CUDA_TRY(cudaMemsetAsync(gx, 0, sizeof(Real) * (size_t)(a.B * a.Ci * a.in_count), s));
  if (gthr != nullptr && a.Co * a.Ci * a.N > 0)
    HT_CUDA_TRY(cudaMemsetAsync(gthr, 0, sizeof(Real) * (size_t)(a.Co * a.Ci * a.N), s));
  if (gw != nullptr && a.Co * a.Ci * a.L * a.M > 0)
    HT_CUDA_TRY(cudaMemsetAsync(gw, 0, sizeof(Real) * (size_t)(a.Co * a.Ci * a.L * a.M), s));
  const int64_t threads = a.B * a.Co * a.out_count;
  if (threads * a.M == 0 || (gx == nullptr && gthr == nullptr && gw == nullptr)) return HT_OK;
  if (g == nullptr) return HT_ERR_INVALID_ARGUMENT;
  if constexpr (std::is_same<Real, float>::value) {
    ConvTileProblem t;
    if (tile_problem(p, a, t)) {
      const size_t records = conv_backward_tiled_workspace_bytes(t);
      if (records != 0 && workspace_bytes >= conv_ordinal_bytes(a) + records + 256) {
        const int tiled = conv_backward_tiled(t, x, thr, a.ord, w, g, gx, gthr, gw,
                                              static_cast<unsigned char *>(workspace) + conv_ordinal_bytes(a), status_word, s);
        if (tiled != HT_ERR_UNSUPPORTED) return tiled;
      }
    }
  }
  if (p->kind == TREE)
    conv_backward_kernel<TREE, Real><<<blocks_for(threads), kBlock, 0, s>>>(a, g, gx, gthr, gw);
  else
    conv_backward_kernel<FERN, Real><<<blocks_for(threads), kBlock, 0, s>>>(a, g, gx, gthr, gw);
  HT_CHECK_LAUNCH();
  return HT_OK;
}

}  // namespace
}  // namespace ht

using namespace ht;

extern "C" {

int ht_conv_output_size(const ht_conv_problem *p, int64_t *osize) {
  ConvArgs a;
  const int rc = check_conv(p, a);
  if (rc != HT_OK) return rc;
  if (osize == nullptr) return HT_ERR_INVALID_ARGUMENT;
  for (int d = 0; d < p->dims; ++d) osize[d] = a.osize[d];
  return HT_OK;
}

size_t ht_conv_workspace_bytes(const ht_conv_problem *p) {
  ConvArgs a;
  if (check_conv(p, a) != HT_OK) return 0;
  return conv_ordinal_bytes(a) + conv_records_bytes(p, a) + 256;
}

int ht_conv_forward_f32(const ht_conv_problem *p, const float *x, const float *thr, const int64_t *ord, const float *w,
                        float *out, void *workspace, size_t workspace_bytes, uint32_t *status_word, ht_stream_t stream) {
  return conv_forward<float>(p, x, thr, ord, w, out, workspace, workspace_bytes, status_word, stream);
}
int ht_conv_forward_f64(const ht_conv_problem *p, const double *x, const double *thr, const int64_t *ord, const double *w,
                        double *out, void *workspace, size_t workspace_bytes, uint32_t *status_word, ht_stream_t stream) {
  return conv_forward<double>(p, x, thr, ord, w, out, workspace, workspace_bytes, status_word, stream);
}

int ht_conv_backward_f32(const ht_conv_problem *p, const float *x, const float *thr, const int64_t *ord, const float *w,
                         const float *g, float *gx, float *gthr, float *gw, void *workspace, size_t workspace_bytes,
                         uint32_t *status_word, ht_stream_t stream) {
  return conv_backward<float>(p, x, thr, ord, w, g, gx, gthr, gw, workspace, workspace_bytes, status_word, stream);
}
int ht_conv_backward_f64(const ht_conv_problem *p, const double *x, const double *thr, const int64_t *ord, const double *w,
                         const double *g, double *gx, double *gthr, double *gw, void *workspace, size_t workspace_bytes,
                         uint32_t *status_word, ht_stream_t stream) {
  return conv_backward<double>(p, x, thr, ord, w, g, gx, gthr, gw, workspace, workspace_bytes, status_word, stream);
}

int ht_contract(int dims, int elem_bytes, const void *image, void *patches, int64_t batch_times_channels,
                const int64_t *size, const int64_t *window, const int64_t *padding, ht_stream_t stream) {
  if (dims < 2 || dims > 3 || size == nullptr || window == nullptr || padding == nullptr) return HT_ERR_INVALID_ARGUMENT;
  int64_t osize[3];
  for (int d = 0; d < dims; ++d) {
    if (window[d] < 1 || padding[d] < 0 || window[d] > size[d] + 2 * padding[d]) return HT_ERR_INVALID_ARGUMENT;
    osize[d] = (size[d] + 2 * padding[d] - window[d]) / window[d] + 1;
  }
  return run_patches(true, dims, elem_bytes, image, patches, batch_times_channels, size, osize, window, padding,
                     reinterpret_cast<cudaStream_t>(stream));
}

int ht_expand(int dims, int elem_bytes, const void *patches, void *image, int64_t batch_times_channels,
              const int64_t *osize, const int64_t *window, const int64_t *padding, ht_stream_t stream) {
  if (dims < 2 || dims > 3 || osize == nullptr || window == nullptr || padding == nullptr) return HT_ERR_INVALID_ARGUMENT;
  int64_t size[3];
  for (int d = 0; d < dims; ++d) {
    if (window[d] < 1 || padding[d] < 0 || osize[d] < 1) return HT_ERR_INVALID_ARGUMENT;
    size[d] = osize[d] * window[d] - ((2 * padding[d]) / window[d]) * window[d];
    if (size[d] < 1) return HT_ERR_INVALID_ARGUMENT;
  }
  return run_patches(false, dims, elem_bytes, patches, image, batch_times_channels, size, osize, window, padding,
                     reinterpret_cast<cudaStream_t>(stream));
}

}  // extern "C"
