// Shared-memory tile kernel for the forward of 1-D / 2-D convolutional hinge trees and ferns
// (one output per leaf).
//
// out[b, j, p] = sum over input channels c (ascending) of tree (j, c) evaluated on the kernel
// window of channel c at output position p.  Work decomposition (one CTA of 1024 threads per SM):
//   * a CTA owns a tile of TY x 32 output positions of one sample and stages, once, the image
//     patch under that tile for EVERY input channel (zero where the window hangs over the image
//     border), so a window cell is a fixed offset from the position's window origin and the 32
//     lanes of a warp (32 consecutive positions of one row) read 32 consecutive banks;
//   * a warp is (tile row, slot): it keeps 4 output channels in flight and, for each, walks the
//     trees (j, 0), (j, 1), ... adding their values in that order in a register, so the sum has the
//     reference's order and the result leaves once, as full 128-byte row segments;
//   * tree records (the forest tile kernel's format, with window cells already turned into patch
//     offsets by the repack kernel) stream through two shared-memory buffers in groups of
//     {4 * slots output channels} x {CC input channels}, one bulk async copy per output channel
//     completing on the group's mbarrier; the last warp to finish a buffer refills it.
// The reference gathers an im2col matrix per (sample, input channel) and runs one tree kernel on
// it, 2 * B * Ci launches per call (hingetree_conv_gpu.cu:368-380).
#include "ht_conv_tiled.cuh"
#include "ht_tile_common.cuh"

#include <algorithm>

namespace ht {

using namespace tile;
using namespace conv_tile;

namespace {

struct ConvTilePlan {
  int TY;              // tile rows; slots = kWarps / TY
  int CC;              // input channels per parameter group
  int patch_h, patch_w;
  int ord_bytes;
  RecordLayout rec;
  size_t smem;
};

bool make_plan(const ConvTileProblem &p, ConvTilePlan &plan) {
  if (p.depth > 10 || p.Ci < 1 || p.Co < 1 || p.B < 1 || p.Ho < 1 || p.Wo < 1) return false;
  if ((double)p.B * p.Ho * p.Wo * (double)p.Co * p.Ci < 1048576.0) return false;  // not worth a 1024-thread CTA
  for (int TY = 8; TY >= 1; TY >>= 1) {
    if (TY > 1 && TY / 2 >= p.Ho) continue;  // no taller than the output needs
    plan.TY = TY;
    const PatchShape shape = patch_shape(p, TY);
    plan.patch_h = shape.h;
    plan.patch_w = shape.w;
    if (shape.far > 65535) continue;
    plan.ord_bytes = shape.far <= 255 ? 1 : 2;
    plan.rec = record_layout(p.kind, p.depth, (uint32_t)plan.ord_bytes, true,
                             paired_ordinals(p.kind, p.depth, (uint32_t)plan.ord_bytes));
    const size_t patches = (size_t)p.Ci * plan.patch_h * plan.patch_w * 4;
    const int JB = (kWarps / TY) * 4;
    for (int CC = 16; CC >= 1; CC >>= 1) {
      if (CC > 1 && CC / 2 >= p.Ci) continue;
      plan.CC = CC;
      plan.smem = align_up(patches, 128) + 2 * (size_t)JB * CC * plan.rec.bytes + 64;
      if (plan.smem <= kSmemBudget && (size_t)JB * CC * plan.rec.bytes < (1u << 20)) return true;
    }
  }
  return false;
}

struct ConvTileArgs {
  const float *x;
  const unsigned char *records;
  float *out;
  uint32_t *status_word;
  int Ci, Co, H, W, Ho, Wo, sy, sx, py, px;
  int TY, CC, patch_h, patch_w, tiles_x, tiles_y;
};

template <int KIND, int DEPTH, typename OrdT>
__global__ void __launch_bounds__(kThreads, 1) conv_forward_tiled_kernel(ConvTileArgs a) {
  extern __shared__ __align__(128) unsigned char smem[];
  constexpr RecordLayout lay =
      record_layout(KIND, DEPTH, (uint32_t)sizeof(OrdT), true, paired_ordinals(KIND, DEPTH, (uint32_t)sizeof(OrdT)));
  const int TY = a.TY, CC = a.CC;
  const int slots = kWarps / TY;
  const int JB = slots * 4;  // output channels per parameter group
  const int patch_elems = a.patch_h * a.patch_w;
  const size_t patch_bytes_all = ((size_t)a.Ci * patch_elems * 4 + 127) & ~(size_t)127;
  float *patches = reinterpret_cast<float *>(smem);
  unsigned char *params = smem + patch_bytes_all;
  const uint32_t buffer_bytes = (uint32_t)JB * (uint32_t)CC * lay.bytes;
  uint64_t *full = reinterpret_cast<uint64_t *>(params + 2 * (size_t)buffer_bytes);
  uint32_t *finished = reinterpret_cast<uint32_t *>(full + 2);

  const int tid = threadIdx.x;
  const int lane = tid & 31, warp = tid >> 5;
  const int tile_row = warp % TY;
  const int slot = warp / TY;
  const int tiles = a.tiles_x * a.tiles_y;
  const int64_t b = blockIdx.x / tiles;
  const int tile = (int)(blockIdx.x - b * tiles);
  const int oy0 = (tile / a.tiles_x) * TY, ox0 = (tile % a.tiles_x) * kTileColumns;

  // blockIdx.y splits the blocks of output channels among CTAs when one sample tile per CTA would
  // leave SMs idle; `it` counts this CTA's groups: (block of output channels) x (chunk of input channels)
  const int c_chunks = (a.Ci + CC - 1) / CC;
  const int all_blocks = (a.Co + JB - 1) / JB;
  const int blocks_per_cta = (all_blocks + (int)gridDim.y - 1) / (int)gridDim.y;
  const int block0 = (int)blockIdx.y * blocks_per_cta;
  const int num_groups = max(0, min(blocks_per_cta, all_blocks - block0)) * c_chunks;
  const uint32_t params_addr = smem_addr(params);

  auto issue = [&](int it) {
    const int j_first = (block0 + it / c_chunks) * JB;
    const int c_first = (it % c_chunks) * CC;
    const int count_j = min(JB, a.Co - j_first), count_c = min(CC, a.Ci - c_first);
    const uint32_t each = (uint32_t)count_c * lay.bytes;
    uint64_t *bar = &full[it & 1];
    mbar_expect_tx(bar, (uint32_t)count_j * each);
    const uint32_t dst = params_addr + (uint32_t)(it & 1) * buffer_bytes;
    for (int jl = 0; jl < count_j; ++jl)
      bulk_load(dst + (uint32_t)jl * (uint32_t)CC * lay.bytes,
                a.records + ((int64_t)(j_first + jl) * a.Ci + c_first) * lay.bytes, each, bar);
  };
  if (tid == 0) {
    mbar_init(&full[0], 1);
    mbar_init(&full[1], 1);
    finished[0] = 0;
    finished[1] = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    if (num_groups > 0) issue(0);
    if (num_groups > 1) issue(1);
  }

  stage_patches(patches, a.x + b * a.Ci * (int64_t)a.H * a.W, a.Ci, a.H, a.W, oy0 * a.sy - a.py, ox0 * a.sx - a.px,
                a.patch_h, a.patch_w);
  __syncthreads();  // patches staged; barrier initialisation visible

  // this lane's window origin inside a patch; a window cell is origin + the offset held in the record
  const uint32_t origin_addr = smem_addr(patches) + (uint32_t)((tile_row * a.sy) * a.patch_w + lane * a.sx) * 4u;
  const uint32_t patch_bytes = (uint32_t)patch_elems * 4u;
  const int oy = oy0 + tile_row, ox = ox0 + lane;
  const bool position_valid = oy < a.Ho && ox < a.Wo;
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  bool poisoned = false;  // a bounded wait ran out: keep the counters matched, stop waiting

  for (int it = 0; it < num_groups; ++it) {
    const int j_first = (block0 + it / c_chunks) * JB;
    const int chunk = it % c_chunks;
    const int c_first = chunk * CC;
    const int count_j = min(JB, a.Co - j_first), count_c = min(CC, a.Ci - c_first);
    if (!poisoned && !mbar_wait(&full[it & 1], (uint32_t)((it >> 1) & 1))) {
      poisoned = true;
      if (a.status_word != nullptr) atomicOr(a.status_word, HT_FLAG_PIPELINE_TIMEOUT);
    }
    if (chunk == 0) {
#pragma unroll
      for (int u = 0; u < 4; ++u) acc[u] = 0.0f;
    }
    const int j_local = slot * 4;
    if (j_local < count_j && !poisoned) {
      const uint32_t base_addr = params_addr + (uint32_t)(it & 1) * buffer_bytes;
      uint32_t rec[4];
#pragma unroll
      for (int u = 0; u < 4; ++u)  // channels beyond the last repeat it (results unused)
        rec[u] = base_addr + (uint32_t)min(j_local + u, count_j - 1) * (uint32_t)CC * lay.bytes;
      uint32_t x_addr = origin_addr + (uint32_t)c_first * patch_bytes;
      for (int ci = 0; ci < count_c; ++ci) {
        float value[4];
        uint32_t path[4];
        walk<KIND, DEPTH, OrdT, 4, true>(rec, x_addr, 4u, value, path);
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          acc[u] = __fadd_rn(acc[u], value[u]);
          rec[u] += lay.bytes;
        }
        x_addr += patch_bytes;
      }
    }
    __syncwarp();
    if (lane == 0) {
      __threadfence_block();
      const uint32_t before = atomicAdd(&finished[it & 1], 1u);
      if (before == kWarps - 1) {
        atomicExch(&finished[it & 1], 0u);
        __threadfence_block();
        if (it + 2 < num_groups) issue(it + 2);
      }
    }
    if (chunk == c_chunks - 1 && position_valid) {
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int j = j_first + j_local + u;
        if (j_local + u < count_j) a.out[((b * a.Co + j) * a.Ho + oy) * (int64_t)a.Wo + ox] = acc[u];
      }
    }
  }
}

template <typename Kernel>
int launch_one(Kernel kernel, const ConvTilePlan &plan, const ConvTileArgs &a, dim3 grid, cudaStream_t stream) {
  HT_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBudget));
  kernel<<<grid, kThreads, plan.smem, stream>>>(a);
  HT_CHECK_LAUNCH();
  return HT_OK;
}

template <int KIND, int DEPTH>
int launch_depth(const ConvTilePlan &plan, const ConvTileArgs &a, dim3 grid, cudaStream_t stream) {
  if (plan.ord_bytes == 1) return launch_one(conv_forward_tiled_kernel<KIND, DEPTH, uint8_t>, plan, a, grid, stream);
  return launch_one(conv_forward_tiled_kernel<KIND, DEPTH, uint16_t>, plan, a, grid, stream);
}

template <int KIND>
int launch_kind(int depth, const ConvTilePlan &plan, const ConvTileArgs &a, dim3 grid, cudaStream_t stream) {
  switch (depth) {
#define HT_DEPTH_CASE(D) \
  case D:                \
    return launch_depth<KIND, D>(plan, a, grid, stream);
    HT_DEPTH_CASE(1)
    HT_DEPTH_CASE(2)
    HT_DEPTH_CASE(3)
    HT_DEPTH_CASE(4)
    HT_DEPTH_CASE(5)
    HT_DEPTH_CASE(6)
    HT_DEPTH_CASE(7)
    HT_DEPTH_CASE(8)
    HT_DEPTH_CASE(9)
    HT_DEPTH_CASE(10)
#undef HT_DEPTH_CASE
    default:
      return HT_ERR_UNSUPPORTED;
  }
}

}  // namespace

size_t conv_tiled_workspace_bytes(const ConvTileProblem &p) {
  ConvTilePlan plan;
  if (!make_plan(p, plan)) return 0;
  return align_up((size_t)(p.Co * p.Ci) * plan.rec.bytes, 256);
}

int conv_forward_tiled(const ConvTileProblem &p, const float *x, const float *thr, const int32_t *ord, const float *w,
                       float *out, void *records, uint32_t *status_word, cudaStream_t stream) {
  ConvTilePlan plan;
  if (!make_plan(p, plan)) return HT_ERR_UNSUPPORTED;
  const int tiles_x = (p.Wo + kTileColumns - 1) / kTileColumns, tiles_y = (p.Ho + plan.TY - 1) / plan.TY;
  const int64_t ctas = p.B * tiles_x * tiles_y;
  if (ctas > 0x7fffffff) return HT_ERR_UNSUPPORTED;

  const int64_t trees = p.Co * p.Ci;
  const int64_t N = threshold_count(p.kind, p.depth);
  const int64_t L = ((int64_t)1) << p.depth;
  const unsigned pack_grid = (unsigned)((trees * (N + L) + 255) / 256);
  unsigned char *rec = static_cast<unsigned char *>(records);
  RecordMap map;
  map.columns = p.kw;
  map.row_step = p.dy * plan.patch_w;
  map.column_step = p.dx;
  if (plan.ord_bytes == 1)
    repack_records_kernel<uint8_t><<<pack_grid, 256, 0, stream>>>(thr, ord, w, rec, p.kind, p.depth, trees, plan.rec, map);
  else
    repack_records_kernel<uint16_t><<<pack_grid, 256, 0, stream>>>(thr, ord, w, rec, p.kind, p.depth, trees, plan.rec, map);
  HT_CHECK_LAUNCH();

  ConvTileArgs a;
  a.x = x;
  a.records = rec;
  a.out = out;
  a.status_word = status_word;
  a.Ci = (int)p.Ci;
  a.Co = (int)p.Co;
  a.H = p.H;
  a.W = p.W;
  a.Ho = p.Ho;
  a.Wo = p.Wo;
  a.sy = p.sy;
  a.sx = p.sx;
  a.py = p.py;
  a.px = p.px;
  a.TY = plan.TY;
  a.CC = plan.CC;
  a.patch_h = plan.patch_h;
  a.patch_w = plan.patch_w;
  a.tiles_x = tiles_x;
  a.tiles_y = tiles_y;
  // few sample tiles: share the blocks of output channels between CTAs (each re-stages the patches)
  const int JB = (kWarps / plan.TY) * 4;
  const int64_t blocks = (p.Co + JB - 1) / JB;
  int64_t splits = 1;
  if (ctas < 2 * 148) splits = std::min<int64_t>(blocks, (2 * 148 + ctas - 1) / ctas);
  const dim3 grid((unsigned)ctas, (unsigned)std::max<int64_t>(splits, 1));
  return p.kind == TREE ? launch_kind<TREE>(p.depth, plan, a, grid, stream)
                        : launch_kind<FERN>(p.depth, plan, a, grid, stream);
}

}  // namespace ht
