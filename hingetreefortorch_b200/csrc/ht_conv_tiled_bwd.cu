// Shared-memory tile kernel for the backward of 1-D / 2-D convolutional hinge trees and ferns
// (one output per leaf).
//
// Same tile as the forward (ht_conv_tiled.cu): a CTA owns TY x 32 output positions of one sample and
// keeps the image patches of all input channels in shared memory.  The loop order is turned round:
// a warp is (tile row, slot) and the slot's warps work on ONE input channel c at a time, walking the
// trees (0, c), (1, c), ... four at a time, so that
//   * the image gradient is collected without atomics in a warp-private array [window cell][lane]
//     (a lane owns its column, whatever cell its tree decided on) over all output channels, and
//     leaves once per (input channel, tile row) as one global reduction per touched pixel;
//   * the threshold and leaf-weight gradients of the trees in flight are collected in shared-memory
//     bins shared by the slot's warps (TY x 32 positions per tree) and leave as one global
//     reduction per touched bin — 1/8 or less of the per-evaluation global atomics of the
//     thread-per-output kernel.
// Tree records are repacked in (input channel, output channel) order so that a slot's stream is
// contiguous; they arrive by bulk async copies on mbarriers, double buffered, like the forward's.
// One traversal serves all three gradients (the reference runs three kernels per (sample, input
// channel), each repeating it, hingetree_conv_gpu.cu:545-606).
//
// For trees of depth <= 7 the shared bins are the slow part (a few bins collect most terms, and a
// float atomic on shared memory is a compare-and-swap loop), so there the parameter gradients come
// from a second kernel further down (one tree per warp, bin columns owned by lanes) and this
// kernel is launched for the image gradient only.  A fused form of the two with 16 warps per CTA
// (both kinds of lane-owned arrays need the shared memory of a whole SM) was measured slower than
// the pair: half the warps hide too little of the traversal's latency.
#include "ht_conv_tiled.cuh"
#include "ht_tile_common.cuh"

#include <algorithm>

namespace ht {

using namespace tile;
using namespace conv_tile;

namespace {

// ---- records with one 8-byte entry per vertex --------------------------------------------------------
//
// The backward's traversal needs the threshold and the patch offset of every vertex it visits, from addresses
// that differ from lane to lane.  In this form of the record vertex v (1-based; ferns: level + 1) has the
// entry {threshold, offset as a 32-bit word} at byte 8 v (bytes 0..7 are unused), so that one address and one
// 8-byte load bring both; the leaf weights follow in path order as in the other records.  Larger than the
// packed form (8 against 5 or 6 bytes a vertex): the plans below take it where it fits.
__host__ __device__ constexpr RecordLayout vertex_pair_layout(int kind, int depth) {
  const uint32_t n = kind == FERN ? (uint32_t)depth : (1u << depth) - 1u;
  const uint32_t w = round16(8u * (n + 1u));
  return RecordLayout{0u, 4u, w, round16(w + 4u * (1u << depth)), false};
}

__global__ void repack_vertex_pairs_kernel(const float *__restrict__ thr, const int32_t *__restrict__ ord,
                                           const float *__restrict__ w, unsigned char *__restrict__ records, int kind,
                                           int depth, int64_t T, RecordLayout lay, RecordMap map) {
  const int64_t N = threshold_count(kind, depth);
  const int64_t L = ((int64_t)1) << depth;
  const int64_t per_tree = N + L;
  const int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= T * per_tree) return;
  const int64_t j = e / per_tree;
  const int64_t r = e - j * per_tree;
  unsigned char *rec = records + map.slot(j) * lay.bytes;
  if (r < N) {
    float t = thr[j * N + r];
    t = t == 0.0f ? 0.0f : t;  // -0 becomes +0
    uint2 entry;
    entry.x = __float_as_uint(t);
    entry.y = map.feature((uint32_t)ord[j * N + r]);
    reinterpret_cast<uint2 *>(rec)[r + 1] = entry;
    if (r == 0) reinterpret_cast<uint2 *>(rec)[0] = make_uint2(0u, 0u);
  } else {
    const int64_t h = r - N;
    reinterpret_cast<float *>(rec + lay.w)[h] = w[j * L + (int64_t)bit_reverse((uint32_t)h, depth)];
  }
}

template <uint32_t OFFSET>
__device__ __forceinline__ uint2 lds_b64_at(uint32_t addr) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0, %1}, [%2+%3];" : "=r"(v.x), "=r"(v.y) : "r"(addr), "n"(OFFSET));
  return v;
}

// walk_full on records of that form: rec[u] and x_addr[u] are the record and the window origin of the u-th walk.
template <int KIND, int DEPTH, int NT>
__device__ __forceinline__ void walk_vertex_pairs(const uint32_t (&rec)[NT], const uint32_t (&x_addr)[NT],
                                                  Walked (&out)[NT]) {
  uint32_t v[NT];
#pragma unroll
  for (int u = 0; u < NT; ++u) v[u] = 1u;
  static_for<0, DEPTH>([&](auto level) {
    constexpr int l = decltype(level)::value;
    static_for<0, NT>([&](auto walk_index) {
      constexpr int u = decltype(walk_index)::value;
      uint2 entry;
      if constexpr (KIND == FERN)
        entry = lds_b64_at<8u * (uint32_t)(l + 1)>(rec[u]);
      else
        entry = lds_b64_at<0u>(rec[u] + 8u * v[u]);
      const float nm = __uint_as_float(entry.x) - lds_f32(x_addr[u] + 4u * entry.y);
      if (l == 0 || fabsf(nm) < fabsf(out[u].nm)) {
        out[u].nm = nm;
        out[u].v = KIND == FERN ? (uint32_t)(l + 1) : v[u];
      }
      v[u] = __funnelshift_l(__float_as_uint(nm), v[u], 1);
    });
  });
#pragma unroll
  for (int u = 0; u < NT; ++u) out[u].path = v[u];
}

struct ConvBwdPlan {
  int TY;  // tile rows; slots = kWarps / TY input channels in progress
  int JJ;  // output channels per parameter group
  int patch_h, patch_w, cells, table_len;
  int ord_bytes;
  bool pairs;  // records with one 8-byte entry per vertex
  RecordLayout rec;
  size_t smem;
};

struct Carve {
  size_t params, bins, cell_sums, table, barriers, total;
};

__host__ __device__ inline Carve carve(int Ci, int patch_elems, int slots, int JJ, uint32_t record_bytes, int bins_per_tree,
                                       int cells, int table_len) {
  Carve c;
  size_t at = ((size_t)Ci * patch_elems * 4 + 127) & ~(size_t)127;
  c.params = at;
  at += 2 * (size_t)slots * JJ * record_bytes;
  c.bins = at;
  at += 2 * (size_t)slots * JJ * bins_per_tree * 4;
  c.cell_sums = at;
  at += (size_t)kWarps * cells * 32 * 4;
  c.table = at;
  at += ((size_t)table_len * 2 + 15) & ~(size_t)15;
  c.barriers = at;
  c.total = at + 64;
  return c;
}

bool make_plan(const ConvTileProblem &p, ConvBwdPlan &plan, bool pairs) {
  plan.pairs = pairs;
  if (p.depth > 10 || p.Ci < 1 || p.Co < 1 || p.B < 1 || p.Ho < 1 || p.Wo < 1) return false;
  if ((double)p.B * p.Ho * p.Wo * (double)p.Co * p.Ci < 1048576.0) return false;
  const int bins_per_tree = (int)(threshold_count(p.kind, p.depth) + (((int64_t)1) << p.depth));
  plan.cells = p.kh * p.kw;
  for (int TY = 8; TY >= 1; TY >>= 1) {
    if (TY > 1 && TY / 2 >= p.Ho) continue;
    if (TY == 2) continue;  // 16 slots would need more named barriers than the 15 a CTA has to spare
    const PatchShape shape = patch_shape(p, TY);
    if (shape.far > 16383) continue;
    plan.TY = TY;
    plan.patch_h = shape.h;
    plan.patch_w = shape.w;
    plan.table_len = (int)shape.far + 1;
    plan.ord_bytes = shape.far <= 255 ? 1 : 2;
    plan.rec = pairs ? vertex_pair_layout(p.kind, p.depth) : record_layout(p.kind, p.depth, (uint32_t)plan.ord_bytes);
    const int slots = kWarps / TY;
    for (int JJ = 16; JJ >= 4; JJ >>= 1) {
      plan.JJ = JJ;
      plan.smem = carve((int)p.Ci, shape.h * shape.w, slots, JJ, plan.rec.bytes, bins_per_tree, plan.cells, plan.table_len).total;
      if (plan.smem <= kSmemBudget && (size_t)slots * JJ * plan.rec.bytes < (1u << 20)) return true;
    }
  }
  return false;
}

struct ConvBwdArgs {
  const float *x;
  const unsigned char *records;  // (input channel, output channel) order
  const float *g;
  float *gx, *gthr, *gw;
  uint32_t *status_word;
  int Ci, Co, H, W, Ho, Wo, sy, sx, py, px, dy, dx, kw;
  int TY, JJ, patch_h, patch_w, cells, table_len, tiles_x, tiles_y;
  RecordMap map;
};

// The window-cell offset that vertex v of the record tests.
template <typename OrdT, bool PAIRS>
__device__ __forceinline__ uint32_t offset_of_vertex(uint32_t rec, uint32_t v, uint32_t ord_at) {
  if (PAIRS) return lds_b32(rec + 8u * v + 4u);
  return lds_ord<OrdT>(rec + (uint32_t)sizeof(OrdT) * v + (ord_at - (uint32_t)sizeof(OrdT)));
}

// PAIRS: the records have one 8-byte entry per vertex (OrdT is then unused).
template <int KIND, int DEPTH, typename OrdT, bool PAIRS>
__global__ void __launch_bounds__(kThreads, 1) conv_backward_tiled_kernel(ConvBwdArgs a) {
  extern __shared__ __align__(128) unsigned char smem[];
  constexpr RecordLayout lay = PAIRS ? vertex_pair_layout(KIND, DEPTH) : record_layout(KIND, DEPTH, (uint32_t)sizeof(OrdT));
  constexpr uint32_t kN = KIND == FERN ? DEPTH : (1u << DEPTH) - 1u;
  constexpr uint32_t kL = 1u << DEPTH;
  constexpr int kBins = (int)(kN + kL);  // per tree: threshold bins, then leaf bins in path order
  const int TY = a.TY, JJ = a.JJ;
  const int slots = kWarps / TY;
  const int patch_elems = a.patch_h * a.patch_w;
  const Carve at = carve(a.Ci, patch_elems, slots, JJ, lay.bytes, kBins, a.cells, a.table_len);
  float *patches = reinterpret_cast<float *>(smem);
  unsigned char *params = smem + at.params;
  float *bins = reinterpret_cast<float *>(smem + at.bins);            // [2][slots][JJ][kBins]
  float *cell_sums = reinterpret_cast<float *>(smem + at.cell_sums);  // [kWarps][cells][32]
  uint16_t *cell_of = reinterpret_cast<uint16_t *>(smem + at.table);  // patch offset -> window cell
  uint64_t *full = reinterpret_cast<uint64_t *>(smem + at.barriers);
  uint32_t *finished = reinterpret_cast<uint32_t *>(full + 2);
  const uint32_t buffer_bytes = (uint32_t)slots * (uint32_t)JJ * lay.bytes;

  const int tid = threadIdx.x;
  const int lane = tid & 31, warp = tid >> 5;
  const int tile_row = warp % TY;
  const int slot = warp / TY;
  const int tiles = a.tiles_x * a.tiles_y;
  const int64_t b = blockIdx.x / tiles;
  const int tile = (int)(blockIdx.x - b * tiles);
  const int oy0 = (tile / a.tiles_x) * TY, ox0 = (tile % a.tiles_x) * kTileColumns;

  // blockIdx.y splits the blocks of input channels among CTAs for small batches; `it` counts this
  // CTA's groups: (block of `slots` input channels) x (chunk of JJ output channels)
  const int j_chunks = (a.Co + JJ - 1) / JJ;
  const int all_blocks = (a.Ci + slots - 1) / slots;
  const int blocks_per_cta = (all_blocks + (int)gridDim.y - 1) / (int)gridDim.y;
  const int block0 = (int)blockIdx.y * blocks_per_cta;
  const int num_groups = max(0, min(blocks_per_cta, all_blocks - block0)) * j_chunks;
  const uint32_t params_addr = smem_addr(params);

  auto issue = [&](int it) {
    const int c_first = (block0 + it / j_chunks) * slots;
    const int j_first = (it % j_chunks) * JJ;
    const int count_c = min(slots, a.Ci - c_first), count_j = min(JJ, a.Co - j_first);
    const uint32_t each = (uint32_t)count_j * lay.bytes;
    uint64_t *bar = &full[it & 1];
    mbar_expect_tx(bar, (uint32_t)count_c * each);
    const uint32_t dst = params_addr + (uint32_t)(it & 1) * buffer_bytes;
    for (int s = 0; s < count_c; ++s)
      bulk_load(dst + (uint32_t)s * (uint32_t)JJ * lay.bytes,
                a.records + ((int64_t)(c_first + s) * a.Co + j_first) * lay.bytes, each, bar);
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
  for (int i = tid; i < 2 * slots * JJ * kBins; i += kThreads) bins[i] = 0.0f;
  for (int i = tid; i < kWarps * a.cells * 32; i += kThreads) cell_sums[i] = 0.0f;
  for (int q = tid; q < a.cells; q += kThreads) cell_of[a.map.feature((uint32_t)q)] = (uint16_t)q;
  __syncthreads();

  const uint32_t origin_addr = smem_addr(patches) + (uint32_t)((tile_row * a.sy) * a.patch_w + lane * a.sx) * 4u;
  const uint32_t patch_bytes = (uint32_t)patch_elems * 4u;
  const uint32_t my_cells_addr = smem_addr(cell_sums) + (uint32_t)(warp * a.cells * 32 + lane) * 4u;
  const int oy = oy0 + tile_row, ox = ox0 + lane;
  const bool position_valid = oy < a.Ho && ox < a.Wo;
  const int slot_threads = TY * 32, tid_in_slot = tile_row * 32 + lane;
  const bool bins_wanted = a.gthr != nullptr || a.gw != nullptr;
  const int64_t g_plane = (int64_t)a.Ho * a.Wo;
  const float *g_here = a.g + b * a.Co * g_plane + (position_valid ? (int64_t)oy * a.Wo + ox : 0);
  bool poisoned = false;

  // chunk = it % j_chunks and block = it / j_chunks, counted instead of divided
  int chunk = -1, block = 0;
  for (int it = 0; it < num_groups; ++it) {
    if (++chunk == j_chunks) {
      chunk = 0;
      ++block;
    }
    const int c_first = (block0 + block) * slots;
    const int j_first = chunk * JJ;
    const int count_c = min(slots, a.Ci - c_first), count_j = min(JJ, a.Co - j_first);
    const int c = c_first + slot;
    const bool active = slot < count_c;
    if (!poisoned && !mbar_wait(&full[it & 1], (uint32_t)((it >> 1) & 1))) {
      poisoned = true;
      if (a.status_word != nullptr) atomicOr(a.status_word, HT_FLAG_PIPELINE_TIMEOUT);
    }
    float *my_bins = bins + ((size_t)(it & 1) * slots + slot) * JJ * kBins;
    if (active && !poisoned) {
      const uint32_t base_addr = params_addr + (uint32_t)(it & 1) * buffer_bytes + (uint32_t)slot * (uint32_t)JJ * lay.bytes;
      const uint32_t x_addr = origin_addr + (uint32_t)c * patch_bytes;
      const float *g_chunk = g_here + (int64_t)j_first * g_plane;  // upstream gradient of channel j_first at this position
      for (int jl = 0; jl < count_j; jl += 4, g_chunk += 4 * g_plane) {
        uint32_t rec[4];
        float gval[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          rec[u] = base_addr + (uint32_t)min(jl + u, count_j - 1) * lay.bytes;
          gval[u] = 0.0f;
          if (position_valid && jl + u < count_j) gval[u] = __ldg(g_chunk + u * g_plane);
        }
        Walked wk[4];
        if constexpr (PAIRS) {
          const uint32_t origins[4] = {x_addr, x_addr, x_addr, x_addr};
          walk_vertex_pairs<KIND, DEPTH, 4>(rec, origins, wk);
        } else {
          walk_full<KIND, DEPTH, OrdT, 4>(rec, x_addr, 4u, wk);
        }
        if (!bins_wanted) {
          // The image gradient alone (the parameter gradients came from the kernel further down).  A walk past the
          // last output channel (it repeats that channel's record) adds nothing.
          if (position_valid) {
            const bool ragged = jl + 4 > count_j;  // the same for the whole CTA
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              if (ragged && jl + u >= count_j) continue;
              const float wg = __fmul_rn(lds_f32(rec[u] + 4u * wk[u].path + (lay.w - 4u * kL)), gval[u]);
              const float dx = signed_term(wk[u].nm, wg);
              const uint32_t off = offset_of_vertex<OrdT, PAIRS>(rec[u], wk[u].v, lay.ord);
              const uint32_t cell_addr = my_cells_addr + (uint32_t)cell_of[off] * 128u;
              sts_f32(cell_addr, __fadd_rn(lds_f32(cell_addr), dx));
            }
          }
          continue;
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          if (jl + u < count_j) {  // the same for the whole warp; lanes off the output contribute zeros
            const float wv = lds_f32(rec[u] + 4u * wk[u].path + (lay.w - 4u * kL));
            const float wg = __fmul_rn(wv, gval[u]);
            // sign(margin) * w * g with margin = -nm
            float dx = signed_term(wk[u].nm, wg);
            float dw = __fmul_rn(fabsf(wk[u].nm), gval[u]);
            if (!position_valid) dx = dw = 0.0f;
            float *tree_bins = my_bins + (jl + u) * kBins;
            if (a.gx != nullptr && position_valid) {
              const uint32_t off = offset_of_vertex<OrdT, PAIRS>(rec[u], wk[u].v, lay.ord);
              const uint32_t cell_addr = my_cells_addr + (uint32_t)cell_of[off] * 128u;
              sts_f32(cell_addr, __fadd_rn(lds_f32(cell_addr), dx));
            }
            bool leader;
            if (a.gthr != nullptr) {
              const float sum = sum_by_key(wk[u].v, -dx, lane, leader);
              if (leader && sum != 0.0f) atomicAdd(tree_bins + (wk[u].v - 1u), sum);
            }
            if (a.gw != nullptr) {
              const float sum = sum_by_key(wk[u].path, dw, lane, leader);
              if (leader && sum != 0.0f) atomicAdd(tree_bins + kN + (wk[u].path - kL), sum);
            }
          }
        }
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

    // The slot's warps have all added to this group's bins: send the touched ones out and clear
    // them.  The buffer is used again two groups on, after the slot has met at this barrier once more.
    if (!bins_wanted)
      ;  // no bins in use
    else if (TY == 1)
      __syncwarp();  // the slot is this warp alone
    else
      named_barrier(1 + slot, slot_threads);
    if (active && bins_wanted) {
      for (int e = tid_in_slot; e < count_j * kBins; e += slot_threads) {
        const float v = my_bins[e];
        if (v != 0.0f) {
          my_bins[e] = 0.0f;
          const int jl = e / kBins, r = e - jl * kBins;
          const int64_t tree = (int64_t)(j_first + jl) * a.Ci + c;
          if (r < (int)kN)
            atomicAdd(a.gthr + tree * kN + r, v);
          else  // bins are in path order; the reference's leaf key has the root decision as bit 0
            atomicAdd(a.gw + tree * kL + (__brev((uint32_t)(r - (int)kN)) >> (32 - DEPTH)), v);
        }
      }
    }
    // last chunk of output channels: this warp's image-gradient sums for channel c are complete
    if (chunk == j_chunks - 1 && active && a.gx != nullptr) {
      const int wy = oy * a.sy - a.py, wx = ox * a.sx - a.px;
      float *image = a.gx + (b * a.Ci + c) * (int64_t)a.H * a.W;
      for (int q = 0; q < a.cells; ++q) {
        const uint32_t addr = my_cells_addr + (uint32_t)q * 128u;
        const float v = lds_f32(addr);
        if (v != 0.0f) {
          sts_f32(addr, 0.0f);
          const int iy = wy + (q / a.kw) * a.dy, ix = wx + (q % a.kw) * a.dx;
          if (iy >= 0 && iy < a.H && ix >= 0 && ix < a.W) atomicAdd(image + (int64_t)iy * a.W + ix, v);  // padding has no gradient
        }
      }
    }
  }
}

// ---- threshold and leaf-weight gradients alone -----------------------------------------------------
//
// The bins of one tree collect one term per output position, and the positions of a tile favour
// few bins (the root decides for many of them; a few leaves take most samples), so shared bins mean
// long chains of colliding updates.  This kernel gives every warp ONE tree and lets it walk that
// tree over all R x 32 positions of the tile itself (4 rows in flight): a lane adds its terms into
// its own column of the warp's bin array [bin][column] with plain loads and stores — lanes that
// share a column (32 / columns of them) never update it together: one group adds its threshold
// terms while its neighbour adds its leaf terms, then they swap — and only after the last row the
// columns are summed (16 bytes at a time) and each touched bin leaves as one global reduction.  No
// atomics on shared memory, and R x 32 evaluations per tree and CTA share one flush.  All warps work
// on the same input channel, so only that channel's patch is needed and R can be large; the patches
// of up to 16 channels are staged at a time, since every warp waits while that is done.  Records
// come in three buffers: a warp runs up to two groups ahead of the slowest before it waits.

struct ParamGradPlan {
  int R;        // tile rows
  int columns;  // lanes' columns per bin: 16, 8 or 4
  int staged;   // input channels whose patches are staged together
  int patch_h, patch_w, ord_bytes;
  bool pairs;
  RecordLayout rec;
  size_t smem;
};

// Record groups in flight or in use: with three, a warp runs up to two groups ahead of the slowest before it waits.
constexpr int kParamBuffers = 3;

bool make_param_plan(const ConvTileProblem &p, ParamGradPlan &plan, bool pairs) {
  plan.pairs = pairs;
  if (p.depth > 7 || p.Ci < 1 || p.Co < 1 || p.B < 1 || p.Ho < 1 || p.Wo < 1) return false;
  if ((double)p.B * p.Ho * p.Wo * (double)p.Co * p.Ci < 1048576.0) return false;
  // a warp's bins: 2^depth rows of {threshold bin, leaf bin}, `columns` lanes' columns each
  const int bins_per_tree = 2 << p.depth;
  plan.columns = 16;
  while (plan.columns > 4 && bins_per_tree * plan.columns * 4 > 4096) plan.columns >>= 1;
  plan.R = std::min(16, (p.Ho + 3) & ~3);
  const PatchShape shape = patch_shape(p, plan.R);
  if (shape.far > 16383) return false;
  plan.patch_h = shape.h;
  plan.patch_w = shape.w;
  plan.ord_bytes = shape.far <= 255 ? 1 : 2;
  plan.rec = pairs ? vertex_pair_layout(p.kind, p.depth) : record_layout(p.kind, p.depth, (uint32_t)plan.ord_bytes);
  // Every warp waits while patches are staged, so as many input channels as fit (16 at most) are staged at a time.
  for (plan.staged = (int)std::min<int64_t>(p.Ci, 16); plan.staged >= 1; --plan.staged) {
    plan.smem = align_up((size_t)plan.staged * shape.h * shape.w * 4, 128) + kParamBuffers * (size_t)kWarps * plan.rec.bytes +
                (size_t)kWarps * bins_per_tree * plan.columns * 4 + 64;
    if (plan.smem <= kSmemBudget) return true;
  }
  return false;
}

struct ParamGradArgs {
  const float *x;
  const unsigned char *records;  // (input channel, output channel) order
  const float *g;
  float *gthr, *gw;
  uint32_t *status_word;
  int Ci, Co, H, W, Ho, Wo, sy, sx, py, px;
  int R, columns, staged, patch_h, patch_w, tiles_x, row_blocks;
};

template <int KIND, int DEPTH, typename OrdT, bool PAIRS>
__global__ void __launch_bounds__(kThreads, 1) conv_backward_params_tiled_kernel(ParamGradArgs a) {
  extern __shared__ __align__(128) unsigned char smem[];
  constexpr RecordLayout lay = PAIRS ? vertex_pair_layout(KIND, DEPTH) : record_layout(KIND, DEPTH, (uint32_t)sizeof(OrdT));
  constexpr uint32_t kN = KIND == FERN ? DEPTH : (1u << DEPTH) - 1u;
  constexpr uint32_t kL = 1u << DEPTH;
  constexpr int kBins = (int)(kN + kL);  // threshold bins, then leaf bins in path order
  const int R = a.R, columns = a.columns;
  const int patch_elems = a.patch_h * a.patch_w;
  float *patch = reinterpret_cast<float *>(smem);
  unsigned char *params = smem + (((size_t)a.staged * patch_elems * 4 + 127) & ~(size_t)127);
  // [kWarps][2^DEPTH rows][threshold bin | leaf bin][columns]: with 16 columns a row is the 32 banks, the lanes adding
  // threshold terms use one half and the lanes adding leaf terms the other, and no two of them meet in a bank
  float *bins = reinterpret_cast<float *>(params + kParamBuffers * (size_t)kWarps * lay.bytes);
  uint64_t *full = reinterpret_cast<uint64_t *>(bins + (size_t)kWarps * 2 * kL * columns);
  uint32_t *finished = reinterpret_cast<uint32_t *>(full + kParamBuffers);

  const int tid = threadIdx.x;
  const int lane = tid & 31, warp = tid >> 5;
  const int tiles = a.tiles_x * a.row_blocks;
  const int64_t b = blockIdx.x / tiles;
  const int tile = (int)(blockIdx.x - b * tiles);
  const int oy0 = (tile / a.tiles_x) * R, ox0 = (tile % a.tiles_x) * kTileColumns;

  // blockIdx.y splits the rounds (32 output channels, one per warp) among CTAs; `it` counts this
  // CTA's groups, input channel outermost
  const int all_rounds = (a.Co + kWarps - 1) / kWarps;
  const int rounds_per_cta = (all_rounds + (int)gridDim.y - 1) / (int)gridDim.y;
  const int round0 = (int)blockIdx.y * rounds_per_cta;
  const int my_rounds = max(0, min(rounds_per_cta, all_rounds - round0));
  const int num_groups = my_rounds * a.Ci;
  const uint32_t params_addr = smem_addr(params);
  const uint32_t buffer_bytes = (uint32_t)kWarps * lay.bytes;

  auto issue = [&](int it) {
    const int c = it / my_rounds;
    const int j_first = (round0 + it % my_rounds) * kWarps;
    const uint32_t bytes = (uint32_t)min(kWarps, a.Co - j_first) * lay.bytes;
    uint64_t *bar = &full[it % kParamBuffers];
    mbar_expect_tx(bar, bytes);
    bulk_load(params_addr + (uint32_t)(it % kParamBuffers) * buffer_bytes, a.records + ((int64_t)c * a.Co + j_first) * lay.bytes, bytes,
              bar);
  };
  if (tid == 0) {
    for (int k = 0; k < kParamBuffers; ++k) {
      mbar_init(&full[k], 1);
      finished[k] = 0;
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    for (int k = 0; k < kParamBuffers; ++k)
      if (k < num_groups) issue(k);
  }
  for (int i = tid; i < kWarps * 2 * (int)kL * columns; i += kThreads) bins[i] = 0.0f;

  const int ox = ox0 + lane;
  const uint32_t lane_addr = smem_addr(patch) + (uint32_t)(lane * a.sx) * 4u;
  const uint32_t row_bytes = (uint32_t)(a.sy * a.patch_w) * 4u;
  const uint32_t my_bins_addr = smem_addr(bins) + (uint32_t)(warp * 2 * (int)kL * columns + lane % columns) * 4u;
  const uint32_t bin_bytes = (uint32_t)columns * 4u, row_bytes_of_bins = 2u * bin_bytes;
  const int turns = 32 / columns, group = lane / columns;
  const int rows_here = min(R, a.Ho - oy0);
  const float *image = a.x + b * a.Ci * (int64_t)a.H * a.W;
  const bool want_thr = a.gthr != nullptr, want_w = a.gw != nullptr;
  bool poisoned = false;

  // c: the group's input channel = it / my_rounds; round = it % my_rounds; channel_slot = c % a.staged (counted, not divided)
  int c = 0, round = 0, channel_slot = 0;
  for (int it = 0; it < num_groups; ++it, ++round) {
    if (round == my_rounds) {
      round = 0;
      ++c;
      if (++channel_slot == a.staged) channel_slot = 0;
    }
    if (round == 0 && channel_slot == 0) {  // next input channels: every warp is done with the previous patches
      __syncthreads();
      stage_patches(patch, image + (int64_t)c * a.H * a.W, min(a.staged, a.Ci - c), a.H, a.W, oy0 * a.sy - a.py,
                    ox0 * a.sx - a.px, a.patch_h, a.patch_w);
      __syncthreads();
    }
    const uint32_t channel_addr = lane_addr + (uint32_t)channel_slot * (uint32_t)patch_elems * 4u;
    if (!poisoned && !mbar_wait(&full[it % kParamBuffers], (uint32_t)((it / kParamBuffers) & 1))) {
      poisoned = true;
      if (a.status_word != nullptr) atomicOr(a.status_word, HT_FLAG_PIPELINE_TIMEOUT);
    }
    const int j = (round0 + round) * kWarps + warp;
    if (j < a.Co && !poisoned) {
      const uint32_t record = params_addr + (uint32_t)(it % kParamBuffers) * buffer_bytes + (uint32_t)warp * lay.bytes;
      // lanes and rows off the output read the last valid element instead and have their terms cleared below
      const float *g_rows = a.g + ((b * a.Co + j) * a.Ho + oy0) * (int64_t)a.Wo + min(ox, a.Wo - 1);
      for (int row0 = 0; row0 < rows_here; row0 += 4) {
        uint32_t rec[4], x_addr[4];
        float gval[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          rec[u] = record;
          x_addr[u] = channel_addr + (uint32_t)(row0 + u) * row_bytes;
          gval[u] = __ldg(g_rows + (int64_t)min(row0 + u, rows_here - 1) * a.Wo);
        }
        Walked wk[4];
        if constexpr (PAIRS)
          walk_vertex_pairs<KIND, DEPTH, 4>(rec, x_addr, wk);
        else
          walk_full<KIND, DEPTH, OrdT, 4>(rec, x_addr, 4u, wk);
        float term_thr[4], term_w[4];
        uint32_t at_thr[4], at_w[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const float wv = lds_f32(record + 4u * wk[u].path + (lay.w - 4u * kL));
          const float wg = __fmul_rn(wv, gval[u]);
          // the threshold term is -sign(margin) * w * g with margin = -nm
          term_thr[u] = -signed_term(wk[u].nm, wg);
          term_w[u] = __fmul_rn(fabsf(wk[u].nm), gval[u]);
          if (!(row0 + u < rows_here && ox < a.Wo)) term_thr[u] = term_w[u] = 0.0f;
          at_thr[u] = my_bins_addr + (wk[u].v - 1u) * row_bytes_of_bins;
          at_w[u] = my_bins_addr + bin_bytes + (wk[u].path - kL) * row_bytes_of_bins;
        }
        // Lanes that share a column (32 / columns of them, `group` apart) must not update it together.  Every term
        // is added, zeros included: a test per term costs a divergent branch each, more than the addition it would
        // save.  (The four bins of one kind may coincide, so a lane's updates of one kind stay in order.)
        if (want_thr && want_w) {
          // A threshold bin and a leaf bin never coincide: while the even group of a pair adds its threshold terms
          // the odd group adds its leaf terms, then they swap.  With two groups nobody idles.
          auto add_one_kind = [&](bool thr_now) {
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              const uint32_t at = thr_now ? at_thr[u] : at_w[u];
              sts_f32(at, __fadd_rn(lds_f32(at), thr_now ? term_thr[u] : term_w[u]));
            }
          };
          if (turns == 2) {
            add_one_kind(group == 0);
            __syncwarp();
            add_one_kind(group != 0);
            __syncwarp();
          } else {
            for (int phase = 0; phase < turns; ++phase) {
              if ((group >> 1) == (phase >> 1)) add_one_kind(((group ^ phase) & 1) == 0);
              __syncwarp();
            }
          }
        } else {
          for (int turn = 0; turn < turns; ++turn) {
            if (turn == group) {
              if (want_thr) {
#pragma unroll
                for (int u = 0; u < 4; ++u) sts_f32(at_thr[u], __fadd_rn(lds_f32(at_thr[u]), term_thr[u]));
              } else if (want_w) {
#pragma unroll
                for (int u = 0; u < 4; ++u) sts_f32(at_w[u], __fadd_rn(lds_f32(at_w[u]), term_w[u]));
              }
            }
            __syncwarp();
          }
        }
      }
      // sum the columns of every bin, clear them, send the touched bins out
      const int64_t tree = (int64_t)j * a.Ci + c;
      const uint32_t warp_bins_addr = smem_addr(bins) + (uint32_t)(warp * 2 * (int)kL * columns) * 4u;
      const int quads = columns >> 2;  // columns is 16, 8 or 4: a bin is 1 to 4 aligned 16-byte pieces
      for (int bin = lane; bin < kBins; bin += 32) {
        float sum = 0.0f;
        for (int k = 0; k < quads; ++k) {
          const int quad = (k + lane) & (quads - 1);  // rotated so that the lanes spread over the banks
          const int piece = bin < (int)kN ? 2 * bin : 2 * (bin - (int)kN) + 1;  // threshold bins in the even halves of the rows
          const uint32_t at = warp_bins_addr + (uint32_t)(piece * columns + 4 * quad) * 4u;
          const uint4 v = lds_b128(at);
          sum += (__uint_as_float(v.x) + __uint_as_float(v.y)) + (__uint_as_float(v.z) + __uint_as_float(v.w));
          sts_b128(at, 0.0f, 0.0f, 0.0f, 0.0f);
        }
        if (sum != 0.0f) {
          if (bin < (int)kN)
            atomicAdd(a.gthr + tree * kN + bin, sum);
          else  // bins are in path order; the reference's leaf key has the root decision as bit 0
            atomicAdd(a.gw + tree * kL + (__brev((uint32_t)(bin - (int)kN)) >> (32 - DEPTH)), sum);
        }
      }
    }
    __syncwarp();
    if (lane == 0) {
      __threadfence_block();
      const uint32_t before = atomicAdd(&finished[it % kParamBuffers], 1u);
      if (before == kWarps - 1) {
        atomicExch(&finished[it % kParamBuffers], 0u);
        __threadfence_block();
        if (it + kParamBuffers < num_groups) issue(it + kParamBuffers);
      }
    }
  }
}

template <typename Kernel>
int launch_params_one(Kernel kernel, const ParamGradPlan &plan, const ParamGradArgs &a, dim3 grid, cudaStream_t stream) {
  HT_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBudget));
  kernel<<<grid, kThreads, plan.smem, stream>>>(a);
  HT_CHECK_LAUNCH();
  return HT_OK;
}

template <int KIND, int DEPTH>
int launch_params_depth(const ParamGradPlan &plan, const ParamGradArgs &a, dim3 grid, cudaStream_t stream) {
  if (plan.pairs)
    return launch_params_one(conv_backward_params_tiled_kernel<KIND, DEPTH, uint32_t, true>, plan, a, grid, stream);
  if (plan.ord_bytes == 1)
    return launch_params_one(conv_backward_params_tiled_kernel<KIND, DEPTH, uint8_t, false>, plan, a, grid, stream);
  return launch_params_one(conv_backward_params_tiled_kernel<KIND, DEPTH, uint16_t, false>, plan, a, grid, stream);
}

template <int KIND>
int launch_params_kind(int depth, const ParamGradPlan &plan, const ParamGradArgs &a, dim3 grid, cudaStream_t stream) {
  switch (depth) {
#define HT_DEPTH_CASE(D) \
  case D:                \
    return launch_params_depth<KIND, D>(plan, a, grid, stream);
    HT_DEPTH_CASE(1)
    HT_DEPTH_CASE(2)
    HT_DEPTH_CASE(3)
    HT_DEPTH_CASE(4)
    HT_DEPTH_CASE(5)
    HT_DEPTH_CASE(6)
    HT_DEPTH_CASE(7)
#undef HT_DEPTH_CASE
    default:
      return HT_ERR_UNSUPPORTED;
  }
}

template <typename Kernel>
int launch_one(Kernel kernel, const ConvBwdPlan &plan, const ConvBwdArgs &a, dim3 grid, cudaStream_t stream) {
  HT_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBudget));
  kernel<<<grid, kThreads, plan.smem, stream>>>(a);
  HT_CHECK_LAUNCH();
  return HT_OK;
}

template <int KIND, int DEPTH>
int launch_depth(const ConvBwdPlan &plan, const ConvBwdArgs &a, dim3 grid, cudaStream_t stream) {
  if (plan.pairs) return launch_one(conv_backward_tiled_kernel<KIND, DEPTH, uint32_t, true>, plan, a, grid, stream);
  if (plan.ord_bytes == 1) return launch_one(conv_backward_tiled_kernel<KIND, DEPTH, uint8_t, false>, plan, a, grid, stream);
  return launch_one(conv_backward_tiled_kernel<KIND, DEPTH, uint16_t, false>, plan, a, grid, stream);
}

template <int KIND>
int launch_kind(int depth, const ConvBwdPlan &plan, const ConvBwdArgs &a, dim3 grid, cudaStream_t stream) {
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

// Both kernels read one set of records.  The form with 8-byte vertex entries is taken when it costs neither kernel
// anything: the same tile and group sizes for the image-gradient kernel, and the parameter kernel still available.
bool choose_plans(const ConvTileProblem &p, ConvBwdPlan &plan, ParamGradPlan &pplan, bool &with_params) {
  if (!make_plan(p, plan, false)) return false;
  auto shared_records = [&]() { return pplan.patch_w == plan.patch_w && (plan.pairs || pplan.ord_bytes == plan.ord_bytes); };
  with_params = make_param_plan(p, pplan, false) && shared_records();
  ConvBwdPlan wide;
  ParamGradPlan wide_params;
  if (make_plan(p, wide, true) && wide.TY == plan.TY && wide.JJ == plan.JJ &&
      (!with_params || (make_param_plan(p, wide_params, true) && wide_params.patch_w == wide.patch_w &&
                        wide_params.staged == pplan.staged))) {
    plan = wide;
    if (with_params) pplan = wide_params;
  }
  return true;
}

}  // namespace

size_t conv_backward_tiled_workspace_bytes(const ConvTileProblem &p) {
  ConvBwdPlan plan;
  ParamGradPlan pplan;
  bool with_params;
  if (!choose_plans(p, plan, pplan, with_params)) return 0;
  return align_up((size_t)(p.Co * p.Ci) * plan.rec.bytes, 256);
}

int conv_backward_tiled(const ConvTileProblem &p, const float *x, const float *thr, const int32_t *ord, const float *w,
                        const float *g, float *gx, float *gthr, float *gw, void *records, uint32_t *status_word,
                        cudaStream_t stream) {
  ConvBwdPlan plan;
  ParamGradPlan pplan;
  bool with_params;
  if (!choose_plans(p, plan, pplan, with_params)) return HT_ERR_UNSUPPORTED;
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
  map.inner = p.Ci;  // tree (j, c) goes to record c * Co + j
  map.outer_count = p.Co;
  if (plan.pairs)
    repack_vertex_pairs_kernel<<<pack_grid, 256, 0, stream>>>(thr, ord, w, rec, p.kind, p.depth, trees, plan.rec, map);
  else if (plan.ord_bytes == 1)
    repack_records_kernel<uint8_t><<<pack_grid, 256, 0, stream>>>(thr, ord, w, rec, p.kind, p.depth, trees, plan.rec, map);
  else
    repack_records_kernel<uint16_t><<<pack_grid, 256, 0, stream>>>(thr, ord, w, rec, p.kind, p.depth, trees, plan.rec, map);
  HT_CHECK_LAUNCH();

  // Shallow trees: the parameter gradients come from the kernel built for them, and the kernel
  // below is left with the image gradient.
  if ((gthr != nullptr || gw != nullptr) && with_params) {
    ParamGradArgs pa;
    pa.x = x;
    pa.records = rec;
    pa.g = g;
    pa.gthr = gthr;
    pa.gw = gw;
    pa.status_word = status_word;
    pa.Ci = (int)p.Ci;
    pa.Co = (int)p.Co;
    pa.H = p.H;
    pa.W = p.W;
    pa.Ho = p.Ho;
    pa.Wo = p.Wo;
    pa.sy = p.sy;
    pa.sx = p.sx;
    pa.py = p.py;
    pa.px = p.px;
    pa.R = pplan.R;
    pa.columns = pplan.columns;
    pa.staged = pplan.staged;
    pa.patch_h = pplan.patch_h;
    pa.patch_w = pplan.patch_w;
    pa.tiles_x = tiles_x;
    pa.row_blocks = (p.Ho + pplan.R - 1) / pplan.R;
    const int64_t tiles = p.B * pa.tiles_x * pa.row_blocks;
    if (tiles <= 0x7fffffff) {
      // enough CTAs for about seven rounds of the machine, so that the last round's idle SMs cost little
      const int64_t rounds = (p.Co + kWarps - 1) / kWarps;
      int64_t splits = 1;
      if (tiles < 7 * 148) splits = std::min<int64_t>(rounds, (7 * 148 + tiles - 1) / tiles);
      const dim3 pgrid((unsigned)tiles, (unsigned)std::max<int64_t>(splits, 1));
      const int rc = p.kind == TREE ? launch_params_kind<TREE>(p.depth, pplan, pa, pgrid, stream)
                                    : launch_params_kind<FERN>(p.depth, pplan, pa, pgrid, stream);
      if (rc != HT_OK) return rc;
      if (gx == nullptr) return HT_OK;
      gthr = nullptr;
      gw = nullptr;
    }
  }

  ConvBwdArgs a;
  a.x = x;
  a.records = rec;
  a.g = g;
  a.gx = gx;
  a.gthr = gthr;
  a.gw = gw;
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
  a.dy = p.dy;
  a.dx = p.dx;
  a.kw = p.kw;
  a.TY = plan.TY;
  a.JJ = plan.JJ;
  a.patch_h = plan.patch_h;
  a.patch_w = plan.patch_w;
  a.cells = plan.cells;
  a.table_len = plan.table_len;
  a.tiles_x = tiles_x;
  a.tiles_y = tiles_y;
  a.map = map;
  const int slots = kWarps / plan.TY;
  const int64_t blocks = (p.Ci + slots - 1) / slots;
  int64_t splits = 1;
  if (ctas < 2 * 148) splits = std::min<int64_t>(blocks, (2 * 148 + ctas - 1) / ctas);
  const dim3 grid((unsigned)ctas, (unsigned)std::max<int64_t>(splits, 1));
  return p.kind == TREE ? launch_kind<TREE>(p.depth, plan, a, grid, stream)
                        : launch_kind<FERN>(p.depth, plan, a, grid, stream);
}

}  // namespace ht
