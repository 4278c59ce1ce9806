// Shared-memory tile kernels for the forest backward on tabular input (K == 1, one output per leaf).
//
// forest_backward_tiled_kernel has the tiling of the forward tile kernel (ht_forest_tiled.cu): a CTA
// owns S consecutive samples, keeps their features feature-major in shared memory and walks ALL
// trees, whose parameter records stream in through bulk async copies; a warp walks 4 consecutive
// trees at once for its 32 samples.  Each lane fetches the 4 upstream gradients g[i, j .. j+3] of its
// sample with one 16-byte load issued before the walk.  One traversal serves all three gradients
// (the reference runs three kernels that each repeat it, hingetree_gpu.cu:699-727); it keeps the
// signed margin and the deciding vertex, with the reference's strict `<` so that the shallowest
// minimum wins.  What happens to the terms depends on the workspace the caller gave:
//   * with room for 12 bytes per evaluation (the record path, both modes): the kernel writes one
//     record per evaluation and two reductions further down add the records in a fixed order —
//     reduce_x_records_kernel for the x gradient, reduce_parameter_records_* for thresholds and
//     leaf weights.  No floating-point atomics anywhere; in fixed-order mode the sums are the
//     reference's sequential CPU sums bit for bit;
//   * without it (default mode only): fire-and-forget global reductions (red.global.add.f32) from
//     the traversal kernel itself.
// There is no block-wide barrier after the feature tile has been staged.
#include "ht_forest_tiled.cuh"
#include "ht_eval_records.cuh"
#include "ht_tile_common.cuh"
#include "ht_tma.cuh"

#include <algorithm>
#include <type_traits>

namespace ht {

using namespace tile;

namespace {

// Warps per CTA of the parameter reduction with bin columns.  Fewer warps leave room for more columns
// per warp (fewer turns per chunk, and a turn costs a full shared-memory wavefront per load and
// store) but hide less latency; C3 forward+backward: 16 warps x 4 columns 17.9 ms, 8 x 8 17.4 ms,
// 4 x 16 18.4 ms.
constexpr int kColumnWarps = 8;

struct BwdPlan {
  int S, G, per_warp, ord_bytes;
  RecordLayout rec;
  size_t smem;
};

// Shared-memory layout of forest_backward_tiled_kernel, from a 1024-byte boundary: the box of upstream
// gradients of the current tree group [S samples x G trees] (filled by a tiled TMA load when the
// gradient admits a tensor map), the feature tile, two parameter buffers, the barriers.
__host__ __device__ inline size_t gradient_box_bytes(int S, int G) {
  return ((size_t)S * G * 4 + 1023) & ~(size_t)1023;
}

// paired: the record path, whose kernels never look a feature index up by vertex, takes the paired form
bool make_bwd_plan(const ht_forest_problem *p, BwdPlan &plan, bool paired = false) {
  if (p->K < 1 || p->M != 1) return false;  // a sample is a (row, inner position) pair
  if (p->C > 65536 || p->depth > 12) return false;
  if (p->B * p->K * p->T < 32 * 1024) return false;
  plan.ord_bytes = p->C <= 256 ? 1 : 2;
  plan.rec = record_layout(p->kind, p->depth, (uint32_t)plan.ord_bytes, true,
                           paired && paired_ordinals(p->kind, p->depth, (uint32_t)plan.ord_bytes));
  for (int S = 256; S >= 32; S >>= 1) {
    const int slots = kWarps / (S / 32);
    for (int per_warp = 4; per_warp >= 1; per_warp >>= 1) {
      const int G = slots * per_warp;
      plan.S = S;
      plan.G = G;
      plan.per_warp = per_warp;
      plan.smem = 1024 + gradient_box_bytes(S, G) + (size_t)p->C * S * 4 + 2 * (size_t)G * plan.rec.bytes + 64;
      if (plan.smem <= kSmemBudget) return true;
    }
  }
  return false;
}

struct BwdArgs {
  CUtensorMap g_map;  // the upstream gradient [B, T] in boxes of S rows x G trees (when tma_g is set)
  int tma_g;
  const float *x;
  const unsigned char *records;
  const float *g;
  float *gx, *gthr, *gw;
  EvalRecords evals;
  uint32_t *status_word;
  int64_t B, T, K;  // B: samples = rows x inner positions; K: inner positions per row
  int C, S, G, per_warp;
};

template <int KIND, int DEPTH, typename OrdT, bool RECORDS>
__global__ void __launch_bounds__(kThreads, 1) forest_backward_tiled_kernel(const __grid_constant__ BwdArgs a) {
  extern __shared__ __align__(1024) unsigned char smem[];
  constexpr bool kPaired = RECORDS && paired_ordinals(KIND, DEPTH, (uint32_t)sizeof(OrdT));
  constexpr RecordLayout lay = record_layout(KIND, DEPTH, (uint32_t)sizeof(OrdT), true, kPaired);
  constexpr uint32_t kN = KIND == FERN ? DEPTH : (1u << DEPTH) - 1u;
  constexpr uint32_t kL = 1u << DEPTH;
  using WhereT = typename std::conditional<(DEPTH <= 8), unsigned short, uint32_t>::type;
  const int S = a.S, G = a.G, C = a.C;
  unsigned char *base = smem + ((1024u - (smem_addr(smem) & 1023u)) & 1023u);
  const uint32_t g_box = smem_addr(base);
  float *xs = reinterpret_cast<float *>(base + gradient_box_bytes(S, G));
  unsigned char *params = reinterpret_cast<unsigned char *>(xs + (size_t)C * S);
  uint64_t *full = reinterpret_cast<uint64_t *>(params + 2 * (size_t)G * lay.bytes);  // [2] parameters landed, [1] gradients landed
  uint32_t *finished = reinterpret_cast<uint32_t *>(full + 3);                        // [2] warps done with a buffer, [1] with the gradients

  const int tid = threadIdx.x;
  const int lane = tid & 31, warp = tid >> 5;
  const int groups_of_samples = S >> 5;
  const int sample_group = warp % groups_of_samples;
  const int slot = warp / groups_of_samples;
  const int per_warp = a.per_warp;
  const int64_t row0 = (int64_t)blockIdx.x * S;
  // the tree groups are split over gridDim.y when the batch alone gives too few tiles
  const int all_groups = (int)((a.T + G - 1) / G);
  const int groups_per_cta = (all_groups + (int)gridDim.y - 1) / (int)gridDim.y;
  const int group0 = (int)blockIdx.y * groups_per_cta;
  const int num_groups = max(0, min(groups_per_cta, all_groups - group0));
  const uint32_t params_addr = smem_addr(params);

  auto issue = [&](int it) {
    const int64_t first_tree = (int64_t)(group0 + it) * G;
    const int64_t count = min((int64_t)G, a.T - first_tree);
    const uint32_t bytes = (uint32_t)(count * lay.bytes);
    uint64_t *bar = &full[it & 1];
    mbar_expect_tx(bar, bytes);
    bulk_load(params_addr + (uint32_t)(it & 1) * (uint32_t)G * lay.bytes, a.records + first_tree * lay.bytes, bytes,
              bar);
  };
  // The upstream gradients of a full tree group arrive as one box [S samples x G trees] through the
  // TMA engine, one group ahead: the last warp to have taken its values out of the box requests the next.
  const int full_groups_all = (int)(a.T / G);
  const bool tma_g = RECORDS && a.tma_g != 0;
  auto issue_gradients = [&](int it) {
    mbar_expect_tx(&full[2], (uint32_t)(S * G * 4));
    tma::load_2d(g_box, &a.g_map, (group0 + it) * G, (int)row0, &full[2]);
  };
  if (tid == 0) {
    mbar_init(&full[0], 1);
    mbar_init(&full[1], 1);
    mbar_init(&full[2], 1);
    finished[0] = 0;
    finished[1] = 0;
    finished[2] = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    if (num_groups > 0) issue(0);
    if (num_groups > 1) issue(1);
    if (tma_g && num_groups > 0 && group0 < full_groups_all) issue_gradients(0);
  }

  // features in
  if (a.K > 1) {
    // consecutive samples are consecutive positions of a row; a thread stages one sample's features
    const int t = tid % S, c_step = kThreads / S;
    const int64_t sample = row0 + t;
    const bool inside = sample < a.B;
    const int64_t row = inside ? sample / a.K : 0, k = inside ? sample - row * a.K : 0;
    const float *src = a.x + row * C * a.K + k;
    for (int c = tid / S; c < C; c += c_step) xs[c * S + t] = inside ? __ldg(src + (int64_t)c * a.K) : 0.0f;
  } else if ((C & 3) == 0) {
    // two 16-byte loads in flight per thread before the first is stored (see the forward kernel)
    const int quads = C >> 2;
    const int total = S * quads;
    for (int idx0 = tid; idx0 < total; idx0 += 2 * kThreads) {
      float4 v[2];
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int idx = idx0 + u * kThreads;
        const int s = idx % S, q = idx / S;
        v[u] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (idx < total && row0 + s < a.B) v[u] = __ldg(reinterpret_cast<const float4 *>(a.x + (row0 + s) * C) + q);
      }
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int idx = idx0 + u * kThreads;
        if (idx < total) {
          const int s = idx % S, q = idx / S;
          xs[(4 * q + 0) * S + s] = v[u].x;
          xs[(4 * q + 1) * S + s] = v[u].y;
          xs[(4 * q + 2) * S + s] = v[u].z;
          xs[(4 * q + 3) * S + s] = v[u].w;
        }
      }
    }
  } else {
    for (int idx = tid; idx < S * C; idx += kThreads) {
      const int s = idx % S, c = idx / S;
      xs[c * S + s] = (row0 + s < a.B) ? __ldg(a.x + (row0 + s) * C + c) : 0.f;
    }
  }
  __syncthreads();

  const int my_sample = sample_group * 32 + lane;
  const bool row_valid = row0 + my_sample < a.B;
  const uint32_t xl_addr = smem_addr(xs + my_sample);
  const uint32_t x_stride = (uint32_t)S * 4u;
  const int64_t my_row = row0 + my_sample;  // the sample's index; with inner positions (row, position) below
  const int64_t my_records = record_index(my_row, 0, a.T);  // tree j's record of this sample: + j * kRecordBlock
  const int64_t outer = row_valid ? my_row / a.K : 0, inner = row_valid ? my_row - outer * a.K : 0;
  // upstream gradient of tree j: g_sample[j * a.K]; x gradient of feature c: gx_sample[c * a.K]
  const float *g_sample = a.g + outer * a.T * a.K + inner;
  float *gx_sample = a.gx == nullptr ? nullptr : a.gx + outer * C * a.K + inner;
  const int full_groups = (int)(a.T / G), tail_trees = (int)(a.T - (int64_t)full_groups * G);
  bool poisoned = false;
  // Full groups with 4 trees per warp on the record path take a body without the bookkeeping of
  // short groups and other tree counts.
  const bool streamlined = RECORDS && per_warp == 4 && (a.T & 3) == 0 && a.K == 1;
  const uint32_t warp_records = (uint32_t)(slot * per_warp) * lay.bytes;
  const float *g_mine = a.g + my_row * a.T + slot * per_warp;
  // this lane's 4 gradients in the swizzled box: row = sample inside the tile, 16-byte chunk = slot
  const uint32_t g_mine_box = g_box + (G == 16 ? tma::swizzled_offset<16>((uint32_t)my_sample, (uint32_t)slot)
                                              : tma::swizzled_offset<32>((uint32_t)my_sample, (uint32_t)slot));
  const int64_t records_mine = my_records + (int64_t)(slot * per_warp) * kRecordBlock;

  // This warp no longer reads parameter buffer (it & 1).  The last warp to say so refills it.
  auto done_with_buffer = [&](int it) {
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
  };

  for (int it = 0; it < num_groups; ++it) {
    const int group = group0 + it;
    const int in_group = group < full_groups ? G : tail_trees;
    const int64_t col0 = (int64_t)group * G;
    if (streamlined && in_group == G) {
      float4 gq = make_float4(0.f, 0.f, 0.f, 0.f);
      if (tma_g) {
        if (!poisoned && !mbar_wait(&full[2], (uint32_t)(it & 1))) {
          poisoned = true;
          if (a.status_word != nullptr) atomicOr(a.status_word, HT_FLAG_PIPELINE_TIMEOUT);
        }
        if (!poisoned) {
          const uint4 q = lds_b128(g_mine_box);
          gq = make_float4(__uint_as_float(q.x), __uint_as_float(q.y), __uint_as_float(q.z), __uint_as_float(q.w));
        }
        __syncwarp();
        if (lane == 0) {
          __threadfence_block();
          const uint32_t before = atomicAdd(&finished[2], 1u);
          if (before == kWarps - 1) {
            atomicExch(&finished[2], 0u);
            __threadfence_block();
            if (it + 1 < num_groups && group + 1 < full_groups_all && !poisoned) issue_gradients(it + 1);
          }
        }
      } else if (row_valid) {
        gq = __ldg(reinterpret_cast<const float4 *>(g_mine + col0));  // requested before the walk
      }
      if (!poisoned && !mbar_wait(&full[it & 1], (uint32_t)((it >> 1) & 1))) {
        poisoned = true;
        if (a.status_word != nullptr) atomicOr(a.status_word, HT_FLAG_PIPELINE_TIMEOUT);
      }
      if (!poisoned) {
        const uint32_t base_addr = params_addr + (uint32_t)(it & 1) * (uint32_t)G * lay.bytes + warp_records;
        uint32_t rec[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) rec[u] = base_addr + (uint32_t)u * lay.bytes;
        Walked wk[4];
        walk_full<KIND, DEPTH, OrdT, 4, kPaired>(rec, xl_addr, x_stride, wk);
        const float gval[4] = {gq.x, gq.y, gq.z, gq.w};
        const int64_t at = records_mine + col0 * kRecordBlock;
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const float wg = __fmul_rn(lds_f32(rec[u] + 4u * wk[u].path + (lay.w - 4u * kL)), gval[u]);
          const float dx = signed_term(wk[u].nm, wg);
          const uint32_t key = __brev(wk[u].path - kL) >> (32 - DEPTH);
          if (row_valid) {
            __stcs(a.evals.dx + at + u * kRecordBlock, dx);
            __stcs(a.evals.dw + at + u * kRecordBlock, __fmul_rn(fabsf(wk[u].nm), gval[u]));
            store_where<WhereT>(a.evals.where, at + u * kRecordBlock, wk[u].v, key);
          }
        }
      }
      done_with_buffer(it);
      continue;
    }

    // upstream gradients of this lane's sample for the warp's trees, requested before the walk
    const int t_first = slot * per_warp;
    float gval[4] = {0.f, 0.f, 0.f, 0.f};
    if (row_valid && t_first < in_group) {
      const float *gp = g_sample + (col0 + t_first) * a.K;
      if (a.K > 1) {
#pragma unroll
        for (int u = 0; u < 4; ++u)
          if (u < per_warp && t_first + u < in_group) gval[u] = __ldg(gp + (int64_t)u * a.K);
      } else if (per_warp == 4 && (a.T & 3) == 0 && t_first + 3 < in_group) {
        const float4 v = __ldg(reinterpret_cast<const float4 *>(gp));
        gval[0] = v.x;
        gval[1] = v.y;
        gval[2] = v.z;
        gval[3] = v.w;
      } else {
#pragma unroll
        for (int u = 0; u < 4; ++u)
          if (u < per_warp && t_first + u < in_group) gval[u] = __ldg(gp + u);
      }
    }

    if (!poisoned && !mbar_wait(&full[it & 1], (uint32_t)((it >> 1) & 1))) {
      poisoned = true;
      if (a.status_word != nullptr) atomicOr(a.status_word, HT_FLAG_PIPELINE_TIMEOUT);
    }
    const uint32_t base_addr = params_addr + (uint32_t)(it & 1) * (uint32_t)G * lay.bytes;
    if (t_first < in_group && !poisoned) {
      auto scatter = [&](const Walked &wk, uint32_t rec, int u) {
        const int t = t_first + u;
        if (t >= in_group || !row_valid) return;
        const int64_t j = col0 + t;
        const float gv = gval[u];
        const float wv = lds_f32(rec + 4u * wk.path + (lay.w - 4u * kL));
        // sign(margin) * w * g with margin = -nm
        const float wg = __fmul_rn(wv, gv);
        const float dx = signed_term(wk.nm, wg);
        if (RECORDS) {
          const uint32_t key = __brev(wk.path - kL) >> (32 - DEPTH);
          const int64_t at = my_records + j * kRecordBlock;
          a.evals.dx[at] = dx;
          a.evals.dw[at] = __fmul_rn(fabsf(wk.nm), gv);
          store_where<WhereT>(a.evals.where, at, wk.v, key);
          return;
        }
        if (a.gx != nullptr) {
          const uint32_t c = lds_ord<OrdT>(rec + (uint32_t)sizeof(OrdT) * wk.v + (lay.ord - (uint32_t)sizeof(OrdT)));
          atomicAdd(gx_sample + (int64_t)c * a.K, dx);
        }
        if (a.gthr != nullptr) atomicAdd(a.gthr + j * kN + (wk.v - 1u), -dx);
        if (a.gw != nullptr) {
          const uint32_t key = __brev(wk.path - kL) >> (32 - DEPTH);  // reference leaf key: bit l = decision at depth l
          atomicAdd(a.gw + j * kL + key, __fmul_rn(fabsf(wk.nm), gv));
        }
      };
      if (per_warp == 4) {
        uint32_t rec[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) rec[u] = base_addr + (uint32_t)min(t_first + u, in_group - 1) * lay.bytes;
        Walked wk[4];
        walk_full<KIND, DEPTH, OrdT, 4, kPaired>(rec, xl_addr, x_stride, wk);
#pragma unroll
        for (int u = 0; u < 4; ++u) scatter(wk[u], rec[u], u);
      } else if (per_warp == 2) {
        uint32_t rec[2];
#pragma unroll
        for (int u = 0; u < 2; ++u) rec[u] = base_addr + (uint32_t)min(t_first + u, in_group - 1) * lay.bytes;
        Walked wk[2];
        walk_full<KIND, DEPTH, OrdT, 2, kPaired>(rec, xl_addr, x_stride, wk);
#pragma unroll
        for (int u = 0; u < 2; ++u) scatter(wk[u], rec[u], u);
      } else {
        uint32_t rec[1] = {base_addr + (uint32_t)t_first * lay.bytes};
        Walked wk[1];
        walk_full<KIND, DEPTH, OrdT, 1, kPaired>(rec, xl_addr, x_stride, wk);
        scatter(wk[0], rec[0], 0);
      }
    }
    done_with_buffer(it);
  }
}

template <typename Kernel>
int launch_one(Kernel kernel, const BwdPlan &plan, const BwdArgs &a, dim3 grid, cudaStream_t stream) {
  HT_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBudget));
  kernel<<<grid, kThreads, plan.smem, stream>>>(a);
  HT_CHECK_LAUNCH();
  return HT_OK;
}

template <int KIND, int DEPTH>
int launch_depth(const BwdPlan &plan, const BwdArgs &a, dim3 grid, cudaStream_t stream) {
  const bool records = a.evals.dx != nullptr;
  if (plan.ord_bytes == 1)
    return records ? launch_one(forest_backward_tiled_kernel<KIND, DEPTH, uint8_t, true>, plan, a, grid, stream)
                   : launch_one(forest_backward_tiled_kernel<KIND, DEPTH, uint8_t, false>, plan, a, grid, stream);
  return records ? launch_one(forest_backward_tiled_kernel<KIND, DEPTH, uint16_t, true>, plan, a, grid, stream)
                 : launch_one(forest_backward_tiled_kernel<KIND, DEPTH, uint16_t, false>, plan, a, grid, stream);
}

// ---- consumers of the evaluation records -----------------------------------------------------------
//
// The x-gradient consumer adds the terms of every element in the order of the reference CPU loop
// (trees ascending), in both modes.  The parameter consumer does so in fixed-order mode (samples
// ascending: equal to the reference CPU loops bit for bit); in default mode it adds them in another,
// fixed association (reproducible from run to run, within rounding of the reference).

// Runs f() on the valid lanes so that lanes sharing `key` execute in lane order.
template <typename F>
__device__ __forceinline__ void lanes_in_order_per_key(bool valid, uint32_t key, F &&f) {
  const unsigned lane = threadIdx.x & 31u;
  const uint32_t tag = valid ? key : (0x80000000u | lane);
  const unsigned peers = __match_any_sync(0xffffffffu, tag);
  const int rank = __popc(peers & ((1u << lane) - 1u));
  const int last = __reduce_max_sync(0xffffffffu, valid ? rank : 0);
  for (int r = 0; r <= last; ++r) {
    if (valid && rank == r) f();
    __syncwarp();
  }
}

// Threshold and leaf-weight gradients: one CTA per tree.  Each of its warps walks a share of the
// tree's records in sample order, 32 at a time (4 chunks prefetched), into its own bins in shared
// memory (lanes that meet in a bin add in lane order); the warps' bins are then summed in warp
// order.  With one warp (fixed-order mode) that is exactly the reference's sequential sum over
// the samples; with several (default mode) it is a reproducible sum with another association.
// ORDERED = false (default mode only): the lanes that meet in a bin first add their terms together
// with shuffles in a logarithmic number of rounds, and the lowest lane of each bin updates it once;
// the ordered form pays one dependent round per lane of the fullest bin, and a few bins (the root
// threshold, the likeliest leaves) collect a third of the lanes of a typical chunk.
template <bool ORDERED, typename WT>
__global__ void __launch_bounds__(512) reduce_parameter_records_kernel(EvalRecords r, int64_t B, int64_t T, int64_t N,
                                                                       int64_t L, float *gthr, float *gw) {
  extern __shared__ float all_bins[];
  const int warps = blockDim.x >> 5, warp = threadIdx.x >> 5;
  float *bins = all_bins + (size_t)warp * (N + L);
  float *thr_bins = bins, *w_bins = bins + N;
  const int64_t j = blockIdx.x;
  const unsigned lane = threadIdx.x & 31u;
  for (int64_t t = lane; t < N + L; t += 32) bins[t] = 0.0f;
  __syncwarp();
  // A batch is kAhead chunks of 32 consecutive samples (all inside one 256-sample record block);
  // the next batch is requested before the current one is consumed.
  constexpr int kAhead = 4;
  const int64_t stride = (int64_t)warps * 32 * kAhead;
  float a[kAhead], b[kAhead], na[kAhead], nb[kAhead];
  uint32_t wh[kAhead], nwh[kAhead];
  auto fetch = [&](int64_t i0, float (&fa)[kAhead], float (&fb)[kAhead], uint32_t (&fw)[kAhead]) {
    const int64_t first = record_index(i0, j, T) + lane;  // i0 is a multiple of 128
#pragma unroll
    for (int u = 0; u < kAhead; ++u) {
      const bool valid = i0 + 32 * u + lane < B;
      fa[u] = valid ? __ldcs(r.dx + first + 32 * u) : 0.0f;
      fb[u] = valid ? __ldcs(r.dw + first + 32 * u) : 0.0f;
      fw[u] = valid ? load_where<WT>(r.where, first + 32 * u) : 1u;
    }
  };
  int64_t i0 = (int64_t)warp * 32 * kAhead;
  if (i0 < B) fetch(i0, a, b, wh);
  for (; i0 < B; i0 += stride) {
    if (i0 + stride < B) fetch(i0 + stride, na, nb, nwh);
#pragma unroll
    for (int u = 0; u < kAhead; ++u) {
      const bool valid = i0 + 32 * u + lane < B;
      // (clamped: a traversal that gave up on a lost copy, and said so in the status word, leaves records unwritten)
      const uint32_t v = min((wh[u] & 0xffffu) - 1u, (uint32_t)N - 1u), key = min(wh[u] >> 16, (uint32_t)L - 1u);
      if (ORDERED) {
        if (gthr != nullptr)
          lanes_in_order_per_key(valid, v, [&]() { thr_bins[v] = __fadd_rn(thr_bins[v], -a[u]); });
        if (gw != nullptr)
          lanes_in_order_per_key(valid, key, [&]() { w_bins[key] = __fadd_rn(w_bins[key], b[u]); });
      } else {
        bool leader;
        if (gthr != nullptr) {
          const float sum = sum_by_key(valid ? v : (0x80000000u | lane), valid ? -a[u] : 0.0f, (int)lane, leader);
          if (leader && valid) thr_bins[v] = __fadd_rn(thr_bins[v], sum);
        }
        if (gw != nullptr) {
          const float sum = sum_by_key(valid ? key : (0x80000000u | lane), valid ? b[u] : 0.0f, (int)lane, leader);
          if (leader && valid) w_bins[key] = __fadd_rn(w_bins[key], sum);
        }
        __syncwarp();
      }
    }
#pragma unroll
    for (int u = 0; u < kAhead; ++u) {
      a[u] = na[u];
      b[u] = nb[u];
      wh[u] = nwh[u];
    }
  }
  __syncthreads();
  for (int64_t t = threadIdx.x; t < N + L; t += blockDim.x) {
    float sum = all_bins[t];
    for (int wi = 1; wi < warps; ++wi) sum = __fadd_rn(sum, all_bins[(size_t)wi * (N + L) + t]);
    if (t < N) {
      if (gthr != nullptr) gthr[j * N + t] = sum;
    } else if (gw != nullptr) {
      gw[j * L + (t - N)] = sum;
    }
  }
}

// Default mode, when the bins fit several times into shared memory: every warp keeps `columns`
// copies of the tree's bins, [bin][column]; a lane adds its terms into column (lane % columns) with
// plain loads and stores, the 32 / columns lanes that share a column taking turns.  No lane has to
// find out which other lanes hit the same bin (a match.any per gradient per chunk bounds the kernel
// above), and the chains of dependent updates of the hot bins are `columns` times shorter.  The
// warps' columns are summed in a fixed order at the end: reproducible, another association.
template <int CHUNKS, typename WT>
__global__ void __launch_bounds__(512, 1) reduce_parameter_records_columns_kernel(EvalRecords r, int64_t B, int64_t T,
                                                                                  int64_t N, int64_t L, int columns,
                                                                                  float *gthr, float *gw) {
  extern __shared__ float all_bins[];  // [warp][bin][column]
  const int warps = blockDim.x >> 5, warp = threadIdx.x >> 5;
  const unsigned lane = threadIdx.x & 31u;
  const int bins_per_tree = (int)(N + L);
  const int64_t j = blockIdx.x;
  for (int t = threadIdx.x; t < warps * bins_per_tree * columns; t += blockDim.x) all_bins[t] = 0.0f;
  __syncthreads();
  const uint32_t my_column = smem_addr(all_bins) + (uint32_t)(warp * bins_per_tree * columns + (int)(lane % columns)) * 4u;
  const uint32_t bin_bytes = (uint32_t)columns * 4u;
  const int turns = 32 / columns, my_turn = (int)lane / columns;

  const int64_t stride = (int64_t)warps * 32 * CHUNKS;
  float a[CHUNKS], b[CHUNKS], na[CHUNKS], nb[CHUNKS];
  uint32_t wh[CHUNKS], nwh[CHUNKS];
  auto fetch = [&](int64_t i0, float (&fa)[CHUNKS], float (&fb)[CHUNKS], uint32_t (&fw)[CHUNKS]) {
    const int64_t first = record_index(i0, j, T) + lane;  // i0 is a multiple of 32 * CHUNKS, which divides 256
#pragma unroll
    for (int u = 0; u < CHUNKS; ++u) {
      const bool valid = i0 + 32 * u + lane < B;
      fa[u] = valid ? __ldcs(r.dx + first + 32 * u) : 0.0f;  // an absent sample adds zeros to bin 0
      fb[u] = valid ? __ldcs(r.dw + first + 32 * u) : 0.0f;
      fw[u] = valid ? load_where<WT>(r.where, first + 32 * u) : 1u;
    }
  };
  int64_t i0 = (int64_t)warp * 32 * CHUNKS;
  if (i0 < B) fetch(i0, a, b, wh);
  for (; i0 < B; i0 += stride) {
    if (i0 + stride < B) fetch(i0 + stride, na, nb, nwh);
    uint32_t at_thr[CHUNKS], at_w[CHUNKS];
#pragma unroll
    for (int u = 0; u < CHUNKS; ++u) {
      at_thr[u] = my_column + min((wh[u] & 0xffffu) - 1u, (uint32_t)N - 1u) * bin_bytes;  // clamped: see above
      at_w[u] = my_column + ((uint32_t)N + min(wh[u] >> 16, (uint32_t)L - 1u)) * bin_bytes;
    }
    for (int turn = 0; turn < turns; ++turn) {
      if (turn == my_turn) {
#pragma unroll
        for (int u = 0; u < CHUNKS; ++u) {
          // the two bins are different words: both updates are in flight together
          const float old_thr = lds_f32(at_thr[u]), old_w = lds_f32(at_w[u]);
          if (gthr != nullptr) sts_f32(at_thr[u], __fadd_rn(old_thr, -a[u]));
          if (gw != nullptr) sts_f32(at_w[u], __fadd_rn(old_w, b[u]));
        }
      }
      __syncwarp();
    }
#pragma unroll
    for (int u = 0; u < CHUNKS; ++u) {
      a[u] = na[u];
      b[u] = nb[u];
      wh[u] = nwh[u];
    }
  }
  __syncthreads();
  for (int t = threadIdx.x; t < bins_per_tree; t += blockDim.x) {
    float sum = 0.0f;
    for (int wi = 0; wi < warps; ++wi)
      for (int c = 0; c < columns; ++c) sum = __fadd_rn(sum, all_bins[((size_t)wi * bins_per_tree + t) * columns + c]);
    if (t < N) {
      if (gthr != nullptr) gthr[j * N + t] = sum;
    } else if (gw != nullptr) {
      gw[j * L + (t - N)] = sum;
    }
  }
}

// Default mode, trees whose bins fit 16 times into a sixth of the shared memory: ONE warp per CTA with
// COLUMNS copies of the tree's bins, rows of {threshold bin r | leaf bin r} x COLUMNS.  With 32 columns a
// lane would own its column outright; with 16 (the form launched) lanes l and l + 16 share one and never
// update it together: while the lower half-warp adds its threshold terms the upper adds its leaf terms,
// then they swap (taking turns instead left half the lanes idle in every instruction: 3.3 against 3.1 ms
// on 2^30 records).  A row is the 32 banks, one half per kind, so the lanes that are active together hit
// distinct banks whatever bins they update and every load and store is one wavefront for 32 terms (the
// 8-column form above pays a wavefront per 8 terms and a conflict on top).  A lane consumes its records
// four at a time: the bin loads of a kind are in flight together, the sums are chained in record order (a
// later record that hits the bin of an earlier one of the four continues from its sum), and the stores
// leave in order, so each lane's column holds exactly the sequential sum of its terms.  The samples are split over gridDim.y; a CTA adds its column totals (in a
// fixed order per bin) to the gradient with one global reduction per bin, or stores them when there is one split.
template <int COLUMNS, int CHUNKS, typename WT>
__global__ void __launch_bounds__(32) reduce_parameter_records_private_kernel(EvalRecords r, int64_t B, int64_t T, int N,
                                                                              int L, int64_t blocks_per_split, float *gthr,
                                                                              float *gw) {
  extern __shared__ float all_bins[];  // [bin][column]
  static_assert(CHUNKS % 8 == 0 && kRecordBlock == 256, "a fetch covers whole record blocks");
  constexpr int kTurns = 32 / COLUMNS;
  constexpr int kBlocksPerFetch = CHUNKS / 8;
  const unsigned lane = threadIdx.x;
  const int bins = N + L;
  const int64_t j = blockIdx.x;
  for (int t = (int)lane; t < 2 * L * COLUMNS; t += 32) all_bins[t] = 0.0f;  // L rows (N <= L)
  __syncwarp();
  constexpr uint32_t kHalfBytes = COLUMNS * 4, kRowBytes = 2 * kHalfBytes;
  const uint32_t my_column = smem_addr(all_bins) + (lane % COLUMNS) * 4u;
  const int my_turn = (int)lane / COLUMNS;
  // two lane groups: the kind a lane adds first (and second), as the half of the row it addresses
  const bool thr_first = my_turn == 0;
  const uint32_t first_half = my_column + (thr_first ? 0u : kHalfBytes), second_half = my_column + (thr_first ? kHalfBytes : 0u);
  const bool first_wanted = thr_first ? gthr != nullptr : gw != nullptr;
  const bool second_wanted = thr_first ? gw != nullptr : gthr != nullptr;
  const int64_t all_blocks = (B + kRecordBlock - 1) / kRecordBlock;
  const int64_t block_first = (int64_t)blockIdx.y * blocks_per_split;
  const int64_t block_last = min(all_blocks, block_first + blocks_per_split);

  float a[CHUNKS], b[CHUNKS], na[CHUNKS], nb[CHUNKS];
  uint32_t wh[CHUNKS], nwh[CHUNKS];
  auto fetch = [&](int64_t blk, float (&fa)[CHUNKS], float (&fb)[CHUNKS], uint32_t (&fw)[CHUNKS]) {
    // whole fetches (all but the last of a split or of the batch) load without a test per chunk
    const bool whole = blk + kBlocksPerFetch <= block_last && (blk + kBlocksPerFetch) * kRecordBlock <= B;
#pragma unroll
    for (int h = 0; h < kBlocksPerFetch; ++h) {
      const int64_t first = ((blk + h) * T + j) * kRecordBlock + lane;
      const float *dxs = r.dx + first, *dws = r.dw + first;
      const WT *wheres = static_cast<const WT *>(r.where) + first;
      if (whole) {
        static_for<0, 8>([&](auto uu) {
          constexpr int u = decltype(uu)::value;
          fa[8 * h + u] = stream_f32_at<32 * u * 4>(dxs);
          fb[8 * h + u] = stream_f32_at<32 * u * 4>(dws);
          fw[8 * h + u] = stream_raw_where_at<WT, 32 * u>(wheres);
        });
        continue;
      }
      static_for<0, 8>([&](auto uu) {
        constexpr int u = decltype(uu)::value;
        const bool valid = blk + h < block_last && (blk + h) * kRecordBlock + 32 * u + lane < B;
        fa[8 * h + u] = 0.0f;  // an absent sample adds zeros to bin 0
        fb[8 * h + u] = 0.0f;
        fw[8 * h + u] = 1u;  // raw form of vertex 1, leaf 0
        if (valid) {
          fa[8 * h + u] = stream_f32_at<32 * u * 4>(dxs);
          fb[8 * h + u] = stream_f32_at<32 * u * 4>(dws);
          fw[8 * h + u] = stream_raw_where_at<WT, 32 * u>(wheres);
        }
      });
    }
  };
  // the terms of one fetch join the bins
  auto consume = [&](const float (&ta)[CHUNKS], const float (&tb)[CHUNKS], const uint32_t (&tw)[CHUNKS]) {
#pragma unroll
    for (int q = 0; q < CHUNKS; q += 4) {
      // adds `term` of the lane's four records to the bins at `at`, in record order
      auto add_four = [&](const uint32_t (&at)[4], const float (&term)[4], bool wanted) {
        float sum[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) sum[u] = lds_f32(at[u]);
#pragma unroll
        for (int u = 0; u < 4; ++u) {
#pragma unroll
          for (int e = 0; e < u; ++e) sum[u] = at[u] == at[e] ? sum[e] : sum[u];  // the latest earlier record on the same bin
          sum[u] = __fadd_rn(sum[u], term[u]);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u)
          if (wanted) sts_f32(at[u], sum[u]);
      };
      uint32_t row_thr[4], row_w[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const uint32_t where = unpack_where<WT>(tw[q + u]);
        row_thr[u] = min((where & 0xffffu) - 1u, (uint32_t)N - 1u);  // clamped
        row_w[u] = min(where >> 16, (uint32_t)L - 1u);
      }
      if constexpr (kTurns == 2) {
        uint32_t at_first[4], at_second[4];
        float term_first[4], term_second[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          at_first[u] = first_half + (thr_first ? row_thr[u] : row_w[u]) * kRowBytes;
          at_second[u] = second_half + (thr_first ? row_w[u] : row_thr[u]) * kRowBytes;
          term_first[u] = thr_first ? -ta[q + u] : tb[q + u];
          term_second[u] = thr_first ? tb[q + u] : -ta[q + u];
        }
        add_four(at_first, term_first, first_wanted);
        __syncwarp();
        add_four(at_second, term_second, second_wanted);
        __syncwarp();
      } else {
        uint32_t at_thr[4], at_w[4];
        float term_thr[4], term_w[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          at_thr[u] = my_column + row_thr[u] * kRowBytes;
          at_w[u] = my_column + kHalfBytes + row_w[u] * kRowBytes;
          term_thr[u] = -ta[q + u];
          term_w[u] = tb[q + u];
        }
#pragma unroll
        for (int turn = 0; turn < kTurns; ++turn) {
          if (kTurns == 1 || turn == my_turn) {
            add_four(at_thr, term_thr, gthr != nullptr);
            add_four(at_w, term_w, gw != nullptr);
          }
          if (kTurns > 1) __syncwarp();
        }
      }
    }
  };
  // two register sets take turns: while one is consumed the next fetch lands in the other (no copies between them)
  int64_t blk = block_first;
  if (blk < block_last) fetch(blk, a, b, wh);
  while (blk < block_last) {
    if (blk + kBlocksPerFetch < block_last) fetch(blk + kBlocksPerFetch, na, nb, nwh);
    consume(a, b, wh);
    blk += kBlocksPerFetch;
    if (blk >= block_last) break;
    if (blk + kBlocksPerFetch < block_last) fetch(blk + kBlocksPerFetch, a, b, wh);
    consume(na, nb, nwh);
    blk += kBlocksPerFetch;
  }
  __syncwarp();
  for (int t = (int)lane; t < bins; t += 32) {
    float sum = 0.0f;
    const int piece = t < N ? 2 * t : 2 * (t - N) + 1;  // threshold bins in the even halves of the rows
#pragma unroll 8
    for (int c = 0; c < COLUMNS; ++c) sum = __fadd_rn(sum, all_bins[piece * COLUMNS + ((c + (int)lane) % COLUMNS)]);
    float *dst = t < N ? (gthr == nullptr ? nullptr : gthr + j * N + t) : (gw == nullptr ? nullptr : gw + j * L + (t - N));
    if (dst == nullptr) continue;
    if (gridDim.y == 1)
      *dst = sum;
    else
      atomicAdd(dst, sum);
  }
}

// x gradient: one thread per sample walks the trees in ascending order and adds into its private
// column of a shared-memory tile gx[c][s]; the tile leaves with plain stores.  Per evaluation it reads
// the term and the deciding vertex (6 or 8 bytes) and looks the vertex's feature up in the compact
// ordinal table, which every thread of the CTA walks in the same order (L1 / L2 resident).
// B: samples (rows x inner positions), K: inner positions per row.
template <typename WT>
__global__ void __launch_bounds__(256) reduce_x_records_kernel(EvalRecords r, const int32_t *__restrict__ ord, int64_t B,
                                                               int64_t K, int64_t T, int64_t N, int C, int S, float *gx) {
  extern __shared__ float tile[];
  const int s = threadIdx.x;
  const int64_t row0 = (int64_t)blockIdx.x * S;
  for (int idx = s; idx < S * C; idx += blockDim.x) tile[idx] = 0.0f;
  __syncthreads();
  const int64_t i = row0 + s;
  if (s < S && i < B) {
    // three stages in flight: records of batch n+2, feature indices of batch n+1, additions of batch n
    constexpr int kAhead = 16;
    const int64_t first = record_index(i, 0, T);  // tree j of this sample sits at first + j * 256
    float a0[kAhead], a1[kAhead], a2[kAhead];
    uint32_t wh1[kAhead], wh2[kAhead];
    uint32_t c0[kAhead], c1[kAhead];
    auto fetch_records = [&](int64_t j0, float (&fa)[kAhead], uint32_t (&fw)[kAhead]) {
      const float *dxs = r.dx + first + j0 * kRecordBlock;
      const WT *wheres = static_cast<const WT *>(r.where) + first + j0 * kRecordBlock;
      static_for<0, kAhead>([&](auto uu) {
        constexpr int u = decltype(uu)::value;
        fa[u] = 0.0f;
        fw[u] = 1u;
        if (j0 + u < T) {
          fa[u] = stream_f32_at<u * kRecordBlock * 4>(dxs);
          fw[u] = stream_raw_where_at<WT, u * kRecordBlock>(wheres);
        }
      });
    };
    auto fetch_features = [&](int64_t j0, const uint32_t (&fw)[kAhead], uint32_t (&fc)[kAhead]) {
#pragma unroll
      for (int u = 0; u < kAhead; ++u)
        fc[u] = j0 + u < T ? min((uint32_t)__ldg(ord + (j0 + u) * N + min((unpack_where<WT>(fw[u]) & 0xffffu) - 1u, (uint32_t)N - 1u)),
                                 (uint32_t)C - 1u)
                           : 0u;  // clamped: see the parameter reductions
    };
    fetch_records(0, a0, wh1);
    fetch_features(0, wh1, c0);
    fetch_records(kAhead, a1, wh1);
    const uint32_t column = smem_addr(tile + s), pitch = (uint32_t)S * 4u;
    for (int64_t j0 = 0; j0 < T; j0 += kAhead) {
      fetch_records(j0 + 2 * kAhead, a2, wh2);
      fetch_features(j0 + kAhead, wh1, c1);
#pragma unroll
      for (int u = 0; u < kAhead; ++u) {  // beyond the last tree: zero into feature 0
        const uint32_t at = column + c0[u] * pitch;
        sts_f32(at, __fadd_rn(lds_f32(at), a0[u]));
      }
#pragma unroll
      for (int u = 0; u < kAhead; ++u) {
        a0[u] = a1[u];
        c0[u] = c1[u];
        a1[u] = a2[u];
        wh1[u] = wh2[u];
      }
    }
  }
  __syncthreads();
  if (K > 1) {  // consecutive samples are consecutive positions: each feature's run of the tile is contiguous
    for (int idx = threadIdx.x; idx < S * C; idx += blockDim.x) {
      const int ss = idx % S, c = idx / S;
      const int64_t sample = row0 + ss;
      if (sample < B) {
        const int64_t row = sample / K, k = sample - row * K;
        gx[(row * C + c) * K + k] = tile[c * S + ss];
      }
    }
  } else if ((C & 3) == 0) {
    const int quads = C >> 2;
    for (int idx = threadIdx.x; idx < S * quads; idx += blockDim.x) {
      const int ss = idx % S, q = idx / S;
      if (row0 + ss < B)
        *(reinterpret_cast<float4 *>(gx + (row0 + ss) * C) + q) =
            make_float4(tile[(4 * q + 0) * S + ss], tile[(4 * q + 1) * S + ss], tile[(4 * q + 2) * S + ss],
                        tile[(4 * q + 3) * S + ss]);
    }
  } else {
    for (int idx = threadIdx.x; idx < S * C; idx += blockDim.x) {
      const int ss = idx % S, c = idx / S;
      if (row0 + ss < B) gx[(row0 + ss) * C + c] = tile[c * S + ss];
    }
  }
}

// ---- the backward from a saved forward ---------------------------------------------------------------
//
// A forward that ran with room for the evaluation records leaves, per evaluation, nm = threshold - feature at
// the deciding vertex and the packed (vertex, leaf).  With them no tree is walked again: expand_saved_kernel
// (sample-stationary, a thread per sample, trees ascending — the reference's order) turns them and the upstream
// gradient into the terms the traversal kernel of the backward would have written, in place (dx = sign * w * g
// over nm, dw = |margin| * g), for the parameter reductions above, and adds the x gradient on the way into its
// column of the shared-memory tile gx[c][s].  Everything it looks up arrives asynchronously, 16 trees at a
// time, two buffers: the leaf weights and compact feature indices of the trees (both contiguous in global
// memory: bulk copies) and the box [S samples x 16 trees] of the upstream gradient (a tiled TMA load, 64-byte
// swizzle: a thread reads the 64 bytes of its own row without bank conflicts).
constexpr int kSavedBatch = 16;  // trees per batch; the saving forward's tree groups are multiples of it
constexpr int kJoin = 4;         // x-gradient terms of a thread whose column updates are in flight together (8: slower)

__host__ __device__ inline size_t saved_table_bytes(int64_t N, int64_t L) { return (size_t)kSavedBatch * (size_t)(N + L) * 4; }

struct ExpandArgs {
  CUtensorMap g_map;
  EvalRecords r;
  const int32_t *ord;
  const float *w;
  float *gx;
  int64_t B, T;
  int N, L, C;
  int write_terms;
};

// TREE_DEPTH > 0: the launch is for trees of that depth, 256 samples per CTA, with the terms written and the x
// gradient wanted — the sizes are then constants, table offsets become immediate operands and the per-term tests go
// (56 -> 41 instructions per evaluation, in a kernel whose few warps wait on every dependent instruction).
template <typename WT, int TREE_DEPTH = 0>
__global__ void __launch_bounds__(256) expand_saved_kernel(const __grid_constant__ ExpandArgs a) {
  constexpr bool kFixed = TREE_DEPTH > 0;
  extern __shared__ __align__(1024) unsigned char saved_smem[];
  const int S = kFixed ? 256 : (int)blockDim.x;
  const int s = threadIdx.x;
  const int L = kFixed ? (1 << TREE_DEPTH) : a.L, N = kFixed ? (1 << TREE_DEPTH) - 1 : a.N, C = a.C;
  const bool write_terms = kFixed ? true : a.write_terms != 0;
  const bool want_gx = kFixed ? true : a.gx != nullptr;
  const int64_t T = a.T;
  unsigned char *base = saved_smem + ((1024u - (smem_addr(saved_smem) & 1023u)) & 1023u);
  const uint32_t box_bytes = (uint32_t)S * kSavedBatch * 4u;
  const uint32_t table_bytes = (uint32_t)saved_table_bytes(N, L);
  const uint32_t boxes = smem_addr(base);                      // [2] gradient boxes
  unsigned char *tables = base + 2 * (size_t)box_bytes;        // [2] {leaf weights, feature indices}
  uint64_t *landed = reinterpret_cast<uint64_t *>(tables + 2 * (size_t)table_bytes);  // [2]
  float *tile = reinterpret_cast<float *>(landed + 2);         // gx[c][s]
  const int64_t row0 = (int64_t)blockIdx.x * S;
  const int batches = (int)(T / kSavedBatch);
  auto issue = [&](int batch) {  // what the evaluations of trees [16 batch, 16 batch + 16) look up
    uint64_t *bar = &landed[batch & 1];
    const uint32_t dst = smem_addr(tables) + (uint32_t)(batch & 1) * table_bytes;
    const uint32_t w_bytes = (uint32_t)(kSavedBatch * L * 4), o_bytes = (uint32_t)(kSavedBatch * N * 4);
    mbar_expect_tx(bar, w_bytes + o_bytes + box_bytes);
    bulk_load(dst, a.w + (int64_t)batch * kSavedBatch * L, w_bytes, bar);
    bulk_load(dst + w_bytes, a.ord + (int64_t)batch * kSavedBatch * N, o_bytes, bar);
    tma::load_2d(boxes + (uint32_t)(batch & 1) * box_bytes, &a.g_map, batch * kSavedBatch, (int)row0, bar);
  };
  if (s == 0) {
    mbar_init(&landed[0], 1);
    mbar_init(&landed[1], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    if (batches > 0) issue(0);
    if (batches > 1) issue(1);
  }
  if (want_gx)
    for (int idx = s; idx < S * C; idx += S) tile[idx] = 0.0f;
  __syncthreads();
  const int64_t i = row0 + s;
  const bool mine = i < a.B;
  const int64_t first = record_index(mine ? i : 0, 0, T);  // tree j of this sample sits at first + j * 256
  // records of the batch after next are requested while the current one is expanded
  float nm0[kSavedBatch], nm1[kSavedBatch], nm2[kSavedBatch];
  uint32_t wh0[kSavedBatch], wh1[kSavedBatch], wh2[kSavedBatch];
  auto fetch = [&](int batch, float (&fn)[kSavedBatch], uint32_t (&fw)[kSavedBatch]) {
    if (batch >= batches || !mine) return;
    const int64_t at = first + (int64_t)batch * kSavedBatch * kRecordBlock;
    const float *margins = a.r.dx + at;
    const WT *wheres = static_cast<const WT *>(a.r.where) + at;
    static_for<0, kSavedBatch>([&](auto u) {
      constexpr int U = decltype(u)::value;
      fn[U] = stream_f32_at<U * kRecordBlock * 4>(margins);
      fw[U] = stream_raw_where_at<WT, U * kRecordBlock>(wheres);
    });
  };
#pragma unroll
  for (int u = 0; u < kSavedBatch; ++u) {
    nm0[u] = nm1[u] = 0.0f;
    wh0[u] = wh1[u] = 1u;
  }
  fetch(0, nm0, wh0);
  fetch(1, nm1, wh1);
  const uint32_t column = smem_addr(tile + s), pitch = (uint32_t)S * 4u;
  bool gave_up = false;
  // one batch: its records are in (nm, wh)
  auto expand = [&](int batch, const float (&nm)[kSavedBatch], const uint32_t (&wh)[kSavedBatch]) {
    const int64_t j0 = (int64_t)batch * kSavedBatch;
    if (!gave_up && !mbar_wait(&landed[batch & 1], (uint32_t)((batch >> 1) & 1))) gave_up = true;  // the copies never came
    if (mine && !gave_up) {
      const uint32_t w_table = smem_addr(tables) + (uint32_t)(batch & 1) * table_bytes;
      const uint32_t o_table = w_table + (uint32_t)(kSavedBatch * L * 4);
      const uint32_t box = boxes + (uint32_t)(batch & 1) * box_bytes;
      float gv[kSavedBatch], wv[kSavedBatch];
      uint32_t c[kSavedBatch];
      float *terms_dx = a.r.dx + first + j0 * kRecordBlock, *terms_dw = a.r.dw + first + j0 * kRecordBlock;
#pragma unroll
      for (int q = 0; q < kSavedBatch / 4; ++q) {
        const uint4 v = lds_b128(box + tma::swizzled_offset<16>((uint32_t)s, (uint32_t)q));
        gv[4 * q + 0] = __uint_as_float(v.x);
        gv[4 * q + 1] = __uint_as_float(v.y);
        gv[4 * q + 2] = __uint_as_float(v.z);
        gv[4 * q + 3] = __uint_as_float(v.w);
      }
#pragma unroll
      for (int u = 0; u < kSavedBatch; ++u) {  // (clamped: a forward that gave up on a lost copy leaves records unwritten)
        const uint32_t where = unpack_where<WT>(wh[u]);
        wv[u] = lds_f32(w_table + 4u * ((uint32_t)(u * L) + min(where >> 16, (uint32_t)L - 1u)));
        if (want_gx)
          c[u] = min(lds_b32(o_table + 4u * ((uint32_t)(u * N) + min((where & 0xffffu) - 1u, (uint32_t)N - 1u))),
                     (uint32_t)C - 1u);
      }
      // The x-gradient terms join the thread's column kJoin at a time: their loads are in flight together, a term
      // whose feature an earlier one of them had continues from that one's sum, and the stores leave in order
      // (one dependent load-add-store per term cost a shared-memory round trip each).
#pragma unroll
      for (int q = 0; q < kSavedBatch; q += kJoin) {
        float dx[kJoin], sum[kJoin];
        uint32_t at[kJoin];
#pragma unroll
        for (int u = 0; u < kJoin; ++u) {
          const float wg = __fmul_rn(wv[q + u], gv[q + u]);
          dx[u] = signed_term(nm[q + u], wg);
          if (write_terms) {
            __stcs(terms_dx + (q + u) * kRecordBlock, dx[u]);
            __stcs(terms_dw + (q + u) * kRecordBlock, __fmul_rn(fabsf(nm[q + u]), gv[q + u]));
          }
          at[u] = column + c[q + u] * pitch;
        }
        if (want_gx) {
#pragma unroll
          for (int u = 0; u < kJoin; ++u) sum[u] = lds_f32(at[u]);
#pragma unroll
          for (int u = 0; u < kJoin; ++u) {
#pragma unroll
            for (int e = 0; e < u; ++e) sum[u] = at[u] == at[e] ? sum[e] : sum[u];
            sum[u] = __fadd_rn(sum[u], dx[u]);
          }
#pragma unroll
          for (int u = 0; u < kJoin; ++u) sts_f32(at[u], sum[u]);
        }
      }
    }
    __syncthreads();  // every thread is done with this buffer
    if (s == 0 && batch + 2 < batches && !gave_up) issue(batch + 2);
  };
  // while one batch is expanded, the records of the two after it are in flight (rotating the register sets costs a
  // few moves per evaluation; three unrolled copies of the body ran slower, measured twice: 9.8 against 8.0 ms for
  // the whole backward of 2^30 evaluations at the time, 12.2 against 11.6 ms per training step with the present kernel)
  for (int batch = 0; batch < batches; ++batch) {
    fetch(batch + 2, nm2, wh2);
    expand(batch, nm0, wh0);
#pragma unroll
    for (int u = 0; u < kSavedBatch; ++u) {
      nm0[u] = nm1[u];
      wh0[u] = wh1[u];
      nm1[u] = nm2[u];
      wh1[u] = wh2[u];
    }
  }
  if (!want_gx) return;
  __syncthreads();
  if ((C & 3) == 0) {
    const int quads = C >> 2;
    for (int idx = s; idx < S * quads; idx += S) {
      const int ss = idx % S, q = idx / S;
      if (row0 + ss < a.B)
        *(reinterpret_cast<float4 *>(a.gx + (row0 + ss) * C) + q) =
            make_float4(tile[(4 * q + 0) * S + ss], tile[(4 * q + 1) * S + ss], tile[(4 * q + 2) * S + ss],
                        tile[(4 * q + 3) * S + ss]);
    }
  } else {
    for (int idx = s; idx < S * C; idx += S) {
      const int ss = idx % S, c = idx / S;
      if (row0 + ss < a.B) a.gx[(row0 + ss) * C + c] = tile[c * S + ss];
    }
  }
}

template <int KIND>
int launch_kind(int depth, const BwdPlan &plan, const BwdArgs &a, dim3 grid, cudaStream_t stream) {
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
    HT_DEPTH_CASE(11)
    HT_DEPTH_CASE(12)
#undef HT_DEPTH_CASE
    default:
      return HT_ERR_UNSUPPORTED;
  }
}

// Launches the threshold / leaf-weight reduction that fits the mode and the tree size.
template <typename WT>
int reduce_parameters(const ht_forest_problem *p, const EvalRecords &evals, int64_t samples, int64_t N, int64_t L,
                      float *gthr, float *gw, cudaStream_t stream) {
  // fixed-order mode: one warp per tree, the reference's sequential sum.  Default mode: as many
  // warps as help (each needs work and its own bins), summed in warp order.
  int warps = 1;
  if ((p->flags & HT_DETERMINISTIC) == 0) {
    warps = 16;
    while (warps > 1 && ((size_t)warps * (N + L) * 4 > 64 * 1024 || samples < (int64_t)warps * 512)) warps >>= 1;
  }
  const size_t smem = sizeof(float) * (size_t)(N + L) * warps;
  if ((p->flags & HT_DETERMINISTIC) != 0) {
    HT_CUDA_TRY(cudaFuncSetAttribute(reduce_parameter_records_kernel<true, WT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     (int)kSmemBudget));
    reduce_parameter_records_kernel<true, WT><<<(unsigned)p->T, 32 * warps, smem, stream>>>(evals, samples, p->T, N, L, gthr, gw);
    HT_CHECK_LAUNCH();
    return HT_OK;
  }
  // copies of the bins per warp (a power of two, at most one per lane) that `column_warps` warps can hold
  const int column_warps = kColumnWarps;
  int columns = 32;
  while (columns > 1 && (size_t)column_warps * (N + L) * columns * 4 > 200 * 1024) columns >>= 1;
  // bins that fit 16 times into a sixth of the shared memory: one warp per CTA, each column shared by two
  // lanes, samples split over gridDim.y so that the machine sees several waves of CTAs
  const int private_columns = 2 * (size_t)L * 16 * 4 <= 36 * 1024 ? 16 : 0;  // L rows of {threshold bin | leaf bin}
  if (private_columns != 0 && samples >= 64 * 1024) {
    const size_t private_smem = 2 * (size_t)L * private_columns * 4;
    const int64_t slots = 148 * (int64_t)(kSmemBudget / (private_smem + 1024));
    const int64_t all_blocks = (samples + kRecordBlock - 1) / kRecordBlock;
    int64_t splits = std::max<int64_t>(1, std::min<int64_t>((6 * slots + p->T - 1) / p->T, all_blocks / 16));
    splits = std::min<int64_t>(splits, 65535);
    const int64_t blocks_per_split = ((all_blocks + splits - 1) / splits + 1) / 2 * 2;  // whole fetches of 2 blocks
    const dim3 reduce_grid((unsigned)p->T, (unsigned)((all_blocks + blocks_per_split - 1) / blocks_per_split));
    // (32 lane-owned columns leave room for 3 warps per SM only and ran slower: 5.3 against 3.2 ms on 2^30 records)
    auto kernel = reduce_parameter_records_private_kernel<16, 16, WT>;
    HT_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBudget));
    kernel<<<reduce_grid, 32, private_smem, stream>>>(evals, samples, p->T, (int)N, (int)L, blocks_per_split, gthr, gw);
  } else if (warps == 16 && columns >= 4) {
    const size_t column_smem = (size_t)column_warps * (N + L) * columns * 4;
    HT_CUDA_TRY(cudaFuncSetAttribute(reduce_parameter_records_columns_kernel<8, WT>,
                                     cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBudget));
    reduce_parameter_records_columns_kernel<8, WT><<<(unsigned)p->T, 32 * column_warps, column_smem, stream>>>(
        evals, samples, p->T, N, L, columns, gthr, gw);
  } else {
    HT_CUDA_TRY(cudaFuncSetAttribute(reduce_parameter_records_kernel<false, WT>,
                                     cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBudget));
    reduce_parameter_records_kernel<false, WT><<<(unsigned)p->T, 32 * warps, smem, stream>>>(evals, samples, p->T, N, L, gthr, gw);
  }
  HT_CHECK_LAUNCH();
  return HT_OK;
}

}  // namespace

size_t backward_records_bytes(const ht_forest_problem *p) {
  BwdPlan plan;
  if (!make_bwd_plan(p, plan) || p->depth > 15) return 0;
  const size_t bytes = 2 * record_array_bytes(p, 4) + record_array_bytes(p, where_bytes(p->depth));
  return bytes <= ((size_t)32 << 30) ? bytes : 0;
}

int backward_tiled(const ht_forest_problem *p, const float *x, const float *thr, const int32_t *ord, const float *w,
                   const float *g, float *gx, float *gthr, float *gw, void *records, void *eval_records,
                   uint32_t *status_word, cudaStream_t stream) {
  BwdPlan plan;
  if (!make_bwd_plan(p, plan, eval_records != nullptr)) return HT_ERR_UNSUPPORTED;
  if (forward_tiled_workspace_bytes(p) == 0) return HT_ERR_UNSUPPORTED;  // the workspace holds no records otherwise
  if (((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(g) | reinterpret_cast<uintptr_t>(gx)) & 15u) != 0)
    return HT_ERR_UNSUPPORTED;
  if (eval_records == nullptr && (p->flags & HT_DETERMINISTIC) != 0) return HT_ERR_UNSUPPORTED;
  const int64_t N = threshold_count(p->kind, p->depth);
  const int64_t L = ((int64_t)1) << p->depth;
  const int64_t elements = p->T * (N + L);
  const unsigned pack_grid = (unsigned)((elements + 255) / 256);
  unsigned char *rec = static_cast<unsigned char *>(records);
  if (plan.ord_bytes == 1)
    repack_records_kernel<uint8_t><<<pack_grid, 256, 0, stream>>>(thr, ord, w, rec, p->kind, p->depth, p->T, plan.rec);
  else
    repack_records_kernel<uint16_t><<<pack_grid, 256, 0, stream>>>(thr, ord, w, rec, p->kind, p->depth, p->T, plan.rec);
  HT_CHECK_LAUNCH();
  BwdArgs a = {};
  a.x = x;
  a.records = rec;
  a.g = g;
  a.gx = gx;
  a.gthr = gthr;
  a.gw = gw;
  a.evals = EvalRecords{nullptr, nullptr, nullptr};
  if (eval_records != nullptr) {
    a.evals = eval_record_arrays(p, eval_records);
  }
  a.status_word = status_word;
  a.B = p->B * p->K;
  a.K = p->K;
  a.T = p->T;
  a.C = (int)p->C;
  a.S = plan.S;
  a.G = plan.G;
  a.per_warp = plan.per_warp;
  // record path, tabular input, groups of 16 or 32 trees: the upstream gradient comes in by tiled TMA loads
  a.tma_g = 0;
  if (eval_records != nullptr && p->K == 1 && plan.per_warp == 4 && (plan.G == 16 || plan.G == 32) && (p->T & 3) == 0 &&
      p->T >= plan.G && tma::encode_matrix_f32(&a.g_map, g, p->B, p->T, plan.S, plan.G))
    a.tma_g = 1;
  // a small batch gives too few sample tiles for 148 SMs: share the tree groups between CTAs
  const int64_t samples = p->B * p->K;
  const int64_t tiles = (samples + plan.S - 1) / plan.S;
  if (tiles > 0x7fffffff) return HT_ERR_UNSUPPORTED;
  const int64_t groups = (p->T + plan.G - 1) / plan.G;
  const dim3 grid((unsigned)tiles, (unsigned)choose_splits(tiles, groups));
  const int rc = p->kind == TREE ? launch_kind<TREE>(p->depth, plan, a, grid, stream)
                                 : launch_kind<FERN>(p->depth, plan, a, grid, stream);
  if (rc != HT_OK || eval_records == nullptr) return rc;

  if (gthr != nullptr || gw != nullptr) {
    const int prc = where_bytes(p->depth) == 2
                        ? reduce_parameters<unsigned short>(p, a.evals, samples, N, L, gthr, gw, stream)
                        : reduce_parameters<uint32_t>(p, a.evals, samples, N, L, gthr, gw, stream);
    if (prc != HT_OK) return prc;
  }
  if (gx != nullptr) {
    int S = 128;  // 3 CTAs per SM at 128 features: the walk over the trees is latency bound
    while (S > 32 && (size_t)S * p->C * 4 > 200 * 1024) S >>= 1;
    const size_t smem = (size_t)S * p->C * 4;
    if (smem > kSmemBudget) return HT_ERR_UNSUPPORTED;
    auto kernel = where_bytes(p->depth) == 2 ? reduce_x_records_kernel<unsigned short> : reduce_x_records_kernel<uint32_t>;
    HT_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBudget));
    kernel<<<(unsigned)((samples + S - 1) / S), S, smem, stream>>>(a.evals, ord, samples, p->K, p->T, N, (int)p->C, S, gx);
    HT_CHECK_LAUNCH();
  }
  return HT_OK;
}

// Samples per CTA of expand_saved_kernel: 256 when the gradient tile, the gradient boxes and the table buffers
// fit, else 128; 0 when even that does not fit.
static size_t expand_smem_bytes(const ht_forest_problem *p, int S, bool with_tile) {
  const size_t tables = 2 * saved_table_bytes(threshold_count(p->kind, p->depth), ((int64_t)1) << p->depth);
  return 1024 + 2 * (size_t)S * kSavedBatch * 4 + tables + 64 + (with_tile ? (size_t)S * p->C * 4 : 0);
}

int saved_samples_per_cta(const ht_forest_problem *p) {
  for (int S = 256; S >= 128; S >>= 1)
    if (expand_smem_bytes(p, S, true) <= kSmemBudget) return S;
  return 0;
}

int backward_saved(const ht_forest_problem *p, const int32_t *ord, const float *w, const float *g, float *gx, float *gthr,
                   float *gw, void *eval_records, cudaStream_t stream) {
  if (!forward_saves(p) || eval_records == nullptr) return HT_ERR_UNSUPPORTED;
  if (((reinterpret_cast<uintptr_t>(g) | reinterpret_cast<uintptr_t>(gx) | reinterpret_cast<uintptr_t>(w) |
        reinterpret_cast<uintptr_t>(ord)) & 15u) != 0)
    return HT_ERR_UNSUPPORTED;
  const int S = saved_samples_per_cta(p);
  if (S == 0) return HT_ERR_UNSUPPORTED;
  const int64_t N = threshold_count(p->kind, p->depth);
  const int64_t L = ((int64_t)1) << p->depth;
  const bool params = gthr != nullptr || gw != nullptr;
  ExpandArgs a = {};
  if (!tma::encode_matrix_f32(&a.g_map, g, p->B, p->T, S, kSavedBatch)) return HT_ERR_UNSUPPORTED;
  a.r = eval_record_arrays(p, eval_records);
  a.ord = ord;
  a.w = w;
  a.gx = gx;
  a.B = p->B;
  a.T = p->T;
  a.N = (int)N;
  a.L = (int)L;
  a.C = (int)p->C;
  a.write_terms = params ? 1 : 0;
  const bool narrow = where_bytes(p->depth) == 2;
  auto kernel = narrow ? expand_saved_kernel<unsigned short> : expand_saved_kernel<uint32_t>;
  if (narrow && p->kind == TREE && S == 256 && params && gx != nullptr) {  // the usual training step: fixed sizes
    if (p->depth == 5) kernel = expand_saved_kernel<unsigned short, 5>;
    if (p->depth == 6) kernel = expand_saved_kernel<unsigned short, 6>;
    if (p->depth == 7) kernel = expand_saved_kernel<unsigned short, 7>;
    if (p->depth == 8) kernel = expand_saved_kernel<unsigned short, 8>;
  }
  HT_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBudget));
  kernel<<<(unsigned)((p->B + S - 1) / S), S, expand_smem_bytes(p, S, gx != nullptr), stream>>>(a);
  HT_CHECK_LAUNCH();
  if (!params) return HT_OK;
  // the records now hold what the backward's traversal kernel writes: the same reductions, either mode
  return narrow ? reduce_parameters<unsigned short>(p, a.r, p->B, N, L, gthr, gw, stream)
                : reduce_parameters<uint32_t>(p, a.r, p->B, N, L, gthr, gw, stream);
}

}  // namespace ht
