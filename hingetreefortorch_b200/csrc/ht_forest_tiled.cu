// Shared-memory tile kernels for the forest forward.
//
// forest_forward_tiled_kernel: tabular input (K == 1), one or several outputs per leaf.
// forest_forward_tiled_inner_kernel: inputs with inner positions (x [B, C, K...]), one output per leaf.
//
// Work decomposition (one CTA of 1024 threads per tile, sized for one CTA per SM):
//   * a CTA owns S consecutive samples and walks ALL trees (or, when the batch alone gives too
//     few tiles for the machine, its share of the tree groups), so every input element is read
//     from HBM once;
//   * the samples' features sit in shared memory feature-major, xs[c][s]: lane l of a warp
//     always reads bank l whatever feature its current vertex tests, so the data gather never
//     conflicts although the 32 lanes are at 32 different vertices;
//   * a warp is (sample group, slot): S/32 sample groups of 32 samples, 32/(S/32) slots.  Trees
//     are processed in groups of G; inside a group slot q owns G/slots consecutive trees and
//     walks them all at once (independent dependent-load chains hide shared-memory latency);
//   * tree parameters arrive as per-tree records {root and its two children for a single
//     broadcast load, thresholds, feature indices, leaf weights in path order}, written once per
//     call by a small repack kernel, and are streamed into shared memory with 1-D bulk async
//     copies (cp.async.bulk, the TMA engine) completing on an mbarrier.  Two buffers; the last
//     warp to finish a group issues the copy that refills its buffer, so no warp ever waits for
//     another in order to keep the pipeline fed.  One-byte feature indices are stored as words
//     {own, left child's, right child's} of the even-level vertices, one load for two levels;
//   * tabular results of a group are transposed through a per-sample-group staging area (named
//     barriers over the 4..32 warps of the sample group only) and leave as row segments; with
//     inner positions consecutive samples are consecutive positions of the same output row, so
//     the results leave straight from registers.
//
// Only the smallest |margin| matters in the forward, so the minimum is tracked on absolute
// values.  CUDA's fminf ignores a NaN operand; the reference keeps a NaN only when the root
// margin is NaN, which is patched after the loop.
//
// The vertex index is kept 1-based (root 1, children 2v and 2v+1) so that one funnel shift
// appends the branch bit.  The bit is the sign of (threshold - feature): it is set exactly
// when the margin (feature - threshold) is positive, given that records hold +0 for a -0
// threshold and that an add producing NaN produces the canonical positive NaN (so NaN margins
// go left, as `margin > 0` does in the reference).  |threshold - feature| equals
// |feature - threshold| bit for bit.
#include "ht_eval_records.cuh"
#include "ht_forest_tiled.cuh"
#include "ht_tile_common.cuh"
#include "ht_tma.cuh"

#include <algorithm>
#include <type_traits>

namespace ht {

using namespace tile;

namespace {


struct TilePlan {
  int S;           // samples per tile
  int G;           // trees per parameter group
  int per_warp;    // trees a warp walks at once: G / slots
  int ord_bytes;   // 1 or 2
  RecordLayout rec;
  size_t smem;
};

// Shared-memory layout of forest_forward_tiled_kernel, from a 1024-byte boundary: the results area (a
// staging row per sample with one output per leaf — boxes the TMA engine can store —, or the warps'
// (margin, leaf) pairs), the feature tile, two parameter buffers, the barriers.
__host__ __device__ inline size_t results_bytes(bool one_output, int S, int G) {
  const size_t bytes = one_output ? (size_t)S * (G + 1) * 4 : (size_t)kWarps * 32 * 4 * 8;
  return (bytes + 1023) & ~(size_t)1023;
}

// 16-byte loads a thread keeps in flight while it stages the feature tile (1, 2, 4, 8 measured on the benchmark shape:
// 3.86, 3.80, 3.89, 3.80 ms; 8 spills a register)
constexpr int kStageLoads = 2;

bool make_plan(const ht_forest_problem *p, TilePlan &plan) {
  if (p->K != 1 || p->M < 1 || p->M > 64) return false;
  if (p->C > 65536 || p->depth > 12) return false;
  if (p->B * p->T < 32 * 1024) return false;  // too small to fill the machine with sample tiles
  plan.ord_bytes = p->C <= 256 ? 1 : 2;
  plan.rec = record_layout(p->kind, p->depth, (uint32_t)plan.ord_bytes, p->M == 1,
                           paired_ordinals(p->kind, p->depth, (uint32_t)plan.ord_bytes));
  for (int S = 256; S >= 32; S >>= 1) {
    const int slots = kWarps / (S / 32);
    for (int per_warp = 4; per_warp >= 1; per_warp >>= 1) {
      const int G = slots * per_warp;
      plan.S = S;
      plan.G = G;
      plan.per_warp = per_warp;
      // results: a staging row per sample (one output per leaf), or the warps' (margin, leaf) pairs
      plan.smem = 1024 + results_bytes(p->M == 1, S, G) + (size_t)p->C * S * 4 + 2 * (size_t)G * plan.rec.bytes + 64;
      if (plan.smem <= kSmemBudget) return true;
    }
  }
  return false;
}

// Inputs with inner positions (x [B, C, K], K > 1; one output per leaf): a sample is a (row, position)
// pair and its features are K elements apart, so consecutive samples of a tile are consecutive
// positions — contiguous in x and, for a fixed tree, in the output.  No staging of results is needed.
bool make_inner_plan(const ht_forest_problem *p, TilePlan &plan) {
  if (p->K <= 1 || p->M != 1) return false;
  if (p->C > 65536 || p->depth > 12) return false;
  if (p->B * p->K * p->T < 32 * 1024) return false;
  plan.ord_bytes = p->C <= 256 ? 1 : 2;
  plan.rec = record_layout(p->kind, p->depth, (uint32_t)plan.ord_bytes, true,
                           paired_ordinals(p->kind, p->depth, (uint32_t)plan.ord_bytes));
  plan.per_warp = 4;
  for (int S = 256; S >= 32; S >>= 1) {
    plan.S = S;
    plan.G = (kWarps / (S / 32)) * plan.per_warp;
    plan.smem = (size_t)p->C * S * 4 + 2 * (size_t)plan.G * plan.rec.bytes + 64;
    if (plan.smem <= kSmemBudget) return true;
  }
  return false;
}

struct TiledArgs {
  CUtensorMap out_map;  // the output [B, T] in boxes of 32 rows x G trees (when tma_store is set)
  const float *x;
  const unsigned char *records;
  const float *w;  // leaf weights in global memory, read when there are several outputs per leaf
  float *out;
  uint32_t *status_word;
  int64_t B, T, K;
  int C, S, G, per_warp, M;
  int tma_store;  // results of full groups leave through the TMA engine (G is 16 or 32)
  // a forward that saves its traversal for the backward (SAVE kernels): threshold - feature at the deciding
  // vertex, and the packed vertex / leaf key, in the evaluation-record layout
  float *save_margin;
  void *save_where;
};

template <int KIND, int DEPTH, typename OrdT, bool WREC, bool SAVE = false>
__global__ void __launch_bounds__(kThreads, 1) forest_forward_tiled_kernel(const __grid_constant__ TiledArgs a) {
  extern __shared__ __align__(1024) unsigned char smem[];
  constexpr RecordLayout lay =
      record_layout(KIND, DEPTH, (uint32_t)sizeof(OrdT), WREC, paired_ordinals(KIND, DEPTH, (uint32_t)sizeof(OrdT)));
  const int S = a.S, G = a.G, C = a.C;
  const int M = WREC ? 1 : a.M;
  // staging row of one sample (one output per leaf): G trees, padded against bank conflicts; dense when
  // the area holds the TMA boxes, so that a sample group's rows stay inside its own box
  const int row_floats = a.tma_store != 0 ? G : G + 1;
  unsigned char *base = smem + ((1024u - (smem_addr(smem) & 1023u)) & 1023u);
  float *outs = reinterpret_cast<float *>(base);
  float *xs = reinterpret_cast<float *>(base + results_bytes(WREC, S, G));
  unsigned char *params = reinterpret_cast<unsigned char *>(xs + (size_t)C * S);
  uint64_t *full = reinterpret_cast<uint64_t *>(params + 2 * (size_t)G * lay.bytes);  // [2] copy landed
  uint32_t *finished = reinterpret_cast<uint32_t *>(full + 2);                         // [2] warps done with a buffer

  const int tid = threadIdx.x;
  const int lane = tid & 31, warp = tid >> 5;
  const int groups_of_samples = S >> 5;
  const int slots = kWarps / groups_of_samples;
  const int sample_group = warp % groups_of_samples;
  const int slot = warp / groups_of_samples;
  const int64_t row0 = (int64_t)blockIdx.x * S;
  // blockIdx.y splits the tree groups among CTAs when there are too few sample tiles to fill the
  // machine; this CTA walks groups [group0, group0 + num_groups), `it` counts them from 0
  const int all_groups = (int)((a.T + G - 1) / G);
  const int groups_per_cta = (all_groups + (int)gridDim.y - 1) / (int)gridDim.y;
  const int group0 = (int)blockIdx.y * groups_per_cta;
  const int num_groups = max(0, min(groups_per_cta, all_groups - group0));
  const uint32_t params_addr = smem_addr(params);

  const int per_warp = a.per_warp;
  auto issue = [&](int it) {
    const int64_t first_tree = (int64_t)(group0 + it) * G;
    const int64_t count = min((int64_t)G, a.T - first_tree);
    const uint32_t bytes = (uint32_t)(count * lay.bytes);
    uint64_t *bar = &full[it & 1];
    mbar_expect_tx(bar, bytes);
    bulk_load(params_addr + (uint32_t)(it & 1) * (uint32_t)G * lay.bytes, a.records + first_tree * lay.bytes, bytes, bar);
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

  // Stage the tile's features: lanes run along samples so that the shared-memory writes are
  // conflict free; each lane fetches 16 bytes of its row at a time when the row allows it.
  if ((C & 3) == 0) {
    // several 16-byte loads in flight per thread before the first is stored: the tile comes from HBM, and a loop that
    // waits for each load in turn spends a memory round trip per pass
    const int quads = C >> 2;
    const int total = S * quads;
    for (int idx0 = tid; idx0 < total; idx0 += kStageLoads * kThreads) {
      float4 v[kStageLoads];
#pragma unroll
      for (int u = 0; u < kStageLoads; ++u) {
        const int idx = idx0 + u * kThreads;
        const int s = idx % S, q = idx / S;
        v[u] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (idx < total && row0 + s < a.B) v[u] = __ldg(reinterpret_cast<const float4 *>(a.x + (row0 + s) * C) + q);
      }
#pragma unroll
      for (int u = 0; u < kStageLoads; ++u) {
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
  __syncthreads();  // features staged; barrier initialisation visible

  const uint32_t xl_addr = smem_addr(xs + sample_group * 32 + lane);
  const uint32_t x_stride = (uint32_t)S * 4u;
  float *stage = outs + (size_t)sample_group * 32 * row_floats;  // this sample group's [32][G*M + 1] staging rows
  const int group_threads = slots * 32;
  const int tid_in_group = slot * 32 + lane;
  constexpr uint32_t kL = 1u << DEPTH;
  bool poisoned = false;  // a bounded wait ran out: keep the barriers matched, stop waiting
  // Output of a full group when its 32 x (G*M/4) 16-byte pieces are one per thread of the sample
  // group (the usual case): which piece is this thread's, worked out once
  const int full_groups = (int)(a.T / G), tail_trees = (int)(a.T - (int64_t)full_groups * G);  // a.T < 2^31 * G
  const int full_quads = (G * M) >> 2;
  const int64_t row_pitch = a.T * M;
  const bool one_piece = ((G * M) & 3) == 0 && (row_pitch & 3) == 0 && 32 * full_quads == group_threads;
  const int piece_row = one_piece ? tid_in_group / full_quads : 0;
  const int piece_quad = one_piece ? tid_in_group - piece_row * full_quads : 0;
  const int64_t piece_sample = row0 + sample_group * 32 + piece_row;
  float *piece_dst = a.out + piece_sample * row_pitch + 4 * piece_quad;
  const float *piece_src = stage + piece_row * row_floats + 4 * piece_quad;
  // Full groups with 4 trees per warp and the weights in the records take a body without the
  // bookkeeping of short groups, other tree counts and several outputs per leaf.
  const bool streamlined = WREC && one_piece && per_warp == 4;
  const uint32_t warp_records = (uint32_t)(slot * per_warp) * lay.bytes;
  float *stage_mine = stage + lane * row_floats + slot * per_warp;
  // TMA form of the streamlined body: this sample group's box of 32 rows x G floats, and where this
  // lane's 4 results (chunk `slot` of row `lane`) sit in it
  const bool tma_store = streamlined && a.tma_store != 0;
  const bool store_issuer = tma_store && slot == 0 && lane == 0;
  const uint32_t box_addr = smem_addr(outs) + (uint32_t)sample_group * 32u * (uint32_t)G * 4u;
  const uint32_t box_mine = box_addr + (G == 16 ? tma::swizzled_offset<16>((uint32_t)lane, (uint32_t)slot)
                                                : tma::swizzled_offset<32>((uint32_t)lane, (uint32_t)slot));

  // This warp no longer reads parameter buffer (it & 1).  The last warp to say so refills it.
  auto done_with_buffer = [&](int it) {
    __syncwarp();
    if (lane == 0) {
      uint32_t before;  // wraps to zero with the last warp: acquire / release order the warps' reads before the refill
      asm volatile("atom.acq_rel.cta.shared::cta.inc.u32 %0, [%1], %2;"
                   : "=r"(before)
                   : "r"(smem_addr(&finished[it & 1])), "r"((uint32_t)kWarps - 1u)
                   : "memory");
      if (before == (uint32_t)kWarps - 1u && it + 2 < num_groups) issue(it + 2);
    }
  };

  int it = 0;
  if (tma_store) {
    // The loop of the benchmark shapes, with nothing in it that the full groups of a forest with the
    // weights in its records do not need: one register addresses the warp's four consecutive records,
    // and the buffer goes back with one atomic (it wraps to zero with the last warp, which refills).
    const int fast = max(0, min(num_groups, full_groups - group0));
    for (; it < fast; ++it) {
      const uint32_t buffer = (uint32_t)(it & 1);
      if (!poisoned && !mbar_wait(&full[buffer], (uint32_t)((it >> 1) & 1))) {
        poisoned = true;
        if (a.status_word != nullptr) atomicOr(a.status_word, HT_FLAG_PIPELINE_TIMEOUT);
      }
      const uint32_t first_record = params_addr + buffer * (uint32_t)G * lay.bytes + warp_records;
      float result[4] = {0.f, 0.f, 0.f, 0.f};
      if constexpr (SAVE) {
        // the walk of the backward (signed margin, deciding vertex, path): the same |margin| * leaf weight leaves as
        // the result, and the traversal itself goes to the evaluation records, from registers (consecutive lanes
        // are consecutive samples: 128 and 64 contiguous bytes per tree)
        using WhereT = typename std::conditional<(DEPTH <= 8), unsigned short, uint32_t>::type;
        const int64_t sample = row0 + sample_group * 32 + lane;
        const int64_t at = record_index(sample, (int64_t)(group0 + it) * G + slot * 4, a.T);
        uint32_t rec[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) rec[u] = first_record + (uint32_t)u * lay.bytes;
        Walked wk[4];
        if (!poisoned) {
          walk_full<KIND, DEPTH, OrdT, 4, lay.paired>(rec, xl_addr, x_stride, wk);
#pragma unroll
          for (int u = 0; u < 4; ++u)
            result[u] = __fmul_rn(fabsf(wk[u].nm), lds_f32(rec[u] + 4u * wk[u].path + (lay.w - 4u * (1u << DEPTH))));
        } else {
#pragma unroll
          for (int u = 0; u < 4; ++u) wk[u] = Walked{0.0f, 1u, 1u << DEPTH};
        }
        if (sample < a.B) {
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            __stcs(a.save_margin + at + u * kRecordBlock, wk[u].nm);
            store_where<WhereT>(a.save_where, at + u * kRecordBlock, wk[u].v, __brev(wk[u].path - (1u << DEPTH)) >> (32 - DEPTH));
          }
        }
      } else {
        const uint32_t rec[4] = {first_record, 0u, 0u, 0u};
        uint32_t unused[4];
        if (!poisoned) walk<KIND, DEPTH, OrdT, 4, WREC, true>(rec, xl_addr, x_stride, result, unused);
      }
      done_with_buffer(it);
      if (store_issuer) tma::wait_stores_read();  // the previous box has been read out of the staging area
      named_barrier(1 + sample_group, group_threads);
      sts_b128(box_mine, result[0], result[1], result[2], result[3]);
      tma::fence_async_shared();
      named_barrier(1 + sample_group, group_threads);  // box complete and visible to the TMA engine
      if (store_issuer) {
        tma::store_2d(&a.out_map, box_addr, (group0 + it) * G, (int)(row0 + sample_group * 32));
        tma::commit_group();
      }
    }
  }
  for (; it < num_groups; ++it) {
    const int group = group0 + it;
    if (!poisoned && !mbar_wait(&full[it & 1], (uint32_t)((it >> 1) & 1))) {
      poisoned = true;
      if (a.status_word != nullptr) atomicOr(a.status_word, HT_FLAG_PIPELINE_TIMEOUT);
    }
    const int in_group = group < full_groups ? G : tail_trees;
    const uint32_t base_addr = params_addr + (uint32_t)(it & 1) * (uint32_t)G * lay.bytes;
    if (streamlined && in_group == G) {
      uint32_t rec[4], unused[4];
      float result[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int u = 0; u < 4; ++u) rec[u] = base_addr + warp_records + (uint32_t)u * lay.bytes;
      if (SAVE) {
        // the walk of the backward (signed margin, deciding vertex, path): the same |margin| * leaf weight
        // leaves as the result, and the traversal itself goes to the evaluation records, from registers
        // (consecutive lanes are consecutive samples: 128 and 64 contiguous bytes per tree)
        using WhereT = typename std::conditional<(DEPTH <= 8), unsigned short, uint32_t>::type;
        const int64_t sample = row0 + sample_group * 32 + lane;
        const int64_t at = record_index(sample, (int64_t)group * G + slot * 4, a.T);
        Walked wk[4];
        if (!poisoned) {
          walk_full<KIND, DEPTH, OrdT, 4, lay.paired>(rec, xl_addr, x_stride, wk);
#pragma unroll
          for (int u = 0; u < 4; ++u)
            result[u] = __fmul_rn(fabsf(wk[u].nm), lds_f32(rec[u] + 4u * wk[u].path + (lay.w - 4u * (1u << DEPTH))));
        } else {
#pragma unroll
          for (int u = 0; u < 4; ++u) wk[u] = Walked{0.0f, 1u, 1u << DEPTH};
        }
        if (sample < a.B) {
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            __stcs(a.save_margin + at + u * kRecordBlock, wk[u].nm);
            store_where<WhereT>(a.save_where, at + u * kRecordBlock, wk[u].v, __brev(wk[u].path - (1u << DEPTH)) >> (32 - DEPTH));
          }
        }
      } else if (!poisoned) {
        walk<KIND, DEPTH, OrdT, 4, WREC>(rec, xl_addr, x_stride, result, unused);  // a buffer that never arrived is not read
      }
      done_with_buffer(it);
      if (tma_store) {
        // The sample group's [32 samples x G trees] block goes to shared memory in the swizzled box layout
        // (a lane writes the 16 bytes of its own row: conflict free) and leaves as ONE tiled TMA store.
        if (store_issuer) tma::wait_stores_read();  // the previous box has been read out of the staging area
        named_barrier(1 + sample_group, group_threads);
        sts_b128(box_mine, result[0], result[1], result[2], result[3]);
        tma::fence_async_shared();
        named_barrier(1 + sample_group, group_threads);  // box complete and visible to the TMA engine
        if (store_issuer) {
          tma::store_2d(&a.out_map, box_addr, group * G, (int)(row0 + sample_group * 32));
          tma::commit_group();
        }
        continue;
      }
      named_barrier(1 + sample_group, group_threads);  // previous group's rows have left the staging area
#pragma unroll
      for (int u = 0; u < 4; ++u) stage_mine[u] = result[u];
      named_barrier(1 + sample_group, group_threads);  // staging area complete
      if (piece_sample < a.B)
        *reinterpret_cast<float4 *>(piece_dst + (int64_t)group * G) =
            make_float4(piece_src[0], piece_src[1], piece_src[2], piece_src[3]);
      continue;
    }
    if (store_issuer) tma::wait_stores_read();  // the body below writes the staging area with plain stores
    const int t_first = slot * per_warp;  // this warp's consecutive trees inside the group
    float result[4] = {0.f, 0.f, 0.f, 0.f};
    uint32_t path[4] = {kL, kL, kL, kL};
    if (t_first < in_group && !poisoned) {  // after a lost copy the buffer is not read: zeros leave instead
      // trees beyond the end of a short last group repeat the last valid one (results unused)
      if (per_warp == 4) {
        uint32_t rec[4];
#pragma unroll
        for (int u = 0; u < 4; ++u)
          rec[u] = base_addr + (uint32_t)(in_group == G ? t_first + u : min(t_first + u, in_group - 1)) * lay.bytes;
        walk<KIND, DEPTH, OrdT, 4, WREC>(rec, xl_addr, x_stride, result, path);
      } else if (per_warp == 2) {
        uint32_t rec[2], p2[2];
#pragma unroll
        for (int u = 0; u < 2; ++u) rec[u] = base_addr + (uint32_t)min(t_first + u, in_group - 1) * lay.bytes;
        float r2[2];
        walk<KIND, DEPTH, OrdT, 2, WREC>(rec, xl_addr, x_stride, r2, p2);
        result[0] = r2[0];
        result[1] = r2[1];
        path[0] = p2[0];
        path[1] = p2[1];
      } else {
        uint32_t rec[1] = {base_addr + (uint32_t)t_first * lay.bytes}, p1[1];
        float r1[1];
        walk<KIND, DEPTH, OrdT, 1, WREC>(rec, xl_addr, x_stride, r1, p1);
        result[0] = r1[0];
        path[0] = p1[0];
      }
    }
    done_with_buffer(it);

    const int64_t col0 = (int64_t)group * G;
    if (!WREC) {
      // Several outputs per leaf: out[i, j, :] = |margin| * w[j, leaf, :], and the warp's trees
      // j .. j + n - 1 of one sample are n * M consecutive outputs.  Every lane leaves its (|margin|, leaf)
      // pairs in the warp's corner of shared memory; then the warp writes the 32 samples' runs one after
      // another, lane by lane along a run, reading the weight rows from global memory (L2 resident)
      // the same way: loads and stores are contiguous whatever leaves the samples reached.
      const int trees_here = min(per_warp, in_group - t_first);  // <= 0: nothing for this warp in a short group
      float2 *pairs = reinterpret_cast<float2 *>(outs) + (size_t)warp * 32 * 4;
      __syncwarp();
#pragma unroll
      for (int u = 0; u < 4; ++u)
        pairs[lane * 4 + u] = make_float2(result[u], __uint_as_float(__brev(path[u] - kL) >> (32 - DEPTH)));
      __syncwarp();
      if (trees_here > 0) {
        const int run = trees_here * M;  // outputs of one sample that this warp owns, contiguous
        const int64_t first_row = row0 + sample_group * 32;
        const int rows_here = (int)min((int64_t)32, a.B - first_row);
        const float *w_first = a.w + (col0 + t_first) * (int64_t)kL * M;
        float *dst = a.out + first_row * row_pitch + (col0 + t_first) * M;
        // Lane l writes element l, l + 32, ... of every sample's run: which tree and which output
        // that is does not depend on the sample, so it is worked out once per pass and the loop
        // over the samples is a pair load, a weight load, a multiply and a store.
        for (int e = lane; e < run; e += 32) {
          const int u = (e >= M) + (e >= 2 * M) + (e >= 3 * M), m = e - u * M;  // run <= 4 * M
          const float *w_tree = w_first + (int64_t)u * kL * M + m;
          const float2 *pair_of = pairs + u;
          float *to = dst + e;
          int sample = 0;
          for (; sample + 4 <= rows_here; sample += 4) {
            float2 pr[4];
            float weight[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) pr[k] = pair_of[(sample + k) * 4];
#pragma unroll
            for (int k = 0; k < 4; ++k) weight[k] = __ldg(w_tree + (int64_t)__float_as_uint(pr[k].y) * M);
#pragma unroll
            for (int k = 0; k < 4; ++k) to[(int64_t)(sample + k) * row_pitch] = pr[k].x * weight[k];
          }
          for (; sample < rows_here; ++sample) {
            const float2 pr = pair_of[sample * 4];
            to[(int64_t)sample * row_pitch] = pr.x * __ldg(w_tree + (int64_t)__float_as_uint(pr.y) * M);
          }
        }
      }
      continue;
    }
    named_barrier(1 + sample_group, group_threads);  // previous group's rows have left the staging area
#pragma unroll
    for (int u = 0; u < 4; ++u)
      if (u < per_warp && t_first + u < in_group) stage[lane * row_floats + t_first + u] = result[u];
    named_barrier(1 + sample_group, group_threads);  // staging area complete

    // the sample group's warps write its [32 x in_group*M] block of results as row segments
    const int64_t row_base = row0 + sample_group * 32;
    const int width = in_group * M;
    const int64_t first_col = col0 * M;
    if (one_piece && in_group == G) {
      if (piece_sample < a.B)
        *reinterpret_cast<float4 *>(piece_dst + first_col) = make_float4(piece_src[0], piece_src[1], piece_src[2], piece_src[3]);
    } else if ((row_pitch & 3) == 0 && (first_col & 3) == 0 && (width & 3) == 0) {
      const int quads = width >> 2;
      for (int idx = tid_in_group; idx < 32 * quads; idx += group_threads) {
        const int s = idx / quads, q = idx - s * quads;
        if (row_base + s < a.B) {
          const float *src = stage + s * row_floats + 4 * q;
          *reinterpret_cast<float4 *>(a.out + (row_base + s) * row_pitch + first_col + 4 * q) =
              make_float4(src[0], src[1], src[2], src[3]);
        }
      }
    } else {
      for (int idx = tid_in_group; idx < 32 * width; idx += group_threads) {
        const int s = idx / width, t = idx - s * width;
        if (row_base + s < a.B) a.out[(row_base + s) * row_pitch + first_col + t] = stage[s * row_floats + t];
      }
    }
  }
  if (store_issuer) tma::wait_stores_read();  // shared memory stays valid until the last box has been read
}

template <int KIND, int DEPTH, typename OrdT>
__global__ void __launch_bounds__(kThreads, 1) forest_forward_tiled_inner_kernel(const __grid_constant__ TiledArgs a) {
  extern __shared__ __align__(1024) unsigned char smem[];
  constexpr RecordLayout lay =
      record_layout(KIND, DEPTH, (uint32_t)sizeof(OrdT), true, paired_ordinals(KIND, DEPTH, (uint32_t)sizeof(OrdT)));
  const int S = a.S, G = a.G, C = a.C;
  float *xs = reinterpret_cast<float *>(smem);
  unsigned char *params = smem + (size_t)C * S * 4;
  uint64_t *full = reinterpret_cast<uint64_t *>(params + 2 * (size_t)G * lay.bytes);
  uint32_t *finished = reinterpret_cast<uint32_t *>(full + 2);

  const int tid = threadIdx.x;
  const int lane = tid & 31, warp = tid >> 5;
  const int groups_of_samples = S >> 5;
  const int sample_group = warp % groups_of_samples;
  const int slot = warp / groups_of_samples;
  const int64_t samples = a.B * a.K;
  const int64_t sample0 = (int64_t)blockIdx.x * S;
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
    bulk_load(params_addr + (uint32_t)(it & 1) * (uint32_t)G * lay.bytes, a.records + first_tree * lay.bytes, bytes, bar);
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

  // features of the tile's samples, feature-major; consecutive samples are consecutive positions.
  // A thread stages the features c0, c0 + step, ... of one sample, or of 4 consecutive positions
  // at a time when the rows allow 16-byte loads (S divides the thread count; a tile starts on a
  // multiple of S, so 4 positions never straddle a row when 4 divides K)
  if ((a.K & 3) == 0) {
    const int quads = S >> 2, t = (tid % quads) * 4, c_step = kThreads / quads;
    const int64_t sample = sample0 + t;
    const bool inside = sample < samples;  // then sample + 3 < samples as well
    const int64_t row = inside ? sample / a.K : 0, k = inside ? sample - row * a.K : 0;
    const float *src = a.x + row * C * a.K + k;
    for (int c = tid / quads; c < C; c += c_step) {
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if (inside) v = __ldg(reinterpret_cast<const float4 *>(src + (int64_t)c * a.K));
      *reinterpret_cast<float4 *>(xs + c * S + t) = v;
    }
  } else {
    const int t = tid % S, c_step = kThreads / S;
    const int64_t sample = sample0 + t;
    const bool inside = sample < samples;
    const int64_t row = inside ? sample / a.K : 0, k = inside ? sample - row * a.K : 0;
    const float *src = a.x + row * C * a.K + k;
    for (int c = tid / S; c < C; c += c_step) xs[c * S + t] = inside ? __ldg(src + (int64_t)c * a.K) : 0.0f;
  }
  __syncthreads();

  const int64_t my_sample = sample0 + sample_group * 32 + lane;
  const bool valid = my_sample < samples;
  const int64_t my_row = valid ? my_sample / a.K : 0, my_k = valid ? my_sample - my_row * a.K : 0;
  float *my_out = a.out + my_row * a.T * a.K + my_k;  // tree j of this sample: + j * K
  const uint32_t xl_addr = smem_addr(xs + sample_group * 32 + lane);
  const uint32_t x_stride = (uint32_t)S * 4u;
  const int t_first = slot * 4;
  bool poisoned = false;

  for (int it = 0; it < num_groups; ++it) {
    const int group = group0 + it;
    if (!poisoned && !mbar_wait(&full[it & 1], (uint32_t)((it >> 1) & 1))) {
      poisoned = true;
      if (a.status_word != nullptr) atomicOr(a.status_word, HT_FLAG_PIPELINE_TIMEOUT);
    }
    const int in_group = (int)min((int64_t)G, a.T - (int64_t)group * G);
    const uint32_t base_addr = params_addr + (uint32_t)(it & 1) * (uint32_t)G * lay.bytes;
    float result[4] = {0.f, 0.f, 0.f, 0.f};
    if (t_first < in_group && !poisoned) {
      uint32_t rec[4], unused[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) rec[u] = base_addr + (uint32_t)min(t_first + u, in_group - 1) * lay.bytes;
      walk<KIND, DEPTH, OrdT, 4, true>(rec, xl_addr, x_stride, result, unused);
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
    if (valid) {
      float *dst = my_out + ((int64_t)group * G + t_first) * a.K;
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (t_first + u < in_group) dst[(int64_t)u * a.K] = result[u];
    }
  }
}

template <typename Kernel>
int launch_one(Kernel kernel, const TilePlan &plan, const TiledArgs &a, dim3 grid, cudaStream_t stream) {
  HT_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBudget));
  kernel<<<grid, kThreads, plan.smem, stream>>>(a);
  HT_CHECK_LAUNCH();
  return HT_OK;
}

template <int KIND, int DEPTH>
int launch_depth(const TilePlan &plan, const TiledArgs &a, dim3 grid, cudaStream_t stream) {
  if (a.K > 1) {
    if (plan.ord_bytes == 1) return launch_one(forest_forward_tiled_inner_kernel<KIND, DEPTH, uint8_t>, plan, a, grid, stream);
    return launch_one(forest_forward_tiled_inner_kernel<KIND, DEPTH, uint16_t>, plan, a, grid, stream);
  }
  const bool wrec = a.M == 1;
  if (a.save_margin != nullptr) {
    if (plan.ord_bytes == 1)
      return launch_one(forest_forward_tiled_kernel<KIND, DEPTH, uint8_t, true, true>, plan, a, grid, stream);
    return launch_one(forest_forward_tiled_kernel<KIND, DEPTH, uint16_t, true, true>, plan, a, grid, stream);
  }
  if (plan.ord_bytes == 1)
    return wrec ? launch_one(forest_forward_tiled_kernel<KIND, DEPTH, uint8_t, true>, plan, a, grid, stream)
                : launch_one(forest_forward_tiled_kernel<KIND, DEPTH, uint8_t, false>, plan, a, grid, stream);
  return wrec ? launch_one(forest_forward_tiled_kernel<KIND, DEPTH, uint16_t, true>, plan, a, grid, stream)
              : launch_one(forest_forward_tiled_kernel<KIND, DEPTH, uint16_t, false>, plan, a, grid, stream);
}

template <int KIND>
int launch_kind(int depth, const TilePlan &plan, const TiledArgs &a, dim3 grid, cudaStream_t stream) {
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

}  // namespace

size_t forward_tiled_workspace_bytes(const ht_forest_problem *p) {
  TilePlan plan;
  if (!(p->K > 1 ? make_inner_plan(p, plan) : make_plan(p, plan))) return 0;
  return align_up((size_t)p->T * plan.rec.bytes, 256);
}

bool forward_saves(const ht_forest_problem *p) {
  TilePlan plan;
  if (p->K != 1 || p->M != 1 || !make_plan(p, plan)) return false;
  // every tree group takes the kernel's streamlined body: 4 trees per warp, no short last group
  // ... and the kernel that expands the records fits its tables into shared memory
  return plan.per_warp == 4 && p->T % plan.G == 0 && p->B <= 0x7fffffff && backward_records_bytes(p) > 0 &&
         saved_samples_per_cta(p) != 0;
}

int forward_tiled(const ht_forest_problem *p, const float *x, const float *thr, const int32_t *ord, const float *w,
                  float *out, void *records, void *eval_records, uint32_t *status_word, cudaStream_t stream) {
  TilePlan plan;
  if (!(p->K > 1 ? make_inner_plan(p, plan) : make_plan(p, plan))) return HT_ERR_UNSUPPORTED;
  if ((reinterpret_cast<uintptr_t>(x) & 15u) != 0 || (reinterpret_cast<uintptr_t>(out) & 15u) != 0)
    return HT_ERR_UNSUPPORTED;
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

  TiledArgs a = {};
  a.x = x;
  a.records = rec;
  a.w = w;
  a.M = (int)p->M;
  a.out = out;
  a.status_word = status_word;
  a.B = p->B;
  a.T = p->T;
  a.K = p->K;
  a.C = (int)p->C;
  a.S = plan.S;
  a.G = plan.G;
  a.per_warp = plan.per_warp;
  a.save_margin = nullptr;
  a.save_where = nullptr;
  if (eval_records != nullptr && forward_saves(p)) {
    const EvalRecords saved = eval_record_arrays(p, eval_records);
    a.save_margin = saved.dx;
    a.save_where = saved.where;
  }
  // Full groups of 16 or 32 trees leave as tiled TMA stores when the output admits a tensor map
  // (rows of a multiple of 16 bytes); otherwise, and for a short last group, as row segments.
  a.tma_store = 0;
  if (p->K == 1 && p->M == 1 && plan.per_warp == 4 && (plan.G == 16 || plan.G == 32) && (p->T & 3) == 0 &&
      p->T >= plan.G && tma::encode_matrix_f32(&a.out_map, out, p->B, p->T, 32, plan.G))
    a.tma_store = 1;
  // With few sample tiles the tree groups are split among CTAs (grid.y) so that the SMs are busy in
  // every round; every split re-stages the feature tile, which is cheap next to the walk.
  const int64_t tiles = (p->B * p->K + plan.S - 1) / plan.S;
  if (tiles > 0x7fffffff) return HT_ERR_UNSUPPORTED;
  const int64_t groups = (p->T + plan.G - 1) / plan.G;
  const dim3 grid((unsigned)tiles, (unsigned)choose_splits(tiles, groups));
  return p->kind == TREE ? launch_kind<TREE>(p->depth, plan, a, grid, stream)
                         : launch_kind<FERN>(p->depth, plan, a, grid, stream);
}

}  // namespace ht

// ---- self test of the bounded wait ---------------------------------------------------------
namespace ht {
namespace {
// One warp waits on a barrier that nothing ever arrives on, with a limit of a few tries: the wait has to
// run out, the kernel has to set the flag and return with its context intact.  This is the path a lost
// parameter copy takes in the tile kernels, exercised without losing a copy.
__global__ void bounded_wait_selftest_kernel(uint32_t *status_word) {
  __shared__ uint64_t never;
  if (threadIdx.x == 0) {
    tile::mbar_init(&never, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  if (!tile::mbar_wait(&never, 0u, 8u) && threadIdx.x == 0) atomicOr(status_word, HT_FLAG_PIPELINE_TIMEOUT);
}
}  // namespace
}  // namespace ht

extern "C" int ht_selftest_bounded_wait(uint32_t *status_word, ht_stream_t stream) {
  if (status_word == nullptr) return HT_ERR_INVALID_ARGUMENT;
  ht::bounded_wait_selftest_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(status_word);
  HT_CHECK_LAUNCH();
  return HT_OK;
}
