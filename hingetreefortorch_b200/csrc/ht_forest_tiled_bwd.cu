// Shared-memory tile kernel for the forest backward on tabular input (K == 1, one output per leaf),
// default (not fixed-order) mode.
//
// Same tiling as the forward tile kernel (ht_forest_tiled.cu): a CTA owns S consecutive samples,
// keeps their features feature-major in shared memory and walks ALL trees, whose parameter
// records stream in through bulk async copies.  In addition:
//   * the x-gradient tile gx[c][s] lives in shared memory next to the features; contributions are
//     added with shared-memory atomics (the warps of a sample group work on different trees and
//     may hit the same element) and the tile leaves once, with plain stores -- no global atomics
//     and no clearing pass for the x gradient;
//   * the block of upstream gradients g[i, j0 .. j0+G) of a tree group is loaded as row segments
//     and transposed through the per-sample-group staging area;
//   * threshold and leaf-weight gradients are scattered with global reductions (red.global.add),
//     one per evaluation each.
// One traversal serves all three gradients (the reference runs three kernels that each repeat it,
// hingetree_gpu.cu:699-727).  The traversal keeps the signed margin and the deciding vertex, with
// the reference's strict `<` so that the shallowest minimum wins.
#include "ht_forest_tiled.cuh"
#include "ht_tile_common.cuh"

namespace ht {

using namespace tile;

namespace {

struct BwdPlan {
  int S, G, per_warp, ord_bytes;
  RecordLayout rec;
  size_t smem;
};

bool make_bwd_plan(const ht_forest_problem *p, BwdPlan &plan) {
  if (p->K != 1 || p->M != 1) return false;
  if (p->C > 65536 || p->depth > 12) return false;
  if (p->B * p->T < 32 * 1024) return false;
  plan.ord_bytes = p->C <= 256 ? 1 : 2;
  plan.rec = record_layout(p->kind, p->depth, (uint32_t)plan.ord_bytes);
  for (int S = 256; S >= 32; S >>= 1) {
    const int slots = kWarps / (S / 32);
    for (int per_warp = 4; per_warp >= 1; per_warp >>= 1) {
      const int G = slots * per_warp;
      plan.S = S;
      plan.G = G;
      plan.per_warp = per_warp;
      plan.smem = 2 * (size_t)p->C * S * 4 + 2 * (size_t)G * plan.rec.bytes + (size_t)S * (G + 1) * 4 + 64;
      if (plan.smem <= kSmemBudget) return true;
    }
  }
  return false;
}

struct BwdArgs {
  const float *x;
  const unsigned char *records;
  const float *g;
  float *gx, *gthr, *gw;
  uint32_t *status_word;
  int64_t B, T;
  int C, S, G, per_warp;
};

struct Walked {
  float nm;      // threshold - feature at the deciding vertex (the negated signed margin)
  uint32_t v;    // 1-based index of the deciding vertex (ferns: level + 1)
  uint32_t path; // 2^DEPTH + path bits, root first (most significant)
};

template <int KIND, int DEPTH, typename OrdT, int NT>
__device__ __forceinline__ void walk_full(const uint32_t (&rec)[NT], uint32_t xl_addr, uint32_t x_stride,
                                          Walked (&out)[NT]) {
  constexpr RecordLayout lay = record_layout(KIND, DEPTH, (uint32_t)sizeof(OrdT));
  uint32_t v[NT];
#pragma unroll
  for (int u = 0; u < NT; ++u) v[u] = 1u;
#pragma unroll
  for (int l = 0; l < DEPTH; ++l) {
#pragma unroll
    for (int u = 0; u < NT; ++u) {
      const uint32_t at = KIND == FERN ? (uint32_t)(l + 1) : v[u];
      const float thr = lds_f32(rec[u] + 4u * at + (lay.thr - 4u));
      const uint32_t c = lds_ord<OrdT>(rec[u] + (uint32_t)sizeof(OrdT) * at + (lay.ord - (uint32_t)sizeof(OrdT)));
      const float nm = thr - lds_f32(c * x_stride + xl_addr);
      if (l == 0 || fabsf(nm) < fabsf(out[u].nm)) {
        out[u].nm = nm;
        out[u].v = at;
      }
      v[u] = __funnelshift_l(__float_as_uint(nm), v[u], 1);
    }
  }
#pragma unroll
  for (int u = 0; u < NT; ++u) out[u].path = v[u];
}

template <int KIND, int DEPTH, typename OrdT>
__global__ void __launch_bounds__(kThreads, 1) forest_backward_tiled_kernel(BwdArgs a) {
  extern __shared__ __align__(128) unsigned char smem[];
  constexpr RecordLayout lay = record_layout(KIND, DEPTH, (uint32_t)sizeof(OrdT));
  constexpr uint32_t kN = KIND == FERN ? DEPTH : (1u << DEPTH) - 1u;
  constexpr uint32_t kL = 1u << DEPTH;
  const int S = a.S, G = a.G, C = a.C;
  float *xs = reinterpret_cast<float *>(smem);
  float *gxs = xs + (size_t)C * S;
  unsigned char *params = reinterpret_cast<unsigned char *>(gxs + (size_t)C * S);
  float *stage_all = reinterpret_cast<float *>(params + 2 * (size_t)G * lay.bytes);
  uint64_t *full = reinterpret_cast<uint64_t *>(stage_all + (size_t)S * (G + 1));
  uint32_t *finished = reinterpret_cast<uint32_t *>(full + 2);

  const int tid = threadIdx.x;
  const int lane = tid & 31, warp = tid >> 5;
  const int groups_of_samples = S >> 5;
  const int slots = kWarps / groups_of_samples;
  const int sample_group = warp % groups_of_samples;
  const int slot = warp / groups_of_samples;
  const int per_warp = a.per_warp;
  const int64_t row0 = (int64_t)blockIdx.x * S;
  const int num_groups = (int)((a.T + G - 1) / G);
  const uint32_t params_addr = smem_addr(params);

  auto issue = [&](int group) {
    const int64_t first_tree = (int64_t)group * G;
    const int64_t count = min((int64_t)G, a.T - first_tree);
    const uint32_t bytes = (uint32_t)(count * lay.bytes);
    uint64_t *bar = &full[group & 1];
    mbar_expect_tx(bar, bytes);
    bulk_load(params_addr + (uint32_t)(group & 1) * (uint32_t)G * lay.bytes, a.records + first_tree * lay.bytes, bytes,
              bar);
  };
  if (tid == 0) {
    mbar_init(&full[0], 1);
    mbar_init(&full[1], 1);
    finished[0] = 0;
    finished[1] = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    issue(0);
    if (num_groups > 1) issue(1);
  }

  // features in, x-gradient tile cleared
  if ((C & 3) == 0) {
    const int quads = C >> 2;
    for (int idx = tid; idx < S * quads; idx += kThreads) {
      const int s = idx % S, q = idx / S;
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if (row0 + s < a.B) v = __ldg(reinterpret_cast<const float4 *>(a.x + (row0 + s) * C) + q);
      xs[(4 * q + 0) * S + s] = v.x;
      xs[(4 * q + 1) * S + s] = v.y;
      xs[(4 * q + 2) * S + s] = v.z;
      xs[(4 * q + 3) * S + s] = v.w;
    }
  } else {
    for (int idx = tid; idx < S * C; idx += kThreads) {
      const int s = idx % S, c = idx / S;
      xs[c * S + s] = (row0 + s < a.B) ? __ldg(a.x + (row0 + s) * C + c) : 0.f;
    }
  }
  for (int idx = tid; idx < S * C; idx += kThreads) gxs[idx] = 0.0f;
  __syncthreads();

  const int my_sample = sample_group * 32 + lane;
  const bool row_valid = row0 + my_sample < a.B;
  const uint32_t xl_addr = smem_addr(xs + my_sample);
  const uint32_t x_stride = (uint32_t)S * 4u;
  float *stage = stage_all + (size_t)sample_group * 32 * (G + 1);
  const int group_threads = slots * 32;
  const int tid_in_group = slot * 32 + lane;
  const int64_t row_base = row0 + sample_group * 32;
  bool poisoned = false;

  for (int group = 0; group < num_groups; ++group) {
    const int in_group = (int)min((int64_t)G, a.T - (int64_t)group * G);
    const int64_t col0 = (int64_t)group * G;

    // upstream gradients of this sample group for the tree group: row segments -> staging rows
    named_barrier(1 + sample_group, group_threads);  // the previous group's values have been consumed
    if ((a.T & 3) == 0 && (in_group & 3) == 0) {
      const int quads = in_group >> 2;
      for (int idx = tid_in_group; idx < 32 * quads; idx += group_threads) {
        const int s = idx / quads, q = idx - s * quads;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (row_base + s < a.B) v = __ldg(reinterpret_cast<const float4 *>(a.g + (row_base + s) * a.T + col0 + 4 * q));
        float *dst = stage + s * (G + 1) + 4 * q;
        dst[0] = v.x;
        dst[1] = v.y;
        dst[2] = v.z;
        dst[3] = v.w;
      }
    } else {
      for (int idx = tid_in_group; idx < 32 * in_group; idx += group_threads) {
        const int s = idx / in_group, t = idx - s * in_group;
        stage[s * (G + 1) + t] = (row_base + s < a.B) ? __ldg(a.g + (row_base + s) * a.T + col0 + t) : 0.f;
      }
    }
    named_barrier(1 + sample_group, group_threads);  // staged

    if (!poisoned && !mbar_wait(&full[group & 1], (uint32_t)((group >> 1) & 1))) {
      poisoned = true;
      if (a.status_word != nullptr) atomicOr(a.status_word, HT_FLAG_PIPELINE_TIMEOUT);
    }
    const uint32_t base_addr = params_addr + (uint32_t)(group & 1) * (uint32_t)G * lay.bytes;
    const int t_first = slot * per_warp;
    if (t_first < in_group && !poisoned) {
      auto scatter = [&](const Walked &wk, uint32_t rec, int t) {
        if (t >= in_group || !row_valid) return;
        const int64_t j = col0 + t;
        const float gval = stage[lane * (G + 1) + t];
        const float wv = lds_f32(rec + 4u * wk.path + (lay.w - 4u * kL));
        // sign(margin) * w * g with margin = -nm
        const float wg = __fmul_rn(wv, gval);
        const float dx = wk.nm < 0.0f ? wg : (wk.nm > 0.0f ? -wg : __fmul_rn(0.0f, wg));
        if (a.gx != nullptr) {
          const uint32_t c = lds_ord<OrdT>(rec + (uint32_t)sizeof(OrdT) * wk.v + (lay.ord - (uint32_t)sizeof(OrdT)));
          atomicAdd(gxs + c * S + my_sample, dx);
        }
        if (a.gthr != nullptr) atomicAdd(a.gthr + j * kN + (wk.v - 1u), -dx);
        if (a.gw != nullptr) {
          const uint32_t key = __brev(wk.path - kL) >> (32 - DEPTH);  // reference leaf key: bit l = decision at depth l
          atomicAdd(a.gw + j * kL + key, __fmul_rn(fabsf(wk.nm), gval));
        }
      };
      if (per_warp == 4) {
        uint32_t rec[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) rec[u] = base_addr + (uint32_t)min(t_first + u, in_group - 1) * lay.bytes;
        Walked wk[4];
        walk_full<KIND, DEPTH, OrdT, 4>(rec, xl_addr, x_stride, wk);
#pragma unroll
        for (int u = 0; u < 4; ++u) scatter(wk[u], rec[u], t_first + u);
      } else if (per_warp == 2) {
        uint32_t rec[2];
#pragma unroll
        for (int u = 0; u < 2; ++u) rec[u] = base_addr + (uint32_t)min(t_first + u, in_group - 1) * lay.bytes;
        Walked wk[2];
        walk_full<KIND, DEPTH, OrdT, 2>(rec, xl_addr, x_stride, wk);
#pragma unroll
        for (int u = 0; u < 2; ++u) scatter(wk[u], rec[u], t_first + u);
      } else {
        uint32_t rec[1] = {base_addr + (uint32_t)t_first * lay.bytes};
        Walked wk[1];
        walk_full<KIND, DEPTH, OrdT, 1>(rec, xl_addr, x_stride, wk);
        scatter(wk[0], rec[0], t_first);
      }
    }
    __syncwarp();
    if (lane == 0) {
      __threadfence_block();
      const uint32_t before = atomicAdd(&finished[group & 1], 1u);
      if (before == kWarps - 1) {
        atomicExch(&finished[group & 1], 0u);
        __threadfence_block();
        if (group + 2 < num_groups) issue(group + 2);
      }
    }
  }

  // the x-gradient tile leaves with plain stores: every element of these rows is written exactly once
  __syncthreads();
  if (a.gx != nullptr) {
    if ((C & 3) == 0) {
      const int quads = C >> 2;
      for (int idx = tid; idx < S * quads; idx += kThreads) {
        const int s = idx % S, q = idx / S;
        if (row0 + s < a.B)
          *(reinterpret_cast<float4 *>(a.gx + (row0 + s) * C) + q) =
              make_float4(gxs[(4 * q + 0) * S + s], gxs[(4 * q + 1) * S + s], gxs[(4 * q + 2) * S + s],
                          gxs[(4 * q + 3) * S + s]);
      }
    } else {
      for (int idx = tid; idx < S * C; idx += kThreads) {
        const int s = idx % S, c = idx / S;
        if (row0 + s < a.B) a.gx[(row0 + s) * C + c] = gxs[c * S + s];
      }
    }
  }
}

template <int KIND, int DEPTH>
int launch_depth(const BwdPlan &plan, const BwdArgs &a, unsigned grid, cudaStream_t stream) {
  if (plan.ord_bytes == 1) {
    auto kernel = forest_backward_tiled_kernel<KIND, DEPTH, uint8_t>;
    HT_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBudget));
    kernel<<<grid, kThreads, plan.smem, stream>>>(a);
  } else {
    auto kernel = forest_backward_tiled_kernel<KIND, DEPTH, uint16_t>;
    HT_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBudget));
    kernel<<<grid, kThreads, plan.smem, stream>>>(a);
  }
  HT_CHECK_LAUNCH();
  return HT_OK;
}

template <int KIND>
int launch_kind(int depth, const BwdPlan &plan, const BwdArgs &a, unsigned grid, cudaStream_t stream) {
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

int backward_tiled(const ht_forest_problem *p, const float *x, const float *thr, const int32_t *ord, const float *w,
                   const float *g, float *gx, float *gthr, float *gw, void *records, uint32_t *status_word,
                   cudaStream_t stream) {
  BwdPlan plan;
  if (!make_bwd_plan(p, plan)) return HT_ERR_UNSUPPORTED;
  if (forward_tiled_workspace_bytes(p) == 0) return HT_ERR_UNSUPPORTED;  // the workspace holds no records otherwise
  if (((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(g) | reinterpret_cast<uintptr_t>(gx)) & 15u) != 0)
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
  BwdArgs a;
  a.x = x;
  a.records = rec;
  a.g = g;
  a.gx = gx;
  a.gthr = gthr;
  a.gw = gw;
  a.status_word = status_word;
  a.B = p->B;
  a.T = p->T;
  a.C = (int)p->C;
  a.S = plan.S;
  a.G = plan.G;
  a.per_warp = plan.per_warp;
  const unsigned grid = (unsigned)((p->B + plan.S - 1) / plan.S);
  return p->kind == TREE ? launch_kind<TREE>(p->depth, plan, a, grid, stream)
                         : launch_kind<FERN>(p->depth, plan, a, grid, stream);
}

}  // namespace ht
