// Shared-memory tile kernel for the forest backward on tabular input with SEVERAL outputs per leaf
// (default mode; the fixed-order mode stays with the ordered any-shape kernels).
//
// Per evaluation the backward needs D = sum_m w[j, leaf, m] * g[i, j, m] (for the x and threshold
// gradients) and adds |margin| * g[i, j, m] to the leaf-weight gradient for every m.  A thread per
// evaluation reads its g row and its leaf's weight row with 32 lanes at 32 unrelated addresses for
// every m, and scatters the weight gradient the same way: about 100 * M 32-byte sectors per warp
// and tree, which is what bounds the any-shape kernel.  Here the traversal has the tiling of the
// forward tile kernel (features feature-major in shared memory, tree records streamed by bulk
// async copies, 4 trees in flight per warp), and the per-m work is done by the warp together:
// every lane leaves (|margin|, leaf) of its sample in shared memory; then, pair by pair, lanes
// along m load the g row and the weight row contiguously, add to the weight gradient contiguously
// and reduce D over the lanes of the pair with shuffles; the owning lane picks D up again and
// scatters the x and threshold terms.
#include "ht_forest_tiled.cuh"
#include "ht_tile_common.cuh"

#include <algorithm>

namespace ht {

using namespace tile;

namespace {

struct MultiPlan {
  int S, G, per_warp, ord_bytes;
  RecordLayout rec;
  size_t smem;
};

constexpr size_t kPairBytes = (size_t)kWarps * 32 * 4 * 8;  // (|margin|, leaf) per sample and tree in flight
constexpr size_t kDotBytes = (size_t)kWarps * 32 * 4 * 4;   // D per sample and tree in flight

bool make_plan(const ht_forest_problem *p, MultiPlan &plan) {
  if (p->K != 1 || p->M < 2 || p->M > 64) return false;
  if (p->C > 65536 || p->depth > 12) return false;
  // Worth it from a few million evaluations on: what bounds this kernel is the rate of the global
  // reductions into the leaf-weight gradient (M per evaluation), which the any-shape kernel pays as
  // well; the gain is in everything else (65536 x 100 trees x 26 outputs: 2.4 -> 1.5 ms; 4096 x 500
  // x 10: 0.23 -> 0.27 ms).
  if (p->B * p->T < 4 * 1024 * 1024) return false;
  plan.ord_bytes = p->C <= 256 ? 1 : 2;
  plan.rec = record_layout(p->kind, p->depth, (uint32_t)plan.ord_bytes, false);
  for (int S = 256; S >= 32; S >>= 1) {
    const int slots = kWarps / (S / 32);
    for (int per_warp = 4; per_warp >= 1; per_warp >>= 1) {
      plan.S = S;
      plan.G = slots * per_warp;
      plan.per_warp = per_warp;
      plan.smem = (size_t)p->C * S * 4 + 2 * (size_t)plan.G * plan.rec.bytes + kPairBytes + kDotBytes + 64;
      if (plan.smem <= kSmemBudget) return true;
    }
  }
  return false;
}

struct MultiArgs {
  const float *x;
  const unsigned char *records;
  const float *w;
  const float *g;
  float *gx, *gthr, *gw;
  uint32_t *status_word;
  int64_t B, T;
  int C, S, G, per_warp, M;
};

template <int KIND, int DEPTH, typename OrdT>
__global__ void __launch_bounds__(kThreads, 1) forest_backward_tiled_multi_kernel(MultiArgs a) {
  extern __shared__ __align__(128) unsigned char smem[];
  constexpr RecordLayout lay = record_layout(KIND, DEPTH, (uint32_t)sizeof(OrdT), false);
  constexpr uint32_t kN = KIND == FERN ? DEPTH : (1u << DEPTH) - 1u;
  constexpr uint32_t kL = 1u << DEPTH;
  const int S = a.S, G = a.G, C = a.C, M = a.M;
  float *xs = reinterpret_cast<float *>(smem);
  unsigned char *params = smem + (size_t)C * S * 4;
  float2 *all_pairs = reinterpret_cast<float2 *>(params + 2 * (size_t)G * lay.bytes);
  float *all_dots = reinterpret_cast<float *>(reinterpret_cast<unsigned char *>(all_pairs) + kPairBytes);
  uint64_t *full = reinterpret_cast<uint64_t *>(reinterpret_cast<unsigned char *>(all_dots) + kDotBytes);
  uint32_t *finished = reinterpret_cast<uint32_t *>(full + 2);

  const int tid = threadIdx.x;
  const int lane = tid & 31, warp = tid >> 5;
  const int groups_of_samples = S >> 5;
  const int sample_group = warp % groups_of_samples;
  const int slot = warp / groups_of_samples;
  const int per_warp = a.per_warp;
  const int64_t row0 = (int64_t)blockIdx.x * S;
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

  if ((C & 3) == 0) {
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

  const int64_t first_row = row0 + sample_group * 32;
  const int64_t my_row = first_row + lane;
  const bool row_valid = my_row < a.B;
  const int rows_here = (int)max((int64_t)0, min((int64_t)32, a.B - first_row));
  const uint32_t xl_addr = smem_addr(xs + sample_group * 32 + lane);
  const uint32_t x_stride = (uint32_t)S * 4u;
  float2 *pairs = all_pairs + (size_t)warp * 32 * 4;
  float *dots = all_dots + (size_t)warp * 32 * 4;
  // lanes of one (sample, tree) pair in the shared phase: the next power of two >= M (so that the
  // shuffle reduction stays inside the pair), at most 32
  int width = 32;
  while (width > 1 && (width >> 1) >= M) width >>= 1;
  const int per_iter = 32 / width, pair_in_iter = lane / width, m0 = lane % width;
  const bool need_dots = a.gx != nullptr || a.gthr != nullptr;
  bool poisoned = false;

  for (int it = 0; it < num_groups; ++it) {
    const int group = group0 + it;
    if (!poisoned && !mbar_wait(&full[it & 1], (uint32_t)((it >> 1) & 1))) {
      poisoned = true;
      if (a.status_word != nullptr) atomicOr(a.status_word, HT_FLAG_PIPELINE_TIMEOUT);
    }
    const int in_group = (int)min((int64_t)G, a.T - (int64_t)group * G);
    const int64_t col0 = (int64_t)group * G;
    const uint32_t base_addr = params_addr + (uint32_t)(it & 1) * (uint32_t)G * lay.bytes;
    const int t_first = slot * per_warp;
    const int trees_here = poisoned ? 0 : min(per_warp, in_group - t_first);

    Walked wk[4];
    uint32_t feature[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      wk[u].nm = 0.0f;
      wk[u].v = 1u;
      wk[u].path = kL;
      feature[u] = 0u;
    }
    if (trees_here > 0) {
      uint32_t rec[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) rec[u] = base_addr + (uint32_t)min(t_first + u, in_group - 1) * lay.bytes;
      if (per_warp == 4) {
        walk_full<KIND, DEPTH, OrdT, 4>(rec, xl_addr, x_stride, wk);
      } else if (per_warp == 2) {
        uint32_t r2[2] = {rec[0], rec[1]};
        Walked w2[2];
        walk_full<KIND, DEPTH, OrdT, 2>(r2, xl_addr, x_stride, w2);
        wk[0] = w2[0];
        wk[1] = w2[1];
      } else {
        uint32_t r1[1] = {rec[0]};
        Walked w1[1];
        walk_full<KIND, DEPTH, OrdT, 1>(r1, xl_addr, x_stride, w1);
        wk[0] = w1[0];
      }
#pragma unroll
      for (int u = 0; u < 4; ++u)  // the feature the deciding vertex tests, while the record is still there
        feature[u] = lds_ord<OrdT>(rec[u] + (uint32_t)sizeof(OrdT) * wk[u].v + (lay.ord - (uint32_t)sizeof(OrdT)));
    }
    // This warp no longer reads the parameter buffer.  The last warp to get here refills it.
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
    if (trees_here <= 0) continue;

#pragma unroll
    for (int u = 0; u < 4; ++u)
      pairs[lane * 4 + u] = make_float2(fabsf(wk[u].nm), __uint_as_float(__brev(wk[u].path - kL) >> (32 - DEPTH)));
    __syncwarp();

    // shared phase: the warp's (sample, tree) pairs, `per_iter` at a time, lanes along m
    for (int u = 0; u < trees_here; ++u) {
      const int64_t j = col0 + t_first + u;
      const float *g_tree = a.g + (first_row * a.T + j) * M;  // sample s: + s * T * M
      const float *w_tree = a.w + j * (int64_t)kL * M;
      float *gw_tree = a.gw == nullptr ? nullptr : a.gw + j * (int64_t)kL * M;
      for (int s0 = 0; s0 < rows_here; s0 += per_iter) {
        const int s = s0 + pair_in_iter;
        const bool active = s < rows_here;
        const float2 pair = active ? pairs[s * 4 + u] : make_float2(0.f, 0.f);
        const int64_t leaf_row = (int64_t)__float_as_uint(pair.y) * M;
        float partial = 0.0f;
        for (int m = m0; m < M && active; m += width) {
          const float gv = __ldg(g_tree + (int64_t)s * a.T * M + m);
          if (need_dots) partial += __ldg(w_tree + leaf_row + m) * gv;
          if (gw_tree != nullptr) atomicAdd(gw_tree + leaf_row + m, pair.x * gv);
        }
        if (need_dots) {
          for (int off = width >> 1; off > 0; off >>= 1) partial += __shfl_xor_sync(0xffffffffu, partial, off);
          if (active && m0 == 0) dots[s * 4 + u] = partial;
        }
      }
    }
    __syncwarp();

    // back with the owning lanes: sign(margin) * D to the x gradient, its negative to the threshold's
    if (need_dots && row_valid) {
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        if (u < trees_here) {
          const float d = dots[lane * 4 + u];
          const float dx = signed_term(wk[u].nm, d);  // margin = -nm
          if (a.gx != nullptr) atomicAdd(a.gx + my_row * C + feature[u], dx);
          if (a.gthr != nullptr) atomicAdd(a.gthr + (col0 + t_first + u) * kN + (wk[u].v - 1u), -dx);
        }
      }
    }
    __syncwarp();  // the pairs and sums are rewritten in the next group
  }
}

template <typename Kernel>
int launch_one(Kernel kernel, const MultiPlan &plan, const MultiArgs &a, dim3 grid, cudaStream_t stream) {
  HT_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBudget));
  kernel<<<grid, kThreads, plan.smem, stream>>>(a);
  HT_CHECK_LAUNCH();
  return HT_OK;
}

template <int KIND, int DEPTH>
int launch_depth(const MultiPlan &plan, const MultiArgs &a, dim3 grid, cudaStream_t stream) {
  if (plan.ord_bytes == 1) return launch_one(forest_backward_tiled_multi_kernel<KIND, DEPTH, uint8_t>, plan, a, grid, stream);
  return launch_one(forest_backward_tiled_multi_kernel<KIND, DEPTH, uint16_t>, plan, a, grid, stream);
}

template <int KIND>
int launch_kind(int depth, const MultiPlan &plan, const MultiArgs &a, dim3 grid, cudaStream_t stream) {
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

int backward_tiled_multi(const ht_forest_problem *p, const float *x, const float *thr, const int32_t *ord, const float *w,
                         const float *g, float *gx, float *gthr, float *gw, void *records, size_t records_bytes,
                         uint32_t *status_word, cudaStream_t stream) {
  MultiPlan plan;
  if ((p->flags & HT_DETERMINISTIC) != 0 || !make_plan(p, plan)) return HT_ERR_UNSUPPORTED;
  if ((size_t)p->T * plan.rec.bytes > records_bytes) return HT_ERR_UNSUPPORTED;
  if ((reinterpret_cast<uintptr_t>(x) & 15u) != 0) return HT_ERR_UNSUPPORTED;
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

  MultiArgs a;
  a.x = x;
  a.records = rec;
  a.w = w;
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
  a.M = (int)p->M;
  const int64_t tiles = (p->B + plan.S - 1) / plan.S;
  if (tiles > 0x7fffffff) return HT_ERR_UNSUPPORTED;
  const int64_t groups = (p->T + plan.G - 1) / plan.G;
  const dim3 grid((unsigned)tiles, (unsigned)choose_splits(tiles, groups));
  return p->kind == TREE ? launch_kind<TREE>(p->depth, plan, a, grid, stream)
                         : launch_kind<FERN>(p->depth, plan, a, grid, stream);
}

}  // namespace ht
