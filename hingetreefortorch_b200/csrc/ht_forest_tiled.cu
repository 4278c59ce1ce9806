// Shared-memory tile kernel for the forest forward on tabular input (K == 1, one output per leaf).
//
// Work decomposition (one CTA of 1024 threads per tile, sized for one CTA per SM):
//   * a CTA owns S consecutive samples and walks ALL trees, so every input element is read
//     from HBM exactly once;
//   * the samples' features sit in shared memory feature-major, xs[c][s]: lane l of a warp
//     always reads bank l whatever feature its current vertex tests, so the data gather never
//     conflicts although the 32 lanes are at 32 different vertices;
//   * a warp is (sample group, tree slot): S/32 sample groups, 32/(S/32) slots; within a tree
//     group a slot takes every `slots`-th tree, two at a time per thread for instruction-level
//     parallelism (the traversal is one dependent chain of shared-memory loads per level);
//   * tree parameters arrive as per-tree records {thresholds, uint8/uint16 feature indices,
//     leaf weights in heap order}, written once per call by a tiny repack kernel, and are
//     streamed into shared memory in groups with 1-D bulk async copies (cp.async.bulk, the TMA
//     engine) completing on an mbarrier, double buffered against the traversal;
//   * the per-group results are staged in shared memory and leave as full-sector row segments.
//
// Only the smallest |margin| matters in the forward, so the minimum is tracked on absolute
// values.  CUDA's fminf ignores a NaN operand; the reference keeps a NaN only when the root
// margin is NaN, which is patched after the loop.
#include "ht_forest_tiled.cuh"

namespace ht {

namespace {

constexpr int kThreads = 1024;
constexpr int kWarps = kThreads / 32;
constexpr size_t kSmemBudget = 227 * 1024;
// Spin limit for the parameter pipeline: far beyond any real copy latency, small enough that a
// lost copy ends the kernel (with a flag) instead of hanging the device.
constexpr uint32_t kMaxSpins = 1u << 22;

struct TilePlan {
  int S;            // samples per tile
  int G;            // trees per parameter group
  int ord_bytes;    // 1 or 2
  int rec_bytes;    // bytes of one tree record (multiple of 16)
  int thr_bytes;    // offset of the ordinals inside a record
  int w_offset;     // offset of the leaf weights inside a record
  size_t smem;      // dynamic shared memory of the tile kernel
  size_t x_bytes, param_bytes, out_bytes;
};

__host__ __device__ inline int round16(int v) { return (v + 15) & ~15; }

bool make_plan(const ht_forest_problem *p, TilePlan &plan) {
  if (p->K != 1 || p->M != 1) return false;
  if (p->C > 65536 || p->depth > 12) return false;
  if (p->B * p->T < 32 * 1024) return false;  // too small to fill the machine with sample tiles
  const int64_t N = threshold_count(p->kind, p->depth);
  const int64_t L = ((int64_t)1) << p->depth;
  plan.ord_bytes = p->C <= 256 ? 1 : 2;
  plan.thr_bytes = round16((int)(4 * N));
  plan.w_offset = plan.thr_bytes + round16((int)(plan.ord_bytes * N));
  plan.rec_bytes = round16(plan.w_offset + (int)(4 * L));
  for (int S = 256; S >= 32; S >>= 1) {
    const int slots = kWarps / (S / 32);
    for (int G = 32; G >= slots && G >= 4; G >>= 1) {
      plan.S = S;
      plan.G = G;
      plan.x_bytes = (size_t)p->C * S * 4;
      plan.param_bytes = 2 * (size_t)G * plan.rec_bytes;
      plan.out_bytes = (size_t)S * (G + 1) * 4;
      plan.smem = plan.x_bytes + plan.param_bytes + plan.out_bytes + 64;
      if (plan.smem <= kSmemBudget) return true;
    }
  }
  return false;
}

__device__ __forceinline__ uint32_t bit_reverse(uint32_t v, int bits) { return __brev(v) >> (32 - bits); }

// One thread per record element: thresholds, compact ordinals, and the leaf weights permuted so
// that the path bits in the order the traversal collects them (root first, most significant)
// address them directly.
template <typename OrdT>
__global__ void repack_records_kernel(const float *__restrict__ thr, const int32_t *__restrict__ ord,
                                      const float *__restrict__ w, unsigned char *__restrict__ records, int kind,
                                      int depth, int64_t T, int rec_bytes, int thr_bytes, int w_offset) {
  const int64_t N = threshold_count(kind, depth);
  const int64_t L = ((int64_t)1) << depth;
  const int64_t per_tree = N + L;
  const int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= T * per_tree) return;
  const int64_t j = e / per_tree;
  const int64_t r = e - j * per_tree;
  unsigned char *rec = records + j * rec_bytes;
  if (r < N) {
    const float t = thr[j * N + r];
    reinterpret_cast<float *>(rec)[r] = t == 0.0f ? 0.0f : t;  // -0 becomes +0
    reinterpret_cast<OrdT *>(rec + thr_bytes)[r] = (OrdT)ord[j * N + r];
  } else {
    const int64_t h = r - N;  // slot in the record
    const int64_t key = (int64_t)bit_reverse((uint32_t)h, depth);  // slot h holds the leaf whose key is h reversed
    reinterpret_cast<float *>(rec + w_offset)[h] = w[j * L + key];
  }
}

__device__ __forceinline__ uint32_t smem_addr(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count));
}

__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}

// 1-D bulk copy global -> shared through the TMA engine; completion is counted in bytes on `bar`.
__device__ __forceinline__ void bulk_load(void *dst, const void *src, uint32_t bytes, uint64_t *bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_addr(dst)),
               "l"(src), "r"(bytes), "r"(smem_addr(bar))
               : "memory");
}

// Bounded wait on a phase of the barrier.  Returns false when the limit ran out.
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity) {
  for (uint32_t spin = 0; spin < kMaxSpins; ++spin) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(smem_addr(bar)), "r"(parity)
        : "memory");
    if (done) return true;
  }
  return false;
}

__device__ __forceinline__ float lds_f32(uint32_t addr) {
  float v;
  asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(addr));
  return v;
}

template <typename OrdT>
__device__ __forceinline__ uint32_t lds_ord(uint32_t addr) {
  uint32_t v;
  if (sizeof(OrdT) == 1)
    asm volatile("ld.shared.u8 %0, [%1];" : "=r"(v) : "r"(addr));
  else
    asm volatile("ld.shared.u16 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}

struct TiledArgs {
  const float *x;
  const unsigned char *records;
  float *out;
  uint32_t *status_word;
  int64_t B, T;
  int C, S, G, rec_bytes, thr_bytes, w_offset;
};

template <int KIND, int DEPTH, typename OrdT>
__global__ void __launch_bounds__(kThreads, 1) forest_forward_tiled_kernel(TiledArgs a) {
  extern __shared__ __align__(128) unsigned char smem[];
  const int S = a.S, G = a.G, C = a.C;
  float *xs = reinterpret_cast<float *>(smem);
  unsigned char *params = smem + (size_t)C * S * 4;
  float *outs = reinterpret_cast<float *>(params + 2 * (size_t)G * a.rec_bytes);
  uint64_t *bars = reinterpret_cast<uint64_t *>(outs + (size_t)S * (G + 1));

  const int tid = threadIdx.x;
  const int lane = tid & 31, warp = tid >> 5;
  const int groups_of_samples = S >> 5;
  const int slots = kWarps / groups_of_samples;
  const int sample_group = warp % groups_of_samples;
  const int slot = warp / groups_of_samples;
  const int64_t row0 = (int64_t)blockIdx.x * S;
  const int num_groups = (int)((a.T + G - 1) / G);

  if (tid == 0) {
    mbar_init(&bars[0], 1);
    mbar_init(&bars[1], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  auto issue = [&](int group) {
    const int64_t first = (int64_t)group * G;
    const int64_t count = min((int64_t)G, a.T - first);
    const uint32_t bytes = (uint32_t)(count * a.rec_bytes);
    uint64_t *bar = &bars[group & 1];
    mbar_expect_tx(bar, bytes);
    bulk_load(params + (size_t)(group & 1) * G * a.rec_bytes, a.records + first * a.rec_bytes, bytes, bar);
  };
  if (tid == 0) issue(0);

  // Stage the tile's features: lanes run along samples so that the shared-memory writes are
  // conflict free; each lane fetches 16 bytes of its row at a time when the row allows it.
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
  __syncthreads();

  // feature c of this lane's sample sits at shared address xl_addr + c * x_stride
  const uint32_t xl_addr = smem_addr(xs + sample_group * 32 + lane);
  const uint32_t x_stride = (uint32_t)S * 4u;
  constexpr uint32_t kN = KIND == FERN ? DEPTH : (1u << DEPTH) - 1u;
  constexpr uint32_t kThrBytes = (4u * kN + 15u) & ~15u;
  constexpr uint32_t kWOffset = kThrBytes + (((uint32_t)sizeof(OrdT) * kN + 15u) & ~15u);
  constexpr uint32_t kRec = (kWOffset + 4u * (1u << DEPTH) + 15u) & ~15u;
  bool timed_out = false;

  for (int group = 0; group < num_groups; ++group) {
    if (tid == 0 && group + 1 < num_groups) issue(group + 1);
    if (!mbar_wait(&bars[group & 1], (uint32_t)((group >> 1) & 1))) timed_out = true;
    if (__syncthreads_or(timed_out)) {
      if (tid == 0 && a.status_word != nullptr) atomicOr(a.status_word, HT_FLAG_PIPELINE_TIMEOUT);
      return;
    }
    const int in_group = (int)min((int64_t)G, a.T - (int64_t)group * G);

    // Two trees per thread per pass.  All addresses are 32-bit shared-memory addresses.  The
    // vertex index is kept 1-based (root = 1, children 2v and 2v+1), so that one funnel shift
    // appends the branch bit: the bit is the sign of (threshold - feature), which is set
    // exactly when the margin is positive (records hold +0 for a -0 threshold, and an add
    // that yields NaN yields the canonical positive NaN, so NaN margins go left as required).
    const uint32_t base_addr = smem_addr(params) + (uint32_t)(group & 1) * (uint32_t)(G * kRec);
    for (int t0 = slot; t0 < in_group; t0 += 2 * slots) {
      const int t1 = t0 + slots;
      const bool has1 = t1 < in_group;
      const uint32_t rec[2] = {base_addr + (uint32_t)t0 * kRec, base_addr + (uint32_t)(has1 ? t1 : t0) * kRec};
      uint32_t v[2] = {1u, 1u};
      float best[2], first[2];
#pragma unroll
      for (int l = 0; l < DEPTH; ++l) {
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          float thr;
          uint32_t c;
          if (KIND == FERN) {
            thr = lds_f32(rec[u] + 4u * l);
            c = lds_ord<OrdT>(rec[u] + kThrBytes + (uint32_t)sizeof(OrdT) * l);
          } else {
            thr = lds_f32(rec[u] + 4u * v[u] - 4u);
            c = lds_ord<OrdT>(rec[u] + (uint32_t)sizeof(OrdT) * v[u] + (kThrBytes - (uint32_t)sizeof(OrdT)));
          }
          const float nm = thr - lds_f32(c * x_stride + xl_addr);
          const float am = fabsf(nm);
          if (l == 0) {
            best[u] = am;
            first[u] = am;
          } else {
            best[u] = fminf(best[u], am);
          }
          v[u] = __funnelshift_l(__float_as_uint(nm), v[u], 1);
        }
      }
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        if (u == 1 && !has1) break;
        const float wv = lds_f32(rec[u] + 4u * v[u] + (kWOffset - 4u * (1u << DEPTH)));
        const float am = (first[u] != first[u]) ? first[u] : best[u];
        outs[(sample_group * 32 + lane) * (G + 1) + (u == 0 ? t0 : t1)] = am * wv;
      }
    }
    __syncthreads();

    // write the [S x in_group] block of results as row segments
    const int64_t col0 = (int64_t)group * G;
    if ((a.T & 3) == 0 && (in_group & 3) == 0) {
      const int quads = in_group >> 2;
      for (int idx = tid; idx < S * quads; idx += kThreads) {
        const int s = idx / quads, q = idx - s * quads;
        if (row0 + s < a.B) {
          const float *src = outs + s * (G + 1) + 4 * q;
          *reinterpret_cast<float4 *>(a.out + (row0 + s) * a.T + col0 + 4 * q) =
              make_float4(src[0], src[1], src[2], src[3]);
        }
      }
    } else {
      for (int idx = tid; idx < S * in_group; idx += kThreads) {
        const int s = idx / in_group, t = idx - s * in_group;
        if (row0 + s < a.B) a.out[(row0 + s) * a.T + col0 + t] = outs[s * (G + 1) + t];
      }
    }
    // no barrier here: the one after the next group's wait also protects the staging buffer
  }
}

template <int KIND, int DEPTH>
int launch_depth(const TilePlan &plan, const TiledArgs &a, unsigned grid, cudaStream_t stream) {
  if (plan.ord_bytes == 1) {
    auto kernel = forest_forward_tiled_kernel<KIND, DEPTH, uint8_t>;
    HT_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBudget));
    kernel<<<grid, kThreads, plan.smem, stream>>>(a);
  } else {
    auto kernel = forest_forward_tiled_kernel<KIND, DEPTH, uint16_t>;
    HT_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBudget));
    kernel<<<grid, kThreads, plan.smem, stream>>>(a);
  }
  HT_CHECK_LAUNCH();
  return HT_OK;
}

template <int KIND>
int launch_kind(int depth, const TilePlan &plan, const TiledArgs &a, unsigned grid, cudaStream_t stream) {
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
  if (!make_plan(p, plan)) return 0;
  return align_up((size_t)p->T * plan.rec_bytes, 256);
}

int forward_tiled(const ht_forest_problem *p, const float *x, const float *thr, const int32_t *ord, const float *w,
                  float *out, void *records, uint32_t *status_word, cudaStream_t stream) {
  TilePlan plan;
  if (!make_plan(p, plan)) return HT_ERR_UNSUPPORTED;
  if ((reinterpret_cast<uintptr_t>(x) & 15u) != 0 || (reinterpret_cast<uintptr_t>(out) & 15u) != 0)
    return HT_ERR_UNSUPPORTED;
  const int64_t N = threshold_count(p->kind, p->depth);
  const int64_t L = ((int64_t)1) << p->depth;
  const int64_t elements = p->T * (N + L);
  const unsigned pack_grid = (unsigned)((elements + 255) / 256);
  unsigned char *rec = static_cast<unsigned char *>(records);
  if (plan.ord_bytes == 1)
    repack_records_kernel<uint8_t><<<pack_grid, 256, 0, stream>>>(thr, ord, w, rec, p->kind, p->depth, p->T,
                                                                   plan.rec_bytes, plan.thr_bytes, plan.w_offset);
  else
    repack_records_kernel<uint16_t><<<pack_grid, 256, 0, stream>>>(thr, ord, w, rec, p->kind, p->depth, p->T,
                                                                    plan.rec_bytes, plan.thr_bytes, plan.w_offset);
  HT_CHECK_LAUNCH();

  TiledArgs a;
  a.x = x;
  a.records = rec;
  a.out = out;
  a.status_word = status_word;
  a.B = p->B;
  a.T = p->T;
  a.C = (int)p->C;
  a.S = plan.S;
  a.G = plan.G;
  a.rec_bytes = plan.rec_bytes;
  a.thr_bytes = plan.thr_bytes;
  a.w_offset = plan.w_offset;
  const unsigned grid = (unsigned)((p->B + plan.S - 1) / plan.S);
  return p->kind == TREE ? launch_kind<TREE>(p->depth, plan, a, grid, stream)
                         : launch_kind<FERN>(p->depth, plan, a, grid, stream);
}

}  // namespace ht
