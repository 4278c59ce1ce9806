// Dense projection on the 5th-generation tensor cores (tcgen05), with the column statistics a batch
// normalisation needs taken in the epilogue:
//
//     z[M, N] = x[M, K] * w[N, K]^T        TF32 operands (the fp32 inputs are read as they are; the tensor core
//                                          uses their upper 19 bits), fp32 accumulation in tensor memory
//     colsum[n]   = sum_m z[m, n]          colsumsq[n] = sum_m z[m, n]^2
//
// This is the Linear -> BatchNorm1d front of the reference's sequential-initialisation pipeline
// (README.md:110-129: Linear(in, trees * (2^depth - 1)) -> BatchNorm1d(affine=False) -> RandomHingeForest with
// init_type="sequential", RandomHingeForest/_RandomHingeForest.py:56-59), where the reference calls torch.nn.Linear
// (cuBLAS) and lets BatchNorm read the activations again for its statistics.
//
// One CTA computes one 128 x 128 tile of z.  Both operands are K-major, so a K-slice of 32 floats of either is
// a box of 128 rows x 128 bytes, which a tiled TMA load (cp.async.bulk.tensor, 128-byte swizzle, no multicast)
// drops into shared memory in exactly the canonical layout a K-major tcgen05 shared-memory descriptor describes.
// Warp roles (192 threads):
//   warp 0     one lane issues the TMA loads of the 3-stage operand ring (full / empty mbarriers);
//   warp 1     allocates 128 columns of tensor memory; one lane issues tcgen05.mma.kind::tf32 (M 128, N 128, K 8,
//              four per stage) and hands each stage back with tcgen05.commit, which also signals the epilogue;
//   warps 2-5  read the accumulator with tcgen05.ld (a warp reads the 32 TMEM lanes of its quarter), stage the
//              tile in shared memory (in the operand ring, idle by then) in the 128-byte swizzled box layout, from
//              where it leaves as four tiled TMA
//              stores while the same threads add the tile's column sums and sums of squares (one thread per
//              column reads its column conflict-free) into the statistics with one global reduction each.
// Rows and columns beyond the matrix are zero on the way in (TMA fill) and clipped on the way out.
// Every wait is bounded: when one runs out the kernel flags HT_FLAG_PIPELINE_TIMEOUT, stops issuing work, waits
// (bounded) for nothing more, frees its tensor memory and returns.
#include "ht_common.cuh"
#include "ht_tile_common.cuh"
#include "ht_tma.cuh"

namespace ht {

using namespace tile;

namespace {

constexpr int kBM = 128, kBN = 128, kBK = 32;  // tile of z, K-slice (32 floats = one 128-byte swizzle row)
constexpr int kStages = 3;  // 96 KB of operand ring: two CTAs per SM, so one's epilogue overlaps the other's main loop
constexpr int kGemmThreads = 192;
constexpr uint32_t kOperandBytes = kBM * kBK * 4;         // 16 KB: one operand box
constexpr uint32_t kStageBytes = 2 * kOperandBytes;       // A then B
constexpr uint32_t kOutBoxBytes = kBM * 32 * 4;           // 16 KB: 128 rows x 32 columns of z
constexpr uint32_t kTmemColumns = 128;
static_assert(4 * kOutBoxBytes <= kStages * kStageBytes, "the tile of z is staged in the operand ring once the MMAs are done");
constexpr size_t kGemmSmem = 1024 + kStages * kStageBytes + 256;

struct GemmArgs {
  CUtensorMap x_map, w_map, z_map;  // boxes of 128 rows x 32 floats, 128-byte swizzle
  float *colsum, *colsumsq;
  uint32_t *status_word;
  int M, N, K;
};

// K-major operand in the 128-byte swizzled layout: rows of 128 bytes, groups of 8 rows 1024 bytes apart.
__device__ __forceinline__ uint64_t operand_descriptor(uint32_t smem_address) {
  uint64_t desc = (uint64_t)((smem_address >> 4) & 0x3fffu);  // start address, 16-byte units
  desc |= (uint64_t)1u << 16;                                 // leading byte offset (unused for swizzled K-major)
  desc |= (uint64_t)(1024u >> 4) << 32;                       // stride byte offset: one 8-row group
  desc |= (uint64_t)1u << 46;                                 // descriptor version of this architecture
  desc |= (uint64_t)2u << 61;                                 // 128-byte swizzle
  return desc;
}

// kind::tf32, fp32 accumulator, both operands K-major, M = 128, N = 128.
constexpr uint32_t kInstruction = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(kBN >> 3) << 17) | ((uint32_t)(kBM >> 4) << 24);

__device__ __forceinline__ void mma_tf32(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
      :
      : "r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(kInstruction), "r"(accumulate), "r"(0u)
      : "memory");
}

// Arrives on the barrier once every tcgen05 operation this thread issued before has completed.
__device__ __forceinline__ void mma_commit(uint64_t *bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_addr(bar)) : "memory");
}

__device__ __forceinline__ void tmem_load_32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

__global__ void __launch_bounds__(kGemmThreads, 2) linear_tf32_stats_kernel(const __grid_constant__ GemmArgs a) {
  extern __shared__ __align__(1024) unsigned char gemm_smem[];
  unsigned char *base = gemm_smem + ((1024u - (smem_addr(gemm_smem) & 1023u)) & 1023u);
  const uint32_t stages = smem_addr(base);                                   // [kStages] {x box, w box}
  const uint32_t out_boxes = stages;  // [4] boxes of z, in the ring (idle by then: every MMA has read its operands)
  uint64_t *full = reinterpret_cast<uint64_t *>(base + kStages * kStageBytes);  // [kStages]
  uint64_t *empty = full + kStages;                                                               // [kStages]
  uint64_t *accumulated = empty + kStages;                                                        // [1]
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(accumulated + 1);
  uint32_t *failed = tmem_slot + 1;  // set by a role whose wait ran out

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = (int)blockIdx.x * kBN, m0 = (int)blockIdx.y * kBM;
  const int k_slices = (a.K + kBK - 1) / kBK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(accumulated, 1);
    *failed = 0u;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {  // the whole warp allocates; the address lands in shared memory
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(tmem_slot)), "r"(kTmemColumns)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = *tmem_slot;

  auto give_up = [&]() {
    *failed = 1u;
    if (a.status_word != nullptr) atomicOr(a.status_word, HT_FLAG_PIPELINE_TIMEOUT);
  };

  if (warp == 0) {
    if (lane == 0) {  // operand loads: slice k goes to stage k % kStages once the MMAs of slice k - kStages are done with it
      for (int k = 0; k < k_slices; ++k) {
        const int s = k % kStages;
        if (!mbar_wait(&empty[s], (uint32_t)(((k / kStages) & 1) ^ 1))) {
          give_up();
          break;
        }
        mbar_expect_tx(&full[s], kStageBytes);
        tma::load_2d(stages + (uint32_t)s * kStageBytes, &a.x_map, k * kBK, m0, &full[s]);
        tma::load_2d(stages + (uint32_t)s * kStageBytes + kOperandBytes, &a.w_map, k * kBK, n0, &full[s]);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      bool ok = true;
      for (int k = 0; k < k_slices && ok; ++k) {
        const int s = k % kStages;
        if (!mbar_wait(&full[s], (uint32_t)((k / kStages) & 1))) {
          give_up();
          ok = false;
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint64_t a_desc = operand_descriptor(stages + (uint32_t)s * kStageBytes);
        const uint64_t b_desc = operand_descriptor(stages + (uint32_t)s * kStageBytes + kOperandBytes);
#pragma unroll
        for (int kk = 0; kk < kBK / 8; ++kk)  // 8 floats = 32 bytes = 2 descriptor units further along K
          mma_tf32(tmem, a_desc + (uint64_t)(2 * kk), b_desc + (uint64_t)(2 * kk), (k | kk) != 0 ? 1u : 0u);
        mma_commit(&empty[s]);  // the stage is free again once these MMAs have read it
      }
      if (ok) mma_commit(accumulated);  // the tile is complete once every MMA has
    }
  } else {
    // epilogue: warps 2..5 own the TMEM lane quarters 2, 3, 0, 1 (a warp may only touch lanes 32 (warp % 4) ...)
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;  // row of the tile = TMEM lane
    const int et = (int)threadIdx.x - 64;  // 0..127 among the epilogue threads
    bool ok = mbar_wait(accumulated, 0u);
    if (!ok) give_up();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (ok) {
#pragma unroll 1
      for (int c = 0; c < kBN / 32; ++c) {
        uint32_t r[32];
        tmem_load_32(tmem + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(c * 32), r);
        const uint32_t box = out_boxes + (uint32_t)c * kOutBoxBytes;
#pragma unroll
        for (int q = 0; q < 8; ++q)
          sts_b128(box + tma::swizzled_offset<32>((uint32_t)row, (uint32_t)q), __uint_as_float(r[4 * q + 0]),
                   __uint_as_float(r[4 * q + 1]), __uint_as_float(r[4 * q + 2]), __uint_as_float(r[4 * q + 3]));
      }
    }
    tma::fence_async_shared();
    named_barrier(1, 128);  // the tile is in shared memory, visible to the TMA engine
    if (ok && *failed == 0u) {
      if (et == 0) {
#pragma unroll
        for (int c = 0; c < kBN / 32; ++c) tma::store_2d(&a.z_map, out_boxes + (uint32_t)c * kOutBoxBytes, n0 + 32 * c, m0);
        tma::commit_group();
      }
      // column statistics: thread et sums column et of the tile (32 consecutive columns of a box row per warp)
      const int n = n0 + et;
      if (n < a.N) {
        const uint32_t box = out_boxes + (uint32_t)(et >> 5) * kOutBoxBytes;
        const uint32_t q = (uint32_t)(et & 31) >> 2, word = (uint32_t)(et & 3) * 4u;
        float sum = 0.0f, sumsq = 0.0f;
#pragma unroll 8
        for (int r2 = 0; r2 < kBM; ++r2) {
          const float v = lds_f32(box + tma::swizzled_offset<32>((uint32_t)r2, q) + word);
          sum += v;
          sumsq = fmaf(v, v, sumsq);
        }
        atomicAdd(a.colsum + n, sum);
        atomicAdd(a.colsumsq + n, sumsq);
      }
      if (et == 0) tma::wait_stores_read();
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemColumns) : "memory");
  }
}

}  // namespace
}  // namespace ht

using namespace ht;

extern "C" int ht_linear_tf32_stats_f32(const float *x, const float *w, float *z, float *colsum, float *colsumsq, int64_t M,
                                        int64_t N, int64_t K, uint32_t *status_word, ht_stream_t stream_) {
  if (M < 0 || N < 0 || K < 1) return HT_ERR_INVALID_ARGUMENT;
  if (M == 0 || N == 0) return HT_OK;
  if (x == nullptr || w == nullptr || z == nullptr || colsum == nullptr || colsumsq == nullptr) return HT_ERR_INVALID_ARGUMENT;
  if (M > 0x7fffffff || N > 0x7fffffff || K > 0x7fffffff) return HT_ERR_UNSUPPORTED;
  if ((K & 3) != 0 || (N & 3) != 0) return HT_ERR_UNSUPPORTED;  // rows of a multiple of 16 bytes (tensor maps)
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  GemmArgs a = {};
  if (!tma::encode_matrix_f32(&a.x_map, x, M, K, kBM, kBK) || !tma::encode_matrix_f32(&a.w_map, w, N, K, kBN, kBK) ||
      !tma::encode_matrix_f32(&a.z_map, z, M, N, kBM, 32))
    return HT_ERR_UNSUPPORTED;
  a.colsum = colsum;
  a.colsumsq = colsumsq;
  a.status_word = status_word;
  a.M = (int)M;
  a.N = (int)N;
  a.K = (int)K;
  HT_CUDA_TRY(cudaMemsetAsync(colsum, 0, sizeof(float) * (size_t)N, stream));
  HT_CUDA_TRY(cudaMemsetAsync(colsumsq, 0, sizeof(float) * (size_t)N, stream));
  HT_CUDA_TRY(cudaFuncSetAttribute(linear_tf32_stats_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kGemmSmem));
  const dim3 grid((unsigned)((N + kBN - 1) / kBN), (unsigned)((M + kBM - 1) / kBM));
  linear_tf32_stats_kernel<<<grid, kGemmThreads, kGemmSmem, stream>>>(a);
  HT_CHECK_LAUNCH();
  return HT_OK;
}
