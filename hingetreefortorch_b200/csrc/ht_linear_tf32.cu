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
// A persistent kernel: one CTA per SM walks tiles of 128 x 256 of z (m-blocks fastest, so the CTAs running at one
// time share the same rows of w in L2).  Both operands are K-major, so a K-slice of 32 floats of either is a box of
// rows x 128 bytes, which a tiled TMA load (cp.async.bulk.tensor, 128-byte swizzle, no multicast) drops into
// shared memory in exactly the canonical layout a K-major tcgen05 shared-memory descriptor describes.
// Warp roles (192 threads):
//   warp 0     one lane issues the TMA loads of the 4-stage operand ring (full / empty mbarriers; 48 KB a stage);
//   warp 1     allocates all 512 columns of tensor memory — two accumulators of 128 lanes x 256 columns — and one
//              lane issues tcgen05.mma.kind::tf32 (M 128, N 256, K 8, four per stage) into the accumulator of the
//              tile, handing each stage back with tcgen05.commit and the finished accumulator to the epilogue;
//   warps 2-5  the epilogue of the PREVIOUS tile, under the main loop of the current one: 32 columns at a time
//              they read the accumulator with tcgen05.ld (a warp reads the 32 TMEM lanes of its quarter), stage
//              them in one of two shared-memory boxes (a lane writes the 128 bytes of its own row, swizzled so that
//              neither this nor the reads below meet in a bank), write the box to z in whole 128-byte row segments
//              and add its column sums and sums of squares (8 columns a warp) into the statistics.
// A 128 x 256 x 8 step reads 12 KB of operands from shared memory for 134 tensor-pipe cycles, 25 % less per
// FLOP than 128 x 128 tiles, which were bound by exactly that.
// Rows and columns beyond the matrix are zero on the way in (TMA fill) and clipped on the way out.
// Every wait is bounded: when one runs out the kernel flags HT_FLAG_PIPELINE_TIMEOUT, every role stops at its own
// next wait, the tensor memory is freed and the kernel returns.
#include <algorithm>

#include "ht_common.cuh"
#include "ht_tile_common.cuh"
#include "ht_tma.cuh"

namespace ht {

using namespace tile;

namespace {

constexpr int kBM = 128, kBN = 256, kBK = 32;  // tile of z, K-slice (32 floats = one 128-byte swizzle row)
constexpr int kStages = 4;
constexpr int kGemmThreads = 192;
constexpr uint32_t kABytes = kBM * kBK * 4;           // 16 KB: the x box of a stage
constexpr uint32_t kBBytes = kBN * kBK * 4;           // 32 KB: the w box
constexpr uint32_t kStageBytes = kABytes + kBBytes;   // 48 KB
constexpr uint32_t kOutBoxBytes = kBM * 32 * 4;       // 16 KB: 128 rows x 32 columns of z
constexpr uint32_t kTmemColumns = 512;                // two accumulators of 256 columns
constexpr size_t kGemmSmem = 1024 + kStages * kStageBytes + 2 * kOutBoxBytes + 256;

struct GemmArgs {
  CUtensorMap x_map, w_map;  // boxes of 128 (x) or 256 (w) rows x 32 floats, 128-byte swizzle
  float *z, *colsum, *colsumsq;
  uint32_t *status_word;
  int M, N, K;
  int m_blocks, tiles;
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

// kind::tf32, fp32 accumulator, both operands K-major, M = 128, N = 256.
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

__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(bar)) : "memory");
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

__global__ void __launch_bounds__(kGemmThreads, 1) linear_tf32_stats_kernel(const __grid_constant__ GemmArgs a) {
  extern __shared__ __align__(1024) unsigned char gemm_smem[];
  unsigned char *base = gemm_smem + ((1024u - (smem_addr(gemm_smem) & 1023u)) & 1023u);
  const uint32_t stages = smem_addr(base);                                        // [kStages] {x box, w box}
  const uint32_t out_boxes = stages + kStages * kStageBytes;                      // [2] boxes of z
  uint64_t *full = reinterpret_cast<uint64_t *>(base + kStages * kStageBytes + 2 * kOutBoxBytes);  // [kStages]
  uint64_t *empty = full + kStages;                                               // [kStages]
  uint64_t *accumulated = empty + kStages;                                        // [2] an accumulator is complete
  uint64_t *drained = accumulated + 2;                                            // [2] ... and has been read out
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(drained + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int k_slices = (a.K + kBK - 1) / kBK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&accumulated[b], 1);
      mbar_init(&drained[b], 4);  // one arrival per epilogue warp
    }
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
    if (a.status_word != nullptr) atomicOr(a.status_word, HT_FLAG_PIPELINE_TIMEOUT);
  };

  if (warp == 0) {
    if (lane == 0) {  // operand loads: slice `it` (counted over all tiles of this CTA) goes to stage it % kStages
      uint32_t it = 0;
      bool ok = true;
      for (int tile = (int)blockIdx.x; tile < a.tiles && ok; tile += (int)gridDim.x) {
        const int m0 = (tile % a.m_blocks) * kBM, n0 = (tile / a.m_blocks) * kBN;
        for (int k = 0; k < k_slices; ++k, ++it) {
          const uint32_t s = it % kStages;
          if (!mbar_wait(&empty[s], ((it / kStages) & 1u) ^ 1u)) {
            give_up();
            ok = false;
            break;
          }
          mbar_expect_tx(&full[s], kStageBytes);
          tma::load_2d(stages + s * kStageBytes, &a.x_map, k * kBK, m0, &full[s]);
          tma::load_2d(stages + s * kStageBytes + kABytes, &a.w_map, k * kBK, n0, &full[s]);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      uint32_t it = 0, t = 0;
      bool ok = true;
      for (int tile = (int)blockIdx.x; tile < a.tiles && ok; tile += (int)gridDim.x, ++t) {
        const uint32_t acc = t & 1u;
        if (!mbar_wait(&drained[acc], ((t >> 1) & 1u) ^ 1u)) {  // the epilogue has read this accumulator's previous tile
          give_up();
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t d = tmem + acc * (uint32_t)kBN;
        for (int k = 0; k < k_slices; ++k, ++it) {
          const uint32_t s = it % kStages;
          if (!mbar_wait(&full[s], (it / kStages) & 1u)) {
            give_up();
            ok = false;
            break;
          }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint64_t a_desc = operand_descriptor(stages + s * kStageBytes);
          const uint64_t b_desc = operand_descriptor(stages + s * kStageBytes + kABytes);
#pragma unroll
          for (int kk = 0; kk < kBK / 8; ++kk)  // 8 floats = 32 bytes = 2 descriptor units further along K
            mma_tf32(d, a_desc + (uint64_t)(2 * kk), b_desc + (uint64_t)(2 * kk), (k | kk) != 0 ? 1u : 0u);
          mma_commit(&empty[s]);  // the stage is free again once these MMAs have read it
        }
        if (ok) mma_commit(&accumulated[acc]);  // the tile is complete once every MMA has
      }
    }
  } else {
    // epilogue: warps 2..5 own the TMEM lane quarters 2, 3, 0, 1 (a warp may only touch lanes 32 (warp % 4) ...)
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;       // row of the tile = TMEM lane
    const int et = (int)threadIdx.x - 64;      // 0..127 among the epilogue threads
    const int ew = et >> 5;                    // 0..3
    // statistics: this warp sums columns 8 ew .. 8 ew + 7 of a box; lane = column + 8 * (group of 32 rows), and the
    // groups start 2 rows apart so that the 32 lanes of one read fall into 32 different banks of the swizzled box
    const uint32_t stat_col = (uint32_t)(8 * ew + (lane & 7)), stat_group = (uint32_t)lane >> 3;
    uint32_t chunk = 0, t = 0;
    // A thread whose wait ran out stops waiting and reading the accumulators but keeps meeting the others at the named
    // barriers (the same count for every thread whatever happened), so that nobody is left waiting there.
    bool dead = false;
    for (int tile = (int)blockIdx.x; tile < a.tiles; tile += (int)gridDim.x, ++t) {
      const int m0 = (tile % a.m_blocks) * kBM, n0 = (tile / a.m_blocks) * kBN;
      const uint32_t acc = t & 1u;
      if (!dead && !mbar_wait(&accumulated[acc], (t >> 1) & 1u)) {
        give_up();
        dead = true;
      }
      dead = __any_sync(0xffffffffu, dead);  // a warp reads tensor memory together or not at all
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll 1
      for (int c = 0; c < kBN / 32; ++c, ++chunk) {
        uint32_t r[32];
        if (!dead) {
          tmem_load_32(tmem + ((uint32_t)(quarter * 32) << 16) + acc * (uint32_t)kBN + (uint32_t)(c * 32), r);
        } else {
#pragma unroll
          for (int u = 0; u < 32; ++u) r[u] = 0u;
        }
        const uint32_t box = out_boxes + (chunk & 1u) * kOutBoxBytes;
        named_barrier(1, 128);  // everybody is through with what this box held two chunks ago
#pragma unroll
        for (int q = 0; q < 8; ++q)
          sts_b128(box + tma::swizzled_offset<32>((uint32_t)row, (uint32_t)q), __uint_as_float(r[4 * q + 0]),
                   __uint_as_float(r[4 * q + 1]), __uint_as_float(r[4 * q + 2]), __uint_as_float(r[4 * q + 3]));
        named_barrier(1, 128);  // the box is complete
        // z leaves in whole 128-byte row segments: 8 lanes along a row's 32 columns, 4 rows per warp instruction,
        // read back from the box without bank conflicts.  (A tiled TMA store per box made every reuse of a box wait
        // for the store engine, which is busy with the operand loads: 0.30 instead of 0.23 ms for the benchmark shape.)
        if (!dead) {
          const int col = n0 + 32 * c + 4 * (lane & 7);
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int r2 = 32 * ew + 4 * i + (lane >> 3);
            const uint4 v = lds_b128(box + tma::swizzled_offset<32>((uint32_t)r2, (uint32_t)(lane & 7)));
            if (m0 + r2 < a.M && col < a.N) __stcs(reinterpret_cast<uint4 *>(a.z + (size_t)(m0 + r2) * (size_t)a.N + col), v);
          }
        }
        const int n = n0 + 32 * c + (int)stat_col;
        float sum = 0.0f, sumsq = 0.0f;
        const uint32_t q = stat_col >> 2, word = (stat_col & 3u) * 4u;
#pragma unroll 8
        for (uint32_t i = 0; i < 32; ++i) {
          const uint32_t r2 = stat_group * 32u + ((i + 2u * stat_group) & 31u);
          const float v = lds_f32(box + tma::swizzled_offset<32>(r2, q) + word);
          sum += v;
          sumsq = fmaf(v, v, sumsq);
        }
        sum += __shfl_xor_sync(0xffffffffu, sum, 8);
        sumsq += __shfl_xor_sync(0xffffffffu, sumsq, 8);
        sum += __shfl_xor_sync(0xffffffffu, sum, 16);
        sumsq += __shfl_xor_sync(0xffffffffu, sumsq, 16);
        if (lane < 8 && n < a.N && !dead) {
          atomicAdd(a.colsum + n, sum);
          atomicAdd(a.colsumsq + n, sumsq);
        }
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(&drained[acc]);  // this warp has read its quarter of the accumulator
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
  if (!tma::encode_matrix_f32(&a.x_map, x, M, K, kBM, kBK) || !tma::encode_matrix_f32(&a.w_map, w, N, K, kBN, kBK))
    return HT_ERR_UNSUPPORTED;
  if ((reinterpret_cast<uintptr_t>(z) & 15u) != 0) return HT_ERR_UNSUPPORTED;  // rows of z are written 16 bytes at a time
  a.z = z;
  a.colsum = colsum;
  a.colsumsq = colsumsq;
  a.status_word = status_word;
  a.M = (int)M;
  a.N = (int)N;
  a.K = (int)K;
  a.m_blocks = (int)((M + kBM - 1) / kBM);
  const int64_t tiles = (int64_t)a.m_blocks * ((N + kBN - 1) / kBN);
  if (tiles > 0x7fffffff) return HT_ERR_UNSUPPORTED;
  a.tiles = (int)tiles;
  int device = 0, sms = 0;
  HT_CUDA_TRY(cudaGetDevice(&device));
  HT_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
  HT_CUDA_TRY(cudaMemsetAsync(colsum, 0, sizeof(float) * (size_t)N, stream));
  HT_CUDA_TRY(cudaMemsetAsync(colsumsq, 0, sizeof(float) * (size_t)N, stream));
  HT_CUDA_TRY(cudaFuncSetAttribute(linear_tf32_stats_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kGemmSmem));
  const unsigned grid = (unsigned)std::min<int64_t>(tiles, std::max(sms, 1));  // one CTA per SM, each walks its tiles
  linear_tf32_stats_kernel<<<grid, kGemmThreads, kGemmSmem, stream>>>(a);
  HT_CHECK_LAUNCH();
  return HT_OK;
}
