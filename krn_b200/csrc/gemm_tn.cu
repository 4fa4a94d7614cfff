// C[M,N] = A[M,K] * B[N,K]^T for 16-bit operands (bf16 / f16) and for unscaled 8-bit float pairs (e4m3 / e5m2, each
// operand its own format), f32 accumulation in tensor memory.
//
// One persistent, warp-specialised kernel per CTA-pair mode:
//   warp 0      TMA producer: one lane streams 128-byte-swizzled A and B tiles into a ring of shared-memory
//               stages (two K blocks of 128 bytes per row each) and arms the stage's "full" mbarrier with the byte count;
//   warp 1      MMA issuer: one lane waits for "full", issues eight tcgen05.mma (32 bytes of K each) per stage
//               into one of two tensor-memory accumulators and commits the stage's "empty" barrier;
//   warps 2..5  epilogue: tcgen05.ld the finished accumulator (each warp owns 32 lanes = 32 rows), round
//               to the output type, stage 32x(128 byte) boxes in swizzled shared memory and TMA-store them,
//               while the MMA warp already fills the other accumulator with the next tile.
// In pair mode (CTA_GROUP = 2) two CTAs on one TPC form a cluster and share a 256x256 output tile: each
// loads its own 128 rows of A and its own 128 of the tile's 256 B rows (no multicast — every byte is
// fetched once by exactly one CTA), the leader issues cta_group::2 MMAs that read both CTAs' shared memory
// and write both CTAs' tensor memory, and barrier arrivals cross the pair through the cluster window.
//
// This is the lowering of `acc += a[rows, ks] @ b[cols, ks].transpose()` in a `pipelined` loop followed by
// `c[rows, cols] = acc.to(T)`; the reference lowers it to mma.sync + ldmatrix + a cp.async ring
// (src/krn/compiler/cuda.py:133-193, src/krn/compiler/emit.py:564-672) and stores with per-element guards
// (src/krn/compiler/emit.py:763-774). TMA gives the same ragged-edge semantics: out-of-range operand
// elements arrive as zeros, out-of-range output elements are clipped.
#include "gemm_common.cuh"

#include <cuda_fp16.h>

namespace krnb {
namespace {

constexpr int kBM = 128;          // rows of C per CTA = tensor-memory lanes
constexpr int kBN = 256;          // columns of C per tile = UMMA N
constexpr int kRowBytes = 128;    // bytes of K per stage row (one swizzle span)
constexpr int kThreads = 192;
constexpr int kTmemColumns = 512; // two 256-column f32 accumulators

template <int CTA_GROUP>
struct Layout {
  static constexpr int kBRows = kBN / CTA_GROUP;
  static constexpr int kABytes = kBM * kRowBytes;
  static constexpr int kBBytes = kBRows * kRowBytes;
  static constexpr int kBlockStageBytes = kABytes + kBBytes;   // one K block (128 bytes of K per row) of A and B
  // A stage is TWO K blocks behind one barrier pair. The issuing thread is the kernel's critical path — a barrier poll
  // costs it about 220 cycles even when it succeeds at once, a commit 60-120, each product about 60 — and one poll and
  // one commit per K block left it at 520-580 cycles per 512 cycles of tensor work.
  static constexpr int kStageBytes = 2 * kBlockStageBytes;
  static constexpr int kStages = CTA_GROUP == 2 ? 3 : 2;
  static constexpr int kEpilogueBytes = 4 * 2 * 4096;  // 4 warps x 2 buffers x (32 rows x 128 bytes)
  static constexpr int kBarrierBytes = 256;
  static constexpr int kSmemBytes = kStages * kStageBytes + kEpilogueBytes + kBarrierBytes + 1024;
};

enum Site { kSiteProducerEmpty = 1, kSiteMmaFull = 2, kSiteMmaTmemEmpty = 3, kSiteEpilogueFull = 4, kSiteRankBarrier = 5 };

// `values[i]` is this thread's accumulator for output column `col + i` (i < 32): add the bias of that column and apply
// the activation, in f32, before the rounding. Lane l fetches the bias of column col + l once; the 32 columns are then
// read from the lanes by shuffle (every lane needs all 32).
template <typename OutT, bool OUT_BF16>
__device__ __forceinline__ void fused_epilogue(uint32_t (&values)[32], const EpilogueSpec& epilogue, int col, int n,
                                               uint32_t lane) {
  const int activation = epilogue.flags >> 1;
  float mine = 0.f;
  if ((epilogue.flags & kEpilogueBias) && col + int(lane) < n) mine = load_bias<OutT, OUT_BF16>(epilogue.bias, col + int(lane));
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    const float x = __uint_as_float(values[i]) + __shfl_sync(0xffffffffu, mine, i);
    values[i] = __float_as_uint(apply_activation(x, activation));
  }
}

template <int CTA_GROUP, int ELEM_BYTES, typename OutT, bool OUT_BF16>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tn_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
               const __grid_constant__ Destinations dst, Problem p, EpilogueSpec epilogue, uint32_t a_format,
               uint32_t b_format, const __grid_constant__ RankSync sync, DeviceStatus* status) {
  using L = Layout<CTA_GROUP>;
  constexpr int kBK = kRowBytes / ELEM_BYTES;                 // K elements per stage
  // b as (K, N): the stage holds [kBK rows of K] x [128 bytes of N] blocks, one per kBlockCols output columns
  constexpr int kBlockCols = kRowBytes / ELEM_BYTES;
  constexpr int kBlockBytes = kBK * kRowBytes;
  constexpr int kChunkCols = kRowBytes / int(sizeof(OutT));   // output columns per 128-byte store row
  constexpr int kChunks = kBN / kChunkCols;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - raw);

  const uint32_t stages_addr = base;
  const uint32_t epilogue_addr = base + L::kStages * L::kStageBytes;
  uint8_t* tail = smem + L::kStages * L::kStageBytes + L::kEpilogueBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(tail);
  const uint32_t full_bar = smem_u32(bars);                       // [kStages]
  const uint32_t empty_bar = full_bar + 8 * L::kStages;           // [kStages]
  const uint32_t tmem_full_bar = empty_bar + 8 * L::kStages;      // [2]
  const uint32_t tmem_empty_bar = tmem_full_bar + 16;             // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tail + 8 * (2 * L::kStages + 4));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const uint32_t lane = lane_id();
  const uint32_t rank = CTA_GROUP == 2 ? cluster_ctarank() : 0u;
  const int cluster_id = blockIdx.x / CTA_GROUP;
  const int num_clusters = gridDim.x / CTA_GROUP;
  const int num_tiles = p.tiles_m * p.tiles_n;
  const int num_kb = (p.k + kBK - 1) / kBK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < L::kStages; ++s) {
      mbar_init(full_bar + 8 * s, 1);
      mbar_init(empty_bar + 8 * s, 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(tmem_full_bar + 8 * i, 1);
      mbar_init(tmem_empty_bar + 8 * i, 4 * CTA_GROUP);
    }
    *abort_flag = 0;
    fence_mbar_init();
    prefetch_tensormap(&map_a);
    prefetch_tensormap(&map_b);
    for (int d = 0; d < dst.count; ++d) prefetch_tensormap(&dst.maps[d]);
  }
  if (warp == 1) {
    tmem_alloc<CTA_GROUP>(smem_u32(tmem_slot), kTmemColumns);
    tmem_relinquish<CTA_GROUP>();
  }
  tc_fence_before();
  __syncthreads();
  if constexpr (CTA_GROUP == 2) {
    cluster_arrive();
    cluster_wait();
  }
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = cluster_id; t < num_tiles && ok; t += num_clusters) {
        int tm, tn;
        tile_coords(t, p, tm, tn);
        const int row_a = tm * (kBM * CTA_GROUP) + int(rank) * kBM;
        const int row_b = tn * kBN + int(rank) * L::kBRows;
        for (int kb0 = 0; kb0 < num_kb; kb0 += 2) {
          if (!mbar_wait(empty_bar + 8 * stage, phase ^ 1u, abort_flag, status, kSiteProducerEmpty)) {
            ok = false;
            break;
          }
          const int blocks = min(2, num_kb - kb0);  // an odd number of K blocks leaves the last stage half full
          const uint32_t leader_full = CTA_GROUP == 2 ? map_to_cta(full_bar + 8 * stage, 0) : full_bar + 8 * stage;
          // in a pair both CTAs' tiles complete on the leader's barrier; the leader alone arms it for both
          if (rank == 0) mbar_arrive_expect_tx(full_bar + 8 * stage, uint32_t(blocks * CTA_GROUP) * L::kBlockStageBytes);
          for (int j = 0; j < blocks; ++j) {
            const int kb = kb0 + j;
            const uint32_t a_dst = stages_addr + stage * L::kStageBytes + j * L::kBlockStageBytes;
            const uint32_t b_dst = a_dst + L::kABytes;
            if constexpr (CTA_GROUP == 1) {
              tma_load_2d(a_dst, &map_a, kb * kBK, row_a, leader_full);
              if (!p.b_kn) {
                tma_load_2d(b_dst, &map_b, kb * kBK, row_b, leader_full);
              } else {
                // b is (K, N): boxes of 128 bytes of N x kBK rows of K, N contiguous; one box per kBlockCols columns
                for (int blk = 0; blk < L::kBRows / kBlockCols; ++blk)
                  tma_load_2d(b_dst + blk * kBlockBytes, &map_b, row_b + blk * kBlockCols, kb * kBK, leader_full);
              }
            } else {
              tma_load_2d_pair(a_dst, &map_a, kb * kBK, row_a, leader_full);
              if (!p.b_kn) {
                tma_load_2d_pair(b_dst, &map_b, kb * kBK, row_b, leader_full);
              } else {
                for (int blk = 0; blk < L::kBRows / kBlockCols; ++blk)
                  tma_load_2d_pair(b_dst + blk * kBlockBytes, &map_b, row_b + blk * kBlockCols, kb * kBK, leader_full);
              }
            }
          }
          if (++stage == L::kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer (leader CTA only)
    // The whole warp runs the loop and one elected lane issues: with every lane on the same path the compiler keeps
    // descriptors, barrier addresses and loop state in uniform registers, which tcgen05 instructions take directly
    // (measured: 23 against 45 cycles per product instruction, 7 against 44 per commit, when issued from a
    // one-lane branch).
    if (rank == 0) {
      const bool leader = elect_one();
      auto wait = [&](uint32_t bar, uint32_t parity, int site) {
        return __all_sync(0xffffffffu, mbar_wait(bar, parity, abort_flag, status, site)) != 0;
      };
      const uint32_t idesc = umma_idesc(a_format, b_format, kBM * CTA_GROUP, kBN, 0, p.b_kn ? 1u : 0u);
      // Descriptor words: b as (N, K) is K-major like a, 32 bytes of K per instruction inside the swizzle span; b as
      // (K, N) is an MN-major operand: blocks of 128 bytes of N are kBlockBytes apart (8192 for 16-bit, 16384 for 8-bit
      // elements), 8-row K groups 1024 bytes apart, and one instruction covers 32 bytes of K = 16 or 32 K rows of 128
      // bytes. Only the low word's start-address field moves (32-bit adds: this thread runs one instruction at a time).
      const uint64_t a_desc0 = umma_desc_kmajor_sw128(stages_addr);
      const uint64_t b_desc0 = p.b_kn ? umma_desc_mnmajor_sw128(stages_addr + L::kABytes, kBlockBytes, 1024)
                                      : umma_desc_kmajor_sw128(stages_addr + L::kABytes);
      const uint32_t a_hi = uint32_t(a_desc0 >> 32), b_hi = uint32_t(b_desc0 >> 32);
      const uint32_t b_step = p.b_kn ? uint32_t(((32 / ELEM_BYTES) * kRowBytes) >> 4) : 2u;
      uint32_t a_lo = uint32_t(a_desc0), b_lo = uint32_t(b_desc0);
      int stage = 0;
      uint32_t phase = 0;
      int iter = 0;
      bool ok = true;
      for (int t = cluster_id; t < num_tiles && ok; t += num_clusters, ++iter) {
        const int acc = iter & 1;
        const uint32_t acc_phase = (iter >> 1) & 1;
        if (!wait(tmem_empty_bar + 8 * acc, acc_phase ^ 1u, kSiteMmaTmemEmpty)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * kBN;
        for (int kb0 = 0; kb0 < num_kb; kb0 += 2) {
          if (!wait(full_bar + 8 * stage, phase, kSiteMmaFull)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const int blocks = min(2, num_kb - kb0);
          if (leader) {
            for (int j = 0; j < blocks; ++j) {
              const uint32_t step = uint32_t(j) * (L::kBlockStageBytes >> 4);
#pragma unroll
              for (int ks = 0; ks < 4; ++ks) {
                umma_ss_halves<CTA_GROUP, ELEM_BYTES == 1>(d_tmem, a_lo + step + 2 * ks, a_hi, b_lo + step + b_step * ks,
                                                           b_hi, idesc, (kb0 + j > 0 || ks > 0) ? 1u : 0u);
              }
            }
            if constexpr (CTA_GROUP == 1) {
              umma_commit(empty_bar + 8 * stage);
            } else {
              umma_commit_pair(empty_bar + 8 * stage, 0x3);
            }
          }
          __syncwarp();
          a_lo += L::kStageBytes >> 4;
          b_lo += L::kStageBytes >> 4;
          if (++stage == L::kStages) {
            stage = 0;
            phase ^= 1u;
            a_lo = uint32_t(a_desc0);
            b_lo = uint32_t(b_desc0);
          }
        }
        if (!ok) break;
        if (leader) {
          if constexpr (CTA_GROUP == 1) {
            umma_commit(tmem_full_bar + 8 * acc);
          } else {
            umma_commit_pair(tmem_full_bar + 8 * acc, 0x3);
          }
        }
        __syncwarp();
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue warps
    const int quarter = warp & 3;  // the 32-lane slice of tensor memory this warp may read
    const uint32_t my_buffers = epilogue_addr + quarter * 2 * 4096;
    const uint32_t leader_tmem_empty = CTA_GROUP == 2 ? map_to_cta(tmem_empty_bar, 0) : tmem_empty_bar;
    int iter = 0;
    bool ok = true;
    int stores = 0;
    for (int t = cluster_id; t < num_tiles && ok; t += num_clusters, ++iter) {
      int tm, tn;
      tile_coords(t, p, tm, tn);
      const int acc = iter & 1;
      const uint32_t acc_phase = (iter >> 1) & 1;
      const int row0 = tm * (kBM * CTA_GROUP) + int(rank) * kBM + quarter * 32;
      const int col0 = tn * kBN;
      // warp-uniform verdict: the aligned tensor-memory loads below need all 32 lanes together
      if (!__all_sync(0xffffffffu, mbar_wait(tmem_full_bar + 8 * acc, acc_phase, abort_flag, status, kSiteEpilogueFull))) {
        ok = false;
        break;
      }
      tc_fence_after();
      const uint32_t t_row = tmem_base + (uint32_t(quarter * 32) << 16) + acc * kBN;
#pragma unroll 1
      for (int chunk = 0; chunk < kChunks; ++chunk) {
        const int col = col0 + chunk * kChunkCols;
        const bool live = row0 < p.m && col < p.n;  // warp-uniform
        uint32_t packed[32];
        if constexpr (sizeof(OutT) == 4) {
          tmem_ld_32x32(t_row + chunk * kChunkCols, packed);
          tmem_ld_wait(packed);
          if (epilogue.flags != 0) fused_epilogue<OutT, OUT_BF16>(packed, epilogue, col, p.n, lane);
        } else {
          uint32_t lo[32], hi[32];
          tmem_ld_32x32(t_row + chunk * kChunkCols, lo);
          tmem_ld_32x32(t_row + chunk * kChunkCols + 32, hi);
          tmem_ld_wait(lo, hi);
          if (epilogue.flags != 0) {
            fused_epilogue<OutT, OUT_BF16>(lo, epilogue, col, p.n, lane);
            fused_epilogue<OutT, OUT_BF16>(hi, epilogue, col + 32, p.n, lane);
          }
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            if constexpr (OUT_BF16) {
              packed[i] = pack_bf16x2(__uint_as_float(lo[2 * i]), __uint_as_float(lo[2 * i + 1]));
              packed[16 + i] = pack_bf16x2(__uint_as_float(hi[2 * i]), __uint_as_float(hi[2 * i + 1]));
            } else {
              packed[i] = pack_f16x2(__uint_as_float(lo[2 * i]), __uint_as_float(lo[2 * i + 1]));
              packed[16 + i] = pack_f16x2(__uint_as_float(hi[2 * i]), __uint_as_float(hi[2 * i + 1]));
            }
          }
        }
        if (live) {
          const uint32_t buffer = my_buffers + (stores & 1) * 4096;
          // the store issued two stores ago read this buffer; wait until it has
          if (lane == 0) tma_store_wait_read<1>();
          __syncwarp();
          const uint32_t row_addr = buffer + lane * 128;
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const uint32_t dst = row_addr + ((uint32_t(j) ^ (lane & 7u)) << 4);
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(packed[4 * j]),
                         "r"(packed[4 * j + 1]), "r"(packed[4 * j + 2]), "r"(packed[4 * j + 3])
                         : "memory");
          }
          fence_async_smem();
          __syncwarp();
          if (lane == 0) {
            // one box, every destination: the own output and, when sharded, each peer's copy of C
            int d = dst.first;
            for (int i = 0; i < dst.count; ++i) {
              tma_store_2d(&dst.maps[d], col + dst.column_offset, row0, buffer);
              if (++d == dst.count) d = 0;
            }
            tma_store_commit();
          }
          ++stores;
        }
      }
      // accumulator drained: hand it back to the MMA warp
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if constexpr (CTA_GROUP == 2) {
          mbar_arrive_cluster(leader_tmem_empty + 8 * acc);
        } else {
          mbar_arrive(tmem_empty_bar + 8 * acc);
        }
      }
    }
    if (lane == 0) {
      tma_store_wait<0>();
      // When the stores went to other ranks, the thread that issued them orders them system-wide itself, before the
      // CTA barrier that precedes the cross-rank flag (completion of a bulk group is a statement about this thread's
      // view of its own copies; the flag is written by another thread).
      if (sync.ranks > 1) {
        asm volatile("fence.proxy.async;" ::: "memory");
        __threadfence_system();
      }
    }
  }

  // ------------------------------------------------------------------ teardown
  if (*abort_flag != 0) {
    // abandoned: give this CTA's own copies in flight time to land before shared memory is released
    for (int i = 0; i < 1000; ++i) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if constexpr (CTA_GROUP == 2) {
    cluster_arrive();
    cluster_wait();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc<CTA_GROUP>(tmem_base, kTmemColumns);
  }
  if (threadIdx.x == 0) rank_barrier_tail(sync, status, kSiteRankBarrier);
}

template <int CTA_GROUP, int ELEM_BYTES, typename OutT, bool OUT_BF16>
int launch(const DeviceContext* ctx, const CUtensorMap& ma, const CUtensorMap& mb, const Destinations& mc, Problem p,
           EpilogueSpec epilogue, uint32_t a_fmt, uint32_t b_fmt, const RankSync& sync, cudaStream_t stream) {
  using L = Layout<CTA_GROUP>;
  auto kernel = gemm_tn_kernel<CTA_GROUP, ELEM_BYTES, OutT, OUT_BF16>;
  KRNB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kSmemBytes));
  const int tiles = p.tiles_m * p.tiles_n;
  int clusters = ctx->sm_count / CTA_GROUP;
  if (clusters > tiles) clusters = tiles;
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(unsigned(clusters * CTA_GROUP), 1, 1);
  config.blockDim = dim3(kThreads, 1, 1);
  config.dynamicSmemBytes = L::kSmemBytes;
  config.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = CTA_GROUP;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  config.attrs = attr;
  config.numAttrs = 1;
  KRNB_CUDA(cudaLaunchKernelEx(&config, kernel, ma, mb, mc, p, epilogue, a_fmt, b_fmt, sync, ctx->status_dev));
  return KRN_B200_OK;
}

template <int ELEM_BYTES>
int launch_for_output(const DeviceContext* ctx, int c_type, int group, const CUtensorMap& ma, const CUtensorMap& mb,
                      const Destinations& mc, Problem p, EpilogueSpec epilogue, uint32_t a_fmt, uint32_t b_fmt,
                      const RankSync& sync, cudaStream_t stream) {
  if (group == 2) {
    if (c_type == KRN_B200_F32) return launch<2, ELEM_BYTES, float, false>(ctx, ma, mb, mc, p, epilogue, a_fmt, b_fmt, sync, stream);
    if (c_type == KRN_B200_BF16) return launch<2, ELEM_BYTES, uint16_t, true>(ctx, ma, mb, mc, p, epilogue, a_fmt, b_fmt, sync, stream);
    return launch<2, ELEM_BYTES, uint16_t, false>(ctx, ma, mb, mc, p, epilogue, a_fmt, b_fmt, sync, stream);
  }
  if (c_type == KRN_B200_F32) return launch<1, ELEM_BYTES, float, false>(ctx, ma, mb, mc, p, epilogue, a_fmt, b_fmt, sync, stream);
  if (c_type == KRN_B200_BF16) return launch<1, ELEM_BYTES, uint16_t, true>(ctx, ma, mb, mc, p, epilogue, a_fmt, b_fmt, sync, stream);
  return launch<1, ELEM_BYTES, uint16_t, false>(ctx, ma, mb, mc, p, epilogue, a_fmt, b_fmt, sync, stream);
}

// Operands whose addresses or row pitches are not multiples of 16 bytes cannot be described to TMA. They take this
// plain tiled kernel instead (64 x 64 outputs per block, 16 of K per step, f32 fma in k order — the same chain the
// reference's scalar fallback runs, src/krn/compiler/emit.py:806-821). It exists so odd shapes such as the
// reference's 50 x 38 x 70 example still run on the device; it is not a performance path.
__device__ __forceinline__ float load_operand(const void* base, long long index, int type) {
  if (type == KRN_B200_BF16) return __uint_as_float(uint32_t(static_cast<const uint16_t*>(base)[index]) << 16);
  if (type == KRN_B200_F16) return __half2float(__ushort_as_half(static_cast<const uint16_t*>(base)[index]));
  const uint32_t code = static_cast<const uint8_t*>(base)[index];
  if (type == KRN_B200_E5M2) return __half2float(__ushort_as_half(uint16_t(code << 8)));  // upper byte of binary16
  uint32_t pair;  // e4m3fn -> f16 is exact
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(pair) : "h"(uint16_t(code)));
  return __half2float(__ushort_as_half(uint16_t(pair & 0xffffu)));
}

__global__ void __launch_bounds__(256)
gemm_tn_unaligned_kernel(const void* __restrict__ a, const void* __restrict__ b, void* __restrict__ c, int m,
                         int n, int k, long long lda, long long ldb, long long ldc, int a_type, int b_type, int c_type,
                         bool b_kn, EpilogueSpec epilogue) {
  __shared__ float as[16][65], bs[16][65];
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int row0 = blockIdx.y * 64, col0 = blockIdx.x * 64;
  float acc[4][4] = {};
  for (int k0 = 0; k0 < k; k0 += 16) {
    for (int i = threadIdx.x; i < 64 * 16; i += 256) {
      const int r = i >> 4, kk = i & 15;
      as[kk][r] = (row0 + r < m && k0 + kk < k) ? load_operand(a, (long long)(row0 + r) * lda + k0 + kk, a_type) : 0.f;
      const long long b_at = b_kn ? (long long)(k0 + kk) * ldb + col0 + r : (long long)(col0 + r) * ldb + k0 + kk;
      bs[kk][r] = (col0 + r < n && k0 + kk < k) ? load_operand(b, b_at, b_type) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < 16; ++kk) {
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(as[kk][ty * 4 + i], bs[kk][tx * 4 + j], acc[i][j]);
    }
    __syncthreads();
  }
  for (int i = 0; i < 4; ++i)
    for (int j = 0; j < 4; ++j) {
      const int r = row0 + ty * 4 + i, col = col0 + tx * 4 + j;
      if (r >= m || col >= n) continue;
      const long long at = (long long)r * ldc + col;
      float value = acc[i][j];
      if (epilogue.flags != 0) {
        if (epilogue.flags & kEpilogueBias) {
          value += c_type == KRN_B200_F32    ? load_bias<float, false>(epilogue.bias, col)
                   : c_type == KRN_B200_BF16 ? load_bias<uint16_t, true>(epilogue.bias, col)
                                             : load_bias<uint16_t, false>(epilogue.bias, col);
        }
        value = apply_activation(value, epilogue.flags >> 1);
      }
      if (c_type == KRN_B200_F32) {
        static_cast<float*>(c)[at] = value;
      } else if (c_type == KRN_B200_BF16) {
        static_cast<uint16_t*>(c)[at] = uint16_t(pack_bf16x2(value, 0.f) & 0xffffu);
      } else {
        static_cast<uint16_t*>(c)[at] = uint16_t(pack_f16x2(value, 0.f) & 0xffffu);
      }
    }
}

__global__ void zero_rows_kernel(uint8_t* c, long long row_bytes, long long pitch_bytes, long long rows) {
  const long long total = rows * row_bytes;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    c[(i / row_bytes) * pitch_bytes + i % row_bytes] = 0;
  }
}

}  // namespace

// CTA pairs (256x256 tiles) whenever the problem has more than one 128-row panel; a single 128-row panel has
// nothing for a second CTA to do.
int gemm_pair_mode(int64_t m) { return m > kBM ? 2 : 1; }

}  // namespace krnb

static bool is_fp8(int type) { return type == KRN_B200_E4M3 || type == KRN_B200_E5M2; }
static bool is_16bit(int type) { return type == KRN_B200_BF16 || type == KRN_B200_F16; }

// Encode the operand and destination maps and launch the tile kernel: C_d[:, offset : offset + n] = A . B^T for every
// destination d (each a row-major matrix of n_total columns with pitch ldc). a_type / b_type are both 16-bit (and then
// equal) or both 8-bit floats (each its own format).
static int tiled_product(const krnb::DeviceContext* ctx, int a_type, int b_type, int c_type, const void* a, const void* b,
                         void* const* destinations, int count, int64_t column_offset, int64_t n_total, int64_t m,
                         int64_t n, int64_t k, int64_t lda, int64_t ldb, int64_t ldc, int group, cudaStream_t stream,
                         bool b_kn = false, krnb::EpilogueSpec epilogue = {nullptr, 0},
                         const krnb::RankSync* rank_sync = nullptr) {
  using namespace krnb;
  const int c_bytes = c_type == KRN_B200_F32 ? 4 : 2;
  const bool fp8 = is_fp8(a_type);
  RankSync sync = {};
  if (rank_sync != nullptr) sync = *rank_sync;
  const int ab_bytes = fp8 ? 1 : 2;
  const uint32_t row_elements = uint32_t(128 / ab_bytes);  // elements in one 128-byte swizzle row
  Problem p;
  p.b_kn = b_kn ? 1 : 0;
  p.m = int(m);
  p.n = int(n);
  p.k = int(k);
  p.tiles_m = int((m + kBM * group - 1) / (kBM * group));
  p.tiles_n = int((n + kBN - 1) / kBN);

  const CUtensorMapDataType ab_dt = fp8                      ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                                    : a_type == KRN_B200_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                              : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  CUtensorMap map_a, map_b;
  {
    uint64_t dims[2] = {uint64_t(k), uint64_t(m)};
    uint64_t strides[1] = {uint64_t(lda) * ab_bytes};
    uint32_t box[2] = {row_elements, uint32_t(kBM)};
    if (int rc = encode_tensor_map(&map_a, ab_dt, 2, a, dims, strides, box, Swizzle::k128B)) return rc;
  }
  if (!b_kn) {
    uint64_t dims[2] = {uint64_t(k), uint64_t(n)};
    uint64_t strides[1] = {uint64_t(ldb) * ab_bytes};
    uint32_t box[2] = {row_elements, uint32_t(kBN / group)};
    if (int rc = encode_tensor_map(&map_b, ab_dt, 2, b, dims, strides, box, Swizzle::k128B)) return rc;
  } else {
    // one box = 128 bytes of N x one stage of K rows (64 for 16-bit, 128 for 8-bit elements)
    uint64_t dims[2] = {uint64_t(n), uint64_t(k)};
    uint64_t strides[1] = {uint64_t(ldb) * ab_bytes};
    uint32_t box[2] = {row_elements, row_elements};
    if (int rc = encode_tensor_map(&map_b, ab_dt, 2, b, dims, strides, box, Swizzle::k128B)) return rc;
  }
  Destinations dst;
  dst.count = count;
  dst.column_offset = int(column_offset);
  dst.first = count > 1 ? int((column_offset / n + 1) % count) : 0;  // column_offset / n = this rank
  for (int d = 0; d < kMaxDestinations; ++d) {
    const CUtensorMapDataType c_dt = c_type == KRN_B200_F32    ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                     : c_type == KRN_B200_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                               : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    uint64_t dims[2] = {uint64_t(n_total), uint64_t(m)};
    uint64_t strides[1] = {uint64_t(ldc) * c_bytes};
    uint32_t box[2] = {uint32_t(128 / c_bytes), 32};
    // unused slots repeat the first destination so that every map in the struct is a valid descriptor
    void* base = destinations[d < count ? d : 0];
    if (int rc = encode_tensor_map(&dst.maps[d], c_dt, 2, base, dims, strides, box, Swizzle::k128B)) return rc;
  }
  if (fp8) {
    const uint32_t a_fmt = a_type == KRN_B200_E4M3 ? kFmtE4M3 : kFmtE5M2;
    const uint32_t b_fmt = b_type == KRN_B200_E4M3 ? kFmtE4M3 : kFmtE5M2;
    return launch_for_output<1>(ctx, c_type, group, map_a, map_b, dst, p, epilogue, a_fmt, b_fmt, sync, stream);
  }
  const uint32_t fmt = a_type == KRN_B200_BF16 ? kFmtBF16 : kFmtF16;
  return launch_for_output<2>(ctx, c_type, group, map_a, map_b, dst, p, epilogue, fmt, fmt, sync, stream);
}

// Argument checks, the K == 0 and unaligned cases and the launch, shared by the two layouts of b and by the 16-bit and
// 8-bit operand kinds.
static int product(int a_type, int b_type, int c_type, const void* a, const void* b, void* c, int64_t m, int64_t n,
                   int64_t k, int64_t lda, int64_t ldb, int64_t ldc, void* stream_handle, bool b_kn,
                   krnb::EpilogueSpec epilogue = {nullptr, 0}) {
  using namespace krnb;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_handle);
  if (!((is_16bit(a_type) && a_type == b_type) || (is_fp8(a_type) && is_fp8(b_type)))) {
    return fail(KRN_B200_ERR_UNSUPPORTED,
                "operand types %d @ %d is not available on sm_100a: the tensor cores multiply two bf16, two f16 or two "
                "8-bit float (e4m3 / e5m2) tiles. Instead: convert the operands to one of those pairs", a_type, b_type);
  }
  if (c_type != KRN_B200_BF16 && c_type != KRN_B200_F16 && c_type != KRN_B200_F32) {
    return fail(KRN_B200_ERR_UNSUPPORTED, "output type %d is not available: use bf16, f16 or f32", c_type);
  }
  if (m < 0 || n < 0 || k < 0) return fail(KRN_B200_ERR_INVALID_ARGUMENT, "negative extent (%lld, %lld, %lld)",
                                           (long long)m, (long long)n, (long long)k);
  if (m == 0 || n == 0) return KRN_B200_OK;
  if (m > INT32_MAX || n > INT32_MAX || k > INT32_MAX) {
    return fail(KRN_B200_ERR_UNSUPPORTED, "extents beyond 2^31-1 are not supported");
  }
  if (c == nullptr || (k > 0 && (a == nullptr || b == nullptr))) {
    return fail(KRN_B200_ERR_INVALID_ARGUMENT, "null tensor address");
  }
  const int c_bytes = c_type == KRN_B200_F32 ? 4 : 2;
  const int ab_bytes = is_fp8(a_type) ? 1 : 2;
  if (ldc < n || (k > 0 && (lda < k || ldb < (b_kn ? n : k)))) {
    return fail(KRN_B200_ERR_INVALID_ARGUMENT, "row pitch shorter than the row (lda %lld, ldb %lld, ldc %lld)",
                (long long)lda, (long long)ldb, (long long)ldc);
  }
  DeviceContext* ctx = current_context();
  if (ctx == nullptr) return KRN_B200_ERR_CUDA;
  if (int rc = require_sm100(ctx)) return rc;

  if (k == 0 && epilogue.flags == 0) {
    // the zero accumulator is stored untouched (src/krn/compiler/emit.py:739-755)
    zero_rows_kernel<<<ctx->sm_count * 4, 256, 0, stream>>>(static_cast<uint8_t*>(c), n * c_bytes, ldc * c_bytes, m);
    KRNB_CUDA(cudaGetLastError());
    return KRN_B200_OK;
  }
  if (k == 0 || !aligned16(a) || !aligned16(b) || !aligned16(c) || (lda * ab_bytes) % 16 != 0 ||
      (ldb * ab_bytes) % 16 != 0 || (ldc * c_bytes) % 16 != 0) {
    // not describable to TMA (or an epilogue over an empty sum): the plain tiled kernel, which needs element-aligned
    // addresses only and never touches a or b when K is 0
    if ((k > 0 && (reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b)) % ab_bytes != 0) ||
        reinterpret_cast<uintptr_t>(c) % c_bytes != 0) {
      return fail(KRN_B200_ERR_INVALID_ARGUMENT, "tensor addresses must be aligned to their element size");
    }
    const dim3 grid(unsigned((n + 63) / 64), unsigned((m + 63) / 64), 1);
    gemm_tn_unaligned_kernel<<<grid, 256, 0, stream>>>(a, b, c, int(m), int(n), int(k), lda, ldb, ldc, a_type, b_type,
                                                       c_type, b_kn, epilogue);
    KRNB_CUDA(cudaGetLastError());
    return KRN_B200_OK;
  }

  const int group = gemm_pair_mode(m);
  void* destinations[1] = {c};
  return tiled_product(ctx, a_type, b_type, c_type, a, b, destinations, 1, 0, n, m, n, k, lda, ldb, ldc, group, stream,
                       b_kn, epilogue);
}

static int refuse_8bit(int ab_type) {
  return krnb::fail(KRN_B200_ERR_UNSUPPORTED,
                    "operand type %d is not available on sm_100a: this entry point multiplies 16-bit tiles. "
                    "Instead: pass KRN_B200_BF16 or KRN_B200_F16 (8-bit float pairs go through krn_b200_gemm_fp8, "
                    "block-scaled ones through krn_b200_gemm_fp8_blockscaled_tn)", ab_type);
}

extern "C" int krn_b200_gemm_fp8(int a_type, int b_type, int c_type, int b_kn, const void* a, const void* b, void* c,
                                 int64_t m, int64_t n, int64_t k, int64_t lda, int64_t ldb, int64_t ldc,
                                 void* stream_handle) {
  if (!is_fp8(a_type) || !is_fp8(b_type)) {
    return krnb::fail(KRN_B200_ERR_UNSUPPORTED,
                      "operand types %d @ %d is not available on sm_100a: this entry point multiplies 8-bit float "
                      "tiles. Instead: pass KRN_B200_E4M3 or KRN_B200_E5M2 for each operand", a_type, b_type);
  }
  return product(a_type, b_type, c_type, a, b, c, m, n, k, lda, ldb, ldc, stream_handle, b_kn != 0);
}

extern "C" int krn_b200_gemm_tn(int ab_type, int c_type, const void* a, const void* b, void* c, int64_t m, int64_t n,
                                int64_t k, int64_t lda, int64_t ldb, int64_t ldc, void* stream_handle) {
  if (!is_16bit(ab_type)) return refuse_8bit(ab_type);
  return product(ab_type, ab_type, c_type, a, b, c, m, n, k, lda, ldb, ldc, stream_handle, false);
}

extern "C" int krn_b200_gemm_nn(int ab_type, int c_type, const void* a, const void* b, void* c, int64_t m, int64_t n,
                                int64_t k, int64_t lda, int64_t ldb, int64_t ldc, void* stream_handle) {
  if (!is_16bit(ab_type)) return refuse_8bit(ab_type);
  return product(ab_type, ab_type, c_type, a, b, c, m, n, k, lda, ldb, ldc, stream_handle, true);
}

extern "C" int krn_b200_matmul(int ab_type, int c_type, int b_kn, int epilogue, const void* a, const void* b,
                               const void* bias, void* c, int64_t m, int64_t n, int64_t k, int64_t lda, int64_t ldb,
                               int64_t ldc, void* stream_handle) {
  using namespace krnb;
  const int activation = epilogue >> 1;
  if (epilogue < 0 || activation > kActivationSilu) {
    return fail(KRN_B200_ERR_INVALID_ARGUMENT, "epilogue flags %d: bit 0 adds the bias, bits 1-2 pick relu (1), gelu "
                "(2) or silu (3)", epilogue);
  }
  if ((epilogue & kEpilogueBias) && bias == nullptr) {
    return fail(KRN_B200_ERR_INVALID_ARGUMENT, "the epilogue adds a bias but the bias address is null");
  }
  const int c_bytes = c_type == KRN_B200_F32 ? 4 : 2;
  if ((epilogue & kEpilogueBias) && reinterpret_cast<uintptr_t>(bias) % c_bytes != 0) {
    return fail(KRN_B200_ERR_INVALID_ARGUMENT, "the bias vector must be aligned to the output element size");
  }
  if (!is_16bit(ab_type)) return refuse_8bit(ab_type);
  return product(ab_type, ab_type, c_type, a, b, c, m, n, k, lda, ldb, ldc, stream_handle, b_kn != 0,
                 EpilogueSpec{bias, epilogue});
}

extern "C" int krn_b200_gemm_tn_gather(int ab_type, int c_type, const void* a, const void* b, void* const* c_of_rank,
                                       int ranks, int rank, int64_t m, int64_t n_local, int64_t k, int64_t lda,
                                       int64_t ldb, int64_t ldc, void* const* sync_of_rank, uint32_t epoch,
                                       void* stream_handle) {
  using namespace krnb;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_handle);
  if (ab_type != KRN_B200_BF16 && ab_type != KRN_B200_F16) {
    return fail(KRN_B200_ERR_UNSUPPORTED, "operand type %d is not available on sm_100a: this entry point multiplies "
                "16-bit tiles. Instead: pass KRN_B200_BF16 or KRN_B200_F16", ab_type);
  }
  if (c_type != KRN_B200_BF16 && c_type != KRN_B200_F16 && c_type != KRN_B200_F32) {
    return fail(KRN_B200_ERR_UNSUPPORTED, "output type %d is not available: use bf16, f16 or f32", c_type);
  }
  if (ranks < 1 || ranks > kMaxDestinations || rank < 0 || rank >= ranks) {
    return fail(KRN_B200_ERR_INVALID_ARGUMENT, "rank %d of %d: between 1 and %d ranks are supported", rank, ranks,
                kMaxDestinations);
  }
  const int c_bytes = c_type == KRN_B200_F32 ? 4 : 2;
  if (m <= 0 || n_local <= 0 || k <= 0 || m > INT32_MAX || n_local * ranks > INT32_MAX || k > INT32_MAX) {
    return fail(KRN_B200_ERR_INVALID_ARGUMENT, "extents must be positive and below 2^31 (m %lld, n_local %lld, k %lld)",
                (long long)m, (long long)n_local, (long long)k);
  }
  if (n_local % (128 / c_bytes) != 0) {
    return fail(KRN_B200_ERR_UNSUPPORTED, "a column block of %lld columns is not a whole number of 128-byte store "
                "rows, so its last store would reach into the next rank's block. Instead: shard N in multiples of "
                "%d columns", (long long)n_local, 128 / c_bytes);
  }
  if (a == nullptr || b == nullptr || c_of_rank == nullptr || lda < k || ldb < k || ldc < n_local * ranks) {
    return fail(KRN_B200_ERR_INVALID_ARGUMENT, "null tensor address or row pitch shorter than the row");
  }
  bool aligned = aligned16(a) && aligned16(b) && (lda * 2) % 16 == 0 && (ldb * 2) % 16 == 0 && (ldc * c_bytes) % 16 == 0;
  void* destinations[kMaxDestinations];
  for (int r = 0; r < ranks; ++r) {
    destinations[r] = c_of_rank[r];
    aligned = aligned && c_of_rank[r] != nullptr && aligned16(c_of_rank[r]);
  }
  if (!aligned) {
    return fail(KRN_B200_ERR_INVALID_ARGUMENT, "the sharded product needs 16-byte aligned addresses and row pitches");
  }
  RankSync sync = {};
  if (int rc = fill_rank_sync(&sync, sync_of_rank, ranks, rank, epoch)) return rc;
  DeviceContext* ctx = current_context();
  if (ctx == nullptr) return KRN_B200_ERR_CUDA;
  if (int rc = require_sm100(ctx)) return rc;
  return tiled_product(ctx, ab_type, ab_type, c_type, a, b, destinations, ranks, rank * n_local, n_local * ranks, m,
                       n_local, k, lda, ldb, ldc, gemm_pair_mode(m), stream, false, EpilogueSpec{nullptr, 0}, &sync);
}
