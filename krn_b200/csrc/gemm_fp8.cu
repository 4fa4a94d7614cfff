// Block-scaled FP8 tile product:
//   C[m,n] = sum over 128-wide K blocks kb of  sa[m,kb] * sb[n/128,kb] * (A8[m,kb-block] . B8[n,kb-block])
// A8, B8 are e4m3fn codes (K-major), sa has one f32 per 1x128 block of A, sb one per 128x128 block of B.
//
// One 128-byte swizzle row of an FP8 operand is exactly one scale block (128 codes), so one pipeline stage is
// one K block. The tensor cores form the UNSCALED partial product of a stage in tensor memory
// (tcgen05.mma kind::f8f6f4, four K=32 instructions, accumulate flag cleared on the first), and while they
// work on the next stage into the other partial buffer the promotion warps read the finished partial
// (tcgen05.ld) and fold it into f32 accumulators held in registers with one packed fma per pair of
// elements: acc += (sa[row,kb] * sb[block,kb]) * partial. The scale therefore rides on the accumulation of
// partial sums — "a coarse scale is applied to the partial sums outside the unit"
// (src/krn/facts/targets.py:127-138) — and no dequantised copy of an operand ever exists. The reference has
// no implementation of this product (QMatrix / QTile are signatures only, src/krn/frontend/memory.py:173-193).
//
// Roles per CTA (384 threads = 3 warpgroups): warp 0 TMA producer, warp 1 MMA issuer, warps 2-3 scale
// loaders (the group gives registers away with setmaxnreg), warps 4..11 promotion + store with 232 registers
// each. A promotion warp owns 32 rows (its tensor-memory lane quarter) x 128 columns (one scale block of B),
// i.e. 128 accumulators per thread.
//
// What the measurements on B200 (M=8192, N=28672, K=8192) say about this kernel:
//  * Operand feed decides the tile shape. One CTA per 128x256 tile moves 48 KB per K block through L2 and
//    shared memory and tops out at 1.40 ms even with the promotion removed; a CTA pair on a 256x256 tile
//    (cta_group::2, each CTA loads 128 rows of A and 128 rows of B) moves 32 KB and reaches 1.27-1.32 ms with
//    the promotion removed. Pairs are therefore used whenever M > 128.
//  * The pair hands a partial buffer back across the cluster every K block. With a release-scope remote
//    arrive each hand-back stalled its warp ~1100 cycles (3.98 ms in total); the relaxed arrive is enough
//    here (see mbar_arrive_cluster_relaxed) and brought the pair to 2.0 ms.
//  * Per-row scale loads straight from global memory (32 lanes, 32 cache lines, every K block) cost 0.15-0.4 ms:
//    two otherwise idle warps now fetch eight K blocks of row scales at a time (one 32-byte sector per row)
//    into a small shared-memory ring, transposed so that a promotion warp reads its 32 scales without conflicts.
//  * Two tcgen05.ld are kept in flight per wait, so a 128-column strip costs two round trips instead of four.
//  * With all of that the kernel runs at 1.92-1.98 ms (1950-2000 TFLOP/s; 2.35 ms before). A cycle trace of one
//    CTA shows what is left: per K block a promotion warp is busy ~950 cycles (barrier poll, two tensor-memory
//    round trips, 64 packed fmas, hand-back) against 540 cycles of tensor-core work, and every poll or
//    shared-memory read on that chain costs 100-250 cycles while the tensor cores and TMA keep shared memory busy.
//    Tried without gain: polling with test_wait, unrolling the issuing thread over the stage ring, fetching the
//    next block's scale early (the in-order warp then waits on that load in front of its fmas), scalar fmas.
#include "gemm_common.cuh"

namespace krnb {
namespace {

constexpr int kBM = 128;
constexpr int kBN = 256;
constexpr int kBK = 128;  // FP8 codes per stage row = one scale block
constexpr int kThreads = 384;  // three warpgroups: {producer, MMA, 2 scale loaders}, promotion x 2
constexpr int kPromotionWarps = 8;
constexpr int kTmemColumns = 512;  // two 256-column partial accumulators
constexpr int kScaleChunk = 8;     // K blocks of row scales per ring slot (8 floats = one 32-byte sector per row)

template <int CTA_GROUP>
struct Layout {
  static constexpr int kBRows = kBN / CTA_GROUP;
  static constexpr int kABytes = kBM * 128;
  static constexpr int kBBytes = kBRows * 128;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStages = CTA_GROUP == 2 ? 6 : 4;
  static constexpr int kStoreBytes = kPromotionWarps * 2048;  // per warp: one 16-row x 128-byte store box
  static constexpr int kScaleBytes = 2 * kScaleChunk * kBM * 4;
  static constexpr int kBarrierBytes = 256;
  static constexpr int kSmemBytes = kStages * kStageBytes + kStoreBytes + kScaleBytes + kBarrierBytes + 1024;
};
static_assert(Layout<2>::kSmemBytes <= 232448 && Layout<1>::kSmemBytes <= 232448, "shared memory budget");

struct Scales {
  const float* sa;
  const float* sb;
  long long ldsa, ldsb;
  int blocks_n;  // ceil(N / 128)
};

enum Site {
  kSiteProducerEmpty = 11,
  kSiteMmaFull = 12,
  kSitePromotionFull = 14,
  kSiteScaleEmpty = 15,
  kSitePromotionScale = 16,
  kSiteRankBarrier = 17,
};

__device__ __forceinline__ void fma_chunk(float2 (&acc)[64], int chunk, const uint32_t (&p)[32], float scale) {
  const float2 s2 = make_float2(scale, scale);
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const float2 v = make_float2(__uint_as_float(p[2 * i]), __uint_as_float(p[2 * i + 1]));
    acc[chunk * 16 + i] = __ffma2_rn(v, s2, acc[chunk * 16 + i]);
  }
}

template <int CTA_GROUP, typename OutT, bool OUT_BF16>
__global__ void __launch_bounds__(kThreads, 1)
gemm_fp8_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                const __grid_constant__ Destinations dst, Problem p, Scales scales,
                const __grid_constant__ RankSync sync, DeviceStatus* status) {
  using L = Layout<CTA_GROUP>;
  constexpr int kChunkCols = 128 / int(sizeof(OutT));  // output columns per 128-byte store row

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - raw);

  const uint32_t stages_addr = base;
  const uint32_t store_addr = base + L::kStages * L::kStageBytes;
  float* scale_ring = reinterpret_cast<float*>(smem + L::kStages * L::kStageBytes + L::kStoreBytes);
  uint8_t* tail = smem + L::kStages * L::kStageBytes + L::kStoreBytes + L::kScaleBytes;
  const uint32_t full_bar = smem_u32(tail);
  const uint32_t empty_bar = full_bar + 8 * L::kStages;
  const uint32_t part_full_bar = empty_bar + 8 * L::kStages;
  const uint32_t scale_full_bar = part_full_bar + 16;
  const uint32_t scale_empty_bar = scale_full_bar + 16;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tail + 8 * (2 * L::kStages + 6));
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
      mbar_init(full_bar + 8 * s, 1 + kPromotionWarps * CTA_GROUP);  // producer + hand-back of the partial buffer
      mbar_init(empty_bar + 8 * s, 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(part_full_bar + 8 * i, 1);
      mbar_init(scale_full_bar + 8 * i, 2);                  // the two loader warps
      mbar_init(scale_empty_bar + 8 * i, kPromotionWarps);   // this CTA's promotion warps
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

  if (warp < 4) reg_dealloc<40>();
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
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(empty_bar + 8 * stage, phase ^ 1u, abort_flag, status, kSiteProducerEmpty)) {
            ok = false;
            break;
          }
          const uint32_t a_dst = stages_addr + stage * L::kStageBytes;
          const uint32_t b_dst = a_dst + L::kABytes;
          if constexpr (CTA_GROUP == 1) {
            mbar_arrive_expect_tx(full_bar + 8 * stage, L::kStageBytes);
            tma_load_2d(a_dst, &map_a, kb * kBK, row_a, full_bar + 8 * stage);
            tma_load_2d(b_dst, &map_b, kb * kBK, row_b, full_bar + 8 * stage);
          } else {
            if (rank == 0) mbar_arrive_expect_tx(full_bar + 8 * stage, 2 * L::kStageBytes);
            const uint32_t leader_full = map_to_cta(full_bar + 8 * stage, 0);
            tma_load_2d_pair(a_dst, &map_a, kb * kBK, row_a, leader_full);
            tma_load_2d_pair(b_dst, &map_b, kb * kBK, row_b, leader_full);
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
    // One thread, every instruction waiting for the one before; beside the promotion warps of its scheduler a
    // barrier poll that succeeds at once still costs it about 250 cycles. So it polls ONE barrier per K block:
    // `full[stage]` counts the producer's arrive (with the stage's bytes) AND the promotion warps' hand-back of the
    // partial buffer this K block will overwrite (they arrive on the full barrier of the K block two ahead).
    // The whole warp runs the loop and one elected lane issues, so that the compiler keeps descriptors, barrier
    // addresses and loop state in uniform registers, which tcgen05 instructions take directly.
    if (rank == 0) {
      const bool leader = elect_one();
      const uint32_t idesc = umma_idesc(kFmtE4M3, kFmtE4M3, kBM * CTA_GROUP, kBN);
      const uint64_t desc0 = umma_desc_kmajor_sw128(stages_addr);
      const uint32_t desc_hi = uint32_t(desc0 >> 32);
      uint32_t a_lo = uint32_t(desc0);
      int stage = 0;
      uint32_t phase = 0;
      uint32_t buf = 0;
      bool ok = true;
      for (int t = cluster_id; t < num_tiles && ok; t += num_clusters) {
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!__all_sync(0xffffffffu, mbar_wait(full_bar + 8 * stage, phase, abort_flag, status, kSiteMmaFull))) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + buf * kBN;
          const uint32_t b_lo = a_lo + (L::kABytes >> 4);
          if (leader) {
#pragma unroll
            for (int ks = 0; ks < 4; ++ks) {
              umma_ss_halves<CTA_GROUP, true>(d_tmem, a_lo + 2 * ks, desc_hi, b_lo + 2 * ks, desc_hi, idesc,
                                              ks > 0 ? 1u : 0u);
            }
            // the promotion warps wait for the first of these: it is on the kernel's critical cycle, the producer's
            // is not
            if constexpr (CTA_GROUP == 1) {
              umma_commit(part_full_bar + 8 * buf);
              umma_commit(empty_bar + 8 * stage);
            } else {
              umma_commit_pair(part_full_bar + 8 * buf, 0x3);
              umma_commit_pair(empty_bar + 8 * stage, 0x3);
            }
          }
          __syncwarp();
          buf ^= 1u;
          a_lo += L::kStageBytes >> 4;
          if (++stage == L::kStages) {
            stage = 0;
            phase ^= 1u;
            a_lo = uint32_t(desc0);
          }
        }
      }
    }
  } else if (warp < 4) {
    // ---------------------------------------------------------------- row-scale loaders (64 threads)
    // Ring slot = kScaleChunk K blocks x 128 rows, stored [block][row] so that a promotion warp reads 32
    // consecutive floats. Each thread fetches the 8 scales of two rows: one 32-byte sector per row.
    const int tid = int(threadIdx.x) - 64;
    const bool vector_ok = (reinterpret_cast<uintptr_t>(scales.sa) % 16 == 0) && (scales.ldsa % 4 == 0);
    uint32_t chunk = 0;
    bool ok = true;
    for (int t = cluster_id; t < num_tiles && ok; t += num_clusters) {
      int tm, tn;
      tile_coords(t, p, tm, tn);
      const int row0 = tm * (kBM * CTA_GROUP) + int(rank) * kBM;
      for (int kb0 = 0; kb0 < num_kb; kb0 += kScaleChunk, ++chunk) {
        const uint32_t slot = chunk & 1u;
        if (!__all_sync(0xffffffffu, mbar_wait(scale_empty_bar + 8 * slot, ((chunk >> 1) & 1u) ^ 1u, abort_flag, status,
                                               kSiteScaleEmpty))) {
          ok = false;
          break;
        }
        float* dst = scale_ring + slot * (kScaleChunk * kBM);
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          const int r = tid + half * 64;
          const int row = row0 + r;
          float v[kScaleChunk];
#pragma unroll
          for (int j = 0; j < kScaleChunk; ++j) v[j] = 0.f;
          if (row < p.m) {
            const float* src = scales.sa + (long long)row * scales.ldsa + kb0;
            if (vector_ok && kb0 + kScaleChunk <= num_kb) {
              const float4 lo = __ldg(reinterpret_cast<const float4*>(src));
              const float4 hi = __ldg(reinterpret_cast<const float4*>(src) + 1);
              v[0] = lo.x, v[1] = lo.y, v[2] = lo.z, v[3] = lo.w;
              v[4] = hi.x, v[5] = hi.y, v[6] = hi.z, v[7] = hi.w;
            } else {
#pragma unroll
              for (int j = 0; j < kScaleChunk; ++j) {
                if (kb0 + j < num_kb) v[j] = __ldg(src + j);
              }
            }
          }
#pragma unroll
          for (int j = 0; j < kScaleChunk; ++j) dst[j * kBM + r] = v[j];
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(scale_full_bar + 8 * slot);
      }
    }
  } else {
    // ---------------------------------------------------------------- promotion + store warps
    reg_alloc<232>();
    const int pw = warp - 4;       // 0..7
    const int quarter = warp & 3;  // tensor-memory lane quarter this warp may read
    const int half = pw >> 2;      // which 128-column scale block of the tile
    const uint32_t my_store = store_addr + pw * 2048;
    const uint32_t leader_full = CTA_GROUP == 2 ? map_to_cta(full_bar, 0) : full_bar;
    // the first two K blocks overwrite partial buffers nobody has to hand back
    if (lane == 0) {
#pragma unroll
      for (int s = 0; s < 2; ++s) {
        if constexpr (CTA_GROUP == 2) {
          mbar_arrive_cluster_relaxed(leader_full + 8 * s);
        } else {
          mbar_arrive(full_bar + 8 * s);
        }
      }
    }
    uint32_t handback_stage = 2;  // stage of K block it + 2
    const float* my_scales = scale_ring + quarter * 32 + lane;
    uint32_t it = 0;
    uint32_t chunk = 0;
    bool ok = true;
    for (int t = cluster_id; t < num_tiles && ok; t += num_clusters) {
      int tm, tn;
      tile_coords(t, p, tm, tn);
      const int row0 = tm * (kBM * CTA_GROUP) + int(rank) * kBM + quarter * 32;
      const int col0 = tn * kBN + half * 128;
      const int nb = col0 / 128;
      const bool nb_ok = nb < scales.blocks_n;
      const float* sb_row = scales.sb + (long long)(nb_ok ? nb : 0) * scales.ldsb;

      float2 acc[64];
#pragma unroll
      for (int i = 0; i < 64; ++i) acc[i] = make_float2(0.f, 0.f);

      float next_sb = (num_kb > 0 && nb_ok) ? __ldg(sb_row) : 0.f;  // one address for the whole warp
      for (int kb = 0; kb < num_kb; ++kb, ++it) {
        const uint32_t buf = it & 1u;
        const uint32_t slot = chunk & 1u;
        const int in_chunk = kb & (kScaleChunk - 1);
        if (in_chunk == 0) {
          if (!__all_sync(0xffffffffu, mbar_wait(scale_full_bar + 8 * slot, (chunk >> 1) & 1u, abort_flag, status,
                                                 kSitePromotionScale))) {
            ok = false;
            break;
          }
        }
        // rows beyond M hold a zero scale in the ring, so their accumulators stay zero
        const float scale = my_scales[slot * (kScaleChunk * kBM) + in_chunk * kBM] * next_sb;
        if (kb + 1 < num_kb && nb_ok) next_sb = __ldg(sb_row + kb + 1);
        // every lane polls the same barrier and gets the same answer: no vote (it is on this warp's critical chain)
        if (!mbar_wait(part_full_bar + 8 * buf, (it >> 1) & 1u, abort_flag, status, kSitePromotionFull)) {
          ok = false;
          break;
        }
        __syncwarp();
        tc_fence_after();
        const uint32_t t_addr = tmem_base + (uint32_t(quarter * 32) << 16) + buf * kBN + half * 128;
        uint32_t p0[32], p1[32];
        tmem_ld_32x32(t_addr, p0);
        tmem_ld_32x32(t_addr + 32, p1);
        tmem_ld_wait(p0, p1);
        fma_chunk(acc, 0, p0, scale);
        tmem_ld_32x32(t_addr + 64, p0);
        fma_chunk(acc, 1, p1, scale);
        tmem_ld_32x32(t_addr + 96, p1);
        tmem_ld_wait(p0, p1);
        // the partial buffer is fully read (its data sits in registers): hand it back before the last fmas
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          if constexpr (CTA_GROUP == 2) {
            mbar_arrive_cluster_relaxed(leader_full + 8 * handback_stage);
          } else {
            mbar_arrive(full_bar + 8 * handback_stage);
          }
          if (in_chunk == kScaleChunk - 1 || kb == num_kb - 1) mbar_arrive(scale_empty_bar + 8 * slot);
        }
        if (in_chunk == kScaleChunk - 1 || kb == num_kb - 1) ++chunk;
        if (++handback_stage == L::kStages) handback_stage = 0;
        fma_chunk(acc, 2, p0, scale);
        fma_chunk(acc, 3, p1, scale);
      }
      if (!ok) break;

      // ---- store this warp's 32 x 128 block through 2 KB of swizzled staging: 128-byte strips, 16 rows per TMA box
      constexpr int kStoreChunks = 128 / kChunkCols;  // 2 for 16-bit outputs, 4 for f32
#pragma unroll
      for (int chunk_index = 0; chunk_index < kStoreChunks; ++chunk_index) {
        uint32_t packed[32];
        if constexpr (sizeof(OutT) == 4) {
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            packed[2 * i] = __float_as_uint(acc[chunk_index * 16 + i].x);
            packed[2 * i + 1] = __float_as_uint(acc[chunk_index * 16 + i].y);
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const float2 v = acc[chunk_index * 32 + i];
            packed[i] = OUT_BF16 ? pack_bf16x2(v.x, v.y) : pack_f16x2(v.x, v.y);
          }
        }
#pragma unroll
        for (int rows_half = 0; rows_half < 2; ++rows_half) {
          if (lane == 0) tma_store_wait_read<0>();
          __syncwarp();
          if (int(lane >> 4) == rows_half) {
            const uint32_t row_addr = my_store + (lane & 15u) * 128;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const uint32_t dst = row_addr + ((uint32_t(j) ^ (lane & 7u)) << 4);
              asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(packed[4 * j]),
                           "r"(packed[4 * j + 1]), "r"(packed[4 * j + 2]), "r"(packed[4 * j + 3])
                           : "memory");
            }
          }
          fence_async_smem();
          __syncwarp();
          if (lane == 0) {
            const int col = col0 + chunk_index * kChunkCols;
            const int row = row0 + rows_half * 16;
            if (row < p.m && col < p.n) {
              // one box, every destination: the own output and, when sharded, each peer's copy of C
              int d = dst.first;
              for (int i = 0; i < dst.count; ++i) {
                tma_store_2d(&dst.maps[d], col + dst.column_offset, row, my_store);
                if (++d == dst.count) d = 0;
              }
            }
            tma_store_commit();
          }
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

template <int CTA_GROUP, typename OutT, bool OUT_BF16>
int launch(const DeviceContext* ctx, const CUtensorMap& ma, const CUtensorMap& mb, const Destinations& mc, Problem p,
           Scales scales, const RankSync& sync, cudaStream_t stream) {
  using L = Layout<CTA_GROUP>;
  auto kernel = gemm_fp8_kernel<CTA_GROUP, OutT, OUT_BF16>;
  KRNB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kSmemBytes));
  // setmaxnreg.inc blocks until the CTA's register pool holds what it asks for: refuse to launch a build
  // whose launch-time allocation cannot cover 2 x 128 x (232 - R) with 128 x (R - 40).
  cudaFuncAttributes attributes;
  KRNB_CUDA(cudaFuncGetAttributes(&attributes, kernel));
  if ((attributes.numRegs - 40) * 128 < (232 - attributes.numRegs) * 256) {
    return fail(KRN_B200_ERR_UNSUPPORTED, "FP8 kernel was built with %d registers per thread; the register "
                "re-partitioning needs at least 168", attributes.numRegs);
  }
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
  KRNB_CUDA(cudaLaunchKernelEx(&config, kernel, ma, mb, mc, p, scales, sync, ctx->status_dev));
  return KRN_B200_OK;
}

__global__ void zero_rows_kernel(uint8_t* c, long long row_bytes, long long pitch_bytes, long long rows) {
  const long long total = rows * row_bytes;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    c[(i / row_bytes) * pitch_bytes + i % row_bytes] = 0;
  }
}

int fp8_pair_mode(int64_t m) { return m > kBM ? 2 : 1; }

}  // namespace
}  // namespace krnb

// Checks, tensor maps and launch shared by the plain and the column-sharded entry points: C_d[:, offset : offset + n]
// for every destination d (each a row-major matrix of n_total columns with pitch ldc).
static int fp8_product(int c_type, const void* a, const float* sa, const void* b, const float* sb,
                       void* const* destinations, int count, int64_t column_offset, int64_t n_total, int64_t m, int64_t n,
                       int64_t k, int64_t lda, int64_t ldb, int64_t ldc, int64_t ldsa, int64_t ldsb, void* stream_handle,
                       const krnb::RankSync* rank_sync = nullptr) {
  using namespace krnb;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_handle);
  RankSync sync = {};
  if (rank_sync != nullptr) sync = *rank_sync;
  if (c_type != KRN_B200_BF16 && c_type != KRN_B200_F16 && c_type != KRN_B200_F32) {
    return fail(KRN_B200_ERR_UNSUPPORTED, "output type %d is not available: use bf16, f16 or f32", c_type);
  }
  if (m < 0 || n < 0 || k < 0) return fail(KRN_B200_ERR_INVALID_ARGUMENT, "negative extent");
  if (m == 0 || n == 0) return KRN_B200_OK;
  if (m > INT32_MAX || n_total > INT32_MAX || k > INT32_MAX) {
    return fail(KRN_B200_ERR_UNSUPPORTED, "extents beyond 2^31-1 are not supported");
  }
  bool null_destination = false, aligned_destinations = true;
  for (int d = 0; d < count; ++d) {
    null_destination = null_destination || destinations[d] == nullptr;
    aligned_destinations = aligned_destinations && aligned16(destinations[d]);
  }
  if (null_destination || (k > 0 && (a == nullptr || b == nullptr || sa == nullptr || sb == nullptr))) {
    return fail(KRN_B200_ERR_INVALID_ARGUMENT, "null tensor address");
  }
  const int c_bytes = c_type == KRN_B200_F32 ? 4 : 2;
  const int64_t blocks_k = (k + 127) / 128;
  if (ldc < n_total || (k > 0 && (lda < k || ldb < k || ldsa < blocks_k || ldsb < blocks_k))) {
    return fail(KRN_B200_ERR_INVALID_ARGUMENT, "row pitch shorter than the row");
  }
  DeviceContext* ctx = current_context();
  if (ctx == nullptr) return KRN_B200_ERR_CUDA;
  if (int rc = require_sm100(ctx)) return rc;
  if (k == 0) {
    for (int d = 0; d < count; ++d) {
      zero_rows_kernel<<<ctx->sm_count * 4, 256, 0, stream>>>(
          static_cast<uint8_t*>(destinations[d]) + column_offset * c_bytes, n * c_bytes, ldc * c_bytes, m);
      KRNB_CUDA(cudaGetLastError());
    }
    return KRN_B200_OK;
  }
  if (!aligned16(a) || !aligned16(b) || !aligned_destinations || lda % 16 != 0 || ldb % 16 != 0 ||
      (ldc * c_bytes) % 16 != 0) {
    return fail(KRN_B200_ERR_INVALID_ARGUMENT,
                "TMA needs 16-byte aligned base addresses and row pitches (lda %lld, ldb %lld bytes, ldc %lld elements)",
                (long long)lda, (long long)ldb, (long long)ldc);
  }
  // CTA pairs whenever there is more than one 128-row panel (see the measurements at the top of this file)
  const int group = fp8_pair_mode(m);
  Problem p;
  p.m = int(m);
  p.n = int(n);
  p.k = int(k);
  p.tiles_m = int((m + kBM * group - 1) / (kBM * group));
  p.tiles_n = int((n + kBN - 1) / kBN);
  p.b_kn = 0;
  Scales scales;
  scales.sa = sa;
  scales.sb = sb;
  scales.ldsa = ldsa;
  scales.ldsb = ldsb;
  scales.blocks_n = int((n + 127) / 128);

  CUtensorMap map_a, map_b;
  {
    uint64_t dims[2] = {uint64_t(k), uint64_t(m)};
    uint64_t strides[1] = {uint64_t(lda)};
    uint32_t box[2] = {128, uint32_t(kBM)};
    if (int rc = encode_tensor_map(&map_a, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, a, dims, strides, box, Swizzle::k128B)) return rc;
  }
  {
    uint64_t dims[2] = {uint64_t(k), uint64_t(n)};
    uint64_t strides[1] = {uint64_t(ldb)};
    uint32_t box[2] = {128, uint32_t(kBN / group)};
    if (int rc = encode_tensor_map(&map_b, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, b, dims, strides, box, Swizzle::k128B)) return rc;
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
    uint32_t box[2] = {uint32_t(128 / c_bytes), 16};
    // unused slots repeat the first destination so that every map in the struct is a valid descriptor
    if (int rc = encode_tensor_map(&dst.maps[d], c_dt, 2, destinations[d < count ? d : 0], dims, strides, box,
                                   Swizzle::k128B)) return rc;
  }
  if (group == 2) {
    if (c_type == KRN_B200_F32) return launch<2, float, false>(ctx, map_a, map_b, dst, p, scales, sync, stream);
    if (c_type == KRN_B200_BF16) return launch<2, uint16_t, true>(ctx, map_a, map_b, dst, p, scales, sync, stream);
    return launch<2, uint16_t, false>(ctx, map_a, map_b, dst, p, scales, sync, stream);
  }
  if (c_type == KRN_B200_F32) return launch<1, float, false>(ctx, map_a, map_b, dst, p, scales, sync, stream);
  if (c_type == KRN_B200_BF16) return launch<1, uint16_t, true>(ctx, map_a, map_b, dst, p, scales, sync, stream);
  return launch<1, uint16_t, false>(ctx, map_a, map_b, dst, p, scales, sync, stream);
}

extern "C" int krn_b200_gemm_fp8_blockscaled_tn(int c_type, const void* a, const float* sa, const void* b,
                                                const float* sb, void* c, int64_t m, int64_t n, int64_t k,
                                                int64_t lda, int64_t ldb, int64_t ldc, int64_t ldsa, int64_t ldsb,
                                                void* stream_handle) {
  void* destinations[1] = {c};
  return fp8_product(c_type, a, sa, b, sb, destinations, 1, 0, n, m, n, k, lda, ldb, ldc, ldsa, ldsb, stream_handle);
}

extern "C" int krn_b200_gemm_fp8_blockscaled_tn_gather(int c_type, const void* a, const float* sa, const void* b,
                                                       const float* sb, void* const* c_of_rank, int ranks, int rank,
                                                       int64_t m, int64_t n_local, int64_t k, int64_t lda, int64_t ldb,
                                                       int64_t ldc, int64_t ldsa, int64_t ldsb,
                                                       void* const* sync_of_rank, uint32_t epoch, void* stream_handle) {
  using namespace krnb;
  if (ranks < 1 || ranks > kMaxDestinations || rank < 0 || rank >= ranks || c_of_rank == nullptr) {
    return fail(KRN_B200_ERR_INVALID_ARGUMENT, "rank %d of %d: between 1 and %d ranks are supported", rank, ranks,
                kMaxDestinations);
  }
  if (m <= 0 || n_local <= 0 || k <= 0) {
    return fail(KRN_B200_ERR_INVALID_ARGUMENT, "extents must be positive (m %lld, n_local %lld, k %lld)", (long long)m,
                (long long)n_local, (long long)k);
  }
  if (n_local % 128 != 0) {
    return fail(KRN_B200_ERR_UNSUPPORTED, "a column block of %lld columns does not end on a 128-column scale block of b. "
                "Instead: shard N in multiples of 128 columns", (long long)n_local);
  }
  void* destinations[kMaxDestinations];
  for (int r = 0; r < ranks; ++r) destinations[r] = c_of_rank[r];
  RankSync sync = {};
  if (int rc = fill_rank_sync(&sync, sync_of_rank, ranks, rank, epoch)) return rc;
  return fp8_product(c_type, a, sa, b, sb, destinations, ranks, rank * n_local, n_local * ranks, m, n_local, k, lda, ldb,
                     ldc, ldsa, ldsb, stream_handle, &sync);
}
