// MXFP8 and NVFP4 tile products with the block scales applied BY the tensor cores. MXFP8:
//   C[m,n] = sum over 32-wide K blocks kb of  2^(sa[m,kb] - 127) * 2^(sb[n,kb] - 127) * (A8[m, kb-block] . B8[n, kb-block])
// A8, B8 are e4m3fn codes (K-major), sa / sb one e8m0 byte per 1 x 32 block: the reference's `MXFP8` block format
// (src/krn/data/formats.py:138-144; `QMatrix` / `QTile` carry it as signatures only, src/krn/frontend/memory.py:173-193,
// 255-269). tcgen05.mma kind::mxf8f6f4.block_scale takes the scale factors as operands of the instruction — "a
// block-scaled MMA" in the literal sense — so nothing is dequantised and no partial sum leaves tensor memory before the
// last K block.
//
// Tiles: a CTA pair on a 256 x 256 tile (cta_group::2: each CTA holds 128 rows of A, 128 of the 256 rows of B, and its
// own 128 x 256 half of the accumulator) whenever M > 128, else one CTA on a 128 x 256 tile. The pair moves 32 KB per K
// block and CTA through L2 and shared memory instead of 48 KB, which is what the single-CTA form is limited by.
//
// Scale bytes. tcgen05.cp (32x128b.warpx4) copies one 512-byte atom — 128 rows x 4 scale bytes, byte offset
// (row % 32) * 16 + (row / 32) * 4 — from shared memory into four tensor-memory columns. The row-major scale matrices
// are therefore first rewritten by a small kernel (tile_scales_kernel, same stream, stream-ordered scratch memory) into
// such atoms, one per group of 128 rows, K block and set of four bytes per row, and the product kernel fetches them by
// TMA together with the operands. (Fetching and transposing them with loader warps inside the product kernel was the
// first design; with 16 scale bytes per row and K block in NVFP4 those warps, competing with TMA and the tensor cores
// for shared memory, set the kernel's pace: 0.80 ms against 0.69 at M = 8192, N = 28672, K = 8192.)
//
// Roles per CTA (192 threads, persistent over tiles):
//   warp 0      TMA producer: per stage the A and B tiles (128 bytes of K per row; two K blocks per stage for MXFP8 —
//               one barrier per 256 codes halves the issuing warp's polls and commits — one for the 4-bit formats) and
//               the stage's scale atoms: this CTA's 128 A rows and ALL 256 B rows of the tile (each CTA of a pair
//               multiplies its A rows by every column, so it needs every column's scale)
//   warp 1      MMA issuer: per K block copies that block's scale atoms into tensor memory (tcgen05.cp; in a pair the
//               leader's one instruction, cta_group::2, makes each CTA copy from its OWN shared memory into its own
//               tensor memory) and issues four instructions (K = 32 codes for MXFP8, whose descriptors select the scale
//               byte of their sub-block; 64 codes for the 4-bit formats)
//   warps 2-5   epilogue: tensor memory -> registers -> output type -> swizzled staging -> TMA store
//
// Tensor memory (512 columns): 256 accumulator columns, then 4 columns of A scales and 8 of B scales. One accumulator
// only — two would not leave room for the scales — so the epilogue's tensor-memory reads (not its stores) are not
// overlapped with the next tile's products: about 5 % of a tile at K = 8192.
//
// The scale-factor columns are rewritten for every K block while earlier products may still be in flight; tcgen05.cp
// and tcgen05.mma issued by one thread execute in issue order, which is what makes that safe.
//
// NVFP4 (template flag FP4; the reference's `NVFP4` block format, src/krn/data/formats.py:147-154):
//   C[m,n] = alpha * sum over 16-wide K blocks kb of  sa[m,kb] * sb[n,kb] * (A4[m, kb-block] . B4[n, kb-block])
// A4, B4 are e2m1 codes packed two per byte (low nibble = lower k), sa / sb one e4m3 byte per 1 x 16 block, alpha the
// product of the two matrices' f32 tensor scales (applied in the epilogue). Same kernel, same roles; what changes:
// a 128-byte stage row is 256 codes, an instruction (kind::mxf4nvf4, scale_vec::4X) covers 64 codes and takes all four
// bytes of a scale-factor column, so each of the four instructions of a K block has its own three scale copies and
// its own twelve tensor-memory columns, and a row has 16 scale bytes per K block (four atoms per group of 128 rows).
#include "gemm_common.cuh"

namespace krnb {
namespace {

constexpr int kBM = 128;
constexpr int kBN = 256;
constexpr int kBK = 128;          // codes per stage row = four 32-wide scale blocks
constexpr int kThreads = 192;      // producer warp, issuing warp, four epilogue warps
constexpr int kABytes = kBM * 128;
constexpr int kEpilogueBytes = 4 * 2048;                // per epilogue warp: one 16-row x 128-byte store box
constexpr int kMxfp8 = 0, kNvfp4 = 1, kMxfp4 = 2;  // FORMAT: what the codes and the scale bytes are

template <int CTA_GROUP, int FORMAT>
struct Layout {
  static constexpr bool FP4 = FORMAT != kMxfp8;            // 4-bit codes, 256 per 128-byte stage row
  // 32-bit words of scale bytes per row and K block = sets of scale copies per K block: MXFP8 one (a byte per 32 codes,
  // its four instructions pick their byte of the one column), NVFP4 four (a byte per 16 codes: every 64-code
  // instruction takes a whole word), MXFP4 two (a byte per 32 codes: two instructions share a word).
  static constexpr int kWordsPerBlock = FORMAT == kNvfp4 ? 4 : FORMAT == kMxfp4 ? 2 : 1;
  static constexpr int kBRows = kBN / CTA_GROUP;           // rows of B this CTA loads
  static constexpr int kBlockBytes = kABytes + kBRows * 128;  // one K block (128 bytes per row): this CTA's A and B rows
  // A stage is two K blocks behind ONE barrier for MXFP8 (one poll and one commit of the issuing warp per 256 codes).
  // The 4-bit formats run a K block in about the time of one TMA round trip, so what their speed needs first is stages
  // in flight: theirs are single K blocks, five of them in a pair (three were measured to starve the issuing warp).
  static constexpr int kBlocksPerStage = FP4 ? 1 : 2;
  // Sets of scale copies per K block: MXFP8's four instructions share one (each picks its byte of the column), NVFP4's
  // four instructions take four bytes each, MXFP4's share a set in twos.
  static constexpr int kScaleSets = kWordsPerBlock;
  // The scale bytes of a stage arrive with its operands, by TMA, from a copy that a small kernel has laid out beforehand
  // the way tcgen05.cp wants them: 512-byte atoms (128 rows x 4 bytes), one per group of 128 rows, K block and set.
  // Behind the operands a stage holds three runs of atoms — this CTA's A rows, B rows 0-127, B rows 128-255 of the tile
  // (each CTA of a pair multiplies its A rows by every column, so it needs every column's scale) — each run with the
  // atoms of the stage's K blocks in order.
  static constexpr int kRunBytes = kBlocksPerStage * kScaleSets * 512;
  static constexpr int kStageScaleBytes = 3 * kRunBytes;
  static constexpr int kStageBytes = kBlocksPerStage * kBlockBytes + kStageScaleBytes;
  static constexpr int kStages = FP4 ? (CTA_GROUP == 2 ? 5 : 4) : (CTA_GROUP == 2 ? 3 : 2);
  static constexpr int kSmemBytes = kStages * kStageBytes + kEpilogueBytes + 256 + 1024;
};
constexpr int kTmemColumns = 512;
constexpr int kTmemScaleA = 256;                        // first column of the scale factors: per set, 4 columns of A
constexpr int kTmemScaleB = 260;                        // and 8 of B; sets are 12 columns apart
static_assert(Layout<1, kMxfp8>::kSmemBytes <= 232448 && Layout<2, kMxfp8>::kSmemBytes <= 232448 &&
              Layout<1, kNvfp4>::kSmemBytes <= 232448 && Layout<2, kNvfp4>::kSmemBytes <= 232448 &&
              Layout<1, kMxfp4>::kSmemBytes <= 232448 && Layout<2, kMxfp4>::kSmemBytes <= 232448, "shared memory budget");

struct MxScales {
  int b_atom0;  // first 512-byte atom of B's scales in the pre-tiled copy (A's atoms start at 0)
  float alpha;  // NVFP4: product of the two tensor scales, applied to the finished accumulator
};

enum Site { kSiteProducerEmpty = 41, kSiteMmaFull = 42, kSiteMmaTmemEmpty = 44, kSiteEpilogueFull = 45 };


// Instruction descriptor of kind::mxf8f6f4.block_scale: B scale id [4,6), A format [7,10), B format [10,13), majors 15 /
// 16, N / 8 at [17,23), scale format (1 = e8m0) at 23, M / 16 at [24,29), A scale id [29,31). The scale id picks which
// of the four bytes of a scale-factor column belongs to this instruction's 32-wide K sub-block.
__device__ __forceinline__ uint32_t mx_idesc(uint32_t sub_block, uint32_t m) {
  return (sub_block << 4) | (kFmtE4M3 << 7) | (kFmtE4M3 << 10) | (uint32_t(kBN >> 3) << 17) | (1u << 23) |
         ((m >> 4) << 24) | (sub_block << 29);
}

// Instruction descriptor of kind::mxf4nvf4.block_scale.scale_vec::4X: the same fields; operand format 1 = e2m1, scale
// format 0 = ue4m3 (the e4m3 code read as unsigned), scale ids 0 because an instruction takes all four bytes.
__device__ __forceinline__ uint32_t nvf4_idesc(uint32_t m) {
  return (1u << 7) | (1u << 10) | (uint32_t(kBN >> 3) << 17) | ((m >> 4) << 24);
}

template <int CTA_GROUP>
__device__ __forceinline__ void umma_nvf4(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t desc_hi, uint32_t idesc,
                                          uint32_t scale_a_tmem, uint32_t scale_b_tmem, uint32_t accumulate) {
  if constexpr (CTA_GROUP == 1) {
    asm volatile(
        "{\n .reg .pred p;\n .reg .b64 da, db;\n setp.ne.b32 p, %7, 0;\n mov.b64 da, {%1, %3};\n mov.b64 db, {%2, %3};\n"
        " tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], da, db, %4, [%5], [%6], p;\n}\n"
        ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(desc_hi), "r"(idesc), "r"(scale_a_tmem), "r"(scale_b_tmem), "r"(accumulate)
        : "memory");
  } else {
    asm volatile(
        "{\n .reg .pred p;\n .reg .b64 da, db;\n setp.ne.b32 p, %7, 0;\n mov.b64 da, {%1, %3};\n mov.b64 db, {%2, %3};\n"
        " tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], da, db, %4, [%5], [%6], p;\n}\n"
        ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(desc_hi), "r"(idesc), "r"(scale_a_tmem), "r"(scale_b_tmem), "r"(accumulate)
        : "memory");
  }
}

// Instruction descriptor of kind::mxf4.block_scale.scale_vec::2X (MXFP4): e2m1 operands, e8m0 scales (bit 23), and
// the scale id picks which half (bytes 0-1 or 2-3) of a scale-factor column belongs to this 64-code instruction.
__device__ __forceinline__ uint32_t mxf4_idesc(uint32_t scale_id, uint32_t m) {
  return (scale_id << 4) | (1u << 7) | (1u << 10) | (uint32_t(kBN >> 3) << 17) | (1u << 23) | ((m >> 4) << 24) | (scale_id << 29);
}

template <int CTA_GROUP>
__device__ __forceinline__ void umma_mxf4(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t desc_hi, uint32_t idesc,
                                          uint32_t scale_a_tmem, uint32_t scale_b_tmem, uint32_t accumulate) {
  if constexpr (CTA_GROUP == 1) {
    asm volatile(
        "{\n .reg .pred p;\n .reg .b64 da, db;\n setp.ne.b32 p, %7, 0;\n mov.b64 da, {%1, %3};\n mov.b64 db, {%2, %3};\n"
        " tcgen05.mma.cta_group::1.kind::mxf4.block_scale.scale_vec::2X [%0], da, db, %4, [%5], [%6], p;\n}\n"
        ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(desc_hi), "r"(idesc), "r"(scale_a_tmem), "r"(scale_b_tmem), "r"(accumulate)
        : "memory");
  } else {
    asm volatile(
        "{\n .reg .pred p;\n .reg .b64 da, db;\n setp.ne.b32 p, %7, 0;\n mov.b64 da, {%1, %3};\n mov.b64 db, {%2, %3};\n"
        " tcgen05.mma.cta_group::2.kind::mxf4.block_scale.scale_vec::2X [%0], da, db, %4, [%5], [%6], p;\n}\n"
        ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(desc_hi), "r"(idesc), "r"(scale_a_tmem), "r"(scale_b_tmem), "r"(accumulate)
        : "memory");
  }
}

// D[tmem] (+)= (A * scale_a) * (B * scale_b): A, B shared-memory descriptors, scales in tensor memory. One thread.
template <int CTA_GROUP>
__device__ __forceinline__ void umma_mx(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t desc_hi, uint32_t idesc,
                                        uint32_t scale_a_tmem, uint32_t scale_b_tmem, uint32_t accumulate) {
  if constexpr (CTA_GROUP == 1) {
    asm volatile(
        "{\n .reg .pred p;\n .reg .b64 da, db;\n setp.ne.b32 p, %7, 0;\n mov.b64 da, {%1, %3};\n mov.b64 db, {%2, %3};\n"
        " tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], da, db, %4, [%5], [%6], p;\n}\n"
        ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(desc_hi), "r"(idesc), "r"(scale_a_tmem), "r"(scale_b_tmem), "r"(accumulate)
        : "memory");
  } else {
    asm volatile(
        "{\n .reg .pred p;\n .reg .b64 da, db;\n setp.ne.b32 p, %7, 0;\n mov.b64 da, {%1, %3};\n mov.b64 db, {%2, %3};\n"
        " tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale [%0], da, db, %4, [%5], [%6], p;\n}\n"
        ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(desc_hi), "r"(idesc), "r"(scale_a_tmem), "r"(scale_b_tmem), "r"(accumulate)
        : "memory");
  }
}

// 512 bytes of shared memory (32 rows of 16 bytes, unswizzled: 8-row groups 128 bytes apart) -> 4 tensor-memory columns,
// the same 32 x 16 bytes into each of the four 32-lane quarters.
template <int CTA_GROUP>
__device__ __forceinline__ void scales_to_tmem(uint32_t tmem_column, uint32_t smem_addr) {
  uint64_t desc = 0;
  desc |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);  // start address, 16-byte units
  desc |= static_cast<uint64_t>(128 >> 4) << 32;               // stride between 8-row groups
  desc |= static_cast<uint64_t>(1) << 46;                      // descriptor version for sm_100
  if constexpr (CTA_GROUP == 1) {
    asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(tmem_column), "l"(desc) : "memory");
  } else {
    asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(tmem_column), "l"(desc) : "memory");
  }
}

template <int CTA_GROUP, int FORMAT, typename OutT, bool OUT_BF16>
__global__ void __launch_bounds__(kThreads, 1)
gemm_mxfp8_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                  const __grid_constant__ CUtensorMap map_c, const __grid_constant__ CUtensorMap map_scales,
                  Problem p, MxScales scales, DeviceStatus* status) {
  constexpr int kChunkCols = 128 / int(sizeof(OutT));  // output columns per 128-byte store row
  constexpr int kChunks = kBN / kChunkCols;
  using L = Layout<CTA_GROUP, FORMAT>;
  constexpr bool FP4 = L::FP4;
  constexpr int kStages = L::kStages;
  constexpr int kStageBytes = L::kStageBytes;
  constexpr int kBlockBytes = L::kBlockBytes;
  constexpr int kBlocksPerStage = L::kBlocksPerStage;
  constexpr int kSets = L::kScaleSets;
  constexpr int kRunBytes = L::kRunBytes;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - raw);

  const uint32_t stages_addr = base;
  const uint32_t epilogue_addr = base + kStages * kStageBytes;
  uint8_t* tail = smem + kStages * kStageBytes + kEpilogueBytes;
  const uint32_t full_bar = smem_u32(tail);                  // [kStages]
  const uint32_t empty_bar = full_bar + 8 * kStages;         // [kStages]
  const uint32_t tmem_full_bar = empty_bar + 8 * kStages;
  const uint32_t tmem_empty_bar = tmem_full_bar + 8;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tail + 8 * (2 * kStages + 2));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const uint32_t lane = lane_id();
  const uint32_t rank = CTA_GROUP == 2 ? cluster_ctarank() : 0u;
  const int first_tile = blockIdx.x / CTA_GROUP;   // this cluster's first tile
  const int tile_step = gridDim.x / CTA_GROUP;     // clusters in the grid
  const int num_tiles = p.tiles_m * p.tiles_n;
  const int num_kb = p.k / kBK;  // p.k counts bytes of K per row: codes for MXFP8, half the codes for NVFP4

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(full_bar + 8 * s, 1);
      mbar_init(empty_bar + 8 * s, 1);
    }
    mbar_init(tmem_full_bar, 1);
    mbar_init(tmem_empty_bar, 4 * CTA_GROUP);            // the epilogue warps of every CTA of the tile
    *abort_flag = 0;
    fence_mbar_init();
    prefetch_tensormap(&map_a);
    prefetch_tensormap(&map_b);
    prefetch_tensormap(&map_c);
    prefetch_tensormap(&map_scales);
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
      for (int t = first_tile; t < num_tiles && ok; t += tile_step) {
        int tm, tn;
        tile_coords(t, p, tm, tn);
        const int row_a = tm * (kBM * CTA_GROUP) + int(rank) * kBM;
        const int row_b = tn * kBN + int(rank) * L::kBRows;
        for (int kb = 0; kb < num_kb; kb += kBlocksPerStage) {
          if (!mbar_wait(empty_bar + 8 * stage, phase ^ 1u, abort_flag, status, kSiteProducerEmpty)) {
            ok = false;
            break;
          }
          const int blocks = min(kBlocksPerStage, num_kb - kb);  // an odd K-block count leaves the last stage half full
          const uint32_t dst = stages_addr + stage * kStageBytes;
          // the stage's scale atoms, already in tcgen05.cp's layout (rows of the copy = atoms of 512 bytes): one run for
          // this CTA's group of 128 A rows and one for each group of the tile's B rows. A run is always fetched whole;
          // behind an odd last K block it ends with atoms that no instruction reads.
          const uint32_t sdst = dst + kBlocksPerStage * kBlockBytes;
          const int a_atom = ((tm * CTA_GROUP + int(rank)) * num_kb + kb) * kSets;
          const int b_atom = scales.b_atom0 + (tn * 2 * num_kb + kb) * kSets;
          if constexpr (CTA_GROUP == 1) {
            const uint32_t full = full_bar + 8 * stage;
            mbar_arrive_expect_tx(full, uint32_t(blocks) * kBlockBytes + L::kStageScaleBytes);
            for (int j = 0; j < blocks; ++j) {
              tma_load_2d(dst + j * kBlockBytes, &map_a, (kb + j) * kBK, row_a, full);
              tma_load_2d(dst + j * kBlockBytes + kABytes, &map_b, (kb + j) * kBK, row_b, full);
            }
            tma_load_2d(sdst, &map_scales, 0, a_atom, full);
            tma_load_2d(sdst + kRunBytes, &map_scales, 0, b_atom, full);
            tma_load_2d(sdst + 2 * kRunBytes, &map_scales, 0, b_atom + num_kb * kSets, full);
          } else {
            // both CTAs' tiles complete on the leader's barrier; the leader alone arms it for both
            if (rank == 0) {
              mbar_arrive_expect_tx(full_bar + 8 * stage, uint32_t(blocks) * 2u * kBlockBytes + 2u * L::kStageScaleBytes);
            }
            const uint32_t leader_full = map_to_cta(full_bar + 8 * stage, 0);
            for (int j = 0; j < blocks; ++j) {
              tma_load_2d_pair(dst + j * kBlockBytes, &map_a, (kb + j) * kBK, row_a, leader_full);
              tma_load_2d_pair(dst + j * kBlockBytes + kABytes, &map_b, (kb + j) * kBK, row_b, leader_full);
            }
            tma_load_2d_pair(sdst, &map_scales, 0, a_atom, leader_full);
            tma_load_2d_pair(sdst + kRunBytes, &map_scales, 0, b_atom, leader_full);
            tma_load_2d_pair(sdst + 2 * kRunBytes, &map_scales, 0, b_atom + num_kb * kSets, leader_full);
          }
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer (leader CTA only)
    // The whole warp runs the loop and one elected lane issues: on one path, the compiler keeps descriptors, barrier
    // addresses and loop state in uniform registers, which tcgen05 instructions take directly.
    if (rank == 0) {
      const bool leader = elect_one();
      auto wait = [&](uint32_t bar, uint32_t parity, int site) {
        return __all_sync(0xffffffffu, mbar_wait(bar, parity, abort_flag, status, site)) != 0;
      };
      const uint64_t desc0 = umma_desc_kmajor_sw128(stages_addr);
      const uint32_t desc_hi = uint32_t(desc0 >> 32);
      int stage = 0;
      uint32_t phase = 0, iter = 0;
      bool ok = true;
      // This thread is the kernel's critical path: every tcgen05 instruction it issues costs about 60 cycles and a
      // barrier poll about 220 even when it succeeds at once (cycle trace with one K block per barrier: 851 cycles per K
      // block — poll 241, three scale copies 164, four products 257, commit 119 — against 512 of tensor work). Hence
      // two K blocks per barrier: one poll and one commit per 256 codes of K.
      for (int t = first_tile; t < num_tiles && ok; t += tile_step, ++iter) {
        // the single accumulator must have been read out by the epilogue of the previous tile
        if (!wait(tmem_empty_bar, (iter & 1u) ^ 1u, kSiteMmaTmemEmpty)) break;
        tc_fence_after();
        for (int kb0 = 0; kb0 < num_kb; kb0 += kBlocksPerStage) {
          if (!wait(full_bar + 8 * stage, phase, kSiteMmaFull)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const int blocks = min(kBlocksPerStage, num_kb - kb0);
          for (int j = 0; j < blocks && ok; ++j) {
            const int kb = kb0 + j;
            // this K block's scale atoms behind the stage's operands: A's sets, then the sets of each group of B rows
            const uint32_t group_a = stages_addr + stage * kStageBytes + kBlocksPerStage * kBlockBytes + j * (kSets * 512);
            const uint32_t group_b0 = group_a + kRunBytes, group_b1 = group_a + 2 * kRunBytes;
            constexpr uint32_t kSetStride = 512;
            if (leader) {
              const uint32_t a_lo = uint32_t(desc0) + ((stage * kStageBytes + j * kBlockBytes) >> 4);
              const uint32_t b_lo = a_lo + (kABytes >> 4);
              if constexpr (!FP4) {
                scales_to_tmem<CTA_GROUP>(tmem_base + kTmemScaleA, group_a);
                scales_to_tmem<CTA_GROUP>(tmem_base + kTmemScaleB, group_b0);
                scales_to_tmem<CTA_GROUP>(tmem_base + kTmemScaleB + 4, group_b1);
#pragma unroll
                for (int ks = 0; ks < 4; ++ks) {
                  umma_mx<CTA_GROUP>(tmem_base, a_lo + 2 * ks, b_lo + 2 * ks, desc_hi, mx_idesc(ks, kBM * CTA_GROUP),
                                     tmem_base + kTmemScaleA, tmem_base + kTmemScaleB, (kb > 0 || ks > 0) ? 1u : 0u);
                }
              } else if constexpr (FORMAT == kNvfp4) {
#pragma unroll
                for (int ks = 0; ks < 4; ++ks) {
                  // each 64-code instruction has its own scale bytes, in its own tensor-memory columns
                  const uint32_t sfa = tmem_base + kTmemScaleA + 12 * ks, sfb = tmem_base + kTmemScaleB + 12 * ks;
                  scales_to_tmem<CTA_GROUP>(sfa, group_a + ks * kSetStride);
                  scales_to_tmem<CTA_GROUP>(sfb, group_b0 + ks * kSetStride);
                  scales_to_tmem<CTA_GROUP>(sfb + 4, group_b1 + ks * kSetStride);
                  umma_nvf4<CTA_GROUP>(tmem_base, a_lo + 2 * ks, b_lo + 2 * ks, desc_hi, nvf4_idesc(kBM * CTA_GROUP), sfa, sfb,
                                       (kb > 0 || ks > 0) ? 1u : 0u);
                }
              } else {
#pragma unroll
                for (int ks = 0; ks < 4; ++ks) {
                  // MXFP4: two 64-code instructions share a set of scale columns; each takes two of the four bytes
                  const uint32_t sfa = tmem_base + kTmemScaleA + 12 * (ks >> 1), sfb = tmem_base + kTmemScaleB + 12 * (ks >> 1);
                  if ((ks & 1) == 0) {
                    scales_to_tmem<CTA_GROUP>(sfa, group_a + (ks >> 1) * kSetStride);
                    scales_to_tmem<CTA_GROUP>(sfb, group_b0 + (ks >> 1) * kSetStride);
                    scales_to_tmem<CTA_GROUP>(sfb + 4, group_b1 + (ks >> 1) * kSetStride);
                  }
                  umma_mxf4<CTA_GROUP>(tmem_base, a_lo + 2 * ks, b_lo + 2 * ks, desc_hi, mxf4_idesc((ks & 1) * 2, kBM * CTA_GROUP), sfa,
                                       sfb, (kb > 0 || ks > 0) ? 1u : 0u);
                }
              }
            }
            __syncwarp();
          }
          if (!ok) break;
          if (leader) {
            if constexpr (CTA_GROUP == 1) {
              umma_commit(empty_bar + 8 * stage);
            } else {
              umma_commit_pair(empty_bar + 8 * stage, 0x3);
            }
          }
          __syncwarp();
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        if (leader) {
          if constexpr (CTA_GROUP == 1) {
            umma_commit(tmem_full_bar);
          } else {
            umma_commit_pair(tmem_full_bar, 0x3);
          }
        }
        __syncwarp();
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue warps
    const int quarter = warp & 3;  // the 32-lane slice of tensor memory this warp may read (warps 2-5: slices 2, 3, 0, 1)
    const uint32_t buffer = epilogue_addr + quarter * 2048;
    const uint32_t leader_tmem_empty = CTA_GROUP == 2 ? map_to_cta(tmem_empty_bar, 0) : tmem_empty_bar;
    uint32_t iter = 0;
    bool ok = true;
    for (int t = first_tile; t < num_tiles && ok; t += tile_step, ++iter) {
      int tm, tn;
      tile_coords(t, p, tm, tn);
      const int row0 = tm * (kBM * CTA_GROUP) + int(rank) * kBM + quarter * 32;
      const int col0 = tn * kBN;
      if (!__all_sync(0xffffffffu, mbar_wait(tmem_full_bar, iter & 1u, abort_flag, status, kSiteEpilogueFull))) {
        ok = false;
        break;
      }
      tc_fence_after();
      const uint32_t t_row = tmem_base + (uint32_t(quarter * 32) << 16);
      auto store_chunk = [&](int chunk, const uint32_t (&words)[32]) {
        // the warp's 32 rows x 128 bytes go out as two 16-row boxes through its 2 KB staging buffer (swizzled as the
        // tensor map expects); shared memory is spent on operand stages instead of a larger buffer
        const int col = col0 + chunk * kChunkCols;
        if (row0 < p.m && col < p.n) {  // warp-uniform
#pragma unroll
          for (int rows_half = 0; rows_half < 2; ++rows_half) {
            if (lane == 0) tma_store_wait_read<0>();  // the previous store has read this buffer
            __syncwarp();
            if (int(lane >> 4) == rows_half) {
              const uint32_t row_addr = buffer + (lane & 15u) * 128;
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                const uint32_t dst = row_addr + ((uint32_t(j) ^ (lane & 7u)) << 4);
                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(words[4 * j]),
                             "r"(words[4 * j + 1]), "r"(words[4 * j + 2]), "r"(words[4 * j + 3])
                             : "memory");
              }
            }
            fence_async_smem();
            __syncwarp();
            if (lane == 0) {
              if (row0 + rows_half * 16 < p.m) tma_store_2d(&map_c, col, row0 + rows_half * 16, buffer);
              tma_store_commit();
            }
          }
        }
      };
      auto hand_back = [&]() {
        // the accumulator has been read completely: the next tile's products may overwrite it
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          if constexpr (CTA_GROUP == 2) {
            // relaxed: the accumulator's values already sit in registers (tcgen05.wait::ld), nothing written by this
            // thread has to be seen by the issuing thread, and a cluster-scope release costs about a thousand cycles
            // of the one phase of a tile that nothing overlaps
            mbar_arrive_cluster_relaxed(leader_tmem_empty);
          } else {
            mbar_arrive(tmem_empty_bar);
          }
        }
      };
      if constexpr (sizeof(OutT) == 4) {
        // f32 output: 256 values per thread do not fit the register file, so the stores sit between the reads
#pragma unroll 1
        for (int chunk = 0; chunk < kChunks; ++chunk) {
          uint32_t words[32];
          tmem_ld_32x32(t_row + chunk * kChunkCols, words);
          tmem_ld_wait(words);
          if constexpr (FORMAT == kNvfp4) {
#pragma unroll
            for (int i = 0; i < 32; ++i) words[i] = __float_as_uint(__uint_as_float(words[i]) * scales.alpha);
          }
          if (chunk == kChunks - 1) hand_back();
          store_chunk(chunk, words);
        }
      } else {
        // 16-bit output: the whole row (256 values) is rounded into 128 registers first, so tensor memory goes back to
        // the tensor cores after four reads, before any store is waited for (with the stores in between, the reads of
        // a tile took as long as the store pipeline: a fifth of the tile's time)
        uint32_t packed[kChunks][32];
#pragma unroll
        for (int chunk = 0; chunk < kChunks; ++chunk) {
          uint32_t lo[32], hi[32];
          tmem_ld_32x32(t_row + chunk * kChunkCols, lo);
          tmem_ld_32x32(t_row + chunk * kChunkCols + 32, hi);
          tmem_ld_wait(lo, hi);
          if constexpr (FORMAT == kNvfp4) {
            const float2 alpha2 = make_float2(scales.alpha, scales.alpha);
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              const float2 l2 = __fmul2_rn(make_float2(__uint_as_float(lo[2 * i]), __uint_as_float(lo[2 * i + 1])), alpha2);
              const float2 h2 = __fmul2_rn(make_float2(__uint_as_float(hi[2 * i]), __uint_as_float(hi[2 * i + 1])), alpha2);
              lo[2 * i] = __float_as_uint(l2.x), lo[2 * i + 1] = __float_as_uint(l2.y);
              hi[2 * i] = __float_as_uint(h2.x), hi[2 * i + 1] = __float_as_uint(h2.y);
            }
          }
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            if constexpr (OUT_BF16) {
              packed[chunk][i] = pack_bf16x2(__uint_as_float(lo[2 * i]), __uint_as_float(lo[2 * i + 1]));
              packed[chunk][16 + i] = pack_bf16x2(__uint_as_float(hi[2 * i]), __uint_as_float(hi[2 * i + 1]));
            } else {
              packed[chunk][i] = pack_f16x2(__uint_as_float(lo[2 * i]), __uint_as_float(lo[2 * i + 1]));
              packed[chunk][16 + i] = pack_f16x2(__uint_as_float(hi[2 * i]), __uint_as_float(hi[2 * i + 1]));
            }
          }
        }
        hand_back();
#pragma unroll
        for (int chunk = 0; chunk < kChunks; ++chunk) store_chunk(chunk, packed[chunk]);
      }
    }
    if (lane == 0) tma_store_wait<0>();
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
}

// Scale bytes of both operands, row-major [rows, num_kb * 4 * SETS], into tcgen05.cp's layout: per group of 128 rows, K
// block and set one atom of 128 words, word (row % 32) * 4 + row / 32 = the set's four scale bytes of that row. A block
// takes one group of 128 rows (A's groups first, then B's) and kTileScalesBlocks K blocks; thread t takes row
// (t % 4) * 32 + t / 4 of the group, whose word is word t: the loads of a thread are contiguous, the stores of a warp
// are. Rows beyond the matrix become zeros (their codes are zero-filled by TMA).
constexpr int kTileScalesBlocks = 8;

template <int SETS>
__global__ void __launch_bounds__(128)
tile_scales_kernel(const uint8_t* __restrict__ sa, long long ldsa, long long rows_a, int groups_a,
                   const uint8_t* __restrict__ sb, long long ldsb, long long rows_b, int num_kb, uint32_t* __restrict__ out) {
  const int group = blockIdx.x, kb0 = blockIdx.y * kTileScalesBlocks, t = threadIdx.x;
  const bool of_a = group < groups_a;
  const long long row = (long long)(of_a ? group : group - groups_a) * 128 + (t & 3) * 32 + (t >> 2);
  const bool live = row < (of_a ? rows_a : rows_b);
  const uint8_t* from = (of_a ? sa + row * ldsa : sb + row * ldsb) + (long long)kb0 * (4 * SETS);
  uint32_t* to = out + ((long long)group * num_kb + kb0) * (SETS * 128) + t;  // B's atoms follow A's
  const int count = min(kTileScalesBlocks, num_kb - kb0);
  uint32_t words[kTileScalesBlocks][SETS] = {};
#pragma unroll
  for (int j = 0; j < kTileScalesBlocks; ++j) {
    if (live && j < count) {
      if constexpr (SETS == 4) {
        const uint4 v = __ldg(reinterpret_cast<const uint4*>(from) + j);
        words[j][0] = v.x, words[j][1] = v.y, words[j][2] = v.z, words[j][3] = v.w;
      } else if constexpr (SETS == 1) {
        words[j][0] = __ldg(reinterpret_cast<const uint32_t*>(from) + j);
      } else {
        const uint2 v = __ldg(reinterpret_cast<const uint2*>(from) + j);
        words[j][0] = v.x, words[j][1] = v.y;
      }
    }
  }
#pragma unroll
  for (int j = 0; j < kTileScalesBlocks; ++j) {
    if (j < count) {
#pragma unroll
      for (int set = 0; set < SETS; ++set) to[(j * SETS + set) * 128] = words[j][set];
    }
  }
}

template <int CTA_GROUP, int FORMAT, typename OutT, bool OUT_BF16>
int launch(const DeviceContext* ctx, const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mc,
           const CUtensorMap& ms, Problem p, MxScales scales, cudaStream_t stream) {
  using L = Layout<CTA_GROUP, FORMAT>;
  auto kernel = gemm_mxfp8_kernel<CTA_GROUP, FORMAT, OutT, OUT_BF16>;
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
  KRNB_CUDA(cudaLaunchKernelEx(&config, kernel, ma, mb, mc, ms, p, scales, ctx->status_dev));
  return KRN_B200_OK;
}

template <int CTA_GROUP, int FORMAT>
int launch_for_output(const DeviceContext* ctx, int c_type, const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mc,
                      const CUtensorMap& ms, Problem p, MxScales scales, cudaStream_t stream) {
  if (c_type == KRN_B200_F32) return launch<CTA_GROUP, FORMAT, float, false>(ctx, ma, mb, mc, ms, p, scales, stream);
  if (c_type == KRN_B200_BF16) return launch<CTA_GROUP, FORMAT, uint16_t, true>(ctx, ma, mb, mc, ms, p, scales, stream);
  return launch<CTA_GROUP, FORMAT, uint16_t, false>(ctx, ma, mb, mc, ms, p, scales, stream);
}

// Checks shared by the two entry points, the tensor maps (operand rows as bytes: 128 per K block) and the launch.
// `k_bytes` is the length of an operand row in bytes, `scale_bytes` of a scale row.
template <int FORMAT>
int block_scaled_product(int c_type, const void* a, const uint8_t* sa, const void* b, const uint8_t* sb, float alpha, void* c,
                         int64_t m, int64_t n, int64_t k_bytes, int64_t scale_bytes, int64_t lda, int64_t ldb, int64_t ldc,
                         int64_t ldsa, int64_t ldsb, cudaStream_t stream) {
  constexpr bool FP4 = FORMAT != kMxfp8;
  const int c_bytes = c_type == KRN_B200_F32 ? 4 : 2;
  if (ldc < n || lda < k_bytes || ldb < k_bytes || ldsa < scale_bytes || ldsb < scale_bytes) {
    return fail(KRN_B200_ERR_INVALID_ARGUMENT, "row pitch shorter than the row");
  }
  if (!aligned16(a) || !aligned16(b) || !aligned16(c) || lda % 16 != 0 || ldb % 16 != 0 || (ldc * c_bytes) % 16 != 0) {
    return fail(KRN_B200_ERR_INVALID_ARGUMENT, "TMA needs 16-byte aligned base addresses and row pitches");
  }
  if (FP4 && !(aligned16(sa) && aligned16(sb) && ldsa % 16 == 0 && ldsb % 16 == 0)) {
    return fail(KRN_B200_ERR_INVALID_ARGUMENT, "the scale matrices of a 4-bit product need 16-byte aligned addresses and row pitches "
                "(a row's scale bytes are fetched as 16-byte vectors)");
  }
  if (!FP4 && (reinterpret_cast<uintptr_t>(sa) % 4 != 0 || reinterpret_cast<uintptr_t>(sb) % 4 != 0 || ldsa % 4 != 0 ||
               ldsb % 4 != 0)) {
    return fail(KRN_B200_ERR_INVALID_ARGUMENT, "scale matrices need 4-byte aligned addresses and row pitches (the four "
                "scale bytes of a 128-wide K step are fetched as one word)");
  }
  DeviceContext* ctx = current_context();
  if (ctx == nullptr) return KRN_B200_ERR_CUDA;
  if (int rc = require_sm100(ctx)) return rc;

  const int group = m > kBM ? 2 : 1;  // a single 128-row panel has nothing for a second CTA to do
  Problem p;
  p.m = int(m);
  p.n = int(n);
  p.k = int(k_bytes);
  p.tiles_m = int((m + kBM * group - 1) / (kBM * group));
  p.tiles_n = int((n + kBN - 1) / kBN);
  p.b_kn = 0;
  MxScales scales = {0, alpha};

  CUtensorMap map_a, map_b, map_c;
  {
    uint64_t dims[2] = {uint64_t(k_bytes), uint64_t(m)};
    uint64_t strides[1] = {uint64_t(lda)};
    uint32_t box[2] = {128, uint32_t(kBM)};
    if (int rc = encode_tensor_map(&map_a, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, a, dims, strides, box, Swizzle::k128B)) return rc;
  }
  {
    uint64_t dims[2] = {uint64_t(k_bytes), uint64_t(n)};
    uint64_t strides[1] = {uint64_t(ldb)};
    uint32_t box[2] = {128, uint32_t(kBN / group)};
    if (int rc = encode_tensor_map(&map_b, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, b, dims, strides, box, Swizzle::k128B)) return rc;
  }
  {
    const CUtensorMapDataType c_dt = c_type == KRN_B200_F32    ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                     : c_type == KRN_B200_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                               : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    uint64_t dims[2] = {uint64_t(n), uint64_t(m)};
    uint64_t strides[1] = {uint64_t(ldc) * c_bytes};
    uint32_t box[2] = {uint32_t(128 / c_bytes), 16};
    if (int rc = encode_tensor_map(&map_c, c_dt, 2, c, dims, strides, box, Swizzle::k128B)) return rc;
  }
  // The kernel reads its scale bytes from a copy in tcgen05.cp's layout, made here by one small kernel on the same
  // stream: 512-byte atoms, one per group of 128 rows, K block and set; A's groups first (as many as the tiles cover,
  // rows beyond the matrix as zeros), then B's. The copy lives in stream-ordered memory for the length of the call.
  constexpr int kSets = Layout<1, FORMAT>::kScaleSets;
  constexpr int kBlocksPerStage = Layout<1, FORMAT>::kBlocksPerStage;
  const int num_kb = int(k_bytes / kBK);
  const long long groups_a = (long long)group * p.tiles_m, groups_b = 2LL * p.tiles_n;
  const long long atoms_a = groups_a * num_kb * kSets, atoms_b = groups_b * num_kb * kSets;
  if (num_kb > 65535 || atoms_a + atoms_b > INT32_MAX) {
    return fail(KRN_B200_ERR_UNSUPPORTED, "a block-scaled product of this size is not available: the copy of its scales "
                "would have %lld atoms. Instead: split the product along M or N", atoms_a + atoms_b);
  }
  uint32_t* tiled = nullptr;
  KRNB_CUDA(cudaMallocFromPoolAsync(reinterpret_cast<void**>(&tiled), size_t(atoms_a + atoms_b) * 512, ctx->scratch_pool,
                                    stream));
  tile_scales_kernel<kSets><<<dim3(unsigned(groups_a + groups_b), unsigned((num_kb + kTileScalesBlocks - 1) / kTileScalesBlocks)),
                              128, 0, stream>>>(sa, ldsa, m, int(groups_a), sb, ldsb, n, num_kb, tiled);
  int rc = KRN_B200_OK;
  if (cudaError_t err = cudaGetLastError(); err != cudaSuccess) {
    rc = fail(KRN_B200_ERR_CUDA, "launch of the scale layout kernel failed: %s", cudaGetErrorString(err));
  }
  CUtensorMap map_scales;
  if (rc == KRN_B200_OK) {
    // one box = the atoms of one 128-row group for the K blocks of a stage
    uint64_t dims[2] = {128, uint64_t(atoms_a + atoms_b)};
    uint64_t strides[1] = {512};
    uint32_t box[2] = {128, uint32_t(kBlocksPerStage * kSets)};
    rc = encode_tensor_map(&map_scales, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, tiled, dims, strides, box, Swizzle::kNone);
  }
  if (rc == KRN_B200_OK) {
    scales.b_atom0 = int(atoms_a);
    rc = group == 2 ? launch_for_output<2, FORMAT>(ctx, c_type, map_a, map_b, map_c, map_scales, p, scales, stream)
                    : launch_for_output<1, FORMAT>(ctx, c_type, map_a, map_b, map_c, map_scales, p, scales, stream);
  }
  cudaFreeAsync(tiled, stream);  // after the product in stream order
  return rc;
}

}  // namespace
}  // namespace krnb

extern "C" int krn_b200_gemm_mxfp8_tn(int c_type, const void* a, const uint8_t* sa, const void* b, const uint8_t* sb, void* c,
                                      int64_t m, int64_t n, int64_t k, int64_t lda, int64_t ldb, int64_t ldc, int64_t ldsa,
                                      int64_t ldsb, void* stream_handle) {
  using namespace krnb;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_handle);
  if (c_type != KRN_B200_BF16 && c_type != KRN_B200_F16 && c_type != KRN_B200_F32) {
    return fail(KRN_B200_ERR_UNSUPPORTED, "output type %d is not available: use bf16, f16 or f32", c_type);
  }
  if (m < 0 || n < 0 || k < 0) return fail(KRN_B200_ERR_INVALID_ARGUMENT, "negative extent");
  if (m == 0 || n == 0) return KRN_B200_OK;
  if (m > INT32_MAX || n > INT32_MAX || k > INT32_MAX) {
    return fail(KRN_B200_ERR_UNSUPPORTED, "extents beyond 2^31-1 are not supported");
  }
  if (k == 0 || k % kBK != 0) {
    return fail(KRN_B200_ERR_UNSUPPORTED, "MXFP8 product with K = %lld is not available on sm_100a: the kernel consumes "
                "four 32-wide scale blocks per step. Instead: pad K to a multiple of 128 with zero codes", (long long)k);
  }
  if (a == nullptr || b == nullptr || c == nullptr || sa == nullptr || sb == nullptr) {
    return fail(KRN_B200_ERR_INVALID_ARGUMENT, "null tensor address");
  }
  return block_scaled_product<kMxfp8>(c_type, a, sa, b, sb, 1.0f, c, m, n, k, k / 32, lda, ldb, ldc, ldsa, ldsb, stream);
}

extern "C" int krn_b200_gemm_nvfp4_tn(int c_type, const void* a, const uint8_t* sa, const void* b, const uint8_t* sb,
                                      float alpha, void* c, int64_t m, int64_t n, int64_t k, int64_t lda, int64_t ldb,
                                      int64_t ldc, int64_t ldsa, int64_t ldsb, void* stream_handle) {
  using namespace krnb;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_handle);
  if (c_type != KRN_B200_BF16 && c_type != KRN_B200_F16 && c_type != KRN_B200_F32) {
    return fail(KRN_B200_ERR_UNSUPPORTED, "output type %d is not available: use bf16, f16 or f32", c_type);
  }
  if (m < 0 || n < 0 || k < 0) return fail(KRN_B200_ERR_INVALID_ARGUMENT, "negative extent");
  if (m == 0 || n == 0) return KRN_B200_OK;
  if (m > INT32_MAX || n > INT32_MAX || k > INT32_MAX) {
    return fail(KRN_B200_ERR_UNSUPPORTED, "extents beyond 2^31-1 are not supported");
  }
  if (k == 0 || k % 256 != 0) {
    return fail(KRN_B200_ERR_UNSUPPORTED, "NVFP4 product with K = %lld is not available on sm_100a: the kernel consumes "
                "256 codes (128 bytes, sixteen 16-wide scale blocks) per step. Instead: pad K to a multiple of 256 with zero "
                "codes", (long long)k);
  }
  if (a == nullptr || b == nullptr || c == nullptr || sa == nullptr || sb == nullptr) {
    return fail(KRN_B200_ERR_INVALID_ARGUMENT, "null tensor address");
  }
  return block_scaled_product<kNvfp4>(c_type, a, sa, b, sb, alpha, c, m, n, k / 2, k / 16, lda, ldb, ldc, ldsa, ldsb, stream);
}

extern "C" int krn_b200_gemm_mxfp4_tn(int c_type, const void* a, const uint8_t* sa, const void* b, const uint8_t* sb, void* c,
                                      int64_t m, int64_t n, int64_t k, int64_t lda, int64_t ldb, int64_t ldc, int64_t ldsa,
                                      int64_t ldsb, void* stream_handle) {
  using namespace krnb;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_handle);
  if (c_type != KRN_B200_BF16 && c_type != KRN_B200_F16 && c_type != KRN_B200_F32) {
    return fail(KRN_B200_ERR_UNSUPPORTED, "output type %d is not available: use bf16, f16 or f32", c_type);
  }
  if (m < 0 || n < 0 || k < 0) return fail(KRN_B200_ERR_INVALID_ARGUMENT, "negative extent");
  if (m == 0 || n == 0) return KRN_B200_OK;
  if (m > INT32_MAX || n > INT32_MAX || k > INT32_MAX) {
    return fail(KRN_B200_ERR_UNSUPPORTED, "extents beyond 2^31-1 are not supported");
  }
  if (k == 0 || k % 512 != 0) {
    return fail(KRN_B200_ERR_UNSUPPORTED, "MXFP4 product with K = %lld is not available on sm_100a: the kernel consumes 256 "
                "codes per step and fetches the scale bytes of two steps as one 16-byte vector. Instead: pad K to a multiple "
                "of 512 with zero codes", (long long)k);
  }
  if (a == nullptr || b == nullptr || c == nullptr || sa == nullptr || sb == nullptr) {
    return fail(KRN_B200_ERR_INVALID_ARGUMENT, "null tensor address");
  }
  return block_scaled_product<kMxfp4>(c_type, a, sa, b, sb, 1.0f, c, m, n, k / 2, k / 32, lda, ldb, ldc, ldsa, ldsb, stream);
}
