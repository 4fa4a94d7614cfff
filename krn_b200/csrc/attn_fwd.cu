// Flash-attention forward for sm_100a: O = softmax(scale * Q K^T [+ causal mask]) V, one pass over the keys.
//
// The statement sequence is the reference's example kernel (examples/04_libraries/08_flash_attention.py:44-59):
// scores carry log2(e)/sqrt(d) so every exponential is exp2, a running row maximum m and row sum l, the output
// accumulator rescaled when the maximum moves, P rounded to the storage type before P.V, one final division.
// The reference lowers each of those statements to a block-wide shared-memory pass with a barrier
// (src/krn/compiler/emit.py:997-1034,1245-1255); here they are fused around the tensor cores:
//
//   warp 0        TMA producer: the CTA's two 128-row query tiles once, then a 2-deep ring of K tiles and a
//                 2-deep ring of V tiles (128 keys each, 128-byte swizzle);
//   warp 1        MMA issuer: S_t = Q_t K^T into tensor memory (tcgen05.mma, A and B from shared memory) and
//                 O_t += P_t V (A = P_t read FROM tensor memory, B = V as an MN-major shared-memory operand),
//                 interleaved over the two query tiles so the tensor cores work on one tile while the other
//                 tile's softmax runs;
//   warps 4..7    softmax of query tile 0; warps 8..11 softmax of tile 1 (224 registers each via setmaxnreg; the
//                 producer / MMA warpgroup keeps 56 so that the MMA issue loop does not spill). A thread owns one query row: it
//                 reads its row of S from tensor memory, applies the mask, updates m and l, writes P (bf16)
//                 back over S, and rescales its row of O in tensor memory when the maximum moved by more than
//                 2^8 (below that the old reference maximum is kept, which leaves the quotient acc/l unchanged).
//                 At the end the same warps divide by l and store O through shared memory with TMA.
//
// Tensor memory (512 columns): S0 | S1 | O0 | O1, 128 columns each; P_t aliases the first 64 columns of S_t.
// Masked scores are -inf instead of the reference's -1.0e30 (both give exactly 0 after exp2); every row sees at
// least key 0 in its first tile, so no row is ever fully masked.
#include "host.cuh"

#include <cmath>

namespace krnb {
namespace {

constexpr int kTileQ = 128;    // query rows per tile = tensor-memory lanes
constexpr int kTileKV = 128;   // keys per K/V tile
constexpr int kThreads = 384;  // warpgroup 0: producer, MMA (+2 idle warps); warpgroups 1, 2: softmax
constexpr float kRescaleThreshold = 8.0f;

template <int D>
struct Layout {
  static constexpr int kBlocks = D / 64;                   // 64-column (128-byte) swizzle blocks per row
  static constexpr int kQBytes = kTileQ * D * 2;           // one query tile
  static constexpr int kKVBytes = kTileKV * D * 2;         // one K or V tile
  static constexpr int kBlockBytes = 128 * 128;            // [128 rows x 128 bytes]
  static constexpr int kSmemBytes = 2 * kQBytes + 4 * kKVBytes + 256 + 1024;
};

struct AttnParams {
  int seq_q, seq_kv, q_heads, kv_heads, batch;
  int q_blocks;  // number of 256-row query blocks
  float scale_log2;
  int causal;
};

enum Site { kSiteLoadK = 21, kSiteLoadV = 22, kSiteMmaQ = 23, kSiteMmaK = 24, kSiteMmaV = 25, kSiteMmaP = 26,
            kSiteSoftmaxS = 27, kSiteSoftmaxO = 28 };

__device__ __forceinline__ void tie(uint32_t (&r)[32]) {
  asm volatile("" : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]),
                   "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15]),
                   "+r"(r[16]), "+r"(r[17]), "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]), "+r"(r[22]), "+r"(r[23]),
                   "+r"(r[24]), "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]), "+r"(r[29]), "+r"(r[30]), "+r"(r[31])
               :: "memory");
}

// Number of 128-key tiles query tile `tile` (0 or 1) of query block `qb` attends to.
__device__ __forceinline__ int kv_tiles(const AttnParams& p, int qb, int tile) {
  const int row0 = qb * 2 * kTileQ + tile * kTileQ;
  if (row0 >= p.seq_q) return 0;
  int keys = p.seq_kv;
  if (p.causal) keys = min(keys, row0 + kTileQ);  // the tile's last row sees keys [0, row0 + 127]
  return (keys + kTileKV - 1) / kTileKV;
}

template <int D, bool BF16>
__global__ void __launch_bounds__(kThreads, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_o, AttnParams p,
                DeviceStatus* status) {
  using L = Layout<D>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - raw);

  const uint32_t q_addr = base;                            // two query tiles, later the output staging
  const uint32_t k_addr = base + 2 * L::kQBytes;           // two K stages
  const uint32_t v_addr = k_addr + 2 * L::kKVBytes;        // two V stages
  uint8_t* tail = smem + 2 * L::kQBytes + 4 * L::kKVBytes;
  const uint32_t bars = smem_u32(tail);
  const uint32_t q_full = bars;
  const uint32_t k_full = bars + 8, k_empty = bars + 24, v_full = bars + 40, v_empty = bars + 56;
  const uint32_t s_full = bars + 72, p_full = bars + 88, o_full = bars + 104;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tail + 128);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const uint32_t lane = lane_id();

  // heaviest query blocks first; the four q heads of a kv head are neighbours in the grid
  const int bh_count = p.q_heads * p.batch;
  const int qb = p.q_blocks - 1 - int(blockIdx.x) / bh_count;
  const int bh = int(blockIdx.x) % bh_count;
  const int b = bh / p.q_heads;
  const int h = bh % p.q_heads;
  const int hk = h / (p.q_heads / p.kv_heads);
  const int n0 = kv_tiles(p, qb, 0), n1 = kv_tiles(p, qb, 1);
  const int n = max(n0, n1);

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(k_full + 8 * i, 1);
      mbar_init(k_empty + 8 * i, 1);
      mbar_init(v_full + 8 * i, 1);
      mbar_init(v_empty + 8 * i, 1);
      mbar_init(s_full + 8 * i, 1);
      mbar_init(p_full + 8 * i, 4);
      mbar_init(o_full + 8 * i, 1);
    }
    *abort_flag = 0;
    fence_mbar_init();
    prefetch_tensormap(&map_q);
    prefetch_tensormap(&map_k);
    prefetch_tensormap(&map_v);
    prefetch_tensormap(&map_o);
  }
  if (warp == 1) {
    tmem_alloc<1>(smem_u32(tmem_slot), 512);
    tmem_relinquish<1>();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp < 4) reg_dealloc<56>();
  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      const int q_row = qb * 2 * kTileQ;
      mbar_arrive_expect_tx(q_full, 2 * L::kQBytes);
      for (int t = 0; t < 2; ++t)
        for (int blk = 0; blk < L::kBlocks; ++blk)
          tma_load_4d(q_addr + t * L::kQBytes + blk * L::kBlockBytes, &map_q, blk * 64, q_row + t * kTileQ, h, b, q_full);
      for (int j = 0; j < n; ++j) {
        const int stage = j & 1;
        const uint32_t parity = ((j >> 1) & 1) ^ 1u;
        if (!mbar_wait(k_empty + 8 * stage, parity, abort_flag, status, kSiteLoadK)) break;
        mbar_arrive_expect_tx(k_full + 8 * stage, L::kKVBytes);
        for (int blk = 0; blk < L::kBlocks; ++blk)
          tma_load_4d(k_addr + stage * L::kKVBytes + blk * L::kBlockBytes, &map_k, blk * 64, j * kTileKV, hk, b,
                      k_full + 8 * stage);
        if (!mbar_wait(v_empty + 8 * stage, parity, abort_flag, status, kSiteLoadV)) break;
        mbar_arrive_expect_tx(v_full + 8 * stage, L::kKVBytes);
        for (int blk = 0; blk < L::kBlocks; ++blk)
          tma_load_4d(v_addr + stage * L::kKVBytes + blk * L::kBlockBytes, &map_v, blk * 64, j * kTileKV, hk, b,
                      v_full + 8 * stage);
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (n > 0) {
      const bool leader = elect_one();
      constexpr uint32_t fmt = BF16 ? kFmtBF16 : kFmtF16;
      const uint32_t idesc_s = umma_idesc(fmt, fmt, kTileQ, kTileKV, 0, 0);
      const uint32_t idesc_pv = umma_idesc(fmt, fmt, kTileQ, D, 0, 1);
      const int nt[2] = {n0, n1};

      // Descriptors are stepped as 32-bit words: the issuing thread runs one instruction at a time, so every
      // 64-bit descriptor rebuild it does not do brings the next product forward.
      const uint64_t kmajor = umma_desc_kmajor_sw128(0);
      const uint64_t mnmajor = umma_desc_mnmajor_sw128(0, L::kBlockBytes, 1024);
      const uint32_t kmajor_hi = uint32_t(kmajor >> 32), mnmajor_hi = uint32_t(mnmajor >> 32);
      const uint32_t q_lo = uint32_t(kmajor) + (q_addr >> 4);
      const uint32_t k_lo = uint32_t(kmajor) + (k_addr >> 4);
      const uint32_t v_lo = uint32_t(mnmajor) + (v_addr >> 4);

      // S_t = Q_t K^T: D/16 instructions of K = 16; operand rows are 128-byte swizzled, 64 columns per block
      auto issue_s = [&](int t, int stage) {
        const uint32_t qa = q_lo + t * (L::kQBytes >> 4);
        const uint32_t ka = k_lo + stage * (L::kKVBytes >> 4);
        if (leader) {
#pragma unroll
          for (int ks = 0; ks < D / 16; ++ks) {
            const uint32_t off = ((ks >> 2) * L::kBlockBytes + (ks & 3) * 32) >> 4;
            umma_ss_halves<1, false>(tmem_base + t * 128, qa + off, kmajor_hi, ka + off, kmajor_hi, idesc_s,
                                     ks > 0 ? 1u : 0u);
          }
          umma_commit(s_full + 8 * t);
        }
        __syncwarp();
      };
      // O_t += P_t V: 8 instructions of K = 16 keys; A = P_t in tensor memory (8 columns per 16 keys), B = V
      // tile with d contiguous: 64-column blocks kBlockBytes apart (leading), 8-key groups 1024 bytes apart
      auto issue_pv = [&](int t, int stage, bool accumulate) {
        const uint32_t va = v_lo + stage * (L::kKVBytes >> 4);
        if (leader) {
#pragma unroll
          for (int ks = 0; ks < kTileKV / 16; ++ks) {
            umma_ts_f16_halves(tmem_base + 256 + t * 128, tmem_base + t * 128 + ks * 8, va + ks * (2048 >> 4), mnmajor_hi,
                               idesc_pv, (accumulate || ks > 0) ? 1u : 0u);
          }
        }
        __syncwarp();
      };

      auto wait = [&](uint32_t bar, uint32_t parity, int site) {
        return __all_sync(0xffffffffu, mbar_wait(bar, parity, abort_flag, status, site)) != 0;
      };
      bool ok = wait(q_full, 0, kSiteMmaQ) && wait(k_full, 0, kSiteMmaK);
      if (ok) {
        tc_fence_after();
        for (int t = 0; t < 2; ++t)
          if (nt[t] > 0) issue_s(t, 0);
        if (leader) umma_commit(k_empty);  // K(0) is free once both score products have read it
      }
      for (int j = 0; j < n && ok; ++j) {
        const int stage = j & 1;
        if (!wait(v_full + 8 * stage, (j >> 1) & 1, kSiteMmaV)) break;
        bool next_k_ready = false;
        for (int t = 0; t < 2 && ok; ++t) {
          if (j >= nt[t]) continue;
          if (!wait(p_full + 8 * t, j & 1, kSiteMmaP)) {
            ok = false;
            break;
          }
          tc_fence_after();
          issue_pv(t, stage, j > 0);
          if (j + 1 < nt[t]) {
            if (!next_k_ready) {
              if (!wait(k_full + 8 * (stage ^ 1), ((j + 1) >> 1) & 1, kSiteMmaK)) {
                ok = false;
                break;
              }
              tc_fence_after();
              next_k_ready = true;
            }
            issue_s(t, stage ^ 1);
          } else {
            if (leader) umma_commit(o_full + 8 * t);  // last P.V of this tile
          }
        }
        if (!ok) break;
        if (leader) {
          umma_commit(v_empty + 8 * stage);
          if (j + 1 < n) umma_commit(k_empty + 8 * (stage ^ 1));
        }
        __syncwarp();
      }
    }
  } else if (warp >= 4) {
    // ---------------------------------------------------------------- softmax + epilogue warps
    reg_alloc<224>();
    const int t = (warp - 4) >> 2;   // query tile of this warpgroup
    const int quarter = warp & 3;    // tensor-memory lane quarter
    const int nt = t == 0 ? n0 : n1;
    const int row_in_tile = quarter * 32 + int(lane);
    const int q_index = qb * 2 * kTileQ + t * kTileQ + row_in_tile;
    const uint32_t lane_base = tmem_base + (uint32_t(quarter * 32) << 16);
    const uint32_t s_tmem = lane_base + t * 128;
    const uint32_t o_tmem = lane_base + 256 + t * 128;
    float m_ref = -INFINITY;  // reference maximum (scaled domain) the accumulators are expressed against
    float l = 0.f;
    bool ok = true;

    for (int j = 0; j < nt; ++j) {
      if (!__all_sync(0xffffffffu, mbar_wait(s_full + 8 * t, j & 1, abort_flag, status, kSiteSoftmaxS))) {
        ok = false;
        break;
      }
      tc_fence_after();
      uint32_t s0[32], s1[32], s2[32], s3[32];
      tmem_ld_32x32(s_tmem, s0);
      tmem_ld_32x32(s_tmem + 32, s1);
      tmem_ld_32x32(s_tmem + 64, s2);
      tmem_ld_32x32(s_tmem + 96, s3);
      tmem_ld_wait(s0);
      tie(s1);
      tie(s2);
      tie(s3);

      // keys past the sequence end, and keys after the query position under the causal mask, take -inf
      const int key0 = j * kTileKV;
      int visible = p.seq_kv - key0;                                 // keys [0, visible) of this tile exist
      if (p.causal) visible = min(visible, q_index - key0 + 1);      // and are not in the future
      if (visible < kTileKV) {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          if (i >= visible) s0[i] = 0xff800000u;
          if (32 + i >= visible) s1[i] = 0xff800000u;
          if (64 + i >= visible) s2[i] = 0xff800000u;
          if (96 + i >= visible) s3[i] = 0xff800000u;
        }
      }
      float mx = -INFINITY;
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        mx = fmaxf(mx, fmaxf(fmaxf(__uint_as_float(s0[i]), __uint_as_float(s1[i])),
                             fmaxf(__uint_as_float(s2[i]), __uint_as_float(s3[i]))));
      }
      const float m_new = fmaxf(m_ref, mx * p.scale_log2);
      if (j == 0) {
        m_ref = m_new;
      } else {
        const bool moved = m_new - m_ref > kRescaleThreshold;
        if (__any_sync(0xffffffffu, moved)) {
          // S_t(j) was issued after P_t(j-1) V(j-1), so O_t is complete and idle until p_full is signalled
          const float corr = moved ? ex2_approx(m_ref - m_new) : 1.0f;
          l *= corr;
          if (moved) m_ref = m_new;
#pragma unroll
          for (int c = 0; c < D / 32; ++c) {
            uint32_t o[32];
            tmem_ld_32x32(o_tmem + c * 32, o);
            tmem_ld_wait(o);
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * corr);
            tmem_st_32x32(o_tmem + c * 32, o);
          }
        }
      }
      // p = exp2(s * scale - m_ref), summed in f32 before the rounding to the storage type
      const float neg_m = -m_ref;
      // packed f32x2 arithmetic for the scale-and-shift and the row sum: half the instructions beside the exponentials
      const float2 scale2 = make_float2(p.scale_log2, p.scale_log2), shift2 = make_float2(neg_m, neg_m);
      float2 sum_a = make_float2(0.f, 0.f), sum_b = sum_a, sum_c = sum_a, sum_d = sum_a;
      uint32_t packed0[32], packed1[32];
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const float2 xa = __ffma2_rn(make_float2(__uint_as_float(s0[2 * i]), __uint_as_float(s0[2 * i + 1])), scale2, shift2);
        const float2 xb = __ffma2_rn(make_float2(__uint_as_float(s1[2 * i]), __uint_as_float(s1[2 * i + 1])), scale2, shift2);
        const float2 xc = __ffma2_rn(make_float2(__uint_as_float(s2[2 * i]), __uint_as_float(s2[2 * i + 1])), scale2, shift2);
        const float2 xd = __ffma2_rn(make_float2(__uint_as_float(s3[2 * i]), __uint_as_float(s3[2 * i + 1])), scale2, shift2);
        const float2 a = make_float2(ex2_approx(xa.x), ex2_approx(xa.y));
        const float2 b2 = make_float2(ex2_approx(xb.x), ex2_approx(xb.y));
        const float2 c = make_float2(ex2_approx(xc.x), ex2_approx(xc.y));
        const float2 d2 = make_float2(ex2_approx(xd.x), ex2_approx(xd.y));
        sum_a = __fadd2_rn(sum_a, a);
        sum_b = __fadd2_rn(sum_b, b2);
        sum_c = __fadd2_rn(sum_c, c);
        sum_d = __fadd2_rn(sum_d, d2);
        packed0[i] = BF16 ? pack_bf16x2(a.x, a.y) : pack_f16x2(a.x, a.y);
        packed0[16 + i] = BF16 ? pack_bf16x2(b2.x, b2.y) : pack_f16x2(b2.x, b2.y);
        packed1[i] = BF16 ? pack_bf16x2(c.x, c.y) : pack_f16x2(c.x, c.y);
        packed1[16 + i] = BF16 ? pack_bf16x2(d2.x, d2.y) : pack_f16x2(d2.x, d2.y);
      }
      const float2 sum2 = __fadd2_rn(__fadd2_rn(sum_a, sum_b), __fadd2_rn(sum_c, sum_d));
      const float sum = sum2.x + sum2.y;
      l += sum;
      tmem_st_32x32(s_tmem, packed0);       // keys 0..63  -> columns 0..31
      tmem_st_32x32(s_tmem + 32, packed1);  // keys 64..127 -> columns 32..63
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full + 8 * t);
    }

    // ---- epilogue: O_t / l through the (now idle) query tile's shared memory
    if (nt > 0 && ok) {
      if (__all_sync(0xffffffffu, mbar_wait(o_full + 8 * t, 0, abort_flag, status, kSiteSoftmaxO))) {
        tc_fence_after();
        const float inv = 1.0f / l;
        const uint32_t stage_addr = q_addr + t * L::kQBytes;
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          uint32_t o[32];
          tmem_ld_32x32(o_tmem + c * 32, o);
          tmem_ld_wait(o);
          // 32 columns = 64 bytes = four 16-byte chunks of the 128-byte swizzled row
          const uint32_t row_addr = stage_addr + (c >> 1) * L::kBlockBytes + row_in_tile * 128;
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint32_t w[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float x = __uint_as_float(o[8 * g + 2 * e]) * inv;
              const float y = __uint_as_float(o[8 * g + 2 * e + 1]) * inv;
              w[e] = BF16 ? pack_bf16x2(x, y) : pack_f16x2(x, y);
            }
            const uint32_t chunk = uint32_t((c & 1) * 4 + g);
            const uint32_t dst = row_addr + ((chunk ^ (uint32_t(row_in_tile) & 7u)) << 4);
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(w[0]), "r"(w[1]), "r"(w[2]),
                         "r"(w[3])
                         : "memory");
          }
        }
        // every warp stores its own 32 rows: no cross-warp barrier, so an abandoned warp cannot block the others
        fence_async_smem();
        __syncwarp();
        if (lane == 0) {
          const int q_row = qb * 2 * kTileQ + t * kTileQ + quarter * 32;
          if (q_row < p.seq_q) {
            for (int blk = 0; blk < L::kBlocks; ++blk)
              tma_store_4d(&map_o, blk * 64, q_row, h, b, stage_addr + blk * L::kBlockBytes + quarter * 4096);
            tma_store_commit();
            tma_store_wait<0>();
          }
        }
      }
    }
  }

  // ------------------------------------------------------------------ teardown
  if (*abort_flag != 0) {
    for (int i = 0; i < 1000; ++i) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc<1>(tmem_base, 512);
  }
}

int encode_bhsd(CUtensorMap* map, CUtensorMapDataType type, const void* base, int64_t d, int64_t seq, int64_t heads,
                int64_t batch, const int64_t* strides, uint32_t box_rows) {
  uint64_t dims[4] = {uint64_t(d), uint64_t(seq), uint64_t(heads), uint64_t(batch)};
  uint64_t strides_bytes[3] = {uint64_t(strides[2]) * 2, uint64_t(strides[1]) * 2, uint64_t(strides[0]) * 2};
  uint32_t box[4] = {64, box_rows, 1, 1};
  return encode_tensor_map(map, type, 4, base, dims, strides_bytes, box, Swizzle::k128B);
}

template <int D, bool BF16>
int launch(const DeviceContext* ctx, const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv,
           const CUtensorMap& mo, AttnParams p, cudaStream_t stream) {
  auto kernel = attn_fwd_kernel<D, BF16>;
  KRNB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Layout<D>::kSmemBytes));
  // setmaxnreg.inc blocks until the CTA's register pool can cover it: 128 x (R - 56) must reach 256 x (224 - R)
  cudaFuncAttributes attributes;
  KRNB_CUDA(cudaFuncGetAttributes(&attributes, kernel));
  if ((attributes.numRegs - 56) * 128 < (224 - attributes.numRegs) * 256) {
    return fail(KRN_B200_ERR_UNSUPPORTED, "attention kernel was built with %d registers per thread; the register "
                "re-partitioning needs at least 168", attributes.numRegs);
  }
  const long long blocks = (long long)p.q_blocks * p.q_heads * p.batch;
  kernel<<<dim3(unsigned(blocks)), dim3(kThreads), Layout<D>::kSmemBytes, stream>>>(mq, mk, mv, mo, p, ctx->status_dev);
  KRNB_CUDA(cudaGetLastError());
  return KRN_B200_OK;
}

}  // namespace
}  // namespace krnb

extern "C" int krn_b200_attn_fwd(int type, const void* q, const void* k, const void* v, void* o, int64_t batch,
                                 int64_t q_heads, int64_t kv_heads, int64_t seq_q, int64_t seq_kv, int64_t d,
                                 float scale_log2, int causal, const int64_t* q_strides, const int64_t* k_strides,
                                 const int64_t* v_strides, const int64_t* o_strides, void* stream_handle) {
  using namespace krnb;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_handle);
  if (type != KRN_B200_BF16 && type != KRN_B200_F16) {
    return fail(KRN_B200_ERR_UNSUPPORTED, "attention element type %d is not available on sm_100a: the kernel takes "
                "16-bit tiles. Instead: pass bf16 or f16 tensors", type);
  }
  if (d != 64 && d != 128) {
    return fail(KRN_B200_ERR_UNSUPPORTED, "head dimension %lld is not available on sm_100a: tiles are built from "
                "128-byte rows. Instead: use d = 64 or d = 128", (long long)d);
  }
  if (batch < 0 || q_heads <= 0 || kv_heads <= 0 || seq_q < 0 || seq_kv < 0 || q_heads % kv_heads != 0) {
    return fail(KRN_B200_ERR_INVALID_ARGUMENT, "bad extents (batch %lld, q_heads %lld, kv_heads %lld)",
                (long long)batch, (long long)q_heads, (long long)kv_heads);
  }
  if (batch == 0 || seq_q == 0) return KRN_B200_OK;
  if (seq_kv == 0) return fail(KRN_B200_ERR_INVALID_ARGUMENT, "attention over zero keys is undefined");
  if (q == nullptr || k == nullptr || v == nullptr || o == nullptr || q_strides == nullptr || k_strides == nullptr ||
      v_strides == nullptr || o_strides == nullptr) {
    return fail(KRN_B200_ERR_INVALID_ARGUMENT, "null tensor address");
  }
  const void* bases[4] = {q, k, v, o};
  const int64_t* strides[4] = {q_strides, k_strides, v_strides, o_strides};
  for (int i = 0; i < 4; ++i) {
    if (!aligned16(bases[i]) || strides[i][0] % 8 != 0 || strides[i][1] % 8 != 0 || strides[i][2] % 8 != 0) {
      return fail(KRN_B200_ERR_INVALID_ARGUMENT, "TMA needs 16-byte aligned addresses and strides");
    }
  }
  if (seq_q > INT32_MAX / 2 || seq_kv > INT32_MAX / 2 || batch * q_heads > INT32_MAX / 4096) {
    return fail(KRN_B200_ERR_UNSUPPORTED, "extents too large for this kernel's 32-bit indices");
  }
  DeviceContext* ctx = current_context();
  if (ctx == nullptr) return KRN_B200_ERR_CUDA;
  if (int rc = require_sm100(ctx)) return rc;

  const CUtensorMapDataType dt = type == KRN_B200_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  CUtensorMap mq, mk, mv, mo;
  if (int rc = encode_bhsd(&mq, dt, q, d, seq_q, q_heads, batch, q_strides, kTileQ)) return rc;
  if (int rc = encode_bhsd(&mk, dt, k, d, seq_kv, kv_heads, batch, k_strides, kTileKV)) return rc;
  if (int rc = encode_bhsd(&mv, dt, v, d, seq_kv, kv_heads, batch, v_strides, kTileKV)) return rc;
  if (int rc = encode_bhsd(&mo, dt, o, d, seq_q, q_heads, batch, o_strides, 32)) return rc;

  AttnParams p;
  p.seq_q = int(seq_q);
  p.seq_kv = int(seq_kv);
  p.q_heads = int(q_heads);
  p.kv_heads = int(kv_heads);
  p.batch = int(batch);
  p.q_blocks = int((seq_q + 2 * kTileQ - 1) / (2 * kTileQ));
  p.scale_log2 = scale_log2;
  p.causal = causal != 0;
  const bool bf16 = type == KRN_B200_BF16;
  if (d == 128) return bf16 ? launch<128, true>(ctx, mq, mk, mv, mo, p, stream) : launch<128, false>(ctx, mq, mk, mv, mo, p, stream);
  return bf16 ? launch<64, true>(ctx, mq, mk, mv, mo, p, stream) : launch<64, false>(ctx, mq, mk, mv, mo, p, stream);
}
