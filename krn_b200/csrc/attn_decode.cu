// Decode attention (one query token per sequence) over a paged FP8 e4m3 KV cache, split over the keys.
//
// Work unit = (sequence b, kv head g, chunk of the context). The four q heads that share kv head g are handled
// together, so every K/V byte is read from HBM once. The path is HBM-bound (about 8 flop per byte); the tensor
// cores are used only to keep the arithmetic off the critical path, with the cache bytes consumed exactly as
// they sit in memory:
//
//   per iteration (128 tokens = two 64-token pages):
//     TMA      K page rows [64 tokens x 128 B] of head g, twice, into one 128-byte-swizzled tile; same for V
//     MMA 1    S^T[token, col] = K_tile . Q8^T        M = 128 tokens, N = 16, K = d = 128 (kind::f8f6f4)
//              Q8 rows 0..3 hold e4m3(q * qscale) of the 4 heads, rows 4..7 the e4m3 of the rounding residual,
//              so column h + column 4+h carry q.k to bf16 accuracy although both operands are FP8
//     threads  one thread per TOKEN reads its 8 scores from tensor memory, forms s = (hi + lo) * scale, the
//              block finds the running maximum per head, p = exp2(s - m); P is written back as an FP8 hi/lo pair
//              (scaled by 2^8) into a [16 x 128 tokens] K-major tile
//     MMA 2    D[d, col] = V_tile^T . P8^T           M = d = 128, N = 16, K = 128 tokens; V is an MN-major
//              operand (d contiguous), i.e. the cache layout itself
//     threads  one thread per OUTPUT COLUMN d: acc[h] = acc[h] * corr[h] + (D[d,h] + D[d,4+h]) * 2^-8
//   end      partial (m, l, acc) per (b, q head, chunk) to the workspace; a second kernel, launched as a programmatic
//            dependent so that its launch overlaps this kernel's tail, merges the chunks, applies v_scale and rounds
//            once to bf16.
//
// Measured alternatives on the benchmark mix (64 sequences, contexts 1024..8192; this layout: 126 us per call):
//   * merging inside this kernel (an arrival counter per (sequence, kv head); the CTA that finishes the last chunk
//     merges): the fence, the atomic and the merge sit on every CTA's critical path, +36 us;
//   * one persistent launch of 3 CTAs per SM taking work units from a ticket counter, with a table of the units that
//     exist so that no CTA is spent on a chunk beyond a context: 141 us — relaunching a CTA per unit costs less than
//     the per-unit bookkeeping, and the hardware scheduler already keeps every slot busy;
//   * a bounds report or a shared-memory flag inside the loop of the thread that issues the copies: +31 / +15 us.
//   * the next iteration's score MMA issued behind this iteration's PV MMA under one commit: +7 us (the wait for the next
//     K tile moves forward and the prefetch distance shrinks); the same with separate K and V barriers and K refetched as
//     soon as the scores are formed: +3 us; chunks as the slowest grid dimension (short last chunks in the last wave): +5 us.
//
// The reference has no implementation of paged decode attention (its roadmap lists it); the arithmetic follows
// its flash-attention statements (examples/04_libraries/08_flash_attention.py:44-59) with K, V = code * scale.
#include "host.cuh"

#include <cuda_fp16.h>

#include <cmath>
#include <mutex>

namespace krnb {
namespace {

constexpr int kD = 128;
constexpr int kPage = 64;
constexpr int kIterTokens = 128;       // two pages
constexpr int kChunkTokens = 1024;     // tokens per work unit (8 iterations)
constexpr int kGroupMax = 4;           // q heads per kv head handled by one CTA
constexpr int kThreads = 128;
constexpr int kStages = 2;
constexpr int kTileBytes = kIterTokens * 128;  // 16 KB: 128 tokens x 128 B
constexpr int kSmemBytes = kStages * 2 * kTileBytes + 2048 /*Q8*/ + 2048 /*P8*/ + 1024 /*misc*/ + 1024 /*align*/;

struct DecodeParams {
  const uint16_t* q;          // bf16 [batch, q_heads, d]
  const int32_t* page_table;  // [batch, max_pages]
  const int32_t* context_len; // [batch]
  const float* k_scale;       // [batch, kv_heads]
  float* workspace;           // partials
  int batch, q_heads, kv_heads, group, max_pages, chunks, num_pages, max_context;
  float scale_log2;
};

constexpr int kErrDeviceIndex = 6;  // mirrors KRN_B200_ERR_DEVICE_INDEX in include/krn_b200.h

enum Site { kSiteKv = 31, kSiteMma1 = 32, kSiteMma2 = 33, kSitePageId = 36 };

__device__ __forceinline__ float bf16_bits_to_float(uint16_t w) { return __uint_as_float(uint32_t(w) << 16); }

// e4m3fn code of x (round to nearest even, saturating) in the low byte.
__device__ __forceinline__ uint32_t to_e4m3(float x) {
  uint16_t r;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(0.0f), "f"(x));
  return r & 0xffu;
}

__device__ __forceinline__ float from_e4m3(uint32_t code) {
  uint32_t h2;
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h2) : "h"(uint16_t(code)));
  return __half2float(__ushort_as_half(uint16_t(h2 & 0xffffu)));
}

// byte address of element (row, byte column) in a K-major tile of 128-byte rows with the 128-byte swizzle
__device__ __forceinline__ uint32_t swizzled(uint32_t base, uint32_t row, uint32_t col) {
  return base + row * 128 + ((((col >> 4) ^ (row & 7u)) << 4) | (col & 15u));
}

__device__ __forceinline__ void st_shared_u8(uint32_t addr, uint32_t v) {
  asm volatile("st.shared.u8 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}

__device__ __forceinline__ void tmem_ld_32x8(uint32_t taddr, uint32_t (&r)[8]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(taddr)
               : "memory");
}

__device__ __forceinline__ void tmem_ld_wait8(uint32_t (&r)[8]) {
  asm volatile("tcgen05.wait::ld.sync.aligned;"
               : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7])
               :
               : "memory");
}

// One warp lane polls, the warp follows; returns a warp-uniform verdict.
__device__ __forceinline__ bool warp_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, DeviceStatus* status,
                                          int site) {
  bool ok = true;
  if (lane_id() == 0) ok = mbar_wait(bar, parity, abort_flag, status, site);
  return __all_sync(0xffffffffu, ok);
}

__global__ void __launch_bounds__(kThreads, 3)
decode_partial_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                      DecodeParams p, DeviceStatus* status) {
  const int chunk = blockIdx.x, g = blockIdx.y, b = blockIdx.z;
  // the context length is clamped into [0, max_context]: a length beyond what the page table row holds can never
  // index past the row
  const int len = max(0, min(p.context_len[b], p.max_context));
  const int token0 = chunk * kChunkTokens;
  if (token0 >= len) return;  // whole CTA leaves together, before any barrier or allocation
  int bad_page = 0;  // thread 0: bit 31 set once a page id outside the pool was met (low bits: part of the id)
  const int tokens = min(kChunkTokens, len - token0);
  const int iters = (tokens + kIterTokens - 1) / kIterTokens;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - raw);
  const uint32_t k_tiles = base;                             // [kStages][16 KB]
  const uint32_t v_tiles = base + kStages * kTileBytes;      // [kStages][16 KB]
  const uint32_t q8_tile = v_tiles + kStages * kTileBytes;   // 16 rows x 128 B
  const uint32_t p8_tile = q8_tile + 2048;                   // 16 rows x 128 B
  uint8_t* misc = smem + 2 * kStages * kTileBytes + 4096;
  const uint32_t kv_full = smem_u32(misc);                   // [kStages]
  const uint32_t mma_bar = kv_full + 8 * kStages;            // one barrier, alternating phases
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(misc + 64);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(misc + 68);
  float* red = reinterpret_cast<float*>(misc + 128);         // [4 warps][4 heads] scratch, then reuse

  const int tid = threadIdx.x, warp = tid >> 5;
  const uint32_t lane = lane_id();
  const int group = p.group;  // q heads per kv head (<= 4)

  if (tid == 0) {
    for (int s = 0; s < kStages; ++s) mbar_init(kv_full + 8 * s, 1);
    mbar_init(mma_bar, 1);
    *abort_flag = 0;
    fence_mbar_init();
    prefetch_tensormap(&map_k);
    prefetch_tensormap(&map_v);
  }
  if (warp == 0) {
    tmem_alloc<1>(smem_u32(tmem_slot), 32);
    tmem_relinquish<1>();
  }
  // zero the Q8 and P8 operand tiles (rows that stay unused must read as zero codes)
  for (int i = tid; i < 4096 / 16; i += kThreads) {
    asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(q8_tile + i * 16), "r"(0u) : "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // ---- TMA issue for one iteration (thread 0): two pages of K and two of V into stage `stage`
  const int32_t* pages = p.page_table + (long long)b * p.max_pages + token0 / kPage;
  auto issue_loads = [&](int it) {
    const int stage = it % kStages;
    const int first = it * 2;
    const int valid_pages = min(2, (tokens - it * kIterTokens + kPage - 1) / kPage);
    mbar_arrive_expect_tx(kv_full + 8 * stage, uint32_t(valid_pages) * 2u * kPage * 128u);
    for (int pg = 0; pg < valid_pages; ++pg) {
      int page = pages[first + pg];
      // A page id outside the pool is never fetched: the copy is aimed one past the pool, where the tensor map's bounds
      // make TMA fill zeros, so those 64 tokens read as zero codes (K = V = 0). Only a compare and a select sit here —
      // this thread's loop is the kernel's critical path (a status report at this point cost 31 us per call, a
      // shared-memory flag read by the softmax threads another 15); the report is made once, at the end.
      if (uint32_t(page) >= uint32_t(p.num_pages)) {
        bad_page = page | int(0x80000000);
        page = p.num_pages;
      }
      tma_load_4d(k_tiles + stage * kTileBytes + pg * kPage * 128, &map_k, 0, g, 0, page, kv_full + 8 * stage);
      tma_load_4d(v_tiles + stage * kTileBytes + pg * kPage * 128, &map_v, 0, g, 0, page, kv_full + 8 * stage);
    }
  };
  if (tid == 0) {
    for (int it = 0; it < min(iters, kStages); ++it) issue_loads(it);
  }

  // ---- Q8 operand: per head, q * 2^e with 2^e chosen so the largest magnitude lands below 448, as hi + lo codes
  // thread `tid` owns column d = tid
  float q_inv_scale[kGroupMax];  // 2^-e per head (folded into the score scale)
  {
    float qv[kGroupMax];
#pragma unroll
    for (int h = 0; h < kGroupMax; ++h) {
      qv[h] = h < group ? bf16_bits_to_float(p.q[((long long)b * p.q_heads + g * group + h) * kD + tid]) : 0.f;
      float a = fabsf(qv[h]);
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, o));
      if (lane == 0) red[warp * 4 + h] = a;
    }
    __syncthreads();
#pragma unroll
    for (int h = 0; h < kGroupMax; ++h) {
      const float amax = fmaxf(fmaxf(red[h], red[4 + h]), fmaxf(red[8 + h], red[12 + h]));
      // power of two: exact to apply and to undo; 256 * amax' <= 448 keeps both codes in range
      int e = 0;
      if (amax > 0.f) {
        frexpf(amax, &e);  // amax = f * 2^e, f in [0.5, 1)
        e = 8 - e;         // q * 2^(8-e) has magnitude in [128, 256)
      }
      const float up = ldexpf(1.0f, e);
      q_inv_scale[h] = ldexpf(1.0f, -e);
      const float scaled = qv[h] * up;
      const uint32_t hi = to_e4m3(scaled);
      const uint32_t lo = to_e4m3(scaled - from_e4m3(hi));
      st_shared_u8(swizzled(q8_tile, h, tid), hi);
      st_shared_u8(swizzled(q8_tile, 4 + h, tid), lo);
    }
    __syncthreads();  // red[] is reused below
  }
  float score_scale[kGroupMax];
  {
    const float ks = p.k_scale[b * p.kv_heads + g] * p.scale_log2;
#pragma unroll
    for (int h = 0; h < kGroupMax; ++h) score_scale[h] = q_inv_scale[h] * ks;
  }
  fence_async_smem();
  __syncthreads();

  const uint32_t idesc1 = umma_idesc(kFmtE4M3, kFmtE4M3, 128, 16, 0, 0);
  const uint32_t idesc2 = umma_idesc(kFmtE4M3, kFmtE4M3, 128, 16, 1, 0);
  const uint32_t lane_base = tmem_base + (uint32_t(warp * 32) << 16);
  float m_run[kGroupMax], l_part[kGroupMax], acc[kGroupMax];
#pragma unroll
  for (int h = 0; h < kGroupMax; ++h) {
    m_run[h] = -INFINITY;
    l_part[h] = 0.f;
    acc[h] = 0.f;
  }
  uint32_t mma_phase = 0;
  bool ok = true;

  for (int it = 0; it < iters && ok; ++it) {
    const int stage = it % kStages;
    const uint32_t k_tile = k_tiles + stage * kTileBytes;
    const uint32_t v_tile = v_tiles + stage * kTileBytes;
    const int valid = min(kIterTokens, tokens - it * kIterTokens);
    if (!warp_wait(kv_full + 8 * stage, (it / kStages) & 1, abort_flag, status, kSiteKv)) {
      ok = false;
      break;
    }
    if (valid < kIterTokens) {
      // rows past the context end hold stale or unloaded bytes: make them zero codes so 0 * x stays 0
      if (tid >= valid) {
        for (int c = 0; c < 8; ++c) {
          asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(k_tile + tid * 128 + c * 16), "r"(0u) : "memory");
          asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(v_tile + tid * 128 + c * 16), "r"(0u) : "memory");
        }
      }
      fence_async_smem();
    }
    tc_fence_before();
    __syncthreads();
    // ---- MMA 1: S^T = K_tile . Q8^T
    if (tid == 0) {
      tc_fence_after();
      const uint64_t a_desc = umma_desc_kmajor_sw128(k_tile);
      const uint64_t b_desc = umma_desc_kmajor_sw128(q8_tile);
#pragma unroll
      for (int ks = 0; ks < 4; ++ks) umma_ss<1, true>(tmem_base, a_desc + 2 * ks, b_desc + 2 * ks, idesc1, ks > 0);
      umma_commit(mma_bar);
    }
    if (!warp_wait(mma_bar, mma_phase, abort_flag, status, kSiteMma1)) {
      ok = false;
      break;
    }
    mma_phase ^= 1u;
    tc_fence_after();
    uint32_t sr[8];
    tmem_ld_32x8(lane_base, sr);
    tmem_ld_wait8(sr);
    // thread = token `tid` of this iteration
    float s[kGroupMax];
#pragma unroll
    for (int h = 0; h < kGroupMax; ++h) {
      s[h] = (__uint_as_float(sr[h]) + __uint_as_float(sr[4 + h])) * score_scale[h];
      if (tid >= valid) s[h] = -INFINITY;
      float mx = s[h];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      if (lane == 0) red[warp * 4 + h] = mx;
    }
    __syncthreads();
    float corr[kGroupMax];
#pragma unroll
    for (int h = 0; h < kGroupMax; ++h) {
      const float mx = fmaxf(fmaxf(red[h], red[4 + h]), fmaxf(red[8 + h], red[12 + h]));
      const float m_new = fmaxf(m_run[h], mx);
      corr[h] = ex2_approx(m_run[h] - m_new);  // 0 on the first iteration (m_run = -inf)
      m_run[h] = m_new;
      const float pv = ex2_approx(s[h] - m_new);
      l_part[h] = l_part[h] * corr[h] + pv;
      const float scaled = pv * 256.0f;
      const uint32_t hi = to_e4m3(scaled);
      const uint32_t lo = to_e4m3(scaled - from_e4m3(hi));
      st_shared_u8(swizzled(p8_tile, h, tid), hi);
      st_shared_u8(swizzled(p8_tile, 4 + h, tid), lo);
    }
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    // ---- MMA 2: D = V_tile^T . P8^T  (A is the MN-major V tile: 8-token groups are 1024 bytes apart)
    if (tid == 0) {
      tc_fence_after();
      const uint64_t b_desc = umma_desc_kmajor_sw128(p8_tile);
#pragma unroll
      for (int ks = 0; ks < 4; ++ks) {
        umma_ss<1, true>(tmem_base + 16, umma_desc_mnmajor_sw128(v_tile + ks * 32 * 128, 0, 1024), b_desc + 2 * ks,
                         idesc2, ks > 0);
      }
      umma_commit(mma_bar);
    }
    if (!warp_wait(mma_bar, mma_phase, abort_flag, status, kSiteMma2)) {
      ok = false;
      break;
    }
    mma_phase ^= 1u;
    tc_fence_after();
    uint32_t dr[8];
    tmem_ld_32x8(lane_base + 16, dr);
    tmem_ld_wait8(dr);
    // thread = output column d = tid
#pragma unroll
    for (int h = 0; h < kGroupMax; ++h) {
      acc[h] = acc[h] * corr[h] + (__uint_as_float(dr[h]) + __uint_as_float(dr[4 + h])) * (1.0f / 256.0f);
    }
    // both tiles of this stage are free again: prefetch the iteration that will reuse it
    if (tid == 0 && it + kStages < iters) issue_loads(it + kStages);
  }

  // ---- partials: l is reduced over the block; (m, l) then acc[d] per q head
  if (ok) {
    __syncthreads();
#pragma unroll
    for (int h = 0; h < kGroupMax; ++h) {
      float v = l_part[h];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      if (lane == 0) red[warp * 4 + h] = v;
    }
    __syncthreads();
    for (int h = 0; h < group; ++h) {
      const long long unit = ((long long)b * p.q_heads + g * group + h) * p.chunks + chunk;
      float* out = p.workspace + unit * (kD + 2);
      if (tid == 0) {
        out[0] = m_run[h];
        out[1] = (red[h] + red[4 + h]) + (red[8 + h] + red[12 + h]);
      }
      out[2 + tid] = acc[h];
    }
  }
  if (tid == 0 && bad_page != 0) report_failure(status, kErrDeviceIndex, kSitePageId, uint32_t(bad_page) & 0x7fffffffu);
  // the merge kernel is launched as a programmatic dependent: let it start arriving while the last CTAs drain
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  if (*abort_flag != 0) {
    for (int i = 0; i < 1000; ++i) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc<1>(tmem_base, 32);
  }
}

// O[b, h, :] = (sum_c 2^(m_c - M) acc_c) / (sum_c 2^(m_c - M) l_c) * v_scale, rounded once to bf16.
__global__ void decode_merge_kernel(const float* __restrict__ workspace, const int32_t* __restrict__ context_len,
                                    const float* __restrict__ v_scale, uint16_t* __restrict__ o, int q_heads,
                                    int kv_heads, int chunks, int max_context) {
  const int h = blockIdx.x, b = blockIdx.y, d = threadIdx.x;
  const int len = max(0, min(context_len[b], max_context));
  const int used = min(chunks, (len + kChunkTokens - 1) / kChunkTokens);
  // launched with programmatic stream serialisation: this grid may be resident before the partial kernel has
  // finished; the partials are valid only after this wait (inputs of the call itself are read above it)
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const float* unit = workspace + ((long long)b * q_heads + h) * chunks * (kD + 2);
  float m = -INFINITY;
  for (int c = 0; c < used; ++c) m = fmaxf(m, unit[c * (kD + 2)]);
  float num = 0.f, den = 0.f;
  for (int c = 0; c < used; ++c) {
    const float w = exp2f(unit[c * (kD + 2)] - m);
    den += w * unit[c * (kD + 2) + 1];
    num += w * unit[c * (kD + 2) + 2 + d];
  }
  const float vs = v_scale[b * kv_heads + h / (q_heads / kv_heads)];
  const float value = used > 0 ? num / den * vs : 0.f;
  o[((long long)b * q_heads + h) * kD + d] = uint16_t(pack_bf16x2(value, 0.f) & 0xffffu);
}

// The merge launch overlaps its own launch latency with the tail of the partial kernel (programmatic dependent launch).
int launch_merge(const float* workspace, const int32_t* context_len, const float* v_scale, uint16_t* o, int q_heads,
                 int kv_heads, int batch, int chunks, int max_context, cudaStream_t stream) {
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(unsigned(q_heads), unsigned(batch), 1);
  config.blockDim = dim3(kD, 1, 1);
  config.dynamicSmemBytes = 0;
  config.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attr;
  config.numAttrs = 1;
  KRNB_CUDA(cudaLaunchKernelEx(&config, decode_merge_kernel, workspace, context_len, v_scale, o, q_heads, kv_heads, chunks,
                               max_context));
  return KRN_B200_OK;
}

int encode_pages(CUtensorMap* map, const void* pages, int64_t num_pages, int64_t kv_heads) {
  uint64_t dims[4] = {uint64_t(kD), uint64_t(kv_heads), uint64_t(kPage), uint64_t(num_pages)};
  uint64_t strides[3] = {uint64_t(kD), uint64_t(kD) * kv_heads, uint64_t(kD) * kv_heads * kPage};
  uint32_t box[4] = {uint32_t(kD), 1, uint32_t(kPage), 1};
  return encode_tensor_map(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, pages, dims, strides, box, Swizzle::k128B);
}

// Floats of split-KV partials a problem needs: (m, l, acc[d]) per (sequence, q head, 1024-token chunk).
long long partial_floats(int64_t batch, int64_t q_heads, int64_t max_context) {
  const long long chunks = (max_context + kChunkTokens - 1) / kChunkTokens;
  return (long long)batch * q_heads * chunks * (kD + 2);
}

struct DecodeArguments {
  const void *q, *k_pages, *v_pages;
  const int32_t *page_table, *context_len;
  const float *k_scale, *v_scale;
  void* o;
  int64_t batch, q_heads, kv_heads, d, page_size, num_pages, max_pages_per_seq, max_context;
  float scale_log2;
};

// Checks shared by the two entry points (everything except where the scratch lives).
int check_arguments(const DecodeArguments& a) {
  if (a.d != kD || a.page_size != kPage) {
    return fail(KRN_B200_ERR_UNSUPPORTED, "paged decode with d = %lld, page size %lld is not available on sm_100a: "
                "the kernel is built for 128-byte rows and 64-token pages. Instead: use d = 128 and page_size = 64",
                (long long)a.d, (long long)a.page_size);
  }
  if (a.batch < 0 || a.q_heads <= 0 || a.kv_heads <= 0 || a.q_heads % a.kv_heads != 0 ||
      a.q_heads / a.kv_heads > kGroupMax) {
    return fail(KRN_B200_ERR_UNSUPPORTED, "q_heads / kv_heads must be an integer of at most %d (got %lld / %lld)",
                kGroupMax, (long long)a.q_heads, (long long)a.kv_heads);
  }
  if (a.batch == 0) return KRN_B200_OK;
  if (a.q == nullptr || a.k_pages == nullptr || a.v_pages == nullptr || a.page_table == nullptr ||
      a.context_len == nullptr || a.k_scale == nullptr || a.v_scale == nullptr || a.o == nullptr) {
    return fail(KRN_B200_ERR_INVALID_ARGUMENT, "null tensor address");
  }
  if (a.max_context <= 0 || a.max_pages_per_seq * kPage < a.max_context) {
    return fail(KRN_B200_ERR_INVALID_ARGUMENT, "max_context %lld does not fit %lld pages per sequence",
                (long long)a.max_context, (long long)a.max_pages_per_seq);
  }
  if (a.batch > 65535 || a.kv_heads > 65535) {
    return fail(KRN_B200_ERR_UNSUPPORTED, "batch %lld x kv_heads %lld is not available: both are grid dimensions of at "
                "most 65535. Instead: split the batch", (long long)a.batch, (long long)a.kv_heads);
  }
  if (a.num_pages <= 0 || a.num_pages >= INT32_MAX || a.batch * a.q_heads > INT32_MAX / 16 || a.max_context > INT32_MAX / 2) {
    return fail(KRN_B200_ERR_INVALID_ARGUMENT, "num_pages %lld must be positive and extents must fit 32-bit indices",
                (long long)a.num_pages);
  }
  if (!aligned16(a.k_pages) || !aligned16(a.v_pages)) {
    return fail(KRN_B200_ERR_INVALID_ARGUMENT, "page pools must be 16-byte aligned");
  }
  return KRN_B200_OK;
}

// Launches the two kernels; `scratch` holds partial_floats() floats and needs no preparation (a call reads back only
// the partials it wrote).
int launch_decode(const DecodeArguments& a, float* scratch, DeviceStatus* status, cudaStream_t stream) {
  CUtensorMap map_k, map_v;
  if (int rc = encode_pages(&map_k, a.k_pages, a.num_pages, a.kv_heads)) return rc;
  if (int rc = encode_pages(&map_v, a.v_pages, a.num_pages, a.kv_heads)) return rc;

  DecodeParams p;
  p.q = static_cast<const uint16_t*>(a.q);
  p.page_table = a.page_table;
  p.context_len = a.context_len;
  p.k_scale = a.k_scale;
  p.workspace = scratch;
  p.batch = int(a.batch);
  p.q_heads = int(a.q_heads);
  p.kv_heads = int(a.kv_heads);
  p.group = int(a.q_heads / a.kv_heads);
  p.max_pages = int(a.max_pages_per_seq);
  p.chunks = int((a.max_context + kChunkTokens - 1) / kChunkTokens);
  p.max_context = int(a.max_context);
  p.num_pages = int(a.num_pages);
  p.scale_log2 = a.scale_log2;

  KRNB_CUDA(cudaFuncSetAttribute(decode_partial_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
  decode_partial_kernel<<<dim3(unsigned(p.chunks), unsigned(a.kv_heads), unsigned(a.batch)), kThreads, kSmemBytes, stream>>>(
      map_k, map_v, p, status);
  KRNB_CUDA(cudaGetLastError());
  return launch_merge(scratch, a.context_len, a.v_scale, static_cast<uint16_t*>(a.o), p.q_heads, p.kv_heads, p.batch,
                      p.chunks, p.max_context, stream);
}

}  // namespace
}  // namespace krnb

extern "C" int64_t krn_b200_attn_decode_workspace_bytes(int64_t batch, int64_t q_heads, int64_t d, int64_t max_context) {
  if (batch <= 0 || q_heads <= 0 || d <= 0 || max_context <= 0) return 0;
  return krnb::partial_floats(batch, q_heads, max_context) * 4;
}

extern "C" int krn_b200_attn_decode_fp8_paged(const void* q, const void* k_pages, const void* v_pages,
                                              const int32_t* page_table, const int32_t* context_len,
                                              const float* k_scale, const float* v_scale, void* o, int64_t batch,
                                              int64_t q_heads, int64_t kv_heads, int64_t d, int64_t page_size,
                                              int64_t num_pages, int64_t max_pages_per_seq, int64_t max_context,
                                              float scale_log2, void* workspace, int64_t workspace_bytes,
                                              void* stream_handle) {
  using namespace krnb;
  const DecodeArguments a = {q, k_pages, v_pages, page_table, context_len, k_scale, v_scale, o, batch, q_heads, kv_heads,
                             d, page_size, num_pages, max_pages_per_seq, max_context, scale_log2};
  if (int rc = check_arguments(a)) return rc;
  if (batch == 0) return KRN_B200_OK;
  const int64_t need = krn_b200_attn_decode_workspace_bytes(batch, q_heads, d, max_context);
  if (workspace == nullptr || workspace_bytes < need) {
    return fail(KRN_B200_ERR_WORKSPACE, "workspace of %lld bytes is too small: %lld needed", (long long)workspace_bytes,
                (long long)need);
  }
  if (!aligned16(workspace)) return fail(KRN_B200_ERR_INVALID_ARGUMENT, "the workspace must be 16-byte aligned");
  DeviceContext* ctx = current_context();
  if (ctx == nullptr) return KRN_B200_ERR_CUDA;
  if (int rc = require_sm100(ctx)) return rc;
  return launch_decode(a, static_cast<float*>(workspace), ctx->status_dev, static_cast<cudaStream_t>(stream_handle));
}

// ---------------------------------------------------------------------------------------------------------
// The same decode attention for callers that must not allocate device memory.
//
// Some hosts of this library cannot call cudaMalloc at the point where they need attention: a serving loop
// that has handed all free HBM to its KV-cache pool, a plugin running inside another runtime's memory budget,
// or code on a path where an allocation (and the implicit synchronisation it can cause) is forbidden. For
// them the split-KV partials live in a fixed array inside the library image instead of a caller workspace. Every GPU that loads the library carries these 16 MiB until the process exits.
namespace krnb {
namespace {

constexpr long long kStaticScratchFloats = 4ll * 1024 * 1024;  // 16 MiB
static __device__ __align__(256) float g_decode_scratch[kStaticScratchFloats];

constexpr int kScratchDevices = 64;
std::mutex g_scratch_mutex;
float* g_scratch_address[kScratchDevices] = {nullptr};

// Device address of g_decode_scratch on the CURRENT device. In host code the array's name is only a handle: the
// address a kernel may dereference comes from cudaGetSymbolAddress, once per device, with that device current.
int static_scratch(float** address) {
  int device = -1;
  KRNB_CUDA(cudaGetDevice(&device));
  if (device < 0 || device >= kScratchDevices) {
    return fail(KRN_B200_ERR_UNSUPPORTED, "device ordinal %d is outside the supported range", device);
  }
  std::lock_guard<std::mutex> lock(g_scratch_mutex);
  if (g_scratch_address[device] == nullptr) {
    int major = 0;
    KRNB_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device));
    if (major != 10) {
      return fail(KRN_B200_ERR_UNSUPPORTED, "tcgen05 kernels is not available on this device: this library holds "
                  "sm_100a code only. Instead: run on a B200 (compute capability 10.x)");
    }
    float* resolved = nullptr;
    KRNB_CUDA(cudaGetSymbolAddress(reinterpret_cast<void**>(&resolved), g_decode_scratch));
    g_scratch_address[device] = resolved;
  }
  *address = g_scratch_address[device];
  return KRN_B200_OK;
}

}  // namespace
}  // namespace krnb

extern "C" int krn_b200_attn_decode_fp8_paged_noalloc(const void* q, const void* k_pages, const void* v_pages,
                                                      const int32_t* page_table, const int32_t* context_len,
                                                      const float* k_scale, const float* v_scale, void* o,
                                                      int64_t batch, int64_t q_heads, int64_t kv_heads, int64_t d,
                                                      int64_t page_size, int64_t num_pages, int64_t max_pages_per_seq,
                                                      int64_t max_context, float scale_log2, void* stream_handle) {
  using namespace krnb;
  const DecodeArguments a = {q, k_pages, v_pages, page_table, context_len, k_scale, v_scale, o, batch, q_heads, kv_heads,
                             d, page_size, num_pages, max_pages_per_seq, max_context, scale_log2};
  if (int rc = check_arguments(a)) return rc;
  if (batch == 0) return KRN_B200_OK;
  const long long need = partial_floats(batch, q_heads, max_context);
  if (need > kStaticScratchFloats) {
    return fail(KRN_B200_ERR_WORKSPACE,
                "batch %lld x q_heads %lld x %lld context chunks needs %lld scratch floats; the built-in scratch holds "
                "%lld (16 MiB). Use krn_b200_attn_decode_fp8_paged with a caller workspace for larger problems",
                (long long)batch, (long long)q_heads, (long long)((max_context + kChunkTokens - 1) / kChunkTokens), need,
                kStaticScratchFloats);
  }
  float* scratch = nullptr;
  if (int rc = static_scratch(&scratch)) return rc;
  // the status word exists only if a regular entry point created it earlier; this call never allocates one
  DeviceContext* ctx = existing_context();
  DeviceStatus* status = ctx != nullptr ? ctx->status_dev : nullptr;
  return launch_decode(a, scratch, status, static_cast<cudaStream_t>(stream_handle));
}
