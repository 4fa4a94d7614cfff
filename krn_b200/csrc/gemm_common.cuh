// Pieces shared by the tile-product kernels: the problem record and the persistent tile order.
#pragma once

#include <cuda_fp16.h>

#include "host.cuh"

namespace krnb {

struct Problem {
  int m, n, k;
  int tiles_m, tiles_n;
  int b_kn;  // 0: b is (N, K), the operand of `b.transpose()`; 1: b is (K, N), the operand of a plain `a @ b`
};

// Where the output goes. One map for a plain product. When the product is sharded by output columns over the GPUs
// of a node, one map per rank: every rank's full C (its own and, through NVLink peer mappings, the others'),
// and this rank's column block is stored into all of them at `column_offset` — the all-gather of the output
// columns happens in the epilogue's TMA stores, tile by tile, while the main loop works on the next tile.
// (TMA STORES to peer memory; no load ever targets a peer and nothing is multicast.)
constexpr int kMaxDestinations = 8;
struct Destinations {
  CUtensorMap maps[kMaxDestinations];
  int count;
  int column_offset;
  int first;  // destination the stores of a box start with: each rank starts one past itself, so that at any moment
              // the ranks of a node aim at different receivers instead of all at rank 0, then all at rank 1, ...
};

// Cross-rank completion of a column-sharded product, done in the kernel's own tail instead of a separate barrier
// kernel. Every rank owns an array of `ranks` 32-bit flags that all ranks can write (peer-mapped memory); flag r of a
// rank holds the number of the last product whose stores FROM rank r have all landed in this rank's C. When a CTA has
// waited for its own bulk stores it counts itself in `arrivals` (local memory); the last CTA of the launch writes the
// product's number (`epoch`, one more per launch) into its flag on every peer and then waits — with a limit — until
// every peer's flag on THIS rank has reached the same number, so the kernel completes only when this rank's C is
// whole. Nothing spins without a limit: on expiry the status word records the site and the kernel returns.
// `ranks == 0` switches all of it off (the caller synchronises the ranks itself).
struct RankSync {
  uint32_t* flags[kMaxDestinations];  // flags[r]: address, valid on this device, of rank r's flag array
  uint32_t* arrivals;                 // this device's count of CTAs that finished their stores; zero between launches
  uint32_t epoch;
  int ranks, rank;
};

__device__ __forceinline__ void rank_barrier_tail(const RankSync& sync, DeviceStatus* status, int site) {
  if (sync.ranks <= 1) return;
  // this CTA's TMA stores have completed (cp.async.bulk.wait_group 0 in the storing lanes, then the CTA barrier);
  // order them, system-wide, before the arrival that may release the flag
  asm volatile("fence.proxy.async;" ::: "memory");
  __threadfence_system();
  if (atomicAdd(sync.arrivals, 1u) + 1u != gridDim.x) return;
  *sync.arrivals = 0u;  // every CTA of this launch has arrived; the next launch on the stream starts from zero
  __threadfence_system();
  for (int r = 0; r < sync.ranks; ++r) {
    if (r == sync.rank) continue;
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(sync.flags[r] + sync.rank), "r"(sync.epoch) : "memory");
  }
  const long long start = clock64();
  for (int r = 0; r < sync.ranks; ++r) {
    if (r == sync.rank) continue;
    const uint32_t* flag = sync.flags[sync.rank] + r;
    while (true) {
      uint32_t seen;
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(flag) : "memory");
      if (int32_t(seen - sync.epoch) >= 0) break;
      if (clock64() - start > kWaitLimitCycles) {
        report_failure(status, kErrDeviceTimeout, site, uint32_t(r));
        return;
      }
      __nanosleep(200);
    }
  }
}

// Host side: `sync_of_rank[r]` is the address on this device of rank r's sync words — `ranks` flags followed by the
// arrival counter, (kMaxDestinations + 1) 32-bit words in all, zero before the first product. A null array leaves the
// in-kernel barrier off.
inline int fill_rank_sync(RankSync* sync, void* const* sync_of_rank, int ranks, int rank, uint32_t epoch) {
  *sync = RankSync{};
  if (sync_of_rank == nullptr) return KRN_B200_OK;
  for (int r = 0; r < ranks; ++r) {
    if (sync_of_rank[r] == nullptr || reinterpret_cast<uintptr_t>(sync_of_rank[r]) % 4 != 0) {
      return fail(KRN_B200_ERR_INVALID_ARGUMENT, "sync words of rank %d: null or not 4-byte aligned", r);
    }
    sync->flags[r] = static_cast<uint32_t*>(sync_of_rank[r]);
  }
  sync->arrivals = static_cast<uint32_t*>(sync_of_rank[rank]) + kMaxDestinations;
  sync->epoch = epoch;
  sync->ranks = ranks;
  sync->rank = rank;
  return KRN_B200_OK;
}

// What happens to the f32 accumulator between the last K step and the rounding to the output type:
// `out = activation(acc + bias[column])`, the statements of the reference's `matmul_epilogue` kernel
// (src/krn/lib/lib_kernels.py:30-48). flags = KRN_B200_EPILOGUE_* of include/krn_b200.h: bit 0 adds the bias (a
// vector of the OUTPUT type, as `Operands.bias`, src/krn/lib/lib.py:155-163), bits 1-2 pick the activation.
struct EpilogueSpec {
  const void* bias;
  int flags;
};
constexpr int kEpilogueBias = 1;
constexpr int kActivationRelu = 1, kActivationGelu = 2, kActivationSilu = 3;

// The reference's element functions in f32 (src/krn/compiler/emit.py:110-114): relu `x < 0 ? 0 : x`, gelu
// `0.5 x (1 + erf(x / sqrt 2))` (the exact Gaussian form), silu `x / (1 + exp(-x))`.
__device__ __forceinline__ float apply_activation(float x, int activation) {
  if (activation == kActivationRelu) return x < 0.f ? 0.f : x;
  if (activation == kActivationGelu) return 0.5f * x * (1.f + erff(x * 0.7071067811865476f));
  if (activation == kActivationSilu) return x / (1.f + expf(-x));
  return x;
}

// Element `index` of a bias vector stored in the output type (f32 words, or 16-bit bf16 / f16 words).
template <typename OutT, bool OUT_BF16>
__device__ __forceinline__ float load_bias(const void* bias, long long index) {
  if constexpr (sizeof(OutT) == 4) {
    return __ldg(static_cast<const float*>(bias) + index);
  } else {
    const uint16_t w = __ldg(static_cast<const uint16_t*>(bias) + index);
    if constexpr (OUT_BF16) return __uint_as_float(uint32_t(w) << 16);
    return __half2float(__ushort_as_half(w));
  }
}

// Tile order: bands of 8 tile rows walked column by column, so that the tiles in flight at any time
// share a few A row-panels and B column-panels in L2.
__device__ __forceinline__ void tile_coords(int t, const Problem& p, int& tm, int& tn) {
  constexpr int kBand = 8;
  const int per_band = kBand * p.tiles_n;
  const int band = t / per_band;
  const int first = band * kBand;
  const int height = min(kBand, p.tiles_m - first);
  const int r = t - band * per_band;
  tm = first + r % height;
  tn = r / height;
}

}  // namespace krnb
