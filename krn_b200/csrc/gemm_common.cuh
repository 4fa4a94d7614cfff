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
