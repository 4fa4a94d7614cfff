// Pieces shared by the tile-product kernels: the problem record and the persistent tile order.
#pragma once

#include "host.cuh"

namespace krnb {

struct Problem {
  int m, n, k;
  int tiles_m, tiles_n;
  int b_kn;  // 0: b is (N, K), the operand of `b.transpose()`; 1: b is (K, N), the operand of a plain `a @ b`
};

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
