#include "host.cuh"
extern "C" int krn_b200_gemm_fp8_blockscaled_tn(int, const void*, const float*, const void*, const float*, void*, int64_t,
                                                int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, void*) {
  return krnb::fail(KRN_B200_ERR_UNSUPPORTED, "block-scaled FP8 product: kernel not built yet");
}
