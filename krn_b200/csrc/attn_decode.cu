#include "host.cuh"
extern "C" int64_t krn_b200_attn_decode_workspace_bytes(int64_t, int64_t, int64_t, int64_t) { return 0; }
extern "C" int krn_b200_attn_decode_fp8_paged(const void*, const void*, const void*, const int32_t*, const int32_t*,
                                              const float*, const float*, void*, int64_t, int64_t, int64_t, int64_t,
                                              int64_t, int64_t, int64_t, float, void*, int64_t, void*) {
  return krnb::fail(KRN_B200_ERR_UNSUPPORTED, "paged decode attention: kernel not built yet");
}
