#include "host.cuh"
extern "C" int krn_b200_attn_fwd(int, const void*, const void*, const void*, void*, int64_t, int64_t, int64_t, int64_t,
                                 int64_t, int64_t, float, int, const int64_t*, const int64_t*, const int64_t*,
                                 const int64_t*, void*) {
  return krnb::fail(KRN_B200_ERR_UNSUPPORTED, "flash attention: kernel not built yet");
}
