// Host-side plumbing shared by the entry points: thread-local error text, the per-device status word,
// TMA descriptor encoding through the driver entry point (no link-time libcuda dependency) and device checks.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>

#include "../../include/krn_b200.h"
#include "ptx.cuh"

namespace krnb {

// ---- error text ----------------------------------------------------------------------------------------

char* error_buffer();            // thread-local, 512 bytes
int fail(int code, const char* format, ...);

#define KRNB_CUDA(call)                                                                                     \
  do {                                                                                                      \
    cudaError_t krnb_err_ = (call);                                                                         \
    if (krnb_err_ != cudaSuccess) {                                                                         \
      return ::krnb::fail(KRN_B200_ERR_CUDA, "%s: %s (%s)", cudaGetErrorName(krnb_err_),                    \
                          cudaGetErrorString(krnb_err_), #call);                                            \
    }                                                                                                       \
  } while (0)

// ---- per-device context ---------------------------------------------------------------------------------

struct DeviceContext {
  int device = -1;
  int sm_count = 0;
  int cc_major = 0;
  int cc_minor = 0;
  DeviceStatus* status_host = nullptr;  // pinned, mapped
  DeviceStatus* status_dev = nullptr;   // device view of the same word
  // Stream-ordered scratch memory that lives for one call (cudaMallocFromPoolAsync / cudaFreeAsync on the call's
  // stream). The pool keeps what it has been given, so only the first call of a size reaches the driver's allocator.
  cudaMemPool_t scratch_pool = nullptr;
};

// Context of the current device; created on first use (allocates the 16-byte status word once).
// Returns nullptr and sets the thread's error text on failure.
DeviceContext* current_context();

// Context of the current device if an earlier call already created it, else nullptr. Never allocates.
DeviceContext* existing_context();

// Refuse anything that is not a compute-capability 10.x device.
int require_sm100(const DeviceContext* ctx);

// ---- TMA descriptors -----------------------------------------------------------------------------------

enum class Swizzle { kNone, k128B };

// Encode a tiled tensor map of `rank` dims. dims/strides innermost first; strides in bytes for dims 1..rank-1.
int encode_tensor_map(CUtensorMap* map, CUtensorMapDataType type, int rank, const void* base, const uint64_t* dims,
                      const uint64_t* strides_bytes, const uint32_t* box, Swizzle swizzle);

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace krnb
