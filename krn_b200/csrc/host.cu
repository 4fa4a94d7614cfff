// Library-wide host state: error text, device contexts, status word, tensor-map encoding.
#include "host.cuh"

#include <cstring>
#include <mutex>

namespace krnb {

char* error_buffer() {
  static thread_local char buffer[512] = {0};
  return buffer;
}

int fail(int code, const char* format, ...) {
  va_list args;
  va_start(args, format);
  vsnprintf(error_buffer(), 512, format, args);
  va_end(args);
  return code;
}

namespace {
constexpr int kMaxDevices = 64;
std::mutex g_mutex;
DeviceContext g_contexts[kMaxDevices];
bool g_ready[kMaxDevices] = {false};

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;

EncodeTiledFn encode_entry() {
  if (g_encode != nullptr) return g_encode;
  std::lock_guard<std::mutex> lock(g_mutex);
  if (g_encode != nullptr) return g_encode;
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult query;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &query) != cudaSuccess ||
      query != cudaDriverEntryPointSuccess) {
    return nullptr;
  }
  g_encode = reinterpret_cast<EncodeTiledFn>(fn);
  return g_encode;
}
}  // namespace

DeviceContext* current_context() {
  int device = -1;
  cudaError_t err = cudaGetDevice(&device);
  if (err != cudaSuccess) {
    fail(KRN_B200_ERR_CUDA, "%s: %s (cudaGetDevice)", cudaGetErrorName(err), cudaGetErrorString(err));
    return nullptr;
  }
  if (device < 0 || device >= kMaxDevices) {
    fail(KRN_B200_ERR_UNSUPPORTED, "device ordinal %d is outside the supported range", device);
    return nullptr;
  }
  std::lock_guard<std::mutex> lock(g_mutex);
  if (g_ready[device]) return &g_contexts[device];
  DeviceContext ctx;
  ctx.device = device;
  cudaDeviceProp prop;
  err = cudaGetDeviceProperties(&prop, device);
  if (err != cudaSuccess) {
    fail(KRN_B200_ERR_CUDA, "%s: %s (cudaGetDeviceProperties)", cudaGetErrorName(err), cudaGetErrorString(err));
    return nullptr;
  }
  ctx.sm_count = prop.multiProcessorCount;
  ctx.cc_major = prop.major;
  ctx.cc_minor = prop.minor;
  err = cudaHostAlloc(reinterpret_cast<void**>(&ctx.status_host), sizeof(DeviceStatus), cudaHostAllocMapped);
  if (err != cudaSuccess) {
    fail(KRN_B200_ERR_CUDA, "%s: %s (status word)", cudaGetErrorName(err), cudaGetErrorString(err));
    return nullptr;
  }
  std::memset(ctx.status_host, 0, sizeof(DeviceStatus));
  err = cudaHostGetDevicePointer(reinterpret_cast<void**>(&ctx.status_dev), ctx.status_host, 0);
  if (err != cudaSuccess) {
    fail(KRN_B200_ERR_CUDA, "%s: %s (status word mapping)", cudaGetErrorName(err), cudaGetErrorString(err));
    return nullptr;
  }
  cudaMemPoolProps pool_props = {};
  pool_props.allocType = cudaMemAllocationTypePinned;
  pool_props.handleTypes = cudaMemHandleTypeNone;
  pool_props.location.type = cudaMemLocationTypeDevice;
  pool_props.location.id = device;
  err = cudaMemPoolCreate(&ctx.scratch_pool, &pool_props);
  if (err == cudaSuccess) {
    uint64_t keep = UINT64_MAX;  // never hand memory back at a synchronisation
    err = cudaMemPoolSetAttribute(ctx.scratch_pool, cudaMemPoolAttrReleaseThreshold, &keep);
  }
  if (err != cudaSuccess) {
    fail(KRN_B200_ERR_CUDA, "%s: %s (scratch memory pool)", cudaGetErrorName(err), cudaGetErrorString(err));
    return nullptr;
  }
  g_contexts[device] = ctx;
  g_ready[device] = true;
  return &g_contexts[device];
}

DeviceContext* existing_context() {
  int device = -1;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kMaxDevices) return nullptr;
  std::lock_guard<std::mutex> lock(g_mutex);
  return g_ready[device] ? &g_contexts[device] : nullptr;
}

int require_sm100(const DeviceContext* ctx) {
  if (ctx->cc_major != 10) {
    return fail(KRN_B200_ERR_UNSUPPORTED,
                "tcgen05 kernels is not available on sm_%d%d: this library holds sm_100a code only. "
                "Instead: run on a B200 (compute capability 10.x)",
                ctx->cc_major, ctx->cc_minor);
  }
  return KRN_B200_OK;
}

int encode_tensor_map(CUtensorMap* map, CUtensorMapDataType type, int rank, const void* base, const uint64_t* dims,
                      const uint64_t* strides_bytes, const uint32_t* box, Swizzle swizzle) {
  EncodeTiledFn encode = encode_entry();
  if (encode == nullptr) return fail(KRN_B200_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t gdims[5];
  cuuint64_t gstrides[4];
  cuuint32_t gbox[5];
  cuuint32_t estrides[5];
  for (int i = 0; i < rank; ++i) {
    gdims[i] = dims[i];
    gbox[i] = box[i];
    estrides[i] = 1;
    if (i > 0) gstrides[i - 1] = strides_bytes[i - 1];
  }
  CUresult res = encode(map, type, static_cast<cuuint32_t>(rank), const_cast<void*>(base), gdims, gstrides, gbox,
                        estrides, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        swizzle == Swizzle::k128B ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (res != CUDA_SUCCESS) {
    return fail(KRN_B200_ERR_INVALID_ARGUMENT,
                "cuTensorMapEncodeTiled failed with CUresult %d (rank %d, dims [%llu, %llu], box [%u, %u])",
                static_cast<int>(res), rank, static_cast<unsigned long long>(dims[0]),
                static_cast<unsigned long long>(rank > 1 ? dims[1] : 0), box[0], rank > 1 ? box[1] : 0);
  }
  return KRN_B200_OK;
}

}  // namespace krnb

extern "C" {

int krn_b200_version(void) { return KRN_B200_ABI_VERSION; }

size_t krn_b200_last_error(char* buffer, size_t size) {
  const char* message = krnb::error_buffer();
  size_t length = std::strlen(message);
  if (buffer != nullptr && size > 0) {
    size_t n = length < size - 1 ? length : size - 1;
    std::memcpy(buffer, message, n);
    buffer[n] = '\0';
  }
  return length;
}

int krn_b200_device_status(int* code, int* site, unsigned int* block) {
  krnb::DeviceContext* ctx = krnb::current_context();
  if (ctx == nullptr) return KRN_B200_ERR_CUDA;
  volatile krnb::DeviceStatus* status = ctx->status_host;
  int c = status->code;
  if (code != nullptr) *code = c;
  if (site != nullptr) *site = status->where;
  if (block != nullptr) *block = status->block;
  if (c != 0) {
    krnb::fail(c, c == KRN_B200_ERR_DEVICE_INDEX ? "index outside its tensor at site %d in block %u (value %u); the access was skipped"
                                                 : "device-side wait expired at site %d in block %u (info %u)",
               status->where, status->block, status->info);
    status->where = 0;
    status->block = 0;
    status->info = 0;
    status->code = 0;
  }
  return KRN_B200_OK;
}

}  // extern "C"
