// Re-layout of all-gathered GEMM output column blocks: slabs[r][M][n_local] -> C_full[M][ranks * n_local].
// After the NCCL all-gather each rank holds `ranks` contiguous slabs (one per rank, in rank order); a
// row-major C wants rank r's columns at [r * n_local, (r + 1) * n_local) of every row. HBM-bound copy with
// 16-byte accesses, grid sized to the SM count.
#include "host.cuh"

namespace krnb {
namespace {

__global__ void scatter_columns_kernel(const uint4* __restrict__ slabs, uint4* __restrict__ full, long long m,
                                       long long vec_per_row_local, long long ranks, long long vec_ld_full) {
  const long long per_slab = m * vec_per_row_local;
  const long long total = per_slab * ranks;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / per_slab;
    const long long rest = i - r * per_slab;
    const long long row = rest / vec_per_row_local;
    const long long col = rest - row * vec_per_row_local;
    full[row * vec_ld_full + r * vec_per_row_local + col] = slabs[i];
  }
}

}  // namespace
}  // namespace krnb

extern "C" int krn_b200_scatter_columns(const void* slabs, void* c_full, int64_t m, int64_t n_local, int64_t ranks,
                                        int64_t ld_full, int elem_bytes, void* stream_handle) {
  using namespace krnb;
  if (slabs == nullptr || c_full == nullptr) return fail(KRN_B200_ERR_INVALID_ARGUMENT, "null tensor address");
  if (m <= 0 || n_local <= 0 || ranks <= 0) return KRN_B200_OK;
  if ((n_local * elem_bytes) % 16 != 0 || (ld_full * elem_bytes) % 16 != 0 || !aligned16(slabs) || !aligned16(c_full)) {
    return fail(KRN_B200_ERR_INVALID_ARGUMENT, "column blocks must be multiples of 16 bytes and 16-byte aligned");
  }
  DeviceContext* ctx = current_context();
  if (ctx == nullptr) return KRN_B200_ERR_CUDA;
  const long long vec_local = n_local * elem_bytes / 16;
  scatter_columns_kernel<<<ctx->sm_count * 8, 256, 0, static_cast<cudaStream_t>(stream_handle)>>>(
      static_cast<const uint4*>(slabs), static_cast<uint4*>(c_full), m, vec_local, ranks, ld_full * elem_bytes / 16);
  KRNB_CUDA(cudaGetLastError());
  return KRN_B200_OK;
}

// A pitched copy between any two of {device memory, page-locked host memory}: `rows` rows of `row_bytes` bytes, each
// side with its own pitch — cudaMemcpy2DAsync behind the library's status convention. The host-operand streaming path
// uses it to return column slabs of a row-major result straight into the caller's host matrix. Replaces nothing in the
// reference, whose host copies are whole-tensor (src/krn/runtime/cuda_backend.py:205-248).
extern "C" int krn_b200_copy_2d(void* dst, int64_t dst_pitch_bytes, const void* src, int64_t src_pitch_bytes,
                                int64_t row_bytes, int64_t rows, void* stream_handle) {
  using namespace krnb;
  if (rows <= 0 || row_bytes <= 0) return KRN_B200_OK;
  if (dst == nullptr || src == nullptr) return fail(KRN_B200_ERR_INVALID_ARGUMENT, "null address");
  if (dst_pitch_bytes < row_bytes || src_pitch_bytes < row_bytes) {
    return fail(KRN_B200_ERR_INVALID_ARGUMENT, "pitch shorter than the row (%lld, %lld < %lld bytes)",
                (long long)dst_pitch_bytes, (long long)src_pitch_bytes, (long long)row_bytes);
  }
  KRNB_CUDA(cudaMemcpy2DAsync(dst, size_t(dst_pitch_bytes), src, size_t(src_pitch_bytes), size_t(row_bytes),
                              size_t(rows), cudaMemcpyDefault, static_cast<cudaStream_t>(stream_handle)));
  return KRN_B200_OK;
}
