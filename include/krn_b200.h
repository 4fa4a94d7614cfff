/* krn_b200.h — C ABI of libkrn_b200.so, the prebuilt sm_100a kernel library behind the B200 device.
 *
 * Every entry point is `extern "C"`, takes raw device addresses and 64-bit extents, enqueues work on the
 * caller's CUDA stream and returns without synchronising. The return value is a status code (0 = ok);
 * `krn_b200_last_error` gives the calling thread's message for the last non-zero status. Nothing here
 * retains caller tensors, and nothing allocates device memory except the three products with tensor-core block scales
 * (krn_b200_gemm_mxfp8_tn, krn_b200_gemm_nvfp4_tn, krn_b200_gemm_mxfp4_tn): each of their calls takes scratch memory the
 * size of the two scale matrices from a stream-ordered pool the library keeps per device (cudaMallocFromPoolAsync on the
 * caller's stream, cudaFreeAsync behind the product), so the driver's allocator is reached only the first time a size
 * is seen. There is no CPU fallback: on a machine without a B200 the compute entry points return KRN_B200_ERR_CUDA /
 * KRN_B200_ERR_UNSUPPORTED.
 *
 * The Python host reaches this file's functions through `krn_b200.hw.Libraries` and ctypes, the way the
 * reference reaches its compiled C programs (src/krn/runtime/cpu.py:168-175) — argument order below is the
 * order the ctypes prototypes in krn_b200/runtime/native.py declare.
 */
#ifndef KRN_B200_H
#define KRN_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define KRN_B200_ABI_VERSION 2 /* 2: the paged decode entries take num_pages, the gather entries sync words; krn_b200_gemm_fp8, krn_b200_gemm_mxfp8_tn, krn_b200_gemm_nvfp4_tn and krn_b200_gemm_mxfp4_tn added */

/* status codes */
#define KRN_B200_OK 0
#define KRN_B200_ERR_INVALID_ARGUMENT 1 /* null pointer, negative extent, misaligned address or stride */
#define KRN_B200_ERR_UNSUPPORTED 2      /* shape / dtype / device this library has no kernel for */
#define KRN_B200_ERR_CUDA 3             /* a CUDA runtime or driver call failed; message names it */
#define KRN_B200_ERR_WORKSPACE 4        /* caller workspace missing or too small */
#define KRN_B200_ERR_DEVICE_TIMEOUT 5   /* a bounded device-side wait expired (read from the status word) */
#define KRN_B200_ERR_DEVICE_INDEX 6     /* a kernel met an index outside its tensor (a page id beyond the pool); the
                                           access was skipped and the status word says where */

/* element types (operands and outputs) */
#define KRN_B200_F32 0
#define KRN_B200_F16 1
#define KRN_B200_BF16 2
#define KRN_B200_E4M3 3
#define KRN_B200_E5M2 4

/* Replaces the reference's version probes of its compiled artefacts (digest of nvrtc version + flags,
 * src/krn/runtime/cuda_backend.py:695-747): the host checks the ABI number before binding prototypes. */
int krn_b200_version(void);

/* Message for the last non-zero status returned on this thread; copies at most `size` bytes including the
 * terminator and returns the full message length. Mirrors CUDAError's "name: message" text
 * (src/krn/runtime/cuda_backend.py:97-105). */
size_t krn_b200_last_error(char* buffer, size_t size);

/* Device-side status word of the current device: bounded waits that expired inside a kernel leave
 * (code, site) here instead of trapping (the reference's device wait traps after 2^26 polls,
 * src/krn/facts/catalog.py:1439-1448). Reads and clears it. Call after the stream has been synchronised —
 * the reference surfaces asynchronous failures at the next event the same way
 * (src/krn/runtime/runtime.py:392-399). */
int krn_b200_device_status(int* code, int* site, unsigned int* block);

/* C[M,N] = A[M,K] * B[N,K]^T, f32 accumulation, one rounding to the output type (round to nearest even).
 * The tile product `a[rows, ks] @ b[cols, ks].transpose()` accumulated over a `pipelined` K loop and stored
 * with `c[rows, cols] = acc.to(T)`: replaces Builder.accumulate + Emitter.pipeline + NvidiaMma.product +
 * emit_TileStore (src/krn/compiler/capture.py:3170-3211, src/krn/compiler/emit.py:564-672,763-774,
 * src/krn/compiler/cuda.py:133-193).
 *   ab_type  KRN_B200_BF16 or KRN_B200_F16 (both operands)
 *   c_type   KRN_B200_BF16, KRN_B200_F16 or KRN_B200_F32
 *   lda/ldb/ldc  row pitches in ELEMENTS. When every base address and pitch * element size is a multiple of 16
 *                bytes the tcgen05 kernel runs; otherwise (e.g. the reference's 50 x 38 x 70 example) a plain
 *                tiled f32-fma kernel computes the same product, slowly. K == 0 stores zeros (the reference
 *                stores the untouched zero accumulator).
 * Ragged M, N, K are handled like the reference's invalid lanes: out-of-range operand elements read as
 * zero, out-of-range outputs are not stored (src/krn/compiler/emit.py:957-974,763-774). */
int krn_b200_gemm_tn(int ab_type, int c_type, const void* a, const void* b, void* c, int64_t m, int64_t n, int64_t k,
                     int64_t lda, int64_t ldb, int64_t ldc, void* stream);

/* C[M,N] = A[M,K] * B[K,N]: the same product with b stored row-major as (K, N), the form the reference's tile example
 * writes (`acc += a[rows, ks] @ b[ks, cols]`, examples/04_libraries/01_gemm_tiles.py:35-40). The b tile reaches the
 * tensor cores as an MN-major operand (64-column x 64-row swizzled boxes), so no transposed copy of b is made.
 * ldb is the pitch of a K row of b (>= N). Everything else as krn_b200_gemm_tn, including the unaligned path and
 * K == 0. */
int krn_b200_gemm_nn(int ab_type, int c_type, const void* a, const void* b, void* c, int64_t m, int64_t n, int64_t k,
                     int64_t lda, int64_t ldb, int64_t ldc, void* stream);

/* C = A * B for two 8-bit float tiles loaded as they are stored — no scales, every code stands for its own value:
 * the product the reference captures for fp8 pairs that are direct tile loads
 * (`acc += a8[rows, ks] @ b8[ks, cols]`, src/krn/compiler/capture.py:3185-3192) and lowers to one unscaled
 * m16n8k32 e4m3/e5m2 instruction per fragment (src/krn/compiler/cuda.py:207-227); here tcgen05 kind::f8f6f4
 * accumulates the whole K extent in tensor memory.
 *   a_type, b_type  KRN_B200_E4M3 or KRN_B200_E5M2, chosen per operand (all four pairs, as the reference tests,
 *                   tests/compiler/test_tensor_cores.py:146,219-239)
 *   b_kn            0: b is (N, K), the operand of b.transpose(); 1: b is (K, N) row-major, the form the reference's
 *                   fp8 kernels write
 *   lda/ldb/ldc     row pitches in ELEMENTS; 16-byte aligned addresses and pitches take the tensor-core kernel,
 *                   anything else (the reference's 50 x 38 x 70 card) the plain fma kernel, which follows the
 *                   reference's k-ordered chain exactly. K == 0 stores zeros. Ragged edges as krn_b200_gemm_tn. */
int krn_b200_gemm_fp8(int a_type, int b_type, int c_type, int b_kn, const void* a, const void* b, void* c, int64_t m,
                      int64_t n, int64_t k, int64_t lda, int64_t ldb, int64_t ldc, void* stream);

/* epilogue flags of krn_b200_matmul: KRN_B200_EPILOGUE_BIAS may be or-ed with one activation */
#define KRN_B200_EPILOGUE_NONE 0
#define KRN_B200_EPILOGUE_BIAS 1
#define KRN_B200_EPILOGUE_RELU 2
#define KRN_B200_EPILOGUE_GELU 4
#define KRN_B200_EPILOGUE_SILU 6

/* out = activation(A * B + bias): the product with the reference's fused epilogues — the statements of its
 * `matmul_epilogue` kernel (src/krn/lib/lib_kernels.py:30-48) behind `lib.matmul(a, b, epilogue=, bias=)`
 * (src/krn/lib/lib.py:580-615), applied to the f32 accumulator in the kernel's epilogue before the one rounding to the
 * output type. relu `x < 0 ? 0 : x`, gelu `0.5 x (1 + erf(x / sqrt 2))`, silu `x / (1 + exp(-x))`
 * (src/krn/compiler/emit.py:110-114).
 *   b_kn      0: b is (N, K) (the operand of b.transpose()); 1: b is (K, N), the layout lib.matmul takes
 *   epilogue  KRN_B200_EPILOGUE_* flags
 *   bias      vector of N elements of the OUTPUT type (`Operands.bias`, src/krn/lib/lib.py:155-163); read only when
 *             the BIAS flag is set
 * Everything else as krn_b200_gemm_tn. With K == 0 the result is activation(bias). */
int krn_b200_matmul(int ab_type, int c_type, int b_kn, int epilogue, const void* a, const void* b, const void* bias,
                    void* c, int64_t m, int64_t n, int64_t k, int64_t lda, int64_t ldb, int64_t ldc, void* stream);

/* The same product sharded by output columns over the GPUs of one node, with the all-gather of the output
 * columns done by the kernel itself: rank `rank` of `ranks` multiplies A[M,K] by ITS rows of B (b: [n_local, K])
 * and its epilogue stores the column block [rank * n_local, (rank + 1) * n_local) into EVERY rank's C —
 * c_of_rank[r] is the address, valid on this device, of rank r's full row-major C[M, ranks * n_local] (its own
 * buffer for r == rank, NVLink peer mappings for the others, e.g. from torch symmetric memory). The stores are TMA
 * stores issued tile by tile while the next tile is being multiplied; no load ever targets a peer and nothing is
 * multicast. Every C is complete once all ranks' kernels have finished their stores: see sync_of_rank below.
 * n_local must be a multiple of 128 bytes of output (64 columns of bf16/f16, 32 of f32); all addresses and pitches
 * 16-byte aligned. `c_of_rank` is a HOST array of `ranks` pointers (ranks <= 8).
 *   sync_of_rank  HOST array of `ranks` addresses (valid on this device) of each rank's 9 32-bit sync words — 8
 *                 flags and an arrival counter, zero before the first product — or NULL. When given, the kernel's
 *                 last CTA tells every peer that this rank's stores of product number `epoch` have landed and waits
 *                 (at most about two seconds; on expiry the status word reports KRN_B200_ERR_DEVICE_TIMEOUT and the
 *                 kernel returns) until every peer has said the same: when the kernel completes, this rank's C holds
 *                 all column blocks and no separate barrier is needed. All ranks must then call with the same
 *                 `epoch`, one more for every product (any start above zero). With NULL the caller runs its own
 *                 cross-rank barrier after the call.
 * No counterpart in the reference, which has no multi-device path. */
int krn_b200_gemm_tn_gather(int ab_type, int c_type, const void* a, const void* b, void* const* c_of_rank, int ranks,
                            int rank, int64_t m, int64_t n_local, int64_t k, int64_t lda, int64_t ldb, int64_t ldc,
                            void* const* sync_of_rank, uint32_t epoch, void* stream);

/* C[M,N] = sum over 128-wide K blocks kb of  sa[m,kb] * sb[n/128,kb] * (A8[m, kb] . B8[n, kb]),
 * A8/B8 e4m3fn codes (one byte each, K-major), sa f32 [M, ceil(K/128)] (one scale per 1x128 block of A,
 * the reference's FP8FN block format, src/krn/data/formats.py:157-164), sb f32 [ceil(N/128), ceil(K/128)]
 * (one per 128x128 block of B). Partial sums of each K block are formed by the tensor cores and scaled
 * when they are added to the f32 accumulator — "a coarse scale ... is applied to the partial sums outside
 * the unit" (src/krn/facts/targets.py:127-138); operands are never dequantised in memory. Output type
 * c_type as above. K must be a multiple of 16 (TMA pitch); lds* in elements. */
int krn_b200_gemm_fp8_blockscaled_tn(int c_type, const void* a, const float* sa, const void* b, const float* sb,
                                     void* c, int64_t m, int64_t n, int64_t k, int64_t lda, int64_t ldb,
                                     int64_t ldc, int64_t ldsa, int64_t ldsb, void* stream);

/* C[M,N] = sum over 32-wide K blocks kb of  2^(sa[m,kb] - 127) * 2^(sb[n,kb] - 127) * (A8[m, kb] . B8[n, kb]):
 * the product of two matrices in the reference's MXFP8 block format — e4m3fn codes with one e8m0 (power-of-two) scale
 * byte per 1 x 32 block of a row (src/krn/data/formats.py:138-144; `QMatrix[MXFP8]`, src/krn/frontend/memory.py:255-269,
 * whose `@` the reference declares and does not implement, :173-193). The scale factors are operands of the tensor-core
 * instruction itself (tcgen05.mma kind::mxf8f6f4.block_scale reads them from tensor memory): nothing is dequantised and
 * no partial sum is rescaled outside the unit.
 *   a, b    e4m3fn codes, K-major: a [M, K], b [N, K]; lda / ldb in elements, multiples of 16
 *   sa, sb  e8m0 bytes: sa [M, K / 32], sb [N, K / 32]; ldsa / ldsb row pitches in BYTES; addresses and pitches
 *           multiples of 4. A small kernel first rewrites both scale matrices into the 512-byte atoms tcgen05.cp copies
 *           (128 rows x 4 bytes per K step), in scratch memory that lives for the call; the product fetches them by TMA
 *   K       a multiple of 128 (four scale blocks per step); M, N ragged as in krn_b200_gemm_tn
 *   c_type  KRN_B200_BF16, KRN_B200_F16 or KRN_B200_F32; ldc in elements */
int krn_b200_gemm_mxfp8_tn(int c_type, const void* a, const uint8_t* sa, const void* b, const uint8_t* sb, void* c, int64_t m,
                           int64_t n, int64_t k, int64_t lda, int64_t ldb, int64_t ldc, int64_t ldsa, int64_t ldsb,
                           void* stream);

/* C[M,N] = alpha * sum over 16-wide K blocks kb of  sa[m,kb] * sb[n,kb] * (A4[m, kb] . B4[n, kb]): the product of two
 * matrices in the reference's NVFP4 block format — e2m1 codes packed two per byte (low nibble first), one e4m3 scale
 * byte per 1 x 16 block of a row, one f32 tensor scale per matrix (src/krn/data/formats.py:147-154; `QMatrix[NVFP4]`,
 * src/krn/frontend/memory.py:255-269, whose `@` the reference declares and does not implement, :173-193). The block
 * scales are operands of the tensor-core instruction (tcgen05.mma kind::mxf4nvf4.block_scale.scale_vec::4X); alpha,
 * the product of the two tensor scales, multiplies the finished accumulator.
 *   a, b    packed e2m1 codes, K-major: a [M, K / 2] bytes, b [N, K / 2] bytes; lda / ldb row pitches in BYTES,
 *           multiples of 16
 *   sa, sb  e4m3 bytes (sign bit clear): sa [M, K / 16], sb [N, K / 16]; ldsa / ldsb row pitches in bytes; addresses and
 *           pitches multiples of 16
 *   K       the number of codes per row, a multiple of 256; M, N ragged as in krn_b200_gemm_tn
 *   c_type  KRN_B200_BF16, KRN_B200_F16 or KRN_B200_F32; ldc in elements */
int krn_b200_gemm_nvfp4_tn(int c_type, const void* a, const uint8_t* sa, const void* b, const uint8_t* sb, float alpha, void* c,
                           int64_t m, int64_t n, int64_t k, int64_t lda, int64_t ldb, int64_t ldc, int64_t ldsa, int64_t ldsb,
                           void* stream);

/* C[M,N] = sum over 32-wide K blocks kb of  2^(sa[m,kb] - 127) * 2^(sb[n,kb] - 127) * (A4[m, kb] . B4[n, kb]): the product
 * of two matrices in the reference's MXFP4 block format — e2m1 codes packed two per byte (low nibble first), one e8m0
 * scale byte per 1 x 32 block of a row (src/krn/data/formats.py:129-135; `QMatrix[MXFP4]`, whose `@` the reference
 * declares and does not implement). tcgen05.mma kind::mxf4.block_scale.scale_vec::2X.
 *   a, b    packed e2m1 codes, K-major: a [M, K / 2] bytes, b [N, K / 2] bytes; lda / ldb row pitches in BYTES,
 *           multiples of 16
 *   sa, sb  e8m0 bytes: sa [M, K / 32], sb [N, K / 32]; ldsa / ldsb row pitches in bytes; addresses and pitches
 *           multiples of 16
 *   K       the number of codes per row, a multiple of 512; M, N ragged as in krn_b200_gemm_tn
 *   c_type  KRN_B200_BF16, KRN_B200_F16 or KRN_B200_F32; ldc in elements */
int krn_b200_gemm_mxfp4_tn(int c_type, const void* a, const uint8_t* sa, const void* b, const uint8_t* sb, void* c, int64_t m,
                           int64_t n, int64_t k, int64_t lda, int64_t ldb, int64_t ldc, int64_t ldsa, int64_t ldsb,
                           void* stream);

/* The block-scaled FP8 product sharded by output columns with the all-gather of the columns done by the kernel's
 * epilogue, exactly as krn_b200_gemm_tn_gather does for the 16-bit product: rank `rank` multiplies A by ITS rows of B
 * (b: [n_local, K] codes, sb: [n_local / 128, ceil(K/128)] scales) and stores the column block
 * [rank * n_local, (rank + 1) * n_local) into every rank's C (c_of_rank: a HOST array of `ranks` addresses valid on
 * this device; TMA stores over NVLink, no peer loads, nothing multicast). n_local must be a multiple of 128.
 * sync_of_rank / epoch as in krn_b200_gemm_tn_gather (NULL: the caller runs a cross-rank barrier after the call).
 * No counterpart in the reference. */
int krn_b200_gemm_fp8_blockscaled_tn_gather(int c_type, const void* a, const float* sa, const void* b, const float* sb,
                                            void* const* c_of_rank, int ranks, int rank, int64_t m, int64_t n_local,
                                            int64_t k, int64_t lda, int64_t ldb, int64_t ldc, int64_t ldsa, int64_t ldsb,
                                            void* const* sync_of_rank, uint32_t epoch, void* stream);

/* Flash-attention forward: O = softmax(scale * Q K^T [+ causal mask]) V per (batch, q head), the statement
 * sequence of the reference's example kernel (examples/04_libraries/08_flash_attention.py:44-59): scores
 * carry scale_log2 = log2(e)/sqrt(d) so every exponential is exp2, masked scores take -1.0e30, running
 * max / sum in f32, P rounded to the storage type before P·V, output (acc / l) rounded once.
 *   q, o : [batch, q_heads, seq_q, d]    k, v : [batch, kv_heads, seq_kv, d]   (bf16, d contiguous)
 *   q_heads % kv_heads == 0 (grouped-query attention: q head h reads kv head h / (q_heads / kv_heads))
 *   causal != 0: key position j is visible to query position i when j <= i (`kpos <= qpos`, as the example masks)
 *   *_stride_b / *_stride_h / *_stride_s: element strides of batch, head and sequence axes.
 * d must be 64 or 128. */
int krn_b200_attn_fwd(int type, const void* q, const void* k, const void* v, void* o, int64_t batch, int64_t q_heads,
                      int64_t kv_heads, int64_t seq_q, int64_t seq_kv, int64_t d, float scale_log2, int causal,
                      const int64_t* q_strides, const int64_t* k_strides, const int64_t* v_strides,
                      const int64_t* o_strides, void* stream);

/* Bytes of caller workspace krn_b200_attn_decode_fp8_paged needs for these extents (split-KV partials). */
int64_t krn_b200_attn_decode_workspace_bytes(int64_t batch, int64_t q_heads, int64_t d, int64_t max_context);

/* Decode attention (one query token per sequence) over a paged e4m3 KV cache. The reference has no
 * implementation of this (roadmap item "Paged attention"); the arithmetic follows the flash-attention
 * statements above with K and V dequantised as code * scale.
 *   q  bf16 [batch, q_heads, d]         o  bf16 [batch, q_heads, d]
 *   k_pages, v_pages  e4m3 codes [num_pages, page_size, kv_heads, d]
 *   num_pages   pages in the pool. It bounds every fetch: a page id outside [0, num_pages) is never read — its 64
 *               tokens read as zero codes (K = V = 0) and KRN_B200_ERR_DEVICE_INDEX is left in the status word.
 *   page_table  int32 [batch, max_pages_per_seq]: page ids of each sequence in order; entries past a sequence's
 *               context are never looked at
 *   context_len int32 [batch]; values are clamped into [0, max_context]; a sequence of length 0 gets zeros
 *   k_scale, v_scale  f32 [batch, kv_heads]
 *   workspace   at least krn_b200_attn_decode_workspace_bytes(...) bytes, 16-byte aligned; contents need no
 *               preparation (a call reads back only the partials it wrote) */
int krn_b200_attn_decode_fp8_paged(const void* q, const void* k_pages, const void* v_pages, const int32_t* page_table,
                                   const int32_t* context_len, const float* k_scale, const float* v_scale, void* o,
                                   int64_t batch, int64_t q_heads, int64_t kv_heads, int64_t d, int64_t page_size,
                                   int64_t num_pages, int64_t max_pages_per_seq, int64_t max_context, float scale_log2,
                                   void* workspace, int64_t workspace_bytes, void* stream);

/* The same computation as krn_b200_attn_decode_fp8_paged, for callers that cannot allocate device memory when
 * they need it — a serving loop whose KV-cache pool owns all remaining HBM, a plugin confined to another
 * runtime's memory budget, a path where cudaMalloc's implicit synchronisation is not allowed. The split-KV
 * partials go to a 16 MiB array built into the library image (each GPU that loads the library holds it until the
 * process exits) instead of a caller workspace; the entry point calls no allocating routine at all.
 *   limit    batch * q_heads * ceil(max_context / 1024) * 130 floats must fit 16 MiB (4 Mi floats); larger
 *            problems are refused with KRN_B200_ERR_WORKSPACE — use the workspace variant for those.
 *   set-up   the first call on each device resolves the array's device address (cudaGetSymbolAddress); make
 *            that first call outside any stream capture.
 *   sharing  every call on a device uses the same array, which keeps the previous call's partials. Nothing in
 *            it has to start at zero (a call reads back only what it wrote), but two calls whose kernels overlap
 *            on the GPU — different streams, or a graph replayed concurrently — race on it: serialise them.
 *   status   a bounded device-side wait that expires (or an out-of-range page id) is recorded in the status word
 *            only if an earlier call of another entry point created that word on this device; this entry point
 *            does not create it.
 * This entry point has no counterpart in the reference. */
int krn_b200_attn_decode_fp8_paged_noalloc(const void* q, const void* k_pages, const void* v_pages,
                                           const int32_t* page_table, const int32_t* context_len, const float* k_scale,
                                           const float* v_scale, void* o, int64_t batch, int64_t q_heads,
                                           int64_t kv_heads, int64_t d, int64_t page_size, int64_t num_pages,
                                           int64_t max_pages_per_seq, int64_t max_context, float scale_log2,
                                           void* stream);

/* Copy this rank's column block C_local[M, n_local] into columns [col0, col0 + n_local) of the row-major
 * C_full[M, N] (ld in elements, elem_bytes 2 or 4). Used after the NCCL all-gather of GEMM output column
 * blocks to lay the gathered slabs out as one row-major matrix. No counterpart in the reference (it has no
 * multi-device path). */
int krn_b200_scatter_columns(const void* slabs, void* c_full, int64_t m, int64_t n_local, int64_t ranks,
                             int64_t ld_full, int elem_bytes, void* stream);

/* Pitched copy of `rows` rows of `row_bytes` bytes between device memory and page-locked host memory (either
 * direction, or device to device), enqueued on `stream`: cudaMemcpy2DAsync behind this library's status codes. Used by
 * the host-operand streaming path to return column slabs of a row-major result into the caller's host matrix. The
 * reference copies whole tensors only (src/krn/runtime/cuda_backend.py:205-248). */
int krn_b200_copy_2d(void* dst, int64_t dst_pitch_bytes, const void* src, int64_t src_pitch_bytes, int64_t row_bytes,
                     int64_t rows, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* KRN_B200_H */
