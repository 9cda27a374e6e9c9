/*
 * quant_ops_b200 -- C ABI of the B200 (sm_100a) W4A4 hot path.
 *
 * Plain pointers and sizes only; no torch types.  Every entry point returns a
 * qo_status (0 = success) and never aborts the process.  After a non-zero
 * return, qo_last_error() gives a human readable reason (thread-local).
 *
 * Unless a function says otherwise, data pointers are DEVICE pointers on the
 * current CUDA device and the work is enqueued on `stream` (a cudaStream_t
 * passed as void*, NULL = the default stream) without synchronising.
 *
 * Each declaration names the interface of the reference project
 * (libarry/quant_ops) that it stands in for, as path:line inside that project.
 *
 * Wire format of packed int4 ("offset binary", shared by all entry points):
 * nibble i (bits 4i..4i+3) of 32-bit word p of a row holds code[8p+i] + 8,
 * codes in [-8, 7].
 */
#ifndef QUANT_OPS_B200_H_
#define QUANT_OPS_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(_WIN32)
#define QO_API __declspec(dllexport)
#else
#define QO_API __attribute__((visibility("default")))
#endif

typedef enum qo_status {
  QO_OK = 0,
  QO_ERR_INVALID_ARGUMENT = 1, /* bad shape, null pointer, misaligned pointer, unknown enum value */
  QO_ERR_UNSUPPORTED = 2,      /* valid request that this build has no kernel for */
  QO_ERR_CUDA = 3,             /* a CUDA runtime/driver call failed; message carries the CUDA error string */
  QO_ERR_NO_DEVICE = 4,        /* no sm_100 device is current */
  QO_ERR_WORKSPACE = 5,        /* workspace missing or too small */
  QO_ERR_DEVICE_TIMEOUT = 6    /* a bounded device-side wait ran out; outputs are not valid */
} qo_status;

typedef enum qo_dtype {
  QO_F32 = 0,
  QO_F16 = 1,
  QO_BF16 = 2
} qo_dtype;

/* Library version as major*10000 + minor*100 + patch. */
QO_API int qo_version(void);
/* Static string for a status code. */
QO_API const char* qo_status_string(int status);
/* Message of the last failure on the calling thread ("" if none). */
QO_API const char* qo_last_error(void);

/*
 * (M, N) with M*N == n, M <= N, from the smallest a >= ceil(sqrt(n)) such that a*a - n is a square.
 * Stands in for: get_decompose_dim, src/quant_ops/utils/decompose.py:11-38.
 * Differs in one point: n = 2 (mod 4) has no such factorisation and the reference loops forever;
 * this returns QO_ERR_INVALID_ARGUMENT.  Host-only, needs no GPU.
 */
QO_API int qo_get_decompose_dim(int64_t n, int64_t* m_out, int64_t* n_out);

/*
 * FlatQuant per-token dynamic int4 quantizer.
 * Stands in for: cuda_kronecker_quant_int8, src/quant_ops/ops/quantization/flatquant/kernels/cuda_quant_kernel.cu:316-390
 * (dispatcher op quant_ops::flatquant_dynamic_quantize, same file :395-413) with the numerics of
 * flatquant_pytorch, src/quant_ops/ops/quantization/flatquant/ops.py:78-130.
 *
 *   x       [tokens, m*n] in `in_dtype`, row stride `ldx` elements (ldx >= m*n)
 *   left    [m, m], right [n, n], contiguous, same dtype as x
 *   codes   pack_int32 == 0: int8  [tokens, m*n]     (contiguous)
 *           pack_int32 != 0: int32 [tokens, m*n / 8] (contiguous; m*n must be a multiple of 8)
 *   scales  [tokens] in `scale_dtype`; the value is the reference's scale, i.e. already rounded to `in_dtype`
 *
 * Per token: Z = round(L^T . round(X . R)), scale = max(round(|min Z| * c), round(max Z * c)) / 7 (rounded,
 * floored at 1e-8), code = clamp(rint(round(Z / scale)), -8, 7); "round" = to in_dtype, nearest even.
 * tokens == 0 is a no-op.
 */
QO_API int qo_flatquant_quantize(const void* x, int64_t ldx, const void* left, const void* right,
                                 void* codes, void* scales, int64_t tokens, int m, int n,
                                 float clip_ratio, int in_dtype, int pack_int32, int scale_dtype,
                                 void* stream);

/*
 * The Kronecker transform alone: z[t] = round(L^T . round(X[t] . R)) as float32 [tokens, m*n] (values are
 * representable in in_dtype).  Stands in for the first two lines of cuda_kronecker_quant_int8,
 * src/quant_ops/ops/quantization/flatquant/kernels/cuda_quant_kernel.cu:337-339 (oracle: flatquant/ops.py:99-103).
 */
QO_API int qo_flatquant_transform(const void* x, int64_t ldx, const void* left, const void* right, float* z,
                                  int64_t tokens, int m, int n, int in_dtype, void* stream);

/*
 * Synchronises `stream` and reports whether any kernel of this library (qo_int4_matmul_static included) gave up on
 * a bounded device-side wait since the last call (QO_ERR_DEVICE_TIMEOUT, and the flag is cleared) -- the
 * reference's counterpart is the cudaGetLastError check after its per-call synchronise, cuda_quant_kernel.cu:380-387.
 * Allocates nothing.
 */
QO_API int qo_device_status(void* stream);

/*
 * Exercises the failure path on purpose, harmlessly: one warp waits (limit 1024 polls, well under a millisecond) on
 * a barrier that nothing arrives on, records a site code in the device status word and returns.  The next
 * qo_device_status() then reports QO_ERR_DEVICE_TIMEOUT once, and the device stays fully usable.  No trap, no
 * fault.  It has no counterpart in the reference, whose only check is cudaGetLastError after a blocking synchronise
 * (cuda_quant_kernel.cu:380-387); it exists so that a host can test its own handling of a timed-out kernel.
 */
QO_API int qo_selftest_wait_timeout(void* stream);

/*
 * int4 codes (int8 or packed) times per-token scale -> float32 [tokens, features].
 * Stands in for: dequantize_int4, src/quant_ops/ops/quantization/flatquant/ops.py:156-178.
 */
QO_API int qo_dequantize_int4(const void* codes, const void* scales, float* out, int64_t tokens,
                              int64_t features, int packed_int32, int scale_dtype, void* stream);

/*
 * Bytes of device scratch qo_int4_matmul wants for this problem (0 if it needs none).
 * New; the reference has no workspace.
 */
QO_API size_t qo_int4_matmul_workspace_bytes(int64_t tokens, int64_t k, int64_t n_out);

/*
 * Packed-int4 GEMM with int32 accumulation and a scale epilogue:
 *   out[t, j] = to_out_dtype( (float(sum_k A[t,k] * B[k,j]) * scale_a[t]) * scale_b[j] )
 * Stands in for: cuda_int4_matmul, src/quant_ops/ops/quantization/int4_matmul/kernels/cuda_int4_matmul_kernel.cu:130-189
 * (dispatcher op quant_ops::int4_matmul, same file :194-214); oracle int4_matmul_pytorch,
 * src/quant_ops/ops/quantization/int4_matmul/ops.py:69-103.
 *
 *   a          int32 [tokens, k/8], row stride `lda` words
 *   b          int32, logical shape [k/8, n_out], element (kp, j) at b[kp*b_stride_k + j*b_stride_n];
 *              the reference layout is (n_out, 1); the transposed view of a [n_out, k/8] weight is (1, k/8)
 *   scale_a    float32 [tokens], scale_b float32 [n_out]
 *   out        [tokens, n_out] contiguous, QO_F16 (the reference's output type) or QO_BF16
 *   acc_out    optional int32 [tokens, n_out]: raw accumulators, for bit-exact checks (NULL to skip)
 *   workspace  device scratch of at least qo_int4_matmul_workspace_bytes(); NULL lets the library use a
 *              per-device buffer it allocates (and keeps) itself.  That buffer is shared by every NULL-workspace
 *              call on the device: issue such calls on one stream at a time.  Callers with several streams or
 *              threads pass their own workspace per call (the torch binding does).
 */
QO_API int qo_int4_matmul(const int32_t* a, int64_t lda, const int32_t* b, int64_t b_stride_k,
                          int64_t b_stride_n, const float* scale_a, const float* scale_b, void* out,
                          int out_dtype, int64_t tokens, int64_t k, int64_t n_out, int32_t* acc_out,
                          void* workspace, size_t workspace_bytes, void* stream);

/*
 * qo_int4_matmul without any allocation.  It has no counterpart in the reference.
 *
 * For hosts that cannot let a library allocate device memory: a serving process that gave all of the GPU's memory
 * to its own pool at start-up has none left for a late cudaMalloc, and a cudaMalloc inside a serving step would
 * synchronise the device.  The scratch for the widened operands lives in a device array inside the library, so the
 * call allocates nothing (no cudaMalloc, no cudaFree, no allocating library routine), and every GPU that loads the
 * library holds qo_int4_matmul_static_max_bytes() (8 MiB) until the process exits.
 *
 * Limits and rules:
 *   - tokens*k bytes (rounded up to 256) + ceil(n_out/256)*256 * ceil(k/128)*128 bytes (the weights are held in
 *     whole blocks of 256 channels x 128 values) must not exceed qo_int4_matmul_static_max_bytes(); larger
 *     problems return QO_ERR_WORKSPACE.  Only the shapes of the tcgen05 kernel are served (k % 16 == 0,
 *     n_out % 8 == 0, b with unit stride along k or along n_out); others return QO_ERR_UNSUPPORTED.
 *   - the first call on a device looks up the array's device address; make it before any stream capture.
 *   - all calls share the one array: calls that may overlap on the GPU (different streams) race; serialise them.
 *   - same arithmetic and same results as qo_int4_matmul (fp16 or bf16 output, no accumulator dump, no bias).
 */
QO_API size_t qo_int4_matmul_static_max_bytes(void);
QO_API int qo_int4_matmul_static(const int32_t* a, int64_t lda, const int32_t* b, int64_t b_stride_k,
                                 int64_t b_stride_n, const float* scale_a, const float* scale_b, void* out,
                                 int out_dtype, int64_t tokens, int64_t k, int64_t n_out, void* stream);

/*
 * Fused W4A4 linear layer: quantize activations (as qo_flatquant_quantize with packing) and multiply by
 * packed weights w [n_out, m*n/8] (K contiguous) with per-output-channel scales.
 * Stands in for the composition a user of the reference writes,
 *   int4_matmul(*flatquant_dynamic_quantize(x, L, R, c, True), w_packed.t(), s_a, s_w),
 * whose layer form is AscendW4A4FlatQuantDynamicLinearMethod.apply, w4a4_flatquant_dynamic.py:168-266.
 *
 *   out        [tokens, n_out] in out_dtype (QO_F16 / QO_BF16); bias (same dtype, [n_out]) may be NULL
 *   workspace  at least qo_w4a4_linear_workspace_bytes(); NULL = library-owned buffer
 */
QO_API size_t qo_w4a4_linear_workspace_bytes(int64_t tokens, int64_t k, int64_t n_out);
QO_API int qo_w4a4_linear(const void* x, int64_t ldx, const void* left, const void* right,
                          const int32_t* w_packed, const float* w_scale, const void* bias, void* out,
                          int64_t tokens, int m, int n, int64_t n_out, float clip_ratio, int in_dtype,
                          int out_dtype, void* workspace, size_t workspace_bytes, void* stream);

/*
 * Fused layer whose outputs are ALL-GATHERED over the row-sharding ranks by the GEMM itself: rank r holds rows
 * [row_offset, row_offset + tokens) of a layer input that is split by rows over the GPUs of one node, and the kernel's
 * epilogue stores its output rows straight into every rank's copy of the gathered output (plain stores to peer memory
 * over NVLink), this rank's own copy included.  No collective kernel runs and no SM is taken from the GEMM.
 * The reference has no counterpart (it is single-GPU); this serves the optional output all-gather of a row-sharded
 * deployment.  Only prefill-sized products take this route (at least 48 tiles of 256 x 256, k a multiple of 256, n_out
 * a multiple of 16); anything else returns QO_ERR_UNSUPPORTED and the caller gathers with its collective library.
 *
 *   dsts        host array of n_dst (1 .. 8) device pointers to buffers [total_rows, n_out] in out_dtype, 32-byte aligned:
 *               this GPU's own buffer and the peers' buffers as mapped into this process (qo_peer_open)
 *   row_offset  first row of this rank's slice in those buffers
 * The caller orders the ranks: a destination buffer may be read once every rank's call has completed on its stream
 * (a barrier across the ranks after a stream synchronise), and must not be rewritten before every reader is done.
 */
QO_API int qo_w4a4_linear_gather(const void* x, int64_t ldx, const void* left, const void* right,
                                 const int32_t* w_packed, const float* w_scale, const void* bias, void* const* dsts,
                                 int n_dst, int64_t row_offset, int64_t tokens, int m, int n, int64_t n_out,
                                 float clip_ratio, int in_dtype, int out_dtype, void* workspace, size_t workspace_bytes,
                                 void* stream);
/*
 * Sharing a device buffer with the other processes of the node (CUDA IPC), for the destinations above.
 * qo_peer_export: handle (64 bytes) of the allocation that contains ptr, and ptr's offset inside it.
 * qo_peer_open:   maps an allocation exported by ANOTHER process into this one (peer access is enabled as needed);
 *                 *base + offset is the exported pointer.  qo_peer_close unmaps it (after the last kernel using it).
 */
QO_API int qo_peer_export(const void* ptr, void* handle64, int64_t* offset);
QO_API int qo_peer_open(const void* handle64, void** base);
QO_API int qo_peer_close(void* base);
/* bytes from this GPU's memory into a mapped peer buffer (or any device buffer) on `stream`: a copy-engine transfer that
 * takes no SM, for gathers that should run beside the kernels of another stream */
QO_API int qo_peer_copy(void* dst, const void* src, size_t bytes, void* stream);

/*
 * Layer form with weights prepared once.  The weights of a layer do not change between calls, so a host that can
 * spend about k bytes per output channel keeps them widened to int8 (qo_prepare_weights, at load time; the buffer is
 * opaque: the GEMM's own layout, blocks of 256 output channels x 128 values, padded to whole blocks) and the
 * per-call work shrinks to: quantize the activations straight to int8 codes, then the tensor-core GEMM; no operand
 * is rewritten per call.  Results are identical to qo_w4a4_linear.  Calls with at most 32 tokens read the packed
 * weights instead (half the bytes), so both buffers are passed.
 * Load-time counterpart in the reference: process_weights_after_loading, w4a4_flatquant_dynamic.py:268-304 (which
 * packs; the int8 copy is this library's addition for sm_100a, where the tensor cores take int8).
 *
 *   prepared   qo_prepared_weights_bytes(n_out, k) bytes, 256-byte aligned, written by qo_prepare_weights
 *   workspace  at least qo_w4a4_linear_prepared_workspace_bytes(); NULL = library-owned buffer
 */
QO_API size_t qo_prepared_weights_bytes(int64_t n_out, int64_t k);
QO_API int qo_prepare_weights(const int32_t* w_packed, void* prepared, int64_t n_out, int64_t k, void* stream);
QO_API size_t qo_w4a4_linear_prepared_workspace_bytes(int64_t tokens, int64_t k, int64_t n_out);
QO_API int qo_w4a4_linear_prepared(const void* x, int64_t ldx, const void* left, const void* right,
                                   const int32_t* w_packed, const void* prepared, const float* w_scale,
                                   const void* bias, void* out, int64_t tokens, int m, int n, int64_t n_out,
                                   float clip_ratio, int in_dtype, int out_dtype, void* workspace,
                                   size_t workspace_bytes, void* stream);

/*
 * int8 codes [rows, features] -> packed int32 [rows, features/8].
 * Stands in for: pack_int4_to_int32, src/quant_ops/ops/quantization/int4_matmul/ops.py:23-45.
 */
QO_API int qo_pack_int4(const int8_t* codes, int32_t* packed, int64_t rows, int64_t features, void* stream);
/* Inverse.  Stands in for: unpack_int32_to_int4, src/quant_ops/ops/quantization/int4_matmul/ops.py:48-66. */
QO_API int qo_unpack_int4(const int32_t* packed, int8_t* codes, int64_t rows, int64_t features, void* stream);

/*
 * Per-output-channel symmetric int4 weight quantizer: scale = max(absmax(row)/7, 1e-8),
 * code = clamp(rint(w/scale), -8, 7), written packed [rows, k/8].  Input float32 [rows, k].
 * New (the reference receives pre-quantized weights, w4a4_flatquant_dynamic.py:118); it is the weight-side
 * of the harness inputs and of model loading.
 */
QO_API int qo_quantize_weights_int4(const float* w, int32_t* packed, float* scale, int64_t rows,
                                    int64_t k, void* stream);

/*
 * Host-buffer form of the quantizer: x, codes and scales are HOST pointers (pinned or pageable); the call
 * copies rows to the device in slices, quantizes, copies results back, overlapping the three on internal
 * streams, and returns when the outputs are complete.  left/right are host pointers too.
 * This is the call a CPU-resident caller of the reference (tensors moved with .cuda() inside
 * flatquant_cuda, src/quant_ops/ops/quantization/flatquant/ops.py:54-75) maps to.
 */
QO_API int qo_flatquant_quantize_host(const void* x_host, const void* left_host, const void* right_host,
                                      void* codes_host, void* scales_host, int64_t tokens, int m, int n,
                                      float clip_ratio, int in_dtype, int pack_int32, int scale_dtype);

/* Number of kernels this library has launched in this process (all threads); used by the benchmark. */
QO_API uint64_t qo_kernel_launch_count(void);
/* Which quantizer kernel the last qo_flatquant_quantize on this thread used: 0 none, 1 generic SIMT, 2 tcgen05. */
QO_API int qo_last_quantizer_path(void);
/* Which GEMM kernel the last qo_int4_matmul on this thread used: 0 none, 1 generic SIMT, 2 tcgen05,
 * 3 weight-streaming kernel for 1 .. 32 rows (automatic policy only). */
QO_API int qo_last_gemm_path(void);
/*
 * Kernel selection for the calling thread: 0 = automatic (tcgen05 kernel when the shape has one, else the
 * generic SIMT kernel), 1 = generic SIMT kernels only, 2 = tcgen05 kernels only (QO_ERR_UNSUPPORTED when the
 * shape has none), 3 = as 2 but without the CTA-pair GEMM kernel (large products then run on the single-CTA
 * tcgen05 kernels).  All kinds compute the same results; the switch exists so that tests can check each.
 */
QO_API int qo_set_kernel_policy(int policy);
/* Free the per-device buffers the library allocated itself. */
QO_API int qo_release_workspaces(void);

#ifdef __cplusplus
}
#endif
#endif /* QUANT_OPS_B200_H_ */
