// Shared host/device helpers for the kernels behind the C ABI.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <atomic>
#include <cstdarg>
#include <cstdint>
#include <cstdio>

#include "../../include/quant_ops_b200.h"

namespace qo {

// ---- error reporting -------------------------------------------------------------------------
void set_error(const char* fmt, ...);  // stores a thread-local message (c_abi.cu)
void clear_error();
extern std::atomic<uint64_t> g_launches;

inline int fail(int status, const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof buf, fmt, ap);
  va_end(ap);
  set_error("%s", buf);
  return status;
}

#define QO_CUDA_TRY(expr)                                                                   \
  do {                                                                                      \
    cudaError_t _e = (expr);                                                                \
    if (_e != cudaSuccess) {                                                                \
      return ::qo::fail(QO_ERR_CUDA, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e), \
                        __FILE__, __LINE__);                                                \
    }                                                                                       \
  } while (0)

// number of SMs of a device, queried once per device (the attribute query costs about a microsecond per call)
inline int sm_count(int dev) {
  static std::atomic<int> cached[64];
  int v = (dev >= 0 && dev < 64) ? cached[dev].load(std::memory_order_relaxed) : 0;
  if (v > 0) return v;
  if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) {
    (void)cudaGetLastError();
    return 148;
  }
  if (dev >= 0 && dev < 64) cached[dev].store(v, std::memory_order_relaxed);
  return v;
}

inline int check_launch(const char* what) {
  cudaError_t e = cudaPeekAtLastError();
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    return fail(QO_ERR_CUDA, "launch of %s failed: %s", what, cudaGetErrorString(e));
  }
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return QO_OK;
}

// ---- working-dtype arithmetic ----------------------------------------------------------------
// The reference evaluates every step in the activation dtype.  For the 16-bit types that is "compute in
// float32, round the result to the 16-bit type"; these helpers are that rounding.
template <typename T>
struct DT;
template <>
struct DT<float> {
  static constexpr int id = QO_F32;
  __device__ __forceinline__ static float load(const float* p) { return *p; }
  __device__ __forceinline__ static void store(float* p, float v) { *p = v; }
  __device__ __forceinline__ static float rnd(float v) { return v; }
  __device__ __forceinline__ static float floor_scale() { return 1e-8f; }
};
template <>
struct DT<__half> {
  static constexpr int id = QO_F16;
  __device__ __forceinline__ static float load(const __half* p) { return __half2float(*p); }
  __device__ __forceinline__ static void store(__half* p, float v) { *p = __float2half_rn(v); }
  __device__ __forceinline__ static float rnd(float v) { return __half2float(__float2half_rn(v)); }
  __device__ __forceinline__ static float floor_scale() { return 0.f; }  // 1e-8 rounds to 0 in fp16
};
template <>
struct DT<__nv_bfloat16> {
  static constexpr int id = QO_BF16;
  __device__ __forceinline__ static float load(const __nv_bfloat16* p) { return __bfloat162float(*p); }
  __device__ __forceinline__ static void store(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }
  __device__ __forceinline__ static float rnd(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
  __device__ __forceinline__ static float floor_scale() { return __bfloat162float(__float2bfloat16_rn(1e-8f)); }
};

// scale of one token from its extreme transformed values (already rounded to the working dtype)
template <typename T>
__device__ __forceinline__ float token_scale(float zmin, float zmax, float clip) {
  float hi = DT<T>::rnd(zmax * clip);
  float lo = fabsf(DT<T>::rnd(zmin * clip));
  float top = fmaxf(lo, hi);
  float s = DT<T>::rnd(__fdiv_rn(top, 7.0f));
  return fmaxf(s, DT<T>::floor_scale());
}

// int4 code of one transformed value; `s` is the token scale.  s == 0 happens only in fp16 (the 1e-8 floor rounds
// to 0 there): the reference then divides by zero, +-inf clamps to 7 / -8 and 0/0 is taken as code 0.
template <typename T>
__device__ __forceinline__ int quantize_one(float z, float s) {
  if (s == 0.f) return z > 0.f ? 7 : (z < 0.f ? -8 : 0);
  float q = DT<T>::rnd(__fdiv_rn(z, s));
  q = fminf(fmaxf(rintf(q), -8.f), 7.f);  // rintf rounds half to even
  return (int)q;
}

__device__ __forceinline__ void store_scale(void* scales, int64_t t, float s, int scale_dtype) {
  if (scale_dtype == QO_F32) {
    reinterpret_cast<float*>(scales)[t] = s;
  } else if (scale_dtype == QO_F16) {
    reinterpret_cast<__half*>(scales)[t] = __float2half_rn(s);
  } else {
    reinterpret_cast<__nv_bfloat16*>(scales)[t] = __float2bfloat16_rn(s);
  }
}

__device__ __forceinline__ float load_scale(const void* scales, int64_t t, int scale_dtype) {
  if (scale_dtype == QO_F32) return reinterpret_cast<const float*>(scales)[t];
  if (scale_dtype == QO_F16) return __half2float(reinterpret_cast<const __half*>(scales)[t]);
  return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(scales)[t]);
}

inline size_t dtype_size(int dt) { return dt == QO_F32 ? 4 : 2; }
inline bool dtype_ok(int dt) { return dt == QO_F32 || dt == QO_F16 || dt == QO_BF16; }

// ---- kernel launchers implemented in the .cu files ---------------------------------------------
int launch_flatquant_generic(const void* x, int64_t ldx, const void* left, const void* right, void* codes,
                             void* scales, int64_t tokens, int m, int n, float clip, int in_dtype, int pack,
                             int scale_dtype, cudaStream_t stream);
// returns QO_ERR_UNSUPPORTED (without setting an error) when the shape has no tcgen05 kernel
int launch_flatquant_sm100(const void* x, int64_t ldx, const void* left, const void* right, void* codes,
                           void* scales, int64_t tokens, int m, int n, float clip, int in_dtype, int pack,
                           int scale_dtype, cudaStream_t stream);
bool flatquant_sm100_supported(int64_t ldx, int m, int n, int in_dtype, const void* x, const void* left, const void* right,
                               float clip);
// mode: 0 int8 codes, 1 packed codes, 2 transform only (float32 Z written to `codes`)
int launch_flatquant_sm100_mode(int mode, const void* x, int64_t ldx, const void* left, const void* right, void* codes,
                                void* scales, int64_t tokens, int m, int n, float clip, int in_dtype, int scale_dtype,
                                cudaStream_t stream);
int launch_transform_generic(const void* x, int64_t ldx, const void* left, const void* right, float* z, int64_t tokens,
                             int m, int n, int in_dtype, cudaStream_t stream);
// device word that kernels set when a bounded wait runs out (nullptr if it could not be allocated)
uint32_t* device_status_word(int dev);
// the same word if some launch on `dev` already created it, else nullptr (never allocates)
uint32_t* device_status_word_if_any(int dev);
// status word of qo_int4_matmul_static (a device array inside the library): read and clear, allocation-free
int static_status_take(int dev, uint32_t* code);

int launch_dequantize(const void* codes, const void* scales, float* out, int64_t tokens, int64_t features,
                      int packed, int scale_dtype, cudaStream_t stream);
int launch_pack(const int8_t* codes, int32_t* packed, int64_t rows, int64_t features, cudaStream_t stream);
int launch_unpack(const int32_t* packed, int8_t* codes, int64_t rows, int64_t features, cudaStream_t stream);
int launch_quantize_weights(const float* w, int32_t* packed, float* scale, int64_t rows, int64_t k,
                            cudaStream_t stream);

int launch_gemm_generic(const int32_t* a, int64_t lda, const int32_t* b, int64_t bsk, int64_t bsn,
                        const float* sa, const float* sb, void* out, int out_dtype, int64_t t, int64_t k,
                        int64_t n, int32_t* acc_out, const void* bias, cudaStream_t stream);
// weight-streaming kernel for 1 .. 32 rows (int4_gemm_skinny.cu); b is [n, k/8] with row stride bsn words
bool gemm_skinny_supported(int64_t t, int64_t k, int64_t n, const void* a, int64_t lda, const void* b, int64_t bsk, int64_t bsn);
int launch_gemm_skinny(const int32_t* a, int64_t lda, const int32_t* b, int64_t bsn, const float* sa, const float* sb, void* out,
                       int out_dtype, int64_t t, int64_t k, int64_t n, int32_t* acc_out, const void* bias, cudaStream_t stream,
                       bool weights_first = false);
size_t gemm_sm100_workspace_bytes(int64_t t, int64_t k, int64_t n);
bool gemm_sm100_supported(int64_t t, int64_t k, int64_t n, int64_t lda, int64_t bsk, int64_t bsn);
int launch_gemm_sm100(const int32_t* a, int64_t lda, const int32_t* b, int64_t bsk, int64_t bsn,
                      const float* sa, const float* sb, void* out, int out_dtype, int64_t t, int64_t k,
                      int64_t n, int32_t* acc_out, const void* bias, void* workspace, size_t workspace_bytes,
                      cudaStream_t stream);

// kernel selection of the calling thread (qo_set_kernel_policy): 0 automatic, 1 generic SIMT only, 2 tcgen05 only,
// 3 tcgen05 only and without the CTA-pair kernel
int current_kernel_policy();
// int8 GEMM on CTA pairs (int4_gemm_sm100_pair.cu); QO_ERR_UNSUPPORTED without a message when it does not apply
int launch_gemm_sm100_pair(const int8_t* a8, const int8_t* b8, const float* sa, const float* sb, void* out, int out_dtype,
                           int64_t t, int64_t k, int64_t n, int32_t* acc_out, const void* bias, uint32_t* status,
                           cudaStream_t stream);

// packed-int4 GEMM that unpacks inside the kernel (int4_gemm_sm100_unpack.cu): b is [n, k/8] with row stride ldb words
bool gemm_unpack_supported(int64_t t, int64_t k, int64_t n, const void* a, int64_t lda, const void* b, int64_t bsk, int64_t bsn);
bool gemm_unpack_preferred(int64_t t, int64_t k, int64_t n);
// destinations of the fused all-gather (see gemm_s4_unpack_kernel): the buffers [total_rows, n] of this GPU and its
// peers; this rank's rows start at row_offset
struct GatherDsts {
  void* ptr[8];
  int n_dst;
  long long row_offset;
};
int launch_gemm_unpack(const int32_t* a, int64_t lda, const int32_t* b, int64_t ldb, const float* sa, const float* sb, void* out,
                       int out_dtype, int64_t t, int64_t k, int64_t n, int32_t* acc_out, const void* bias, uint32_t* status,
                       cudaStream_t stream, const GatherDsts* gather = nullptr);

// pieces of the tcgen05 GEMM, used separately by the fused layer
int launch_widen_rows(const int32_t* in, int64_t ld_words, int8_t* out, int64_t rows, int64_t k, cudaStream_t stream, bool blocked,
                      bool beside_previous = false);  // beside_previous: may run beside the kernel before it (see int4_gemm_sm100.cu)
size_t gemm_b8_bytes(int64_t n, int64_t k);  // bytes of the int8 B operand in the GEMM's blocked layout
int launch_gemm_sm100_s8(const int8_t* a8, const int8_t* b8, const float* sa, const float* sb, void* out, int out_dtype,
                         int64_t t, int64_t k, int64_t n, int32_t* acc_out, const void* bias, cudaStream_t stream,
                         bool b_early = false);  // b_early: b8 was not written by the kernel that precedes the GEMM in the stream

int launch_widen_b(const int32_t* b, int64_t bsk, int64_t bsn, int8_t* b8, int64_t n, int64_t k, cudaStream_t stream);
int launch_gemm_sm100_s8_status(const int8_t* a8, const int8_t* b8, const float* sa, const float* sb, void* out,
                                int out_dtype, int64_t t, int64_t k, int64_t n, int32_t* acc_out, uint32_t* status,
                                cudaStream_t stream);

}  // namespace qo
