// extern "C" entry points: argument validation, kernel selection, workspaces.  No kernels live here.
#include <cuda.h>

#include <cstring>
#include <mutex>
#include <vector>

#include "qo_internal.cuh"

namespace qo {

static thread_local char t_error[512] = "";
static thread_local int t_policy = 0;
static thread_local int t_quant_path = 0;
static thread_local int t_gemm_path = 0;
std::atomic<uint64_t> g_launches{0};

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(t_error, sizeof t_error, fmt, ap);
  va_end(ap);
}
void clear_error() { t_error[0] = 0; }
int current_kernel_policy() { return t_policy; }

namespace {

constexpr int kMaxDevices = 64;

// The kernels are built for sm_100a only; anything else cannot run them.
int require_device(int* dev_out) {
  static std::atomic<int> ok[kMaxDevices];  // 0 unknown, 1 good, 2 bad
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    return fail(QO_ERR_NO_DEVICE, "no CUDA device available: %s", cudaGetErrorString(e));
  }
  if (dev_out) *dev_out = dev;
  if (dev < 0 || dev >= kMaxDevices) return fail(QO_ERR_NO_DEVICE, "device index %d out of range", dev);
  int state = ok[dev].load(std::memory_order_relaxed);
  if (state == 0) {
    int major = 0;
    QO_CUDA_TRY(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
    state = (major == 10) ? 1 : 2;
    ok[dev].store(state, std::memory_order_relaxed);
  }
  if (state != 1) return fail(QO_ERR_NO_DEVICE, "device %d is not an sm_100 GPU; this library has sm_100a kernels only", dev);
  return QO_OK;
}

// Grow-only per-device scratch the library owns when the caller passes no workspace.  ONE buffer per device, shared
// by every call that passes no workspace: such calls must be issued on one stream at a time (calls on different
// streams would overwrite each other's operands).  A buffer that has become too small is not freed when a larger
// one replaces it -- kernels already enqueued may still use it -- but kept until qo_release_workspaces(), so growing
// neither synchronises the device nor frees memory under a running kernel.
struct Scratch {
  std::mutex mu;
  void* ptr[kMaxDevices] = {};
  size_t bytes[kMaxDevices] = {};
  struct Retired { int dev; void* ptr; };
  std::vector<Retired> retired;
};
Scratch g_scratch;       // GEMM / fused layer
Scratch g_host_staging;  // device side of the host-buffer quantizer

int scratch_get(Scratch& s, int dev, size_t need, void** out) {
  std::lock_guard<std::mutex> lock(s.mu);
  if (s.bytes[dev] < need) {
    const size_t grow = need + need / 4;
    void* fresh = nullptr;
    QO_CUDA_TRY(cudaMalloc(&fresh, grow));
    if (s.ptr[dev]) s.retired.push_back({dev, s.ptr[dev]});
    s.ptr[dev] = fresh;
    s.bytes[dev] = grow;
  }
  *out = s.ptr[dev];
  return QO_OK;
}

inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

int check_quant_args(const void* x, int64_t ldx, const void* left, const void* right, const void* codes,
                     const void* scales, int64_t tokens, int m, int n, int in_dtype, int pack, int scale_dtype) {
  if (tokens < 0) return fail(QO_ERR_INVALID_ARGUMENT, "flatquant: tokens = %lld is negative", (long long)tokens);
  if (m <= 0 || n <= 0) return fail(QO_ERR_INVALID_ARGUMENT, "flatquant: transform sizes must be positive (m=%d n=%d)", m, n);
  if (!dtype_ok(in_dtype)) return fail(QO_ERR_INVALID_ARGUMENT, "flatquant: unknown in_dtype %d", in_dtype);
  if (!dtype_ok(scale_dtype)) return fail(QO_ERR_INVALID_ARGUMENT, "flatquant: unknown scale_dtype %d", scale_dtype);
  const int64_t feat = (int64_t)m * n;
  if (feat > (1 << 20)) return fail(QO_ERR_INVALID_ARGUMENT, "flatquant: m*n = %lld is not a plausible feature count", (long long)feat);
  if (ldx < feat) return fail(QO_ERR_INVALID_ARGUMENT, "flatquant: row stride %lld is smaller than m*n = %lld", (long long)ldx, (long long)feat);
  if (pack && feat % 8) return fail(QO_ERR_INVALID_ARGUMENT, "flatquant: features (%lld) must be divisible by 8 for int32 packing", (long long)feat);
  if (tokens > 0 && (!x || !left || !right || !codes || !scales)) return fail(QO_ERR_INVALID_ARGUMENT, "flatquant: null pointer argument");
  return QO_OK;
}

}  // namespace
}  // namespace qo

using namespace qo;

extern "C" {

int qo_version(void) { return 100; }

const char* qo_status_string(int status) {
  switch (status) {
    case QO_OK: return "ok";
    case QO_ERR_INVALID_ARGUMENT: return "invalid argument";
    case QO_ERR_UNSUPPORTED: return "unsupported";
    case QO_ERR_CUDA: return "CUDA error";
    case QO_ERR_NO_DEVICE: return "no sm_100 device";
    case QO_ERR_WORKSPACE: return "workspace too small";
    case QO_ERR_DEVICE_TIMEOUT: return "device-side wait timed out";
  }
  return "unknown status";
}

const char* qo_last_error(void) { return t_error; }

uint64_t qo_kernel_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }
int qo_last_quantizer_path(void) { return t_quant_path; }
int qo_last_gemm_path(void) { return t_gemm_path; }

int qo_set_kernel_policy(int policy) {
  if (policy < 0 || policy > 3) return fail(QO_ERR_INVALID_ARGUMENT, "kernel policy must be 0, 1, 2 or 3");
  t_policy = policy;
  return QO_OK;
}

int qo_get_decompose_dim(int64_t n, int64_t* m_out, int64_t* n_out) {
  if (!m_out || !n_out) return fail(QO_ERR_INVALID_ARGUMENT, "get_decompose_dim: null output pointer");
  if (n <= 0) return fail(QO_ERR_INVALID_ARGUMENT, "get_decompose_dim: n must be positive");
  if (n % 4 == 2) return fail(QO_ERR_INVALID_ARGUMENT, "get_decompose_dim: %lld = 2 (mod 4) is not a difference of two squares", (long long)n);
  auto isqrt = [](int64_t v) {
    int64_t r = (int64_t)__builtin_sqrtl((long double)v);
    while (r * r > v) --r;
    while ((r + 1) * (r + 1) <= v) ++r;
    return r;
  };
  int64_t a = isqrt(n);
  if (a * a < n) ++a;
  for (;; ++a) {
    const int64_t d = a * a - n, b = isqrt(d);
    if (b * b == d) {
      *m_out = a - b;
      *n_out = a + b;
      return QO_OK;
    }
  }
}

int qo_flatquant_quantize(const void* x, int64_t ldx, const void* left, const void* right, void* codes, void* scales,
                          int64_t tokens, int m, int n, float clip_ratio, int in_dtype, int pack_int32,
                          int scale_dtype, void* stream) {
  clear_error();
  int rc = check_quant_args(x, ldx, left, right, codes, scales, tokens, m, n, in_dtype, pack_int32, scale_dtype);
  if (rc) return rc;
  if (tokens == 0) return QO_OK;
  if ((rc = require_device(nullptr))) return rc;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const bool fast_ok = flatquant_sm100_supported(ldx, m, n, in_dtype, x, left, right, clip_ratio);
  if (t_policy >= 2 && !fast_ok)
    return fail(QO_ERR_UNSUPPORTED, "flatquant: no tcgen05 kernel for m=%d n=%d dtype=%d ldx=%lld", m, n, in_dtype, (long long)ldx);
  if (fast_ok && t_policy != 1) {
    t_quant_path = 2;
    return launch_flatquant_sm100(x, ldx, left, right, codes, scales, tokens, m, n, clip_ratio, in_dtype, pack_int32,
                                  scale_dtype, st);
  }
  t_quant_path = 1;
  return launch_flatquant_generic(x, ldx, left, right, codes, scales, tokens, m, n, clip_ratio, in_dtype, pack_int32 ? 1 : 0,
                                  scale_dtype, st);
}

int qo_flatquant_transform(const void* x, int64_t ldx, const void* left, const void* right, float* z, int64_t tokens,
                           int m, int n, int in_dtype, void* stream) {
  clear_error();
  int rc = check_quant_args(x, ldx, left, right, z, z, tokens, m, n, in_dtype, 0, QO_F32);
  if (rc) return rc;
  if (tokens == 0) return QO_OK;
  if ((rc = require_device(nullptr))) return rc;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const bool fast_ok = flatquant_sm100_supported(ldx, m, n, in_dtype, x, left, right, 1.0f);
  if (t_policy >= 2 && !fast_ok)
    return fail(QO_ERR_UNSUPPORTED, "flatquant_transform: no tcgen05 kernel for m=%d n=%d dtype=%d", m, n, in_dtype);
  if (fast_ok && t_policy != 1) {
    t_quant_path = 2;
    return launch_flatquant_sm100_mode(2, x, ldx, left, right, z, nullptr, tokens, m, n, 1.0f, in_dtype, QO_F32, st);
  }
  t_quant_path = 1;
  return launch_transform_generic(x, ldx, left, right, z, tokens, m, n, in_dtype, st);
}

int qo_device_status(void* stream) {
  clear_error();
  int dev = 0, rc = require_device(&dev);
  if (rc) return rc;
  QO_CUDA_TRY(cudaStreamSynchronize(reinterpret_cast<cudaStream_t>(stream)));
  // two words can carry a report: the one the regular entry points share (it exists once any of them has launched a
  // tcgen05 kernel on this device) and the one inside the library that qo_int4_matmul_static uses.  Reading them
  // allocates nothing, so a host that may not allocate can call this too.
  uint32_t code = 0, code_static = 0;
  if (uint32_t* word = device_status_word_if_any(dev)) {
    QO_CUDA_TRY(cudaMemcpy(&code, word, sizeof code, cudaMemcpyDeviceToHost));
    if (code != 0) QO_CUDA_TRY(cudaMemset(word, 0, sizeof code));
  }
  if ((rc = static_status_take(dev, &code_static))) return rc;
  if (code == 0) code = code_static;
  if (code == 0) return QO_OK;
  return fail(QO_ERR_DEVICE_TIMEOUT, "a kernel gave up waiting (site 0x%x); its outputs are not valid", code);
}

int qo_dequantize_int4(const void* codes, const void* scales, float* out, int64_t tokens, int64_t features,
                       int packed_int32, int scale_dtype, void* stream) {
  clear_error();
  if (tokens < 0 || features < 0) return fail(QO_ERR_INVALID_ARGUMENT, "dequantize: negative size");
  if (!dtype_ok(scale_dtype)) return fail(QO_ERR_INVALID_ARGUMENT, "dequantize: unknown scale_dtype %d", scale_dtype);
  if (packed_int32 && features % 8) return fail(QO_ERR_INVALID_ARGUMENT, "dequantize: packed input needs features %% 8 == 0");
  if (tokens == 0 || features == 0) return QO_OK;
  if (!codes || !scales || !out) return fail(QO_ERR_INVALID_ARGUMENT, "dequantize: null pointer argument");
  if (reinterpret_cast<uintptr_t>(out) % 16) return fail(QO_ERR_INVALID_ARGUMENT, "dequantize: out must be 16-byte aligned");
  int rc = require_device(nullptr);
  if (rc) return rc;
  return launch_dequantize(codes, scales, out, tokens, features, packed_int32, scale_dtype,
                           reinterpret_cast<cudaStream_t>(stream));
}

size_t qo_int4_matmul_workspace_bytes(int64_t tokens, int64_t k, int64_t n_out) {
  return gemm_sm100_workspace_bytes(tokens, k, n_out);
}

static int int4_matmul_impl(const int32_t* a, int64_t lda, const int32_t* b, int64_t bsk, int64_t bsn,
                            const float* sa, const float* sb, void* out, int out_dtype, int64_t t, int64_t k,
                            int64_t n, int32_t* acc_out, const void* bias, void* workspace, size_t workspace_bytes,
                            cudaStream_t st, bool b_is_layer_weight = false) {
  if (t < 0 || k < 0 || n < 0) return fail(QO_ERR_INVALID_ARGUMENT, "int4_matmul: negative size");
  if (k % 8) return fail(QO_ERR_INVALID_ARGUMENT, "int4_matmul: k = %lld must be a multiple of 8", (long long)k);
  if (k > 262143) return fail(QO_ERR_INVALID_ARGUMENT, "int4_matmul: k = %lld is beyond the supported reduction length", (long long)k);
  if (out_dtype != QO_F16 && out_dtype != QO_BF16) return fail(QO_ERR_INVALID_ARGUMENT, "int4_matmul: out_dtype must be QO_F16 or QO_BF16");
  if (t == 0 || n == 0) return QO_OK;
  if (!a || !b || !sa || !sb || !out) return fail(QO_ERR_INVALID_ARGUMENT, "int4_matmul: null pointer argument");
  if (lda < k / 8) return fail(QO_ERR_INVALID_ARGUMENT, "int4_matmul: lda smaller than k/8");
  int dev = 0, rc = require_device(&dev);
  if (rc) return rc;
  // a few rows: stream the packed weights once instead of widening them for the tensor-memory kernel
  if (t_policy == 0 && gemm_skinny_supported(t, k, n, a, lda, b, bsk, bsn)) {
    t_gemm_path = 3;
    // (b_is_layer_weight: B was not written by the kernel that precedes this one in the stream, see qo_w4a4_linear)
    return launch_gemm_skinny(a, lda, b, bsn, sa, sb, out, out_dtype, t, k, n, acc_out, bias, st, b_is_layer_weight);
  }
  const bool fast_ok = k > 0 && gemm_sm100_supported(t, k, n, lda, bsk, bsn);
  if (t_policy >= 2 && !fast_ok)
    return fail(QO_ERR_UNSUPPORTED, "int4_matmul: no tcgen05 kernel for t=%lld k=%lld n=%lld", (long long)t, (long long)k, (long long)n);
  if (fast_ok && t_policy != 1) {
    const size_t need = gemm_sm100_workspace_bytes(t, k, n);
    if (workspace == nullptr && need > 0) {
      if ((rc = scratch_get(g_scratch, dev, need, &workspace))) return rc;
      workspace_bytes = need;
    }
    if (workspace_bytes < need) return fail(QO_ERR_WORKSPACE, "int4_matmul: workspace of %zu bytes, need %zu", workspace_bytes, need);
    t_gemm_path = 2;
    return launch_gemm_sm100(a, lda, b, bsk, bsn, sa, sb, out, out_dtype, t, k, n, acc_out, bias, workspace,
                             workspace_bytes, st);
  }
  t_gemm_path = 1;
  return launch_gemm_generic(a, lda, b, bsk, bsn, sa, sb, out, out_dtype, t, k, n, acc_out, bias, st);
}

int qo_int4_matmul(const int32_t* a, int64_t lda, const int32_t* b, int64_t b_stride_k, int64_t b_stride_n,
                   const float* scale_a, const float* scale_b, void* out, int out_dtype, int64_t tokens, int64_t k,
                   int64_t n_out, int32_t* acc_out, void* workspace, size_t workspace_bytes, void* stream) {
  clear_error();
  return int4_matmul_impl(a, lda, b, b_stride_k, b_stride_n, scale_a, scale_b, out, out_dtype, tokens, k, n_out,
                          acc_out, nullptr, workspace, workspace_bytes, reinterpret_cast<cudaStream_t>(stream));
}

size_t qo_w4a4_linear_workspace_bytes(int64_t tokens, int64_t k, int64_t n_out) {
  if (tokens <= 0 || k <= 0) return 0;
  return align_up((size_t)tokens * (size_t)(k / 8) * 4, 256) + align_up((size_t)tokens * 4, 256) +
         gemm_sm100_workspace_bytes(tokens, k, n_out);
}

int qo_w4a4_linear(const void* x, int64_t ldx, const void* left, const void* right, const int32_t* w_packed,
                   const float* w_scale, const void* bias, void* out, int64_t tokens, int m, int n, int64_t n_out,
                   float clip_ratio, int in_dtype, int out_dtype, void* workspace, size_t workspace_bytes,
                   void* stream) {
  clear_error();
  if (n_out < 0) return fail(QO_ERR_INVALID_ARGUMENT, "w4a4_linear: negative n_out");
  const int64_t k = (int64_t)m * n;
  if (m <= 0 || n <= 0 || k % 8) return fail(QO_ERR_INVALID_ARGUMENT, "w4a4_linear: m*n must be a positive multiple of 8");
  if (out_dtype != QO_F16 && out_dtype != QO_BF16) return fail(QO_ERR_INVALID_ARGUMENT, "w4a4_linear: out_dtype must be QO_F16 or QO_BF16");
  if (tokens < 0) return fail(QO_ERR_INVALID_ARGUMENT, "w4a4_linear: negative token count");
  if (tokens == 0 || n_out == 0) return QO_OK;
  if (!x || !left || !right || !w_packed || !w_scale || !out) return fail(QO_ERR_INVALID_ARGUMENT, "w4a4_linear: null pointer argument");
  int dev = 0, rc = require_device(&dev);
  if (rc) return rc;
  const size_t need = qo_w4a4_linear_workspace_bytes(tokens, k, n_out);
  if (workspace == nullptr) {
    if ((rc = scratch_get(g_scratch, dev, need, &workspace))) return rc;
    workspace_bytes = need;
  }
  if (workspace_bytes < need) return fail(QO_ERR_WORKSPACE, "w4a4_linear: workspace of %zu bytes, need %zu", workspace_bytes, need);
  char* ws = reinterpret_cast<char*>(workspace);
  // prefill sizes: the quantizer packs, and the GEMM that unpacks in the kernel takes the packed codes and the packed
  // weights as they are (the packed route below); otherwise ...
  const bool unpack_route = t_policy != 1 && gemm_unpack_preferred(tokens, k, n_out) &&
                            gemm_unpack_supported(tokens, k, n_out, workspace, k / 8, w_packed, 1, k / 8);
  if (!unpack_route && t_policy != 1 && tokens > 32 && gemm_sm100_supported(tokens, k, n_out, k / 8, 1, k / 8)) {
    // ... tensor-core route with int8 operands: the quantizer writes int8 codes, which is that GEMM's A operand as it
    // is; only the weights are widened.  Layout: int8 codes [tokens, k] | scales | int8 weights (blocked).
    int8_t* a8 = reinterpret_cast<int8_t*>(ws);
    const size_t o_scale = align_up((size_t)tokens * (size_t)k, 256);
    float* a_scale8 = reinterpret_cast<float*>(ws + o_scale);
    const size_t o_b = o_scale + align_up((size_t)tokens * 4, 256);
    int8_t* b8 = reinterpret_cast<int8_t*>(ws + o_b);
    rc = qo_flatquant_quantize(x, ldx, left, right, a8, a_scale8, tokens, m, n, clip_ratio, in_dtype, 0, QO_F32, stream);
    if (rc) return rc;
    // the weights are widened beside the quantizer just launched: it neither reads the packed weights nor writes b8
    if ((rc = launch_widen_rows(w_packed, k / 8, b8, n_out, k, reinterpret_cast<cudaStream_t>(stream), true, true))) return rc;
    t_gemm_path = 2;
    return launch_gemm_sm100_s8(a8, b8, a_scale8, w_scale, out, out_dtype, tokens, k, n_out, nullptr, bias,
                                reinterpret_cast<cudaStream_t>(stream));
  }
  int32_t* a_packed = reinterpret_cast<int32_t*>(ws);
  const size_t off_scale = align_up((size_t)tokens * (size_t)(k / 8) * 4, 256);
  float* a_scale = reinterpret_cast<float*>(ws + off_scale);
  const size_t off_gemm = off_scale + align_up((size_t)tokens * 4, 256);
  rc = qo_flatquant_quantize(x, ldx, left, right, a_packed, a_scale, tokens, m, n, clip_ratio, in_dtype, 1, QO_F32, stream);
  if (rc) return rc;
  // weights are [n_out, k/8] with K contiguous: as the GEMM's B operand that is strides (1, k/8).  The kernel before
  // the GEMM in the stream is this call's quantizer, which writes only the workspace, and it lets dependents start
  // only after everything older has completed: the GEMM may fetch weights while the quantizer still runs.
  return int4_matmul_impl(a_packed, k / 8, w_packed, 1, k / 8, a_scale, w_scale, out, out_dtype, tokens, k, n_out,
                          nullptr, bias, ws + off_gemm, workspace_bytes - off_gemm,
                          reinterpret_cast<cudaStream_t>(stream), /*b_is_layer_weight=*/t_quant_path == 2);
}

int qo_w4a4_linear_gather(const void* x, int64_t ldx, const void* left, const void* right, const int32_t* w_packed,
                          const float* w_scale, const void* bias, void* const* dsts, int n_dst, int64_t row_offset,
                          int64_t tokens, int m, int n, int64_t n_out, float clip_ratio, int in_dtype, int out_dtype,
                          void* workspace, size_t workspace_bytes, void* stream) {
  clear_error();
  const int64_t k = (int64_t)m * n;
  if (m <= 0 || n <= 0 || k % 8) return fail(QO_ERR_INVALID_ARGUMENT, "w4a4_linear_gather: m*n must be a positive multiple of 8");
  if (out_dtype != QO_F16 && out_dtype != QO_BF16) return fail(QO_ERR_INVALID_ARGUMENT, "w4a4_linear_gather: out_dtype must be QO_F16 or QO_BF16");
  if (tokens < 0 || n_out < 0 || row_offset < 0) return fail(QO_ERR_INVALID_ARGUMENT, "w4a4_linear_gather: negative size or offset");
  if (n_dst < 1 || n_dst > 8 || !dsts) return fail(QO_ERR_INVALID_ARGUMENT, "w4a4_linear_gather: 1 .. 8 destinations");
  if (tokens == 0 || n_out == 0) return QO_OK;
  if (!x || !left || !right || !w_packed || !w_scale) return fail(QO_ERR_INVALID_ARGUMENT, "w4a4_linear_gather: null pointer argument");
  int dev = 0, rc = require_device(&dev);
  if (rc) return rc;
  const size_t need = qo_w4a4_linear_workspace_bytes(tokens, k, n_out);
  if (workspace == nullptr) {
    if ((rc = scratch_get(g_scratch, dev, need, &workspace))) return rc;
    workspace_bytes = need;
  }
  if (workspace_bytes < need) return fail(QO_ERR_WORKSPACE, "w4a4_linear_gather: workspace of %zu bytes, need %zu", workspace_bytes, need);
  if (t_policy == 1 || !gemm_unpack_preferred(tokens, k, n_out) ||
      !gemm_unpack_supported(tokens, k, n_out, workspace, k / 8, w_packed, 1, k / 8) || n_out % 16)
    return fail(QO_ERR_UNSUPPORTED, "w4a4_linear_gather: only prefill-sized products gather in the kernel (tokens=%lld k=%lld n_out=%lld)",
                (long long)tokens, (long long)k, (long long)n_out);
  GatherDsts g = {};
  g.n_dst = n_dst;
  g.row_offset = row_offset;
  for (int d = 0; d < n_dst; ++d) g.ptr[d] = dsts[d];
  char* ws = reinterpret_cast<char*>(workspace);
  int32_t* a_packed = reinterpret_cast<int32_t*>(ws);
  const size_t off_scale = align_up((size_t)tokens * (size_t)(k / 8) * 4, 256);
  float* a_scale = reinterpret_cast<float*>(ws + off_scale);
  rc = qo_flatquant_quantize(x, ldx, left, right, a_packed, a_scale, tokens, m, n, clip_ratio, in_dtype, 1, QO_F32, stream);
  if (rc) return rc;
  uint32_t* status = device_status_word(dev);
  if (!status) return fail(QO_ERR_CUDA, "w4a4_linear_gather: could not allocate the device status word");
  t_gemm_path = 2;
  rc = launch_gemm_unpack(a_packed, k / 8, w_packed, k / 8, a_scale, w_scale, nullptr, out_dtype, tokens, k, n_out, nullptr, bias,
                          status, reinterpret_cast<cudaStream_t>(stream), &g);
  if (rc == QO_ERR_UNSUPPORTED && qo_last_error()[0] == 0)
    return fail(QO_ERR_UNSUPPORTED, "w4a4_linear_gather: this device cannot co-schedule the CTA pairs of the kernel");
  return rc;
}

// ---- sharing device buffers between the processes of a node (CUDA IPC) -------------------------------------------------
namespace {
typedef CUresult (*PointerGetAttributeFn)(void*, CUpointer_attribute, CUdeviceptr);
PointerGetAttributeFn pointer_attribute_fn() {
  static PointerGetAttributeFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuPointerGetAttribute", &p, cudaEnableDefault, &qres) == cudaSuccess && qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<PointerGetAttributeFn>(p);
    else
      (void)cudaGetLastError();
  });
  return fn;
}
}  // namespace

int qo_peer_export(const void* ptr, void* handle64, int64_t* offset) {
  clear_error();
  if (!ptr || !handle64 || !offset) return fail(QO_ERR_INVALID_ARGUMENT, "peer_export: null pointer argument");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
  int rc = require_device(nullptr);
  if (rc) return rc;
  PointerGetAttributeFn attr = pointer_attribute_fn();
  if (!attr) return fail(QO_ERR_CUDA, "peer_export: cuPointerGetAttribute is not available");
  CUdeviceptr base = 0;
  const CUresult r = attr(&base, CU_POINTER_ATTRIBUTE_RANGE_START_ADDR, reinterpret_cast<CUdeviceptr>(ptr));
  if (r != CUDA_SUCCESS || base == 0) return fail(QO_ERR_CUDA, "peer_export: not a device allocation (driver code %d)", (int)r);
  cudaIpcMemHandle_t h;
  QO_CUDA_TRY(cudaIpcGetMemHandle(&h, reinterpret_cast<void*>(base)));
  memcpy(handle64, &h, sizeof(h));
  *offset = (int64_t)(reinterpret_cast<CUdeviceptr>(ptr) - base);
  return QO_OK;
}

int qo_peer_open(const void* handle64, void** base) {
  clear_error();
  if (!handle64 || !base) return fail(QO_ERR_INVALID_ARGUMENT, "peer_open: null pointer argument");
  int rc = require_device(nullptr);
  if (rc) return rc;
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  QO_CUDA_TRY(cudaIpcOpenMemHandle(base, h, cudaIpcMemLazyEnablePeerAccess));
  return QO_OK;
}

int qo_peer_close(void* base) {
  clear_error();
  if (!base) return QO_OK;
  QO_CUDA_TRY(cudaIpcCloseMemHandle(base));
  return QO_OK;
}

int qo_peer_copy(void* dst, const void* src, size_t bytes, void* stream) {
  clear_error();
  if (bytes == 0) return QO_OK;
  if (!dst || !src) return fail(QO_ERR_INVALID_ARGUMENT, "peer_copy: null pointer argument");
  QO_CUDA_TRY(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, reinterpret_cast<cudaStream_t>(stream)));
  return QO_OK;
}

size_t qo_prepared_weights_bytes(int64_t n_out, int64_t k) {
  if (n_out <= 0 || k <= 0) return 0;
  return gemm_b8_bytes(n_out, k);
}

int qo_prepare_weights(const int32_t* w_packed, void* prepared, int64_t n_out, int64_t k, void* stream) {
  clear_error();
  if (n_out < 0 || k < 0 || k % 8) return fail(QO_ERR_INVALID_ARGUMENT, "prepare_weights: k (%lld) must be a non-negative multiple of 8", (long long)k);
  if (n_out == 0 || k == 0) return QO_OK;
  if (!w_packed || !prepared) return fail(QO_ERR_INVALID_ARGUMENT, "prepare_weights: null pointer argument");
  if (reinterpret_cast<uintptr_t>(prepared) % 256) return fail(QO_ERR_INVALID_ARGUMENT, "prepare_weights: the prepared buffer must be 256-byte aligned");
  int rc = require_device(nullptr);
  if (rc) return rc;
  return launch_widen_rows(w_packed, k / 8, reinterpret_cast<int8_t*>(prepared), n_out, k, reinterpret_cast<cudaStream_t>(stream), true);
}

// layout of the prepared layer's workspace: int8 codes [tokens, k] | float scales [tokens]
size_t qo_w4a4_linear_prepared_workspace_bytes(int64_t tokens, int64_t k, int64_t n_out) {
  if (tokens <= 0 || k <= 0) return 0;
  const size_t direct = align_up((size_t)tokens * (size_t)k, 256) + align_up((size_t)tokens * 4, 256);
  const size_t packed = qo_w4a4_linear_workspace_bytes(tokens, k, n_out);  // shapes that take the packed-weight route
  return direct > packed ? direct : packed;
}

int qo_w4a4_linear_prepared(const void* x, int64_t ldx, const void* left, const void* right, const int32_t* w_packed,
                            const void* prepared, const float* w_scale, const void* bias, void* out, int64_t tokens, int m,
                            int n, int64_t n_out, float clip_ratio, int in_dtype, int out_dtype, void* workspace,
                            size_t workspace_bytes, void* stream) {
  clear_error();
  if (n_out < 0) return fail(QO_ERR_INVALID_ARGUMENT, "w4a4_linear: negative n_out");
  const int64_t k = (int64_t)m * n;
  if (m <= 0 || n <= 0 || k % 8) return fail(QO_ERR_INVALID_ARGUMENT, "w4a4_linear: m*n must be a positive multiple of 8");
  if (tokens == 0 || n_out == 0) return QO_OK;
  if (!x || !left || !right || !w_packed || !prepared || !w_scale || !out) return fail(QO_ERR_INVALID_ARGUMENT, "w4a4_linear: null pointer argument");
  if (out_dtype != QO_F16 && out_dtype != QO_BF16) return fail(QO_ERR_INVALID_ARGUMENT, "w4a4_linear: out_dtype must be QO_F16 or QO_BF16");
  int dev = 0, rc = require_device(&dev);
  if (rc) return rc;
  const size_t need = qo_w4a4_linear_prepared_workspace_bytes(tokens, k, n_out);
  if (workspace == nullptr) {
    if ((rc = scratch_get(g_scratch, dev, need, &workspace))) return rc;
    workspace_bytes = need;
  }
  if (workspace_bytes < need) return fail(QO_ERR_WORKSPACE, "w4a4_linear: workspace of %zu bytes, need %zu", workspace_bytes, need);
  // few tokens (weight-streaming kernel), prefill sizes (the GEMM that unpacks in the kernel is the faster one there and
  // needs no int8 copy), or a shape / policy the int8 tensor-core kernel does not take: packed route
  const bool unpack_route = t_policy != 1 && gemm_unpack_preferred(tokens, k, n_out) &&
                            gemm_unpack_supported(tokens, k, n_out, workspace, k / 8, w_packed, 1, k / 8);
  const bool direct = !unpack_route && t_policy != 1 && tokens > 32 && gemm_sm100_supported(tokens, k, n_out, k / 8, 1, k / 8) &&
                      reinterpret_cast<uintptr_t>(prepared) % 256 == 0;
  if (!direct)
    return qo_w4a4_linear(x, ldx, left, right, w_packed, w_scale, bias, out, tokens, m, n, n_out, clip_ratio, in_dtype, out_dtype,
                          workspace, workspace_bytes, stream);
  char* ws = reinterpret_cast<char*>(workspace);
  int8_t* a8 = reinterpret_cast<int8_t*>(ws);
  const size_t off_scale = align_up((size_t)tokens * (size_t)k, 256);
  float* a_scale = reinterpret_cast<float*>(ws + off_scale);
  rc = qo_flatquant_quantize(x, ldx, left, right, a8, a_scale, tokens, m, n, clip_ratio, in_dtype, 0, QO_F32, stream);
  if (rc) return rc;
  t_gemm_path = 2;
  // the prepared weights were not written by the quantizer just launched: the GEMM may request them before it waits
  return launch_gemm_sm100_s8(a8, reinterpret_cast<const int8_t*>(prepared), a_scale, w_scale, out, out_dtype, tokens, k, n_out,
                              nullptr, bias, reinterpret_cast<cudaStream_t>(stream), true);
}

int qo_pack_int4(const int8_t* codes, int32_t* packed, int64_t rows, int64_t features, void* stream) {
  clear_error();
  if (rows < 0 || features < 0 || features % 8) return fail(QO_ERR_INVALID_ARGUMENT, "pack_int4: features (%lld) must be divisible by 8", (long long)features);
  if (rows == 0 || features == 0) return QO_OK;
  if (!codes || !packed) return fail(QO_ERR_INVALID_ARGUMENT, "pack_int4: null pointer argument");
  if (reinterpret_cast<uintptr_t>(codes) % 8) return fail(QO_ERR_INVALID_ARGUMENT, "pack_int4: codes must be 8-byte aligned");
  int rc = require_device(nullptr);
  if (rc) return rc;
  return launch_pack(codes, packed, rows, features, reinterpret_cast<cudaStream_t>(stream));
}

int qo_unpack_int4(const int32_t* packed, int8_t* codes, int64_t rows, int64_t features, void* stream) {
  clear_error();
  if (rows < 0 || features < 0 || features % 8) return fail(QO_ERR_INVALID_ARGUMENT, "unpack_int4: features (%lld) must be divisible by 8", (long long)features);
  if (rows == 0 || features == 0) return QO_OK;
  if (!codes || !packed) return fail(QO_ERR_INVALID_ARGUMENT, "unpack_int4: null pointer argument");
  if (reinterpret_cast<uintptr_t>(codes) % 8) return fail(QO_ERR_INVALID_ARGUMENT, "unpack_int4: codes must be 8-byte aligned");
  int rc = require_device(nullptr);
  if (rc) return rc;
  return launch_unpack(packed, codes, rows, features, reinterpret_cast<cudaStream_t>(stream));
}

int qo_quantize_weights_int4(const float* w, int32_t* packed, float* scale, int64_t rows, int64_t k, void* stream) {
  clear_error();
  if (rows < 0 || k < 0 || k % 8) return fail(QO_ERR_INVALID_ARGUMENT, "quantize_weights: k (%lld) must be divisible by 8", (long long)k);
  if (rows == 0 || k == 0) return QO_OK;
  if (!w || !packed || !scale) return fail(QO_ERR_INVALID_ARGUMENT, "quantize_weights: null pointer argument");
  int rc = require_device(nullptr);
  if (rc) return rc;
  return launch_quantize_weights(w, packed, scale, rows, k, reinterpret_cast<cudaStream_t>(stream));
}

// Host-buffer quantizer: rows go through a ring of device slots, one stream per slot, so the copy in of slice
// i+1, the kernel on slice i and the copy out of slice i-1 overlap.
int qo_flatquant_quantize_host(const void* x_host, const void* left_host, const void* right_host, void* codes_host,
                               void* scales_host, int64_t tokens, int m, int n, float clip_ratio, int in_dtype,
                               int pack_int32, int scale_dtype) {
  clear_error();
  int rc = check_quant_args(x_host, (int64_t)m * n, left_host, right_host, codes_host, scales_host, tokens, m, n,
                            in_dtype, pack_int32, scale_dtype);
  if (rc) return rc;
  if (tokens == 0) return QO_OK;
  int dev = 0;
  if ((rc = require_device(&dev))) return rc;

  constexpr int kSlots = 4;
  static std::mutex mu;
  static cudaStream_t streams[kMaxDevices][kSlots] = {};
  std::lock_guard<std::mutex> lock(mu);  // one host-buffer call at a time per process: the slots are shared
  for (int s = 0; s < kSlots; ++s)
    if (!streams[dev][s]) QO_CUDA_TRY(cudaStreamCreateWithFlags(&streams[dev][s], cudaStreamNonBlocking));

  const size_t feat = (size_t)m * n, esz = dtype_size(in_dtype), ssz = dtype_size(scale_dtype);
  const size_t code_row = pack_int32 ? feat / 2 : feat;
  int64_t slice = (int64_t)((24u << 20) / (feat * esz));  // about 24 MB of activations per slice (8 MB slices measured 15 % slower end to end)
  if (slice < 1) slice = 1;
  if (slice > tokens) slice = tokens;
  const size_t x_bytes = align_up((size_t)slice * feat * esz, 256), c_bytes = align_up((size_t)slice * code_row, 256),
               s_bytes = align_up((size_t)slice * ssz, 256), lr_bytes = align_up(((size_t)m * m + (size_t)n * n) * esz, 256);
  void* base = nullptr;
  if ((rc = scratch_get(g_host_staging, dev, lr_bytes + kSlots * (x_bytes + c_bytes + s_bytes), &base))) return rc;
  char* p = reinterpret_cast<char*>(base);
  char* d_left = p;
  char* d_right = p + (size_t)m * m * esz;
  p += lr_bytes;
  QO_CUDA_TRY(cudaMemcpyAsync(d_left, left_host, (size_t)m * m * esz, cudaMemcpyHostToDevice, streams[dev][0]));
  QO_CUDA_TRY(cudaMemcpyAsync(d_right, right_host, (size_t)n * n * esz, cudaMemcpyHostToDevice, streams[dev][0]));
  static cudaEvent_t lr_ready[kMaxDevices] = {};
  if (!lr_ready[dev]) QO_CUDA_TRY(cudaEventCreateWithFlags(&lr_ready[dev], cudaEventDisableTiming));
  QO_CUDA_TRY(cudaEventRecord(lr_ready[dev], streams[dev][0]));
  for (int s = 1; s < kSlots; ++s) QO_CUDA_TRY(cudaStreamWaitEvent(streams[dev][s], lr_ready[dev], 0));  // the transforms are on the device

  int slot = 0;
  for (int64_t t0 = 0; t0 < tokens; t0 += slice, slot = (slot + 1) % kSlots) {
    const int64_t cnt = (tokens - t0 < slice) ? tokens - t0 : slice;
    char* dx = p + slot * (x_bytes + c_bytes + s_bytes);
    char* dc = dx + x_bytes;
    char* ds = dc + c_bytes;
    cudaStream_t st = streams[dev][slot];
    QO_CUDA_TRY(cudaMemcpyAsync(dx, reinterpret_cast<const char*>(x_host) + (size_t)t0 * feat * esz,
                                (size_t)cnt * feat * esz, cudaMemcpyHostToDevice, st));
    rc = qo_flatquant_quantize(dx, (int64_t)feat, d_left, d_right, dc, ds, cnt, m, n, clip_ratio, in_dtype, pack_int32,
                               scale_dtype, st);
    if (rc) break;
    QO_CUDA_TRY(cudaMemcpyAsync(reinterpret_cast<char*>(codes_host) + (size_t)t0 * code_row, dc, (size_t)cnt * code_row,
                                cudaMemcpyDeviceToHost, st));
    QO_CUDA_TRY(cudaMemcpyAsync(reinterpret_cast<char*>(scales_host) + (size_t)t0 * ssz, ds, (size_t)cnt * ssz,
                                cudaMemcpyDeviceToHost, st));
  }
  for (int s = 0; s < kSlots; ++s) {
    cudaError_t e = cudaStreamSynchronize(streams[dev][s]);
    if (e != cudaSuccess && rc == QO_OK) rc = fail(QO_ERR_CUDA, "host-buffer quantizer: %s", cudaGetErrorString(e));
  }
  return rc;
}

int qo_release_workspaces(void) {
  clear_error();
  int rc = QO_OK, cur = 0;
  if (cudaGetDevice(&cur) != cudaSuccess) {
    (void)cudaGetLastError();
    return QO_OK;
  }
  for (Scratch* s : {&g_scratch, &g_host_staging}) {
    std::lock_guard<std::mutex> lock(s->mu);
    for (int d = 0; d < kMaxDevices; ++d) {
      if (!s->ptr[d]) continue;
      s->retired.push_back({d, s->ptr[d]});
      s->ptr[d] = nullptr;
      s->bytes[d] = 0;
    }
    for (const Scratch::Retired& r : s->retired) {
      if (cudaSetDevice(r.dev) == cudaSuccess) {
        cudaDeviceSynchronize();
        if (cudaFree(r.ptr) != cudaSuccess) rc = fail(QO_ERR_CUDA, "cudaFree of a library workspace failed");
      }
    }
    s->retired.clear();
  }
  cudaSetDevice(cur);
  return rc;
}

}  // extern "C"
