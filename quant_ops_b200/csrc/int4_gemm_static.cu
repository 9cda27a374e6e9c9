// qo_int4_matmul_static: the packed-int4 GEMM for hosts that must not allocate device memory.
//
// Some callers of this library cannot let it call cudaMalloc: an inference server that handed (nearly) all of the
// device memory to its own pool at start-up has nothing left for a late allocation, and a cudaMalloc in the middle
// of a serving step would also synchronise the device.  The regular entry point needs scratch for the widened
// operands (from the caller, or from a buffer the library allocates); this one keeps that scratch, and the word the
// kernels report a timed-out wait in, in the two file-scope device arrays below.  They are part of the loaded
// module, so every GPU that loads the library holds kStaticScratchBytes of device memory until the process exits.
//
// In host code the names of those arrays are host-side stand-ins, not device addresses.  The device addresses come
// from cudaGetSymbolAddress, looked up once per device with that device current.  The first call on a device does
// this look-up; make that first call before any stream capture.
#include <mutex>

#include "qo_internal.cuh"

namespace qo {
namespace {

constexpr size_t kStaticScratchBytes = 8u << 20;  // 8 MiB: tokens*k bytes + the blocked int8 weights (whole 256 x 128 blocks) must fit

static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];
static __device__ __align__(256) uint32_t g_static_status[64];

struct DeviceAddresses {
  unsigned char* scratch = nullptr;
  uint32_t* status = nullptr;
};

std::mutex g_addr_mu;
DeviceAddresses g_addr_table[64];

// the addresses of device `dev` if a call already resolved them
bool static_addresses_if_resolved(int dev, DeviceAddresses* out) {
  std::lock_guard<std::mutex> lock(g_addr_mu);
  if (!g_addr_table[dev].scratch) return false;
  *out = g_addr_table[dev];
  return true;
}

// Device addresses of the two arrays on the current device (index `dev`), resolved on first use.
int static_addresses(int dev, DeviceAddresses* out) {
  std::mutex& mu = g_addr_mu;
  DeviceAddresses* table = g_addr_table;
  if (dev < 0 || dev >= 64) return fail(QO_ERR_NO_DEVICE, "int4_matmul_static: device index %d out of range", dev);
  std::lock_guard<std::mutex> lock(mu);
  if (!table[dev].scratch) {
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_static_scratch);
    if (e != cudaSuccess) {
      (void)cudaGetLastError();
      return fail(QO_ERR_CUDA, "int4_matmul_static: cudaGetSymbolAddress(scratch) failed: %s", cudaGetErrorString(e));
    }
    void* q = nullptr;
    e = cudaGetSymbolAddress(&q, g_static_status);
    if (e != cudaSuccess) {
      (void)cudaGetLastError();
      return fail(QO_ERR_CUDA, "int4_matmul_static: cudaGetSymbolAddress(status) failed: %s", cudaGetErrorString(e));
    }
    table[dev].status = reinterpret_cast<uint32_t*>(q);
    table[dev].scratch = reinterpret_cast<unsigned char*>(p);
  }
  *out = table[dev];
  return QO_OK;
}

inline size_t align256(size_t v) { return (v + 255) & ~size_t(255); }

}  // namespace

// Reads and clears the status word of qo_int4_matmul_static on device `dev` (which must be current and idle on the
// caller's stream).  Plain cudaMemcpy from / to the resolved symbol address: nothing is allocated.  *code stays 0 when
// the entry point has not been used on this device yet.
int static_status_take(int dev, uint32_t* code) {
  *code = 0;
  if (dev < 0 || dev >= 64) return QO_OK;
  uint32_t* word = nullptr;
  {
    // only a device on which the entry point already ran has anything to report; do not resolve the symbol here
    DeviceAddresses probe;
    if (static_addresses_if_resolved(dev, &probe)) word = probe.status;
  }
  if (!word) return QO_OK;
  QO_CUDA_TRY(cudaMemcpy(code, word, sizeof *code, cudaMemcpyDeviceToHost));
  if (*code != 0) {
    const uint32_t zero = 0;
    QO_CUDA_TRY(cudaMemcpy(word, &zero, sizeof zero, cudaMemcpyHostToDevice));
  }
  return QO_OK;
}

}  // namespace qo

using namespace qo;

extern "C" {

size_t qo_int4_matmul_static_max_bytes(void) { return kStaticScratchBytes; }

int qo_int4_matmul_static(const int32_t* a, int64_t lda, const int32_t* b, int64_t b_stride_k, int64_t b_stride_n,
                          const float* scale_a, const float* scale_b, void* out, int out_dtype, int64_t tokens,
                          int64_t k, int64_t n_out, void* stream) {
  clear_error();
  if (tokens < 0 || k < 0 || n_out < 0) return fail(QO_ERR_INVALID_ARGUMENT, "int4_matmul_static: negative size");
  if (out_dtype != QO_F16 && out_dtype != QO_BF16) return fail(QO_ERR_INVALID_ARGUMENT, "int4_matmul_static: out_dtype must be QO_F16 or QO_BF16");
  if (tokens == 0 || n_out == 0) return QO_OK;
  if (!a || !b || !scale_a || !scale_b || !out) return fail(QO_ERR_INVALID_ARGUMENT, "int4_matmul_static: null pointer argument");
  if (k % 8 || lda < k / 8) return fail(QO_ERR_INVALID_ARGUMENT, "int4_matmul_static: k must be a multiple of 8 and lda >= k/8");
  if (!gemm_sm100_supported(tokens, k, n_out, lda, b_stride_k, b_stride_n))
    return fail(QO_ERR_UNSUPPORTED, "int4_matmul_static: only the shapes of the tcgen05 kernel are served here (k %% 16 == 0, n_out %% 8 == 0, unit stride along k or n_out); got t=%lld k=%lld n=%lld", (long long)tokens, (long long)k, (long long)n_out);
  const size_t a_bytes = align256((size_t)tokens * (size_t)k), need = a_bytes + gemm_b8_bytes(n_out, k);
  if (need > kStaticScratchBytes)
    return fail(QO_ERR_WORKSPACE, "int4_matmul_static: the widened operands take %zu bytes, which exceeds the built-in scratch of %zu bytes; use qo_int4_matmul with a workspace", need, (size_t)kStaticScratchBytes);
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    return fail(QO_ERR_NO_DEVICE, "int4_matmul_static: no CUDA device: %s", cudaGetErrorString(e));
  }
  int major = 0;
  QO_CUDA_TRY(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
  if (major != 10) return fail(QO_ERR_NO_DEVICE, "int4_matmul_static: device %d is not an sm_100 GPU", dev);
  DeviceAddresses addr;
  int rc = static_addresses(dev, &addr);
  if (rc) return rc;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  int8_t* a8 = reinterpret_cast<int8_t*>(addr.scratch);
  int8_t* b8 = a8 + a_bytes;
  // every byte the GEMM reads is rewritten by the two widen passes, so nothing has to be cleared between calls
  if ((rc = launch_widen_rows(a, lda, a8, tokens, k, st, false))) return rc;
  if ((rc = launch_widen_b(b, b_stride_k, b_stride_n, b8, n_out, k, st))) return rc;
  return launch_gemm_sm100_s8_status(a8, b8, scale_a, scale_b, out, out_dtype, tokens, k, n_out, nullptr, addr.status, st);
}

}  // extern "C"
