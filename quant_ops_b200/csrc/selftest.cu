// Self-test of the failure path: what the host sees when a bounded device-side wait runs out.
//
// Every mbarrier wait in this library gives up after a poll limit, records a site code in the device status word and
// lets its CTA leave in an orderly way; qo_device_status() then reports QO_ERR_DEVICE_TIMEOUT.  A healthy pipeline never
// gets there, so the path is exercised here on purpose and harmlessly: one warp waits, with a limit of 1024 polls
// (about a hundred microseconds), on a barrier that nothing will ever arrive on, records the code and returns.  No
// trap, no fault, no unbounded loop; the context stays usable and the next launch runs normally.
#include "qo_internal.cuh"
#include "sm100_ptx.cuh"

namespace qo {
namespace {

constexpr uint32_t kSelfTestSite = 0xE00u;

__global__ void __launch_bounds__(32)
wait_timeout_probe_kernel(uint32_t* __restrict__ status, uint32_t limit_polls) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    ptx::mbar_init(ptx::smem_u32(&bar), 1);
    ptx::fence_barrier_init();
  }
  __syncwarp();
  // phase 0 of a freshly initialised barrier completes only after one arrival; none is ever made
  const bool ok = ptx::mbar_wait(ptx::smem_u32(&bar), 0, limit_polls);
  if (!ok && threadIdx.x == 0) atomicCAS(status, 0u, kSelfTestSite);
}

}  // namespace
}  // namespace qo

using namespace qo;

extern "C" int qo_selftest_wait_timeout(void* stream) {
  clear_error();
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    return fail(QO_ERR_NO_DEVICE, "selftest: no CUDA device: %s", cudaGetErrorString(e));
  }
  int major = 0;
  QO_CUDA_TRY(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
  if (major != 10) return fail(QO_ERR_NO_DEVICE, "selftest: device %d is not an sm_100 GPU", dev);
  uint32_t* status = device_status_word(dev);
  if (!status) return fail(QO_ERR_CUDA, "selftest: could not allocate the device status word");
  wait_timeout_probe_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(status, 1024u);
  return check_launch("wait_timeout_probe_kernel");
}
