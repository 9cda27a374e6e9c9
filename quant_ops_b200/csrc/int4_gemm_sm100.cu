#include "qo_internal.cuh"
namespace qo {
size_t gemm_sm100_workspace_bytes(int64_t, int64_t, int64_t) { return 0; }
bool gemm_sm100_supported(int64_t, int64_t, int64_t, int64_t, int64_t, int64_t) { return false; }
int launch_gemm_sm100(const int32_t*, int64_t, const int32_t*, int64_t, int64_t, const float*, const float*, void*, int,
                      int64_t, int64_t, int64_t, int32_t*, const void*, void*, size_t, cudaStream_t) { return QO_ERR_UNSUPPORTED; }
}
