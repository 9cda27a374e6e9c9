#include "qo_internal.cuh"
namespace qo {
bool flatquant_sm100_supported(int64_t, int, int, int, const void*) { return false; }
int launch_flatquant_sm100(const void*, int64_t, const void*, const void*, void*, void*, int64_t, int, int, float, int,
                           int, int, cudaStream_t) { return QO_ERR_UNSUPPORTED; }
}
