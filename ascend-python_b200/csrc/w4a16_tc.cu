// W4A16 tcgen05 kernel (placeholder until the tensor-core path is validated).
#include "qmm_common.cuh"
#include "w4a16_simt.cuh"

namespace qmm {
bool w4a16_tc_supported(const W4Params &, int) { return false; }
int launch_w4a16_tc(const W4Params &, int, cudaStream_t) {
    return fail(QMM_ERR_UNSUPPORTED, "w4a16 tcgen05 kernel is not available");
}
}  // namespace qmm
