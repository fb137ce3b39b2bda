// W4A16 matmul (npu_weight_quant_batchmatmul): entry point and kernel choice.
#include "qmm_common.cuh"
#include "w4a16_simt.cuh"

namespace qmm {
// Implemented in w4a16_tc.cu: tcgen05 kernel for 16-byte aligned operands.
bool w4a16_tc_supported(const W4Params &p, int x_dtype);
size_t w4a16_tc_workspace_bytes(int64_t M, int64_t N, int64_t K, int64_t group);
int launch_w4a16_tc(const W4Params &p, int x_dtype, void *workspace, cudaStream_t stream);
// Implemented in w4a16_mma.cu: register-operand kernel for decode (M <= 16).
bool w4a16_mma_supported(const W4Params &p, int x_dtype);
size_t w4a16_mma_workspace_bytes(int64_t M, int64_t N, int64_t K, int64_t group);
int launch_w4a16_mma(const W4Params &p, int x_dtype, void *workspace, cudaStream_t stream);
}  // namespace qmm

extern "C" int qmm_weight_quant_batchmatmul_workspace_size(int64_t M, int64_t N, int64_t K, int64_t group,
                                                           size_t *bytes) {
    using namespace qmm;
    QMM_REQUIRE(bytes != nullptr, "qmm_weight_quant_batchmatmul_workspace_size: bytes is NULL");
    QMM_REQUIRE(M >= 0 && N >= 0 && K >= 0 && group >= 0,
                "qmm_weight_quant_batchmatmul_workspace_size: negative argument");
    const size_t tc = w4a16_tc_workspace_bytes(M, N, K, group > 0 ? group : K);
    const size_t mma = w4a16_mma_workspace_bytes(M, N, K, group > 0 ? group : K);
    *bytes = tc > mma ? tc : mma;
    return QMM_OK;
}

extern "C" int qmm_weight_quant_batchmatmul(const void *x, int x_dtype, int64_t ld_x, const int32_t *weight,
                                            int64_t ld_w, const void *antiquant_scale, const void *antiquant_offset,
                                            int64_t group, const void *bias, void *out, int64_t ld_out, int64_t M,
                                            int64_t N, int64_t K, void *workspace, size_t workspace_bytes,
                                            void *stream) {
    using namespace qmm;
    QMM_REQUIRE(M >= 0 && N >= 0 && K >= 0, "qmm_weight_quant_batchmatmul: negative dimension");
    QMM_REQUIRE(x_dtype == QMM_DTYPE_BF16 || x_dtype == QMM_DTYPE_F16,
                "qmm_weight_quant_batchmatmul: x must be bf16 or f16");
    QMM_REQUIRE(N % 8 == 0, "qmm_weight_quant_batchmatmul: N must be a multiple of 8 (8 int4 per int32)");
    if (M == 0 || N == 0) return QMM_OK;
    QMM_REQUIRE(out != nullptr, "qmm_weight_quant_batchmatmul: out is NULL");
    QMM_REQUIRE(ld_out >= N, "qmm_weight_quant_batchmatmul: ld_out smaller than N");
    if (K > 0) {
        QMM_REQUIRE(x != nullptr && weight != nullptr && antiquant_scale != nullptr,
                    "qmm_weight_quant_batchmatmul: NULL operand");
        QMM_REQUIRE(ld_x >= K, "qmm_weight_quant_batchmatmul: ld_x smaller than K");
        QMM_REQUIRE(ld_w >= N / 8, "qmm_weight_quant_batchmatmul: ld_w smaller than N/8");
        QMM_REQUIRE(group > 0 && K % group == 0, "qmm_weight_quant_batchmatmul: group must divide K");
        QMM_REQUIRE(group % 32 == 0 || group == K,
                    "qmm_weight_quant_batchmatmul: group must be a multiple of 32 (or equal to K)");
    }
    W4Params p;
    p.x = x;
    p.ld_x = ld_x;
    p.w = weight;
    p.ld_w = ld_w;
    p.scale = antiquant_scale;
    p.offset = antiquant_offset;
    p.group = group > 0 ? group : 1;
    p.bias = bias;
    p.out = out;
    p.ld_out = ld_out;
    p.M = M;
    p.N = N;
    p.K = K;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // Both tensor-core kernels need operands that meet TMA's 16-byte rules and 256-byte aligned
    // scratch.  Up to 16 token rows the weights stay packed until they are in registers; beyond
    // that the tcgen05 kernel takes over.
    const bool ws_ok = workspace != nullptr && (reinterpret_cast<uintptr_t>(workspace) & 255) == 0;
    if (K > 0 && ws_ok && w4a16_mma_supported(p, x_dtype) &&
        workspace_bytes >= w4a16_mma_workspace_bytes(M, N, K, p.group))
        return launch_w4a16_mma(p, x_dtype, workspace, s);
    if (K > 0 && w4a16_tc_supported(p, x_dtype) && workspace != nullptr &&
        (reinterpret_cast<uintptr_t>(workspace) & 255) == 0 &&
        workspace_bytes >= w4a16_tc_workspace_bytes(M, N, K, p.group))
        return launch_w4a16_tc(p, x_dtype, workspace, s);
    if (x_dtype == QMM_DTYPE_BF16) return launch_w4a16_simt<__nv_bfloat16>(p, s);
    return launch_w4a16_simt<__half>(p, s);
}
