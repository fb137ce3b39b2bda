// npu_quant_matmul: int8 x int8 matmul with fused dequantization.
//
// Argument checks, output shape rules and allocation follow the reference's
// dense matmul host code (op_plugin/ops/base_ops/opapi/MmKernelNpuOpApi.cpp:24-42,
// MatmulKernelNpuOpApi.cpp:28-78 for batched left operands); the launch goes
// through the two-phase workspace-size + launch boundary.
#include "op_plugin/OpApiInterface.h"
#include "op_plugin/utils/qmm_api_common.h"

namespace op_api {

at::Tensor npu_quant_matmul(const at::Tensor &x1, const at::Tensor &x2, const at::Tensor &scale,
                            const c10::optional<at::Tensor> &offset, const c10::optional<at::Tensor> &pertoken_scale,
                            const c10::optional<at::Tensor> &bias, c10::optional<at::ScalarType> output_dtype)
{
    TORCH_CHECK(x1.is_cuda() && x2.is_cuda(), "npu_quant_matmul expects CUDA tensors, but x1 is on ", x1.device(),
                " and x2 is on ", x2.device());
    TORCH_CHECK(x1.scalar_type() == at::kChar && x2.scalar_type() == at::kChar,
                "Both inputs of npu_quant_matmul are required to be int8, but the actual dtypes are ",
                x1.scalar_type(), " and ", x2.scalar_type());
    TORCH_CHECK(x1.dim() >= 2 && x2.dim() == 2, "x1 of npu_quant_matmul should be at least 2D and x2 2D, but the "
                "actual inputs are ", x1.dim(), "D and ", x2.dim(), "D");
    TORCH_CHECK(x1.size(-1) == x2.size(0),
                "The K-axis in the two inputs of Matmul must be equal, but in reality, the K-axis of x1 is ",
                x1.size(-1), " and the K-axis of x2 is ", x2.size(0));
    // output_dtype=None is the int8 (requantized) output, as for the operator this signature comes from
    const at::ScalarType out_type = output_dtype.value_or(at::kChar);
    TORCH_CHECK(out_type == at::kBFloat16 || out_type == at::kHalf || out_type == at::kInt || out_type == at::kChar,
                "output_dtype of npu_quant_matmul should be int8, bfloat16, float16 or int32, but it is ", out_type);
    const at::Tensor &offset_real = offset.value_or(at::Tensor());
    TORCH_CHECK(!offset_real.defined() || out_type == at::kChar,
                "npu_quant_matmul: offset only applies to an int8 output, but output_dtype is ", out_type);
    c10::cuda::CUDAGuard guard(x1.device());

    const int64_t K = x1.size(-1);
    const int64_t N = x2.size(1);
    const int64_t M = c10::multiply_integers(x1.sizes().slice(0, x1.dim() - 1));
    const at::Tensor &pertoken_real = pertoken_scale.value_or(at::Tensor());
    const at::Tensor &bias_real = bias.value_or(at::Tensor());

    if (out_type != at::kInt) {
        TORCH_CHECK(scale.scalar_type() == at::kFloat, "scale of npu_quant_matmul should be float32, but it is ",
                    scale.scalar_type());
        TORCH_CHECK(scale.numel() == N || scale.numel() == 1, "scale of npu_quant_matmul should have N=", N,
                    " elements or one, but it has ", scale.numel());
    }
    if (pertoken_real.defined()) {
        TORCH_CHECK(pertoken_real.scalar_type() == at::kFloat && pertoken_real.numel() == M,
                    "pertoken_scale of npu_quant_matmul should be float32 with M=", M, " elements, but it is ",
                    pertoken_real.scalar_type(), " with ", pertoken_real.numel());
    }
    if (bias_real.defined()) {
        TORCH_CHECK(bias_real.numel() == N, "bias of npu_quant_matmul should have N=", N, " elements, but it has ",
                    bias_real.numel());
        if (out_type == at::kInt || out_type == at::kChar) {
            TORCH_CHECK(bias_real.scalar_type() == at::kInt, "bias must be int32 when output_dtype is int32 or int8, "
                        "but it is ", bias_real.scalar_type());
        } else {
            TORCH_CHECK(bias_real.scalar_type() == at::kBFloat16 || bias_real.scalar_type() == at::kHalf ||
                            bias_real.scalar_type() == at::kFloat,
                        "bias must be bfloat16, float16 or float32 for a floating-point output, but it is ",
                        bias_real.scalar_type());
        }
    }

    auto output_size = x1.sizes().vec();
    output_size.back() = N;
    at::Tensor result = at::empty(output_size, x1.options().dtype(out_type));
    if (result.numel() == 0) {
        return result;
    }

    at::Tensor a = x1.contiguous();
    // x2 is used as stored when it is row-major [K,N] or the transposed view of a row-major [N,K]
    at::Tensor b = x2;
    const bool b_row_major = (b.stride(1) == 1 || N == 1) && (b.stride(0) >= N || K <= 1);
    const bool b_col_major = (b.stride(0) == 1 || K == 1) && (b.stride(1) >= K || N <= 1);
    if (!b_row_major && !b_col_major) {
        b = x2.contiguous();
    }
    const int64_t stride_k = (b_row_major || (!b_row_major && !b_col_major)) ? std::max<int64_t>(b.stride(0), N) : 1;
    const int64_t stride_n = (b_row_major || (!b_row_major && !b_col_major)) ? 1 : std::max<int64_t>(b.stride(1), K);
    at::Tensor scale_c = scale.defined() ? scale.contiguous() : scale;
    at::Tensor pertoken_c = pertoken_real.defined() ? pertoken_real.contiguous() : pertoken_real;
    at::Tensor bias_c = bias_real.defined() ? bias_real.contiguous() : bias_real;

    if (out_type == at::kChar) {
        if (offset_real.defined()) {
            TORCH_CHECK(offset_real.scalar_type() == at::kFloat && (offset_real.numel() == N || offset_real.numel() == 1),
                        "offset of npu_quant_matmul should be float32 with N=", N, " elements or one, but it is ",
                        offset_real.scalar_type(), " with ", offset_real.numel());
        }
        at::Tensor offset_c = offset_real.defined() ? offset_real.contiguous() : offset_real;
        size_t ws_size = 0;
        EXEC_QMM_CMD(qmm_quant_matmul_int8_workspace_size, M, N, K, &ws_size);
        at::Tensor ws = op_plugin_utils::qmm_workspace(a, ws_size, /*family=*/3);
        EXEC_QMM_CMD(qmm_quant_matmul_int8, static_cast<const int8_t *>(a.const_data_ptr()), std::max<int64_t>(K, 1),
                     static_cast<const int8_t *>(b.const_data_ptr()), stride_k, stride_n,
                     static_cast<const float *>(scale_c.const_data_ptr()), scale_c.numel(),
                     static_cast<const float *>(op_plugin_utils::opt_ptr(offset_c)),
                     offset_c.defined() ? offset_c.numel() : 0,
                     static_cast<const float *>(op_plugin_utils::opt_ptr(pertoken_c)),
                     static_cast<const int32_t *>(op_plugin_utils::opt_ptr(bias_c)),
                     static_cast<int8_t *>(result.data_ptr()), N, M, N, K, ws.defined() ? ws.data_ptr() : nullptr,
                     ws_size, op_plugin_utils::current_stream(a));
        return result;
    }
    size_t workspace_size = 0;
    EXEC_QMM_CMD(qmm_quant_matmul_workspace_size, M, N, K, QMM_ALGO_AUTO, &workspace_size);
    at::Tensor workspace = op_plugin_utils::qmm_workspace(a, workspace_size);
    EXEC_QMM_CMD(qmm_quant_matmul, static_cast<const int8_t *>(a.const_data_ptr()), std::max<int64_t>(K, 1),
                 static_cast<const int8_t *>(b.const_data_ptr()), stride_k, stride_n,
                 static_cast<const float *>(op_plugin_utils::opt_ptr(scale_c)), scale_c.defined() ? scale_c.numel() : 0,
                 static_cast<const float *>(op_plugin_utils::opt_ptr(pertoken_c)), op_plugin_utils::opt_ptr(bias_c),
                 bias_c.defined() ? op_plugin_utils::qmm_dtype(bias_c.scalar_type()) : QMM_DTYPE_NONE,
                 result.data_ptr(), op_plugin_utils::qmm_dtype(out_type), N, M, N, K, QMM_ALGO_AUTO,
                 workspace.defined() ? workspace.data_ptr() : nullptr, workspace_size,
                 op_plugin_utils::current_stream(a));
    return result;
}

}  // namespace op_api
