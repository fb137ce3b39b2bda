// npu_mm_all_reduce_base: row-parallel W8A8 matmul followed by allreduce(sum).
//
// Same shape as the reference's fused matmul + collective operator
// npu_mm_reduce_scatter_base
// (op_plugin/ops/base_ops/opapi/MatmulReduceScatterBaseKernelNpuOpApi.cpp:22-42):
// 2-D inputs, K-axis check, communicator passed by name (`hcom`), reduce_op as
// a string, comm_turn as the communication granularity, output allocated from
// the options of x1, arguments forwarded in the order inputs, attributes,
// outputs.  Each rank passes its K shard of x1/x2 and its own pertoken_scale;
// `dequant_scale` is the per-channel weight scale.
#include <string>

#include "op_plugin/OpApiInterface.h"
#include "op_plugin/utils/qmm_api_common.h"

namespace op_api {

at::Tensor npu_mm_all_reduce_base(const at::Tensor &x1, const at::Tensor &x2, c10::string_view hcom,
                                  c10::string_view reduce_op, const c10::optional<at::Tensor> &bias,
                                  const c10::optional<at::Tensor> &antiquant_scale,
                                  const c10::optional<at::Tensor> &antiquant_offset,
                                  const c10::optional<at::Tensor> &x3, const c10::optional<at::Tensor> &dequant_scale,
                                  const c10::optional<at::Tensor> &pertoken_scale, int64_t antiquant_group_size,
                                  int64_t comm_turn)
{
    TORCH_CHECK(x1.is_cuda() && x2.is_cuda(), "npu_mm_all_reduce_base expects CUDA tensors, but x1 is on ",
                x1.device(), " and x2 is on ", x2.device());
    TORCH_CHECK(x1.dim() == 2 && x2.dim() == 2, "Both inputs of mm are required to be 2D, but the actual inputs are ",
                x1.dim(), "D and ", x2.dim(), "D");
    TORCH_CHECK(x1.size(1) == x2.size(0),
                "The K-axis in the two inputs of Matmul must be equal, but in reality, the K-axis of x1 is ",
                x1.size(1), " and the K-axis of x2 is ", x2.size(0));
    TORCH_CHECK(x1.scalar_type() == at::kChar && x2.scalar_type() == at::kChar,
                "npu_mm_all_reduce_base of this build multiplies int8 inputs, but the actual dtypes are ",
                x1.scalar_type(), " and ", x2.scalar_type());
    TORCH_CHECK(reduce_op == "sum", "reduce_op of npu_mm_all_reduce_base should be 'sum', but it is '",
                std::string(reduce_op), "'");
    TORCH_CHECK(!antiquant_scale.has_value() || !antiquant_scale->defined(),
                "npu_mm_all_reduce_base: antiquant_scale (weight-only quantization) is not supported, pass None");
    TORCH_CHECK(!antiquant_offset.has_value() || !antiquant_offset->defined(),
                "npu_mm_all_reduce_base: antiquant_offset (weight-only quantization) is not supported, pass None");
    TORCH_CHECK(!x3.has_value() || !x3->defined(), "npu_mm_all_reduce_base: x3 is not supported, pass None");
    TORCH_CHECK(antiquant_group_size == 0, "npu_mm_all_reduce_base: antiquant_group_size should be 0, but it is ",
                antiquant_group_size);
    TORCH_CHECK(dequant_scale.has_value() && dequant_scale->defined(),
                "npu_mm_all_reduce_base: dequant_scale (per-channel float32 weight scale) is required for int8 inputs");
    TORCH_CHECK(comm_turn >= 0, "comm_turn should be non-negative, but the actual value is ", comm_turn);
    c10::cuda::CUDAGuard guard(x1.device());

    const int64_t M = x1.size(0);
    const int64_t K = x1.size(1);
    const int64_t N = x2.size(1);
    const at::Tensor &scale_real = dequant_scale.value();
    const at::Tensor &pertoken_real = pertoken_scale.value_or(at::Tensor());
    const at::Tensor &bias_real = bias.value_or(at::Tensor());
    TORCH_CHECK(scale_real.scalar_type() == at::kFloat && (scale_real.numel() == N || scale_real.numel() == 1),
                "dequant_scale should be float32 with N=", N, " elements or one, but it is ", scale_real.scalar_type(),
                " with ", scale_real.numel());
    if (pertoken_real.defined()) {
        TORCH_CHECK(pertoken_real.scalar_type() == at::kFloat && pertoken_real.numel() == M,
                    "pertoken_scale should be float32 with M=", M, " elements, but it is ",
                    pertoken_real.scalar_type(), " with ", pertoken_real.numel());
    }
    at::ScalarType out_type = at::kBFloat16;
    if (bias_real.defined()) {
        TORCH_CHECK(bias_real.numel() == N, "bias should have N=", N, " elements, but it has ", bias_real.numel());
        TORCH_CHECK(bias_real.scalar_type() == at::kBFloat16 || bias_real.scalar_type() == at::kHalf ||
                        bias_real.scalar_type() == at::kFloat,
                    "bias should be bfloat16, float16 or float32, but it is ", bias_real.scalar_type());
        if (bias_real.scalar_type() == at::kHalf) {
            out_type = at::kHalf;  // the output follows a 16-bit bias, bfloat16 otherwise
        }
    }

    auto output_size = {M, N};
    at::Tensor result = at::empty(output_size, x1.options().dtype(out_type));
    std::string hcom_str(hcom);
    std::string reduce_op_str(reduce_op);

    at::Tensor a = x1.contiguous();
    at::Tensor b = x2;
    const bool b_row_major = (b.stride(1) == 1 || N == 1) && (b.stride(0) >= N || K <= 1);
    const bool b_col_major = (b.stride(0) == 1 || K == 1) && (b.stride(1) >= K || N <= 1);
    if (!b_row_major && !b_col_major) {
        b = x2.contiguous();
    }
    const bool as_row_major = b_row_major || !b_col_major;
    const int64_t stride_k = as_row_major ? std::max<int64_t>(b.stride(0), N) : 1;
    const int64_t stride_n = as_row_major ? 1 : std::max<int64_t>(b.stride(1), K);
    at::Tensor scale_c = scale_real.contiguous();
    at::Tensor pertoken_c = pertoken_real.defined() ? pertoken_real.contiguous() : pertoken_real;
    at::Tensor bias_c = bias_real.defined() ? bias_real.contiguous() : bias_real;

    size_t workspace_size = 0;
    EXEC_QMM_CMD(qmm_quant_matmul_workspace_size, M, N, K, QMM_ALGO_AUTO, &workspace_size);
    at::Tensor workspace = op_plugin_utils::qmm_workspace(a, workspace_size);
    const int ret = qmm_mm_all_reduce(
        static_cast<const int8_t *>(a.const_data_ptr()), std::max<int64_t>(K, 1),
        static_cast<const int8_t *>(b.const_data_ptr()), stride_k, stride_n,
        static_cast<const float *>(scale_c.const_data_ptr()), scale_c.numel(),
        static_cast<const float *>(op_plugin_utils::opt_ptr(pertoken_c)), op_plugin_utils::opt_ptr(bias_c),
        bias_c.defined() ? op_plugin_utils::qmm_dtype(bias_c.scalar_type()) : QMM_DTYPE_NONE, result.data_ptr(),
        op_plugin_utils::qmm_dtype(out_type), N, M, N, K, hcom_str.c_str(), reduce_op_str.c_str(), comm_turn,
        workspace.defined() ? workspace.data_ptr() : nullptr, workspace_size, op_plugin_utils::current_stream(a));
    if (ret == QMM_ERR_DEVICE_TIMEOUT) {
        // an earlier kernel was cut short: its scratch may hold partial sums, hand out fresh buffers from now on
        op_plugin_utils::qmm_workspace_reset();
    }
    TORCH_CHECK(ret == 0, "call qmm_mm_all_reduce failed, detail:", qmm_last_error());
    return result;
}

}  // namespace op_api
