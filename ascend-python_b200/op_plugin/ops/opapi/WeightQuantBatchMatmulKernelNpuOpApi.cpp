// npu_weight_quant_batchmatmul: activations in bf16/f16, weights in packed int4
// with per-group (or per-channel) antiquant scale and offset.
//
// Host conventions follow the reference's dense matmul
// (op_plugin/ops/base_ops/opapi/MmKernelNpuOpApi.cpp:24-42) and the optional
// bias handling of op_plugin/ops/base_ops/aclops/LinearKernelNpu.cpp:29-45.
// Weight layout: int32 tensor [K, N/8]; nibble j of word i is column 8*i+j,
// two's complement.  W = (w + antiquant_offset) * antiquant_scale.
#include "op_plugin/OpApiInterface.h"
#include "op_plugin/utils/qmm_api_common.h"

namespace op_api {

at::Tensor npu_weight_quant_batchmatmul(const at::Tensor &x, const at::Tensor &weight,
                                        const at::Tensor &antiquant_scale,
                                        const c10::optional<at::Tensor> &antiquant_offset,
                                        const c10::optional<at::Tensor> &quant_scale,
                                        const c10::optional<at::Tensor> &quant_offset,
                                        const c10::optional<at::Tensor> &bias, int64_t antiquant_group_size)
{
    TORCH_CHECK(x.is_cuda() && weight.is_cuda(), "npu_weight_quant_batchmatmul expects CUDA tensors, but x is on ",
                x.device(), " and weight is on ", weight.device());
    TORCH_CHECK(x.scalar_type() == at::kBFloat16 || x.scalar_type() == at::kHalf,
                "x of npu_weight_quant_batchmatmul should be bfloat16 or float16, but the actual dtype is ",
                x.scalar_type());
    TORCH_CHECK(weight.scalar_type() == at::kInt,
                "weight of npu_weight_quant_batchmatmul should be int32 (8 int4 values per element), but it is ",
                weight.scalar_type());
    TORCH_CHECK(x.dim() >= 2 && weight.dim() == 2, "x should be at least 2D and weight 2D, but the actual inputs are ",
                x.dim(), "D and ", weight.dim(), "D");
    TORCH_CHECK(x.size(-1) == weight.size(0),
                "The K-axis in the two inputs of Matmul must be equal, but in reality, the K-axis of x is ",
                x.size(-1), " and the K-axis of weight is ", weight.size(0));
    TORCH_CHECK(!quant_scale.has_value() || !quant_scale->defined(),
                "npu_weight_quant_batchmatmul: quant_scale (int8 output) is not supported by this build, pass None");
    TORCH_CHECK(!quant_offset.has_value() || !quant_offset->defined(),
                "npu_weight_quant_batchmatmul: quant_offset (int8 output) is not supported by this build, pass None");
    TORCH_CHECK(antiquant_group_size >= 0, "antiquant_group_size should be non-negative, but it is ",
                antiquant_group_size);
    c10::cuda::CUDAGuard guard(x.device());

    const int64_t K = x.size(-1);
    const int64_t N = weight.size(1) * 8;
    const int64_t M = c10::multiply_integers(x.sizes().slice(0, x.dim() - 1));
    const int64_t group = antiquant_group_size > 0 ? antiquant_group_size : K;
    TORCH_CHECK(K == 0 || (group > 0 && K % group == 0), "antiquant_group_size=", antiquant_group_size,
                " should divide K=", K);
    const int64_t ngroups = K == 0 ? 0 : K / group;
    const at::Tensor &offset_real = antiquant_offset.value_or(at::Tensor());
    const at::Tensor &bias_real = bias.value_or(at::Tensor());
    TORCH_CHECK(antiquant_scale.scalar_type() == x.scalar_type() && antiquant_scale.numel() == ngroups * N,
                "antiquant_scale should have the dtype of x and ", ngroups, "x", N, " elements, but it is ",
                antiquant_scale.scalar_type(), " with ", antiquant_scale.numel());
    if (offset_real.defined()) {
        TORCH_CHECK(offset_real.scalar_type() == x.scalar_type() && offset_real.numel() == ngroups * N,
                    "antiquant_offset should have the dtype of x and ", ngroups, "x", N, " elements, but it is ",
                    offset_real.scalar_type(), " with ", offset_real.numel());
    }
    if (bias_real.defined()) {
        TORCH_CHECK(bias_real.scalar_type() == x.scalar_type() && bias_real.numel() == N,
                    "bias should have the dtype of x and N=", N, " elements, but it is ", bias_real.scalar_type(),
                    " with ", bias_real.numel());
    }

    auto output_size = x.sizes().vec();
    output_size.back() = N;
    at::Tensor result = at::empty(output_size, x.options());
    if (result.numel() == 0) {
        return result;
    }
    at::Tensor xc = x.contiguous();
    at::Tensor wc = weight.contiguous();
    at::Tensor sc = antiquant_scale.contiguous();
    at::Tensor oc = offset_real.defined() ? offset_real.contiguous() : offset_real;
    at::Tensor bc = bias_real.defined() ? bias_real.contiguous() : bias_real;
    size_t workspace_size = 0;
    EXEC_QMM_CMD(qmm_weight_quant_batchmatmul_workspace_size, M, N, K, group, &workspace_size);
    at::Tensor workspace = op_plugin_utils::qmm_workspace(xc, workspace_size, /*family=*/1);
    EXEC_QMM_CMD(qmm_weight_quant_batchmatmul, xc.const_data_ptr(), op_plugin_utils::qmm_dtype(xc.scalar_type()),
                 std::max<int64_t>(K, 1), static_cast<const int32_t *>(wc.const_data_ptr()),
                 std::max<int64_t>(N / 8, 1), sc.const_data_ptr(), op_plugin_utils::opt_ptr(oc), group,
                 op_plugin_utils::opt_ptr(bc), result.data_ptr(), N, M, N, K,
                 workspace.defined() ? workspace.data_ptr() : nullptr, workspace_size,
                 op_plugin_utils::current_stream(xc));
    return result;
}

}  // namespace op_api
