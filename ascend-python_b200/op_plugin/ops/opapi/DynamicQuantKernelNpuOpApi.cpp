// npu_dynamic_quant: per-token symmetric int8 quantization of activations.
//
// The operator is not part of the reference snapshot; the host conventions
// follow its nearest relatives: output dtype/allocation as in
// op_plugin/ops/base_ops/aclops/QuantizePerChannelKernelNpu.cpp:69-92, the
// (values, fp32 statistics) tuple as in
// op_plugin/ops/base_ops/opapi/RmsNormKernelOpApi.cpp:24-35.
#include "op_plugin/OpApiInterface.h"
#include "op_plugin/utils/qmm_api_common.h"

namespace op_api {

::std::tuple<at::Tensor, at::Tensor> npu_dynamic_quant(const at::Tensor &input,
                                                       const c10::optional<at::Tensor> &smooth_scales)
{
    TORCH_CHECK(input.is_cuda(), "npu_dynamic_quant expects a CUDA tensor, but the input is on ", input.device());
    TORCH_CHECK(input.dim() >= 1, "The input of npu_dynamic_quant should have at least 1 dimension, but it has ",
                input.dim());
    TORCH_CHECK(input.scalar_type() == at::kBFloat16 || input.scalar_type() == at::kHalf,
                "The input of npu_dynamic_quant should be bfloat16 or float16, but the actual dtype is ",
                input.scalar_type());
    TORCH_CHECK(!smooth_scales.has_value() || !smooth_scales->defined(),
                "npu_dynamic_quant: smooth_scales is not supported by this build, pass None");
    c10::cuda::CUDAGuard guard(input.device());

    const int64_t cols = input.size(-1);
    const int64_t rows = cols == 0 ? 0 : input.numel() / cols;
    at::Tensor x = input.contiguous();
    at::Tensor y = at::empty(input.sizes(), input.options().dtype(at::kChar));
    at::Tensor scale = at::empty(input.sizes().slice(0, input.dim() - 1), input.options().dtype(at::kFloat));
    if (input.numel() == 0) {
        scale.zero_();
        return ::std::tuple<at::Tensor, at::Tensor>(y, scale);
    }
    EXEC_QMM_CMD(qmm_dynamic_quant, x.const_data_ptr(), op_plugin_utils::qmm_dtype(x.scalar_type()), rows, cols, cols,
                 static_cast<int8_t *>(y.data_ptr()), cols, static_cast<float *>(scale.data_ptr()),
                 op_plugin_utils::current_stream(x));
    return ::std::tuple<at::Tensor, at::Tensor>(y, scale);
}

}  // namespace op_api
