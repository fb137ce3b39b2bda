// npu_rms_norm and npu_rms_norm_dynamic_quant.
//
// npu_rms_norm mirrors the reference host function
// (op_plugin/ops/base_ops/opapi/RmsNormKernelOpApi.cpp:24-35): y takes the input's
// options, rstd is fp32 with the shape of the input whose normalised (trailing,
// gamma-shaped) dimensions are 1, and the call order is inputs, attribute, outputs.
// npu_rms_norm_dynamic_quant has no counterpart there: it is that operator fused with
// npu_dynamic_quant, the step that consumes y in a quantized decoder block, and returns
// (int8 values, per-token scale, rstd).
#include "op_plugin/OpApiInterface.h"
#include "op_plugin/utils/qmm_api_common.h"

namespace op_api {

namespace {

void check_rms_norm_inputs(const char *op, const at::Tensor &self, const at::Tensor &gamma, bool allow_float)
{
    TORCH_CHECK(self.is_cuda() && gamma.is_cuda(), op, " expects CUDA tensors, but self is on ", self.device(),
                " and gamma is on ", gamma.device());
    TORCH_CHECK(self.dim() >= 1 && gamma.dim() >= 1 && gamma.dim() <= self.dim(), op,
                ": self should have at least as many dimensions as gamma, but they have ", self.dim(), " and ",
                gamma.dim());
    for (int64_t i = 1; i <= gamma.dim(); ++i) {
        TORCH_CHECK(self.size(-i) == gamma.size(-i), op,
                    ": the trailing dimensions of self must equal the shape of gamma, but self is ", self.sizes(),
                    " and gamma is ", gamma.sizes());
    }
    const auto t = self.scalar_type();
    TORCH_CHECK(t == at::kBFloat16 || t == at::kHalf || (allow_float && t == at::kFloat), op,
                ": unsupported dtype ", t);
    TORCH_CHECK(gamma.scalar_type() == t, op, ": gamma should have the dtype of self (", t, "), but it is ",
                gamma.scalar_type());
    TORCH_CHECK(gamma.numel() > 0, op, ": gamma must not be empty");
}

std::vector<int64_t> rstd_sizes(const at::Tensor &self, const at::Tensor &gamma)
{
    auto sizes = self.sizes().vec();
    for (int64_t i = 1; i <= gamma.dim(); ++i) {
        sizes[sizes.size() - i] = 1;
    }
    return sizes;
}

}  // namespace

::std::tuple<at::Tensor, at::Tensor> npu_rms_norm(const at::Tensor &self, const at::Tensor &gamma, double epsilon)
{
    check_rms_norm_inputs("npu_rms_norm", self, gamma, /*allow_float=*/true);
    c10::cuda::CUDAGuard guard(self.device());
    at::Tensor y = at::empty(self.sizes(), self.options());
    at::Tensor rstd = at::empty(rstd_sizes(self, gamma), self.options().dtype(at::kFloat));
    if (self.numel() == 0) {
        return ::std::tuple<at::Tensor, at::Tensor>(y, rstd);
    }
    const int64_t cols = gamma.numel();
    const int64_t rows = self.numel() / cols;
    at::Tensor x = self.contiguous();
    at::Tensor g = gamma.contiguous();
    EXEC_QMM_CMD(qmm_rms_norm, x.const_data_ptr(), op_plugin_utils::qmm_dtype(x.scalar_type()), rows, cols, cols,
                 g.const_data_ptr(), epsilon, y.data_ptr(), cols, static_cast<float *>(rstd.data_ptr()),
                 op_plugin_utils::current_stream(x));
    return ::std::tuple<at::Tensor, at::Tensor>(y, rstd);
}

::std::tuple<at::Tensor, at::Tensor, at::Tensor> npu_rms_norm_dynamic_quant(const at::Tensor &self,
                                                                            const at::Tensor &gamma, double epsilon)
{
    check_rms_norm_inputs("npu_rms_norm_dynamic_quant", self, gamma, /*allow_float=*/false);
    TORCH_CHECK(gamma.dim() == 1, "npu_rms_norm_dynamic_quant: gamma should be 1D (the token dimension is the last "
                "one), but it has ", gamma.dim(), " dimensions");
    c10::cuda::CUDAGuard guard(self.device());
    at::Tensor q = at::empty(self.sizes(), self.options().dtype(at::kChar));
    at::Tensor scale = at::empty(self.sizes().slice(0, self.dim() - 1), self.options().dtype(at::kFloat));
    at::Tensor rstd = at::empty(rstd_sizes(self, gamma), self.options().dtype(at::kFloat));
    if (self.numel() == 0) {
        scale.zero_();
        return ::std::tuple<at::Tensor, at::Tensor, at::Tensor>(q, scale, rstd);
    }
    const int64_t cols = gamma.numel();
    const int64_t rows = self.numel() / cols;
    at::Tensor x = self.contiguous();
    at::Tensor g = gamma.contiguous();
    EXEC_QMM_CMD(qmm_rms_norm_dynamic_quant, x.const_data_ptr(), op_plugin_utils::qmm_dtype(x.scalar_type()), rows,
                 cols, cols, g.const_data_ptr(), epsilon, static_cast<int8_t *>(q.data_ptr()), cols,
                 static_cast<float *>(scale.data_ptr()), static_cast<float *>(rstd.data_ptr()),
                 op_plugin_utils::current_stream(x));
    return ::std::tuple<at::Tensor, at::Tensor, at::Tensor>(q, scale, rstd);
}

}  // namespace op_api
