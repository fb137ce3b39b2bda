// npu_all_gather_base_mm: x1 is gathered over the ranks of a communicator along its rows and
// multiplied by this rank's x2.
//
// Host function after the reference's
// (op_plugin/ops/base_ops/opapi/AllGatherBaseMatmulKernelNpuOpApi.cpp:22-60): the same two checks and
// the same two output-size helpers (the matmul output has world_size times the rows of x1; the gather
// output is x1's shape with world_size times the rows, or an empty tensor when gather_output is false).
// The device side is qmm_all_gather_mm.  Only gather_index == 0 exists here.
#include <string>

#include "op_plugin/OpApiInterface.h"
#include "op_plugin/utils/qmm_api_common.h"

namespace op_api {

static c10::SmallVector<int64_t, 2> get_output_size_gather_mm(const at::Tensor &x1, const at::Tensor &x2,
                                                              int64_t world_size, int64_t gather_index)
{
    const int64_t out_x = gather_index == 0 ? x1.size(0) * world_size : x1.size(0);
    return {out_x, x2.size(1)};
}

static c10::SmallVector<int64_t, 2> get_output_size_gather(const at::Tensor &x1, const at::Tensor &x2,
                                                           int64_t world_size, int64_t gather_index)
{
    const at::Tensor &gather_out = gather_index == 0 ? x1 : x2;
    return {gather_out.size(0) * world_size, gather_out.size(1)};
}

::std::tuple<at::Tensor, at::Tensor> npu_all_gather_base_mm(const at::Tensor &self, const at::Tensor &x2,
                                                            c10::string_view hcom, int64_t world_size,
                                                            const c10::optional<at::Tensor> &bias,
                                                            int64_t gather_index, bool gather_output,
                                                            int64_t comm_turn)
{
    TORCH_CHECK(self.dim() == 2 && x2.dim() == 2, "Both inputs of mm are required to be 2D, but the actual inputs are ",
                self.dim(), "D and ", x2.dim(), "D");
    TORCH_CHECK(self.size(1) == x2.size(0),
                "The K-axis in the two inputs of Matmul must be equal, but in reality, the K-axis of x1 is ",
                self.size(1), " and the K-axis of x2 is ", x2.size(0));
    TORCH_CHECK(world_size > 0, "world_size should be greater than 0, but the actual value is ", world_size);
    TORCH_CHECK(gather_index == 0, "npu_all_gather_base_mm of this build gathers x1 (gather_index=0), but the actual "
                "value is ", gather_index);
    TORCH_CHECK(self.is_cuda() && x2.is_cuda(), "npu_all_gather_base_mm expects CUDA tensors, but self is on ",
                self.device(), " and x2 is on ", x2.device());
    TORCH_CHECK((self.scalar_type() == at::kHalf || self.scalar_type() == at::kBFloat16) &&
                    x2.scalar_type() == self.scalar_type(),
                "npu_all_gather_base_mm multiplies float16 or bfloat16 inputs of one dtype, but the actual dtypes are ",
                self.scalar_type(), " and ", x2.scalar_type());
    TORCH_CHECK(comm_turn >= 0, "comm_turn should be non-negative, but the actual value is ", comm_turn);
    c10::cuda::CUDAGuard guard(self.device());
    std::string hcom_str(hcom);
    int nranks = 0;
    int rank = 0;
    EXEC_QMM_CMD(qmm_comm_info, hcom_str.c_str(), &nranks, &rank);
    TORCH_CHECK(nranks == world_size, "world_size=", world_size, " does not match the size of communicator '", hcom_str,
                "' (", nranks, ")");

    auto out_gather_mm_size = get_output_size_gather_mm(self, x2, world_size, gather_index);
    auto out_gather_size = get_output_size_gather(self, x2, world_size, gather_index);
    at::Tensor out_gather_mm = at::empty(out_gather_mm_size, self.options());
    at::Tensor out_gather = at::empty({0}, self.options());
    if (gather_output) {
        out_gather = at::empty(out_gather_size, self.options());
    }
    const int64_t M = self.size(0);
    const int64_t K = self.size(1);
    const int64_t N = x2.size(1);
    const at::Tensor &bias_real = bias.value_or(at::Tensor());
    if (bias_real.defined()) {
        TORCH_CHECK(bias_real.scalar_type() == self.scalar_type() && bias_real.numel() == N,
                    "bias should have the dtype of self and N=", N, " elements, but it is ", bias_real.scalar_type(),
                    " with ", bias_real.numel());
    }
    if (M == 0) {
        return std::tie(out_gather_mm, out_gather);
    }
    at::Tensor a = self.contiguous();
    op_plugin_utils::MatmulOperandB bdesc = op_plugin_utils::describe_operand_b(x2, K, N);
    at::Tensor bias_c = bias_real.defined() ? bias_real.contiguous() : bias_real;
    size_t workspace_size = 0;
    at::Tensor workspace;
    if (!gather_output) {
        EXEC_QMM_CMD(qmm_all_gather_mm_workspace_size, M, N, K, nranks, &workspace_size);
        workspace = at::empty({static_cast<int64_t>(workspace_size)}, self.options().dtype(at::kByte));
    }
    EXEC_QMM_CMD(qmm_all_gather_mm, a.const_data_ptr(), op_plugin_utils::qmm_dtype(a.scalar_type()),
                 std::max<int64_t>(K, 1), bdesc.tensor.const_data_ptr(), bdesc.stride_k, bdesc.stride_n,
                 op_plugin_utils::opt_ptr(bias_c), out_gather_mm.data_ptr(), N,
                 gather_output ? out_gather.data_ptr() : nullptr, std::max<int64_t>(K, 1), M, N, K, hcom_str.c_str(),
                 gather_index, comm_turn, workspace.defined() ? workspace.data_ptr() : nullptr, workspace_size,
                 op_plugin_utils::current_stream(a));
    return std::tie(out_gather_mm, out_gather);
}

}  // namespace op_api
