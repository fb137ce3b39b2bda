// npu_mm_reduce_scatter_base: matmul whose result is summed over the ranks of a communicator and
// scattered by rows.
//
// Host function after the reference's
// (op_plugin/ops/base_ops/opapi/MatmulReduceScatterBaseKernelNpuOpApi.cpp:22-42): the same four checks,
// the output [M / world_size, N] allocated from the options of `self`, the communicator passed by
// name, arguments forwarded in the order inputs, attributes, outputs.  The device side is
// qmm_mm_reduce_scatter: a tcgen05 bf16/f16 matmul whose epilogue delivers its fp32 rows to the
// ranks that own them, and one reduce kernel per rank.
#include <string>

#include "op_plugin/OpApiInterface.h"
#include "op_plugin/utils/qmm_api_common.h"

namespace op_api {

at::Tensor npu_mm_reduce_scatter_base(const at::Tensor &self, const at::Tensor &x2, c10::string_view hcom,
                                      int64_t world_size, c10::string_view reduce_op,
                                      const c10::optional<at::Tensor> &bias, int64_t comm_turn)
{
    TORCH_CHECK(world_size > 0, "world_size should be greater than 0, but the actual value is ", world_size);
    TORCH_CHECK(self.dim() == 2 && x2.dim() == 2, "Both inputs of mm are required to be 2D, but the actual inputs are ",
                self.dim(), "D and ", x2.dim(), "D");
    TORCH_CHECK(self.size(1) == x2.size(0),
                "The K-axis in the two inputs of Matmul must be equal, but in reality, the K-axis of x1 is ",
                self.size(1), " and the K-axis of x2 is ", x2.size(0));
    TORCH_CHECK(self.size(0) % world_size == 0, "The M-axis in input of Matmul should be be divisible by world_size");
    TORCH_CHECK(self.is_cuda() && x2.is_cuda(), "npu_mm_reduce_scatter_base expects CUDA tensors, but self is on ",
                self.device(), " and x2 is on ", x2.device());
    TORCH_CHECK((self.scalar_type() == at::kHalf || self.scalar_type() == at::kBFloat16) &&
                    x2.scalar_type() == self.scalar_type(),
                "npu_mm_reduce_scatter_base multiplies float16 or bfloat16 inputs of one dtype, but the actual dtypes are ",
                self.scalar_type(), " and ", x2.scalar_type());
    TORCH_CHECK(reduce_op == "sum", "reduce_op of npu_mm_reduce_scatter_base should be 'sum', but it is '",
                std::string(reduce_op), "'");
    TORCH_CHECK(comm_turn >= 0, "comm_turn should be non-negative, but the actual value is ", comm_turn);
    c10::cuda::CUDAGuard guard(self.device());
    std::string hcom_str(hcom);
    std::string reduce_op_str(reduce_op);
    int nranks = 0;
    int rank = 0;
    EXEC_QMM_CMD(qmm_comm_info, hcom_str.c_str(), &nranks, &rank);
    TORCH_CHECK(nranks == world_size, "world_size=", world_size, " does not match the size of communicator '", hcom_str,
                "' (", nranks, ")");

    const int64_t M = self.size(0);
    const int64_t K = self.size(1);
    const int64_t N = x2.size(1);
    auto output_size = {M / world_size, N};
    at::Tensor result = at::empty(output_size, self.options());
    const at::Tensor &bias_real = bias.value_or(at::Tensor());
    if (bias_real.defined()) {
        TORCH_CHECK(bias_real.scalar_type() == self.scalar_type() && bias_real.numel() == N,
                    "bias should have the dtype of self and N=", N, " elements, but it is ", bias_real.scalar_type(),
                    " with ", bias_real.numel());
    }
    if (result.numel() == 0) {
        return result;
    }
    at::Tensor a = self.contiguous();
    at::Tensor b = x2;
    op_plugin_utils::MatmulOperandB bdesc = op_plugin_utils::describe_operand_b(b, K, N);
    at::Tensor bias_c = bias_real.defined() ? bias_real.contiguous() : bias_real;
    size_t workspace_size = 0;
    EXEC_QMM_CMD(qmm_mm_reduce_scatter_workspace_size, M, N, K, nranks, &workspace_size);
    // the fp32 partial is only needed when NCCL carries the reduction; the library says which path it takes by
    // refusing a missing workspace, so one is always offered (from the caching allocator: no allocation in steady state)
    at::Tensor workspace = at::empty({static_cast<int64_t>(workspace_size)}, self.options().dtype(at::kByte));
    EXEC_QMM_CMD(qmm_mm_reduce_scatter, a.const_data_ptr(), op_plugin_utils::qmm_dtype(a.scalar_type()),
                 std::max<int64_t>(K, 1), bdesc.tensor.const_data_ptr(), bdesc.stride_k, bdesc.stride_n,
                 op_plugin_utils::opt_ptr(bias_c), result.data_ptr(), N, M, N, K, hcom_str.c_str(),
                 reduce_op_str.c_str(), comm_turn, workspace.data_ptr(), workspace_size,
                 op_plugin_utils::current_stream(a));
    return result;
}

}  // namespace op_api
