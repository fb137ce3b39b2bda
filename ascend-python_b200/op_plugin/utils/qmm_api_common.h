// Launch boundary between the operator host functions and the kernel library.
//
// Counterpart of the reference's op_plugin/utils/op_api_common.h: there
// `EXEC_NPU_CMD(aclnnX, args...)` (:520-570) resolves two C symbols, queries a
// workspace size, allocates the workspace from the caching allocator and
// enqueues the launch on the current stream, turning a non-zero status into a
// TORCH_CHECK failure that quotes the library's error text (:546,555).
// `EXEC_QMM_CMD(qmm_x, args...)` keeps that contract for libqmm_b200: plain
// pointers and sizes go in, the current CUDA stream is the last argument by
// convention of each entry point, status 0 is success.  CUDA launches are
// asynchronous already, so there is no task queue and no executor cache.
#ifndef OP_PLUGIN_UTILS_QMM_API_COMMON_H_
#define OP_PLUGIN_UTILS_QMM_API_COMMON_H_

#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

#include "qmm_b200.h"

#define EXEC_QMM_CMD(qmm_api, ...)                                                              \
    do {                                                                                        \
        int qmm_api_ret = qmm_api(__VA_ARGS__);                                                 \
        TORCH_CHECK(qmm_api_ret == 0, "call " #qmm_api " failed, detail:", qmm_last_error());   \
    } while (false)

namespace op_plugin_utils {

// Element type code of the C ABI for a tensor dtype (QMM_DTYPE_NONE if it has none).
int qmm_dtype(at::ScalarType t);

// Current CUDA stream of `device` as the `void*` the C ABI takes.
void *current_stream(const at::Tensor &like);

// Zero-initialised scratch of at least `bytes`, cached per (device, stream) and
// grown on demand.  The kernels that use it leave it zeroed, so one buffer is
// reused by consecutive launches of the same stream (stream order serializes them).
// `family` separates kernel families: each relies on the state it left in its own buffer.
at::Tensor qmm_workspace(const at::Tensor &like, size_t bytes, int family = 0);

// Drops every cached scratch buffer: the next request gets a fresh zero-filled one.  For the case that a kernel
// was cut short (a bounded device-side wait gave up) and left its scratch in an unknown state.
void qmm_workspace_reset();

// The second matmul operand as the C ABI addresses it, x2[k * stride_k + n * stride_n] with one unit stride:
// a row-major [K, N] tensor and the transposed view of a row-major [N, K] tensor are taken as stored
// (cf. the transpose-aware matmul of the reference, op_plugin/ops/base_ops/aclops/MmKernelNpu.cpp:40-53),
// anything else is made contiguous first.
struct MatmulOperandB {
    at::Tensor tensor;
    int64_t stride_k;
    int64_t stride_n;
};
MatmulOperandB describe_operand_b(const at::Tensor &x2, int64_t K, int64_t N);

// data pointer of an optional tensor (nullptr when absent)
inline const void *opt_ptr(const at::Tensor &t) { return t.defined() ? t.const_data_ptr() : nullptr; }

}  // namespace op_plugin_utils

#endif  // OP_PLUGIN_UTILS_QMM_API_COMMON_H_
