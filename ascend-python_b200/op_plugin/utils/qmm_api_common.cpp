#include "op_plugin/utils/qmm_api_common.h"

#include <map>
#include <mutex>
#include <tuple>
#include <utility>

namespace op_plugin_utils {

int qmm_dtype(at::ScalarType t)
{
    switch (t) {
        case at::kBFloat16:
            return QMM_DTYPE_BF16;
        case at::kHalf:
            return QMM_DTYPE_F16;
        case at::kFloat:
            return QMM_DTYPE_F32;
        case at::kInt:
            return QMM_DTYPE_I32;
        default:
            return QMM_DTYPE_NONE;
    }
}

void *current_stream(const at::Tensor &like)
{
    return static_cast<void *>(at::cuda::getCurrentCUDAStream(like.device().index()).stream());
}

namespace {
std::mutex &workspace_mutex()
{
    static std::mutex m;
    return m;
}
std::map<std::tuple<int, int, void *>, at::Tensor> &workspace_cache()
{
    // leaked on purpose: tensors must not be destroyed after the CUDA runtime at process exit
    static auto &cache = *new std::map<std::tuple<int, int, void *>, at::Tensor>();
    return cache;
}
}  // namespace

void qmm_workspace_reset()
{
    std::lock_guard<std::mutex> lock(workspace_mutex());
    workspace_cache().clear();
}

MatmulOperandB describe_operand_b(const at::Tensor &x2, int64_t K, int64_t N)
{
    MatmulOperandB d;
    d.tensor = x2;
    const bool row_major = (x2.stride(1) == 1 || N == 1) && (x2.stride(0) >= N || K <= 1);
    const bool col_major = (x2.stride(0) == 1 || K == 1) && (x2.stride(1) >= K || N <= 1);
    if (!row_major && !col_major) {
        d.tensor = x2.contiguous();
    }
    const bool as_row_major = row_major || !col_major;
    d.stride_k = as_row_major ? std::max<int64_t>(d.tensor.stride(0), N) : 1;
    d.stride_n = as_row_major ? 1 : std::max<int64_t>(d.tensor.stride(1), K);
    return d;
}

at::Tensor qmm_workspace(const at::Tensor &like, size_t bytes, int family)
{
    std::mutex &mutex = workspace_mutex();
    auto &cache = workspace_cache();
    if (bytes == 0) {
        return at::Tensor();
    }
    std::lock_guard<std::mutex> lock(mutex);
    auto key = std::make_tuple(family, static_cast<int>(like.device().index()), current_stream(like));
    auto it = cache.find(key);
    if (it == cache.end() || static_cast<size_t>(it->second.numel()) < bytes) {
        at::Tensor ws = at::zeros({static_cast<int64_t>(bytes)}, like.options().dtype(at::kByte));
        cache[key] = ws;
        return ws;
    }
    return it->second;
}

}  // namespace op_plugin_utils
