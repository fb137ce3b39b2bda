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

at::Tensor qmm_workspace(const at::Tensor &like, size_t bytes, int family)
{
    static std::mutex mutex;
    // leaked on purpose: tensors must not be destroyed after the CUDA runtime at process exit
    static auto &cache = *new std::map<std::tuple<int, int, void *>, at::Tensor>();
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
