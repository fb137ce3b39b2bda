// npu_weight_quant_batchmatmul: activations in bf16/f16, weights in packed int4
// with per-group (or per-channel) antiquant scale and offset.
//
// Host conventions follow the reference's dense matmul
// (op_plugin/ops/base_ops/opapi/MmKernelNpuOpApi.cpp:24-42) and the optional
// bias handling of op_plugin/ops/base_ops/aclops/LinearKernelNpu.cpp:29-45.
// Weight layout: int32 tensor [K, N/8]; nibble j of word i is column 8*i+j,
// two's complement.  W = (w + antiquant_offset) * antiquant_scale.
//
// Weight format.  The reference keeps matmul weights in a private device format and casts between it and
// the plain layout around the matmul (ND <-> FRACTAL_NZ, op_plugin/ops/base_ops/aclops/MmKernelNpu.cpp:80-94,
// :301-316).  The counterpart here is the k-major int4 stream of qmm_w4a16_prepack: the first call that
// benefits from it (more than eight token rows) rewrites the weight once, and a cache keyed by the data
// pointers of weight, scale and offset serves every later call.  An entry stays valid while the three
// storages are alive and their version counters are unchanged (an in-place update re-packs); the cache holds
// a second copy of the weights, bounded by QMM_W4_PREPACK_MAX_MB (default 16384; QMM_W4_PREPACK=0 switches
// the format off).  Callers that want a single copy prepack explicitly through the C ABI and drop the original.
#include <cstdlib>
#include <map>
#include <mutex>
#include <optional>
#include <tuple>

#include "op_plugin/OpApiInterface.h"
#include "op_plugin/utils/qmm_api_common.h"

namespace op_api {

namespace {

struct PrepackEntry {
    at::Tensor packed;
    std::optional<c10::weak_intrusive_ptr<c10::StorageImpl>> storages[3];
    uint32_t versions[3] = {0, 0, 0};
};

using PrepackKey = std::tuple<const void *, const void *, const void *, int64_t, int64_t, int64_t, int>;

uint32_t version_of(const at::Tensor &t)
{
    return t.is_inference() ? 0u : t.unsafeGetTensorImpl()->version_counter().current_version();
}

bool prepack_enabled()
{
    static const bool on = [] {
        const char *e = std::getenv("QMM_W4_PREPACK");
        return !(e != nullptr && std::string(e) == "0");
    }();
    return on;
}

size_t prepack_budget_bytes()
{
    static const size_t n = [] {
        const char *e = std::getenv("QMM_W4_PREPACK_MAX_MB");
        const long long mb = e ? std::atoll(e) : 16384;
        return static_cast<size_t>(mb < 0 ? 0 : mb) << 20;
    }();
    return n;
}

// The prepacked form of (weight, scale, offset), from the cache or packed now; undefined when the shape has
// no prepacked form or the budget is exhausted.
at::Tensor prepacked_weight(const at::Tensor &w, const at::Tensor &scale, const at::Tensor &offset, int64_t group,
                            int64_t N, int64_t K)
{
    static std::mutex mutex;
    // leaked on purpose: tensors must not be destroyed after the CUDA runtime at process exit
    static auto &cache = *new std::map<PrepackKey, PrepackEntry>();
    static size_t cached_bytes = 0;
    size_t bytes = 0;
    EXEC_QMM_CMD(qmm_w4a16_prepack_size, N, K, group, &bytes);
    if (bytes == 0) {
        return at::Tensor();
    }
    const at::Tensor *parts[3] = {&w, &scale, &offset};
    const PrepackKey key{w.const_data_ptr(), scale.const_data_ptr(), op_plugin_utils::opt_ptr(offset), K, N, group,
                         static_cast<int>(scale.scalar_type())};
    std::lock_guard<std::mutex> lock(mutex);
    auto it = cache.find(key);
    if (it != cache.end()) {
        bool valid = true;
        for (int i = 0; i < 3 && valid; ++i) {
            if (!it->second.storages[i].has_value()) {
                valid = !parts[i]->defined();
                continue;
            }
            auto alive = it->second.storages[i]->lock();
            valid = parts[i]->defined() && alive && alive.get() == parts[i]->storage().unsafeGetStorageImpl() &&
                    it->second.versions[i] == version_of(*parts[i]);
        }
        if (valid) {
            return it->second.packed;
        }
        cached_bytes -= static_cast<size_t>(it->second.packed.numel());
        cache.erase(it);
    }
    if (bytes > prepack_budget_bytes()) {
        return at::Tensor();
    }
    if (cached_bytes + bytes > prepack_budget_bytes()) {  // over budget: start over rather than track recency
        cache.clear();
        cached_bytes = 0;
    }
    PrepackEntry e;
    e.packed = at::empty({static_cast<int64_t>(bytes)}, w.options().dtype(at::kByte));
    EXEC_QMM_CMD(qmm_w4a16_prepack, static_cast<const int32_t *>(w.const_data_ptr()), N / 8, scale.const_data_ptr(),
                 op_plugin_utils::opt_ptr(offset), op_plugin_utils::qmm_dtype(scale.scalar_type()), group, N, K,
                 e.packed.data_ptr(), bytes, op_plugin_utils::current_stream(w));
    for (int i = 0; i < 3; ++i) {
        if (parts[i]->defined()) {
            e.storages[i].emplace(
                c10::intrusive_ptr<c10::StorageImpl>::reclaim_copy(parts[i]->storage().unsafeGetStorageImpl()));
            e.versions[i] = version_of(*parts[i]);
        }
    }
    cached_bytes += bytes;
    at::Tensor packed = e.packed;
    cache.emplace(key, std::move(e));
    return packed;
}

}  // namespace

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
    // one or two token rows (integer dot products at the speed of the weight stream) and more than eight (operand
    // unpacked into tensor memory): the kernels over the prepacked stream are the faster ones
    if (prepack_enabled() && (M <= 2 || M > 8) && K > 0) {
        at::Tensor packed = prepacked_weight(wc, sc, oc, group, N, K);
        if (packed.defined()) {
            size_t ws_size = 0;
            EXEC_QMM_CMD(qmm_weight_quant_batchmatmul_prepacked_workspace_size, M, N, K, &ws_size);
            at::Tensor ws = op_plugin_utils::qmm_workspace(xc, ws_size, /*family=*/2);
            EXEC_QMM_CMD(qmm_weight_quant_batchmatmul_prepacked, xc.const_data_ptr(),
                         op_plugin_utils::qmm_dtype(xc.scalar_type()), K, packed.const_data_ptr(),
                         static_cast<size_t>(packed.numel()), op_plugin_utils::opt_ptr(bc), result.data_ptr(), N, M, N,
                         K, ws.defined() ? ws.data_ptr() : nullptr, ws_size, op_plugin_utils::current_stream(xc));
            return result;
        }
    }
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
