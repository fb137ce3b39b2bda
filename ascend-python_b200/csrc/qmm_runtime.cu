// Host-side runtime shared by all entry points: last-error text, the device
// status word, SM count cache and tensor-map encoding.
//
// Error convention mirrors the reference launch boundary: status 0 is success,
// anything else carries a message the caller turns into a TORCH_CHECK failure
// (op_plugin/utils/op_api_common.h:546,555 use aclGetRecentErrMsg() the same way).
#include <cudaTypedefs.h>

#include <mutex>

#include "qmm_common.cuh"

namespace qmm {

static thread_local std::string g_last_error;

void set_last_error(const std::string &msg) { g_last_error = msg; }

int fail(int code, const std::string &msg) {
    g_last_error = msg;
    return code;
}

static std::mutex g_mutex;
static uint32_t *g_status_host = nullptr;
static uint32_t *g_status_dev = nullptr;

uint32_t *device_status_word() {
    std::lock_guard<std::mutex> lock(g_mutex);
    if (g_status_dev == nullptr) {
        void *h = nullptr;
        if (cudaHostAlloc(&h, 64, cudaHostAllocMapped | cudaHostAllocPortable) != cudaSuccess) {
            (void)cudaGetLastError();
            return nullptr;
        }
        memset(h, 0, 64);
        void *d = nullptr;
        if (cudaHostGetDevicePointer(&d, h, 0) != cudaSuccess) {
            (void)cudaGetLastError();
            cudaFreeHost(h);
            return nullptr;
        }
        g_status_host = static_cast<uint32_t *>(h);
        g_status_dev = static_cast<uint32_t *>(d);
    }
    return g_status_dev;
}

// Counts the times a non-zero status word was cleared: device-side state that a kernel leaves behind only
// when it completes (arrival counters) is cleaned by its owner when this number has moved.
static uint64_t g_status_generation = 1;

// Current value of the status word as the host sees it (0 if it was never created); `clear` resets it.
uint32_t device_status_peek(bool clear) {
    std::lock_guard<std::mutex> lock(g_mutex);
    if (g_status_host == nullptr) return 0;
    const uint32_t v = *reinterpret_cast<volatile uint32_t *>(g_status_host);
    if (clear && v != 0) {
        *reinterpret_cast<volatile uint32_t *>(g_status_host) = 0;
        ++g_status_generation;
    }
    return v;
}

uint64_t device_status_generation() {
    std::lock_guard<std::mutex> lock(g_mutex);
    return g_status_generation;
}

int sm_count() {
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

static PFN_cuTensorMapEncodeTiled_v12000 get_encode_fn() {
    static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess) {
            fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(p);
        } else {
            (void)cudaGetLastError();
        }
    });
    return fn;
}

int make_tmap_2d(CUtensorMap *map, const void *base, int elem_bytes, uint64_t inner, uint64_t outer, uint64_t ld,
                 uint32_t box_inner, uint32_t box_outer, bool swizzle128) {
    auto fn = get_encode_fn();
    if (fn == nullptr) return fail(QMM_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    if ((reinterpret_cast<uintptr_t>(base) & 15) != 0)
        return fail(QMM_ERR_UNSUPPORTED, "tensor map: base address is not 16-byte aligned");
    if (((ld * elem_bytes) & 15) != 0)
        return fail(QMM_ERR_UNSUPPORTED, "tensor map: row pitch is not a multiple of 16 bytes");
    CUtensorMapDataType dt = elem_bytes == 1   ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                             : elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_UINT16
                                               : CU_TENSOR_MAP_DATA_TYPE_UINT32;
    cuuint64_t dims[2] = {inner, outer};
    cuuint64_t strides[1] = {ld * static_cast<uint64_t>(elem_bytes)};
    cuuint32_t box[2] = {box_inner, box_outer};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, dt, 2, const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(QMM_ERR_CUDA, "cuTensorMapEncodeTiled failed with code " + std::to_string(r));
    return QMM_OK;
}

}  // namespace qmm

extern "C" {

const char *qmm_last_error(void) { return qmm::g_last_error.c_str(); }

int qmm_version(void) { return 100; }

int qmm_device_status(int reset) {
    (void)qmm::device_status_word();
    std::lock_guard<std::mutex> lock(qmm::g_mutex);
    if (qmm::g_status_host == nullptr) return 0;
    int v = static_cast<int>(*reinterpret_cast<volatile uint32_t *>(qmm::g_status_host));
    if (reset && v != 0) {
        *reinterpret_cast<volatile uint32_t *>(qmm::g_status_host) = 0;
        ++qmm::g_status_generation;
    }
    return v;
}
}
