// Communicator registry and the row-parallel W8A8 matmul + allreduce
// (npu_mm_all_reduce_base).
//
// The reference hands its fused matmul+collective kernels a communicator NAME
// (op_plugin/ops/base_ops/opapi/MatmulReduceScatterBaseKernelNpuOpApi.cpp:35-40);
// the device library resolves it.  Here a name resolves to an NCCL communicator
// plus one communication stream and a few events.  NCCL is bound at run time
// with dlopen/dlsym, the way the reference binds its device library
// (op_plugin/utils/op_api_common.h:80-123), so that the process uses the one
// libnccl its framework already loaded.
//
// Overlap (comm_turn > 1): M is cut into chunks; chunk c's matmul runs on the caller's
// stream, an event hands the finished rows to the communication stream, whose
// in-place ncclAllReduce of chunk c runs while chunk c+1 is being multiplied.
// The matmul leaves a few SMs free while a collective may be in flight.
//
// When the ranks have attached peer memory to the communicator (qmm_comm_attach_peer_memory) and the
// call fits it, NCCL is not involved: the matmul writes its partial output into this rank's region
// and one kernel per rank (peer_all_reduce.cuh) reduces and gathers over NVLink loads.
#include <cstdio>
#include <dlfcn.h>
#include <nccl.h>

#include <map>
#include <mutex>
#include <vector>

#include "dense_gemm.cuh"
#include "peer_all_reduce.cuh"
#include "peer_fused.cuh"
#include "peer_scatter_gather.cuh"
#include "qmm_common.cuh"
#include "w8a8_epilogue.cuh"

namespace qmm {

int quant_matmul_dispatch(const int8_t *x1, int64_t ld_x1, const int8_t *x2, int64_t x2_sk, int64_t x2_sn,
                          const EpilogueParams &ep, int out_dtype, int64_t K, int algo, void *workspace,
                          size_t workspace_bytes, cudaStream_t stream, LaunchOptions *opts);
int validate_quant_matmul(const int8_t *x1, int64_t ld_x1, const int8_t *x2, int64_t x2_sk, int64_t x2_sn,
                          const float *scale, int64_t scale_len, const void *bias, int bias_dtype, void *out,
                          int out_dtype, int64_t ld_out, int64_t M, int64_t N, int64_t K);

namespace {

struct NcclApi {
    void *handle = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId *) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t *, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommInitRankConfig)(ncclComm_t *, int, ncclUniqueId, int, ncclConfig_t *) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*CommAbort)(ncclComm_t) = nullptr;
    ncclResult_t (*AllReduce)(const void *, void *, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t,
                              cudaStream_t) = nullptr;
    ncclResult_t (*ReduceScatter)(const void *, void *, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t,
                                  cudaStream_t) = nullptr;
    ncclResult_t (*AllGather)(const void *, void *, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*CommGetAsyncError)(ncclComm_t, ncclResult_t *) = nullptr;
    const char *(*GetErrorString)(ncclResult_t) = nullptr;
    std::string error;
};

NcclApi &nccl() {
    static NcclApi api;
    static std::once_flag once;
    std::call_once(once, [] {
        std::vector<std::string> names;
        if (const char *env = getenv("QMM_NCCL_LIB")) names.emplace_back(env);
        names.emplace_back("libnccl.so.2");
        names.emplace_back("libnccl.so");
        for (const auto &n : names) {
            api.handle = dlopen(n.c_str(), RTLD_NOW | RTLD_GLOBAL);
            if (api.handle) break;
        }
        if (!api.handle) {
            api.error = "cannot dlopen libnccl.so.2 (set QMM_NCCL_LIB to its path)";
            return;
        }
        auto sym = [&](const char *name) -> void * {
            void *p = dlsym(api.handle, name);
            if (!p && api.error.empty()) api.error = std::string("libnccl lacks symbol ") + name;
            return p;
        };
        api.GetUniqueId = reinterpret_cast<decltype(api.GetUniqueId)>(sym("ncclGetUniqueId"));
        api.CommInitRank = reinterpret_cast<decltype(api.CommInitRank)>(sym("ncclCommInitRank"));
        // optional: absent from very old NCCL builds, then the communicator is created without a CTA cap
        api.CommInitRankConfig =
            reinterpret_cast<decltype(api.CommInitRankConfig)>(dlsym(api.handle, "ncclCommInitRankConfig"));
        api.CommDestroy = reinterpret_cast<decltype(api.CommDestroy)>(sym("ncclCommDestroy"));
        api.CommAbort = reinterpret_cast<decltype(api.CommAbort)>(sym("ncclCommAbort"));
        api.AllReduce = reinterpret_cast<decltype(api.AllReduce)>(sym("ncclAllReduce"));
        api.ReduceScatter = reinterpret_cast<decltype(api.ReduceScatter)>(sym("ncclReduceScatter"));
        api.AllGather = reinterpret_cast<decltype(api.AllGather)>(sym("ncclAllGather"));
        api.CommGetAsyncError = reinterpret_cast<decltype(api.CommGetAsyncError)>(sym("ncclCommGetAsyncError"));
        api.GetErrorString = reinterpret_cast<decltype(api.GetErrorString)>(sym("ncclGetErrorString"));
    });
    return api;
}

int nccl_ready() {
    NcclApi &a = nccl();
    if (!a.error.empty()) return fail(QMM_ERR_NCCL, a.error);
    return QMM_OK;
}

#define QMM_NCCL_OK(expr)                                                                          \
    do {                                                                                           \
        ncclResult_t _r = (expr);                                                                  \
        if (_r != ncclSuccess && _r != ncclInProgress)                                             \
            return ::qmm::fail(QMM_ERR_NCCL, std::string(#expr) + ": " + nccl().GetErrorString(_r)); \
    } while (0)

constexpr int kMaxChunks = 16;

// CTAs a collective of ours may use, and therefore SMs the matmul leaves idle while a collective can
// be in flight: the matmul's persistent CTAs fill the shared memory of the SMs they run on, so a
// collective CTA only ever lands on an SM the matmul left free; a collective that wanted more CTAs
// than that would finish only after the matmul chunk beside it, and nothing would overlap.
int comm_ctas() {
    static int n = [] {
        const char *e = getenv("QMM_COMM_MAX_CTAS");
        int v = e ? atoi(e) : 32;
        return v < 1 ? 1 : (v > 64 ? 64 : v);
    }();
    return n;
}

// Regions of all ranks of the node as mapped into this process, for the peer-memory allreduce.
struct PeerMem {
    uint8_t *base[kPeerMaxRanks] = {};
    uint8_t *mc_base = nullptr;  // the same regions through the NVLink multicast mapping, if there is one
    size_t bytes = 0;     // size of every region
    uint32_t epoch = 0;   // number of collective calls made through the regions
    uint32_t rs_calls = 0;  // reduce-scatter / all-gather calls so far (targets of their CTA counters)
    uint32_t ag_calls = 0;
    uint64_t fused_clean_gen = 0;  // device_status_generation() when the fused kernel's counters were last cleared
};

struct Comm {
    PeerMem peer;
    ncclComm_t comm = nullptr;
    int nranks = 0;
    int rank = 0;
    int device = 0;
    bool owned = false;
    int64_t stat_peer = 0;         // calls whose allreduce ran in the library's own kernel over peer memory
    int64_t stat_peer_pushed = 0;  // ... of which the matmul delivered its tiles to the owners itself
    int64_t stat_peer_fused = 0;   // ... of which the matmul kernel also reduced and gathered (no second kernel)
    int64_t stat_nccl = 0;         // calls whose allreduce NCCL carried
    cudaStream_t stream = nullptr;  // communication stream
    cudaEvent_t chunk_ready[kMaxChunks] = {};
    cudaEvent_t done = nullptr;
};

std::mutex g_comm_mutex;
std::map<std::string, Comm> g_comms;

int create_stream_events(Comm &c) {
    QMM_CUDA_OK(cudaGetDevice(&c.device));
    int lo = 0, hi = 0;
    QMM_CUDA_OK(cudaDeviceGetStreamPriorityRange(&lo, &hi));
    QMM_CUDA_OK(cudaStreamCreateWithPriority(&c.stream, cudaStreamNonBlocking, hi));
    for (auto &e : c.chunk_ready) QMM_CUDA_OK(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
    QMM_CUDA_OK(cudaEventCreateWithFlags(&c.done, cudaEventDisableTiming));
    return QMM_OK;
}

void release(Comm &c, bool abort) {
    if (c.stream) cudaStreamSynchronize(c.stream);
    if (c.owned && c.comm) {
        if (abort)
            nccl().CommAbort(c.comm);
        else
            nccl().CommDestroy(c.comm);
    }
    for (auto &e : c.chunk_ready)
        if (e) cudaEventDestroy(e);
    if (c.done) cudaEventDestroy(c.done);
    if (c.stream) cudaStreamDestroy(c.stream);
    c = Comm();
}

}  // namespace

}  // namespace qmm

extern "C" int qmm_comm_unique_id(void *id_out) {
    using namespace qmm;
    static_assert(sizeof(ncclUniqueId) <= QMM_UNIQUE_ID_BYTES, "unique id does not fit");
    QMM_REQUIRE(id_out != nullptr, "qmm_comm_unique_id: id_out is NULL");
    int rc = nccl_ready();
    if (rc != QMM_OK) return rc;
    ncclUniqueId id;
    QMM_NCCL_OK(nccl().GetUniqueId(&id));
    memset(id_out, 0, QMM_UNIQUE_ID_BYTES);
    memcpy(id_out, &id, sizeof(id));
    return QMM_OK;
}

extern "C" int qmm_comm_init_rank(const char *name, const void *id, int nranks, int rank) {
    using namespace qmm;
    QMM_REQUIRE(name != nullptr && name[0] != '\0', "qmm_comm_init_rank: empty communicator name");
    QMM_REQUIRE(id != nullptr, "qmm_comm_init_rank: id is NULL");
    QMM_REQUIRE(nranks >= 1 && rank >= 0 && rank < nranks, "qmm_comm_init_rank: rank outside [0, nranks)");
    int rc = nccl_ready();
    if (rc != QMM_OK) return rc;
    {
        std::lock_guard<std::mutex> lock(g_comm_mutex);
        if (g_comms.count(name)) return fail(QMM_ERR_INVALID_ARGUMENT, std::string("communicator '") + name +
                                                                           "' is already registered");
    }
    Comm c;
    c.nranks = nranks;
    c.rank = rank;
    c.owned = true;
    ncclUniqueId uid;
    memcpy(&uid, id, sizeof(uid));
    if (nccl().CommInitRankConfig != nullptr) {
        ncclConfig_t config = NCCL_CONFIG_INITIALIZER;
        config.maxCTAs = comm_ctas();
        QMM_NCCL_OK(nccl().CommInitRankConfig(&c.comm, nranks, uid, rank, &config));
    } else {
        QMM_NCCL_OK(nccl().CommInitRank(&c.comm, nranks, uid, rank));
    }
    rc = create_stream_events(c);
    if (rc != QMM_OK) {
        release(c, true);
        return rc;
    }
    std::lock_guard<std::mutex> lock(g_comm_mutex);
    g_comms[name] = c;
    return QMM_OK;
}

extern "C" int qmm_comm_register(const char *name, void *nccl_comm, int nranks, int rank) {
    using namespace qmm;
    QMM_REQUIRE(name != nullptr && name[0] != '\0', "qmm_comm_register: empty communicator name");
    QMM_REQUIRE(nccl_comm != nullptr, "qmm_comm_register: communicator is NULL");
    QMM_REQUIRE(nranks >= 1 && rank >= 0 && rank < nranks, "qmm_comm_register: rank outside [0, nranks)");
    int rc = nccl_ready();
    if (rc != QMM_OK) return rc;
    {
        std::lock_guard<std::mutex> lock(g_comm_mutex);
        if (g_comms.count(name)) return fail(QMM_ERR_INVALID_ARGUMENT, std::string("communicator '") + name +
                                                                           "' is already registered");
    }
    Comm c;
    c.comm = static_cast<ncclComm_t>(nccl_comm);
    c.nranks = nranks;
    c.rank = rank;
    c.owned = false;
    rc = create_stream_events(c);
    if (rc != QMM_OK) {
        release(c, true);
        return rc;
    }
    std::lock_guard<std::mutex> lock(g_comm_mutex);
    g_comms[name] = c;
    return QMM_OK;
}

namespace qmm {
namespace {

size_t align256(size_t v) { return (v + 255) / 256 * 256; }

// A region is its flags followed by two halves of equal size whose position depends on the region's
// size only: partial outputs ([M][N], or [world][rows_per][N] with rows_per rounded up to 32) in the
// first, the reduced output [M][N] in the second.  Because the halves never move, a call of one shape
// may follow a call of another without a barrier between them (see peer_all_reduce.cuh).
size_t peer_half_need(int64_t M, int64_t N, int world) {
    const int64_t rows_per = ((M + world - 1) / world + 31) / 32 * 32;
    const size_t a = align256(static_cast<size_t>(world) * rows_per * N * 2);
    const size_t b = align256(static_cast<size_t>(M) * N * 2);
    return a > b ? a : b;
}
size_t peer_half_bytes(size_t region_bytes) {
    return region_bytes <= kPeerFlagBytes ? 0 : ((region_bytes - kPeerFlagBytes) / 2) & ~static_cast<size_t>(255);
}
// Bytes of a region that an allreduce of [M][N] 16-bit values over `world` ranks needs.
size_t peer_region_bytes(int64_t M, int64_t N, int world) { return kPeerFlagBytes + 2 * peer_half_need(M, N, world); }

// Row chunks of the peer-memory path (QMM_PEER_CHUNKS, 1..8).
int peer_chunks() {
    static const int n = [] {
        const char *e = getenv("QMM_PEER_CHUNKS");
        const int v = e ? atoi(e) : 1;
        return v < 1 ? 1 : (v > 8 ? 8 : v);
    }();
    return n;
}

// QMM_PEER_PUSH=0 keeps the matmul's output local (the reduce kernel then pulls it over NVLink).
bool push_disabled() {
    static const bool off = [] {
        const char *e = getenv("QMM_PEER_PUSH");
        return e != nullptr && std::string(e) == "0";
    }();
    return off;
}

// Whether the matmul kernel also reduces and gathers (communication warps, peer_fused.cuh).  Measured on
// B200s (M=4096, K=28672, N=8192, per call): 2 ranks 360 us fused against 383 us with the separate kernel;
// 4 ranks 294-313 us against 261 us - with more ranks the 192 communication threads per SM move their share of
// the exchange more slowly than a kernel that owns the whole GPU, and the tail outgrows what was hidden.  So the
// default is fused for two ranks only; QMM_PEER_FUSED=1 forces it for any rank count, =0 switches it off.
bool fused_wanted(int nranks) {
    static const int mode = [] {
        const char *e = getenv("QMM_PEER_FUSED");
        return e == nullptr ? -1 : (std::string(e) == "0" ? 0 : 1);
    }();
    return mode < 0 ? nranks == 2 : mode == 1;
}

// Column chunks of the fused kernel (QMM_PEER_FUSED_CHUNKS, 1..8): what is left to exchange when the matmul
// ends is one chunk; every chunk costs a round of flags.
int fused_chunks() {
    static const int n = [] {
        const char *e = getenv("QMM_PEER_FUSED_CHUNKS");
        const int v = e ? atoi(e) : 4;
        return v < 1 ? 1 : (v > kFusedMaxChunks ? kFusedMaxChunks : v);
    }();
    return n;
}

bool peer_path_disabled() {
    static const bool off = [] {
        const char *e = getenv("QMM_ALLREDUCE");
        return e != nullptr && std::string(e) == "nccl";
    }();
    return off;
}

}  // namespace
}  // namespace qmm

extern "C" int qmm_comm_peer_memory_size(int64_t M, int64_t N, int nranks, size_t *bytes) {
    using namespace qmm;
    QMM_REQUIRE(bytes != nullptr, "qmm_comm_peer_memory_size: bytes is NULL");
    QMM_REQUIRE(M >= 0 && N >= 0 && nranks >= 1, "qmm_comm_peer_memory_size: bad argument");
    *bytes = peer_region_bytes(M, N, nranks);
    return QMM_OK;
}

extern "C" int qmm_comm_attach_peer_memory(const char *name, const void *const *regions, const void *multicast,
                                           size_t bytes) {
    using namespace qmm;
    QMM_REQUIRE(name != nullptr, "qmm_comm_attach_peer_memory: name is NULL");
    QMM_REQUIRE(regions != nullptr || bytes == 0, "qmm_comm_attach_peer_memory: regions is NULL");
    std::lock_guard<std::mutex> lock(g_comm_mutex);
    auto it = g_comms.find(name);
    if (it == g_comms.end())
        return fail(QMM_ERR_NOT_FOUND, std::string("communicator '") + name + "' is not registered");
    Comm &c = it->second;
    if (bytes == 0) {  // detach
        c.peer = PeerMem();
        return QMM_OK;
    }
    QMM_REQUIRE(c.nranks <= kPeerMaxRanks, "qmm_comm_attach_peer_memory: at most 8 ranks");
    QMM_REQUIRE(bytes >= kPeerFlagBytes, "qmm_comm_attach_peer_memory: region smaller than its flag area");
    PeerMem pm;
    for (int r = 0; r < c.nranks; ++r) {
        QMM_REQUIRE(regions[r] != nullptr && (reinterpret_cast<uintptr_t>(regions[r]) & 255) == 0,
                    "qmm_comm_attach_peer_memory: regions must be non-NULL and 256-byte aligned");
        pm.base[r] = static_cast<uint8_t *>(const_cast<void *>(regions[r]));
    }
    QMM_REQUIRE((reinterpret_cast<uintptr_t>(multicast) & 255) == 0,
                "qmm_comm_attach_peer_memory: the multicast address must be 256-byte aligned");
    pm.mc_base = static_cast<uint8_t *>(const_cast<void *>(multicast));
    pm.bytes = bytes;
    pm.epoch = 0;
    c.peer = pm;
    return QMM_OK;
}

extern "C" int qmm_comm_info(const char *name, int *nranks, int *rank) {
    using namespace qmm;
    QMM_REQUIRE(name != nullptr, "qmm_comm_info: name is NULL");
    std::lock_guard<std::mutex> lock(g_comm_mutex);
    auto it = g_comms.find(name);
    if (it == g_comms.end())
        return fail(QMM_ERR_NOT_FOUND, std::string("communicator '") + name + "' is not registered");
    if (nranks) *nranks = it->second.nranks;
    if (rank) *rank = it->second.rank;
    return QMM_OK;
}

extern "C" int qmm_comm_stats(const char *name, int64_t *peer_calls, int64_t *peer_pushed_calls,
                              int64_t *peer_fused_calls, int64_t *nccl_calls) {
    using namespace qmm;
    QMM_REQUIRE(name != nullptr, "qmm_comm_stats: name is NULL");
    std::lock_guard<std::mutex> lock(g_comm_mutex);
    auto it = g_comms.find(name);
    if (it == g_comms.end())
        return fail(QMM_ERR_NOT_FOUND, std::string("communicator '") + name + "' is not registered");
    if (peer_calls) *peer_calls = it->second.stat_peer;
    if (peer_pushed_calls) *peer_pushed_calls = it->second.stat_peer_pushed;
    if (peer_fused_calls) *peer_fused_calls = it->second.stat_peer_fused;
    if (nccl_calls) *nccl_calls = it->second.stat_nccl;
    return QMM_OK;
}

extern "C" int qmm_comm_destroy(const char *name) {
    using namespace qmm;
    QMM_REQUIRE(name != nullptr, "qmm_comm_destroy: name is NULL");
    Comm c;
    {
        std::lock_guard<std::mutex> lock(g_comm_mutex);
        auto it = g_comms.find(name);
        if (it == g_comms.end())
            return fail(QMM_ERR_NOT_FOUND, std::string("communicator '") + name + "' is not registered");
        c = it->second;
        g_comms.erase(it);
    }
    release(c, false);
    return QMM_OK;
}

extern "C" int qmm_mm_all_reduce(const int8_t *x1, int64_t ld_x1, const int8_t *x2, int64_t x2_stride_k,
                                 int64_t x2_stride_n, const float *scale, int64_t scale_len,
                                 const float *pertoken_scale, const void *bias, int bias_dtype, void *out,
                                 int out_dtype, int64_t ld_out, int64_t M, int64_t N, int64_t K, const char *hcom,
                                 const char *reduce_op, int64_t comm_turn, void *workspace, size_t workspace_bytes,
                                 void *stream) {
    using namespace qmm;
    QMM_REQUIRE(hcom != nullptr && hcom[0] != '\0', "qmm_mm_all_reduce: empty communicator name");
    QMM_REQUIRE(reduce_op != nullptr && std::string(reduce_op) == "sum",
                std::string("qmm_mm_all_reduce: reduce_op must be 'sum', got '") + (reduce_op ? reduce_op : "") + "'");
    QMM_REQUIRE(out_dtype == QMM_DTYPE_BF16 || out_dtype == QMM_DTYPE_F16,
                "qmm_mm_all_reduce: output dtype must be bf16 or f16");
    QMM_REQUIRE(comm_turn >= 0, "qmm_mm_all_reduce: comm_turn must be non-negative");
    int rc = validate_quant_matmul(x1, ld_x1, x2, x2_stride_k, x2_stride_n, scale, scale_len, bias, bias_dtype, out,
                                   out_dtype, ld_out, M, N, K);
    if (rc != QMM_OK) return rc;
    // A bounded wait that gave up in an earlier kernel (a peer that never arrived) left that call's result
    // incomplete: report it here, where the next collective would otherwise build on it.  The word is cleared.
    if (const uint32_t st = device_status_peek(true)) {
        char msg[160];
        snprintf(msg, sizeof(msg), "qmm_mm_all_reduce: an earlier kernel's bounded device-side wait gave up (status 0x%x); "
                 "that call's result is incomplete (status cleared)", st);
        return fail(QMM_ERR_DEVICE_TIMEOUT, msg);
    }
    Comm c;
    {
        std::lock_guard<std::mutex> lock(g_comm_mutex);
        auto it = g_comms.find(hcom);
        if (it == g_comms.end())
            return fail(QMM_ERR_NOT_FOUND, std::string("communicator '") + hcom + "' is not registered");
        c = it->second;
    }
    if (M == 0 || N == 0) return QMM_OK;
    QMM_REQUIRE(ld_out == N || M == 1, "qmm_mm_all_reduce: out must be contiguous (ld_out == N)");
    int dev = 0;
    QMM_CUDA_OK(cudaGetDevice(&dev));
    QMM_REQUIRE(dev == c.device, "qmm_mm_all_reduce: communicator belongs to another device");
    cudaStream_t s = static_cast<cudaStream_t>(stream);

    // Peer-memory path: matmul into this rank's region, then one reduce + gather kernel.  Whether a call
    // takes it depends only on values every rank shares (shape, attached size, comm_turn, the QMM_ALLREDUCE
    // setting), so that ranks cannot part ways; what only this rank can see (capture state, alignment of
    // `out`) is an error instead of a silent switch to NCCL that the peers would not follow.
    if (c.nranks > 1 && c.nranks <= kPeerMaxRanks && comm_turn == 0 && !peer_path_disabled() && N % 8 == 0 &&
        peer_half_bytes(c.peer.bytes) >= peer_half_need(M, N, c.nranks)) {
        cudaStreamCaptureStatus capture = cudaStreamCaptureStatusNone;
        QMM_CUDA_OK(cudaStreamIsCapturing(s, &capture));
        if (capture != cudaStreamCaptureStatusNone)
            return fail(QMM_ERR_UNSUPPORTED,
                        "qmm_mm_all_reduce: the peer-memory allreduce cannot be captured in a CUDA graph (its epoch "
                        "advances on the host); pass comm_turn > 0 or set QMM_ALLREDUCE=nccl on every rank");
        QMM_REQUIRE((reinterpret_cast<uintptr_t>(out) & 15) == 0,
                    "qmm_mm_all_reduce: out must be 16-byte aligned for the peer-memory allreduce");
        // Row chunks (QMM_PEER_CHUNKS, default 1): chunk c's reduce + gather kernel can run on the
        // communication stream while chunk c+1 is multiplied on the caller's stream.  Measured on two
        // B200s that costs far more than it hides (804-1105 us against 377 us unchunked: the two kernels
        // share the SMs badly), so the overlap is left to the matmul's epilogue, which pushes finished
        // tiles to their owners; chunking stays available for experiments.
        int chunks = peer_chunks();
        if (M < 512 * chunks) chunks = 1;
        int64_t rows_chunk = (M + chunks - 1) / chunks;
        rows_chunk = (rows_chunk + 255) / 256 * 256;
        const size_t elt = 2;
        const int64_t rows_per_full = ((M + c.nranks - 1) / c.nranks + 31) / 32 * 32;
        const size_t red_area = kPeerFlagBytes + peer_half_bytes(c.peer.bytes);
        const bool push_ok = chunks == 1 && !push_disabled();
        int ci = 0;
        for (int64_t m0 = 0; m0 < M; m0 += rows_chunk, ++ci) {
            const int64_t rows = (M - m0) < rows_chunk ? (M - m0) : rows_chunk;
            const size_t row_bytes0 = static_cast<size_t>(m0) * N * elt;
            PeerParams pp;
            for (int r = 0; r < kPeerMaxRanks; ++r) pp.base[r] = c.peer.base[r];
            pp.mc_base = c.peer.mc_base;
            pp.world = c.nranks;
            pp.rank = c.rank;
            pp.epoch = 0;  // drawn below, once the matmul is in the stream
            pp.M = rows;
            pp.N = N;
            pp.rows_per = chunks == 1 ? rows_per_full : (rows + c.nranks - 1) / c.nranks;
            pp.pushed = 0;
            {
                const size_t own_bytes = static_cast<size_t>(pp.rows_per) * N * elt;
                size_t n = (own_bytes + kPeerChunkBytes - 1) / kPeerChunkBytes;
                pp.nchunks = static_cast<int>(n < 1 ? 1 : (n > kPeerChunks ? kPeerChunks : n));
            }
            pp.partial_off = kPeerFlagBytes + row_bytes0;
            pp.red_off = red_area + row_bytes0;
            pp.out = static_cast<uint8_t *>(out) + row_bytes0;
            pp.status = device_status_word();
            pp.status_at_launch = device_status_peek(false);
            EpilogueParams ep;
            ep.scale = scale;
            ep.pertoken_scale = pertoken_scale ? pertoken_scale + m0 : nullptr;
            ep.bias = (c.rank == 0) ? bias : nullptr;  // bias enters the sum once
            ep.bias_dtype = ep.bias ? bias_dtype : QMM_DTYPE_NONE;
            ep.scale_is_scalar = (scale_len == 1 && N != 1) ? 1 : 0;
            ep.out = c.peer.base[c.rank] + pp.partial_off;
            ep.ld_out = N;
            ep.M = rows;
            ep.N = N;
            // The epoch is drawn before the matmul (a fused launch raises flags itself) and given back if nothing
            // was launched: a call that fails has touched no flag, so the ranks' epochs stay in step as long as
            // every rank either launches or fails before launching.
            {
                std::lock_guard<std::mutex> lock(g_comm_mutex);
                auto it = g_comms.find(hcom);
                if (it == g_comms.end())
                    return fail(QMM_ERR_NOT_FOUND, std::string("communicator '") + hcom + "' is not registered");
                pp.epoch = ++it->second.peer.epoch;
            }
            // the CTA-pair matmul stores each output tile into the region of the rank that owns its rows, and
            // (plain peer loads, one chunk of rows) reduces and gathers finished column chunks itself
            PushSpec spec;
            FusedComm fspec;
            LaunchOptions opts;
            if (push_ok) {
                for (int r = 0; r < kPeerMaxRanks; ++r) spec.base[r] = c.peer.base[r];
                spec.area_off = pp.partial_off;
                spec.world = c.nranks;
                spec.rank = c.rank;
                spec.rows_per = pp.rows_per;
                opts.push = &spec;
                if (pp.mc_base == nullptr && fused_wanted(c.nranks)) {
                    for (int r = 0; r < kPeerMaxRanks; ++r) fspec.base[r] = c.peer.base[r];
                    fspec.world = c.nranks;
                    fspec.rank = c.rank;
                    fspec.epoch = pp.epoch;
                    fspec.chunks = fused_chunks();
                    fspec.M = rows;
                    fspec.N = N;
                    fspec.rows_per = pp.rows_per;
                    fspec.partial_off = pp.partial_off;
                    fspec.red_off = pp.red_off;
                    fspec.out = pp.out;
                    fspec.status = pp.status;
                    fspec.status_at_launch = pp.status_at_launch;
                    fspec.enabled = 0;
                    // arrival counters of the fused kernel: zero unless a call was cut short (or never used yet)
                    {
                        const uint64_t gen = device_status_generation();
                        bool clean = false;
                        {
                            std::lock_guard<std::mutex> lock(g_comm_mutex);
                            auto it = g_comms.find(hcom);
                            if (it != g_comms.end()) {
                                clean = it->second.peer.fused_clean_gen == gen;
                                it->second.peer.fused_clean_gen = gen;
                            }
                        }
                        if (!clean)
                            QMM_CUDA_OK(cudaMemsetAsync(c.peer.base[c.rank] + kFusedFlagOffset + kFusedPushCountOffset, 0,
                                                        kFusedCounterBytes, s));
                    }
                    opts.fused = &fspec;
                }
            }
            rc = quant_matmul_dispatch(x1 + m0 * ld_x1, ld_x1, x2, x2_stride_k, x2_stride_n, ep, out_dtype, K,
                                       K == 0 ? QMM_ALGO_SIMT : QMM_ALGO_AUTO, workspace, workspace_bytes, s, &opts);
            pp.pushed = opts.push_applied ? 1 : 0;
            {
                std::lock_guard<std::mutex> lock(g_comm_mutex);
                auto it = g_comms.find(hcom);
                if (it != g_comms.end()) {
                    if (rc != QMM_OK) {
                        --it->second.peer.epoch;
                    } else if (ci == 0) {
                        ++it->second.stat_peer;
                        if (pp.pushed) ++it->second.stat_peer_pushed;
                        if (opts.fused_applied) ++it->second.stat_peer_fused;
                    }
                }
            }
            if (rc != QMM_OK) return rc;
            if (opts.fused_applied) continue;  // the matmul kernel has done the exchange
            cudaStream_t ks = s;
            if (chunks > 1) {
                QMM_CUDA_OK(cudaEventRecord(c.chunk_ready[ci], s));
                QMM_CUDA_OK(cudaStreamWaitEvent(c.stream, c.chunk_ready[ci], 0));
                ks = c.stream;
            }
            // every CTA must be resident (ranks wait on one another's CTAs): one per SM
            const int grid = sm_count();
            const bool mc = pp.mc_base != nullptr;
            if (out_dtype == QMM_DTYPE_BF16) {
                if (mc)
                    peer_all_reduce_kernel<__nv_bfloat16, true><<<grid, kPeerThreads, 0, ks>>>(pp);
                else
                    peer_all_reduce_kernel<__nv_bfloat16, false><<<grid, kPeerThreads, 0, ks>>>(pp);
            } else {
                if (mc)
                    peer_all_reduce_kernel<__half, true><<<grid, kPeerThreads, 0, ks>>>(pp);
                else
                    peer_all_reduce_kernel<__half, false><<<grid, kPeerThreads, 0, ks>>>(pp);
            }
            QMM_CUDA_OK(cudaGetLastError());
        }
        if (chunks > 1) {
            QMM_CUDA_OK(cudaEventRecord(c.done, c.stream));
            QMM_CUDA_OK(cudaStreamWaitEvent(s, c.done, 0));
        }
        return QMM_OK;
    }

    // Number of M chunks.  Measured on 2, 4 and 8 B200s (M=4096, N=8192): every extra ncclAllReduce call
    // costs tens of microseconds and a collective confined to the SMs the matmul leaves free runs far
    // below link speed, so cutting M into chunks lost more than the overlap won back (2 GPUs: 423 us
    // unchunked, 486 us in 4 chunks).  The default is therefore one chunk; comm_turn > 0 asks for more.
    int chunks = comm_turn > 0 ? static_cast<int>(comm_turn < kMaxChunks ? comm_turn : kMaxChunks) : 1;
    if (chunks < 1) chunks = 1;
    if (chunks > kMaxChunks) chunks = kMaxChunks;
    int64_t rows_per = (M + chunks - 1) / chunks;
    rows_per = (rows_per + 127) / 128 * 128;
    const size_t elt = 2;
    const ncclDataType_t dt = out_dtype == QMM_DTYPE_BF16 ? ncclBfloat16 : ncclFloat16;

    int ci = 0;
    for (int64_t m0 = 0; m0 < M; m0 += rows_per, ++ci) {
        const int64_t rows = (M - m0) < rows_per ? (M - m0) : rows_per;
        EpilogueParams ep;
        ep.scale = scale;
        ep.pertoken_scale = pertoken_scale ? pertoken_scale + m0 : nullptr;
        ep.bias = (c.rank == 0) ? bias : nullptr;  // bias enters the sum once
        ep.bias_dtype = ep.bias ? bias_dtype : QMM_DTYPE_NONE;
        ep.scale_is_scalar = (scale_len == 1 && N != 1) ? 1 : 0;
        ep.out = static_cast<uint8_t *>(out) + static_cast<size_t>(m0) * ld_out * elt;
        ep.ld_out = ld_out;
        ep.M = rows;
        ep.N = N;
        // leave SMs to a collective that may be running beside this chunk
        LaunchOptions opts;
        opts.sm_reserve = (c.nranks > 1 && ci > 0) ? comm_ctas() : 0;
        rc = quant_matmul_dispatch(x1 + m0 * ld_x1, ld_x1, x2, x2_stride_k, x2_stride_n, ep, out_dtype, K,
                                   K == 0 ? QMM_ALGO_SIMT : QMM_ALGO_AUTO, workspace, workspace_bytes, s, &opts);
        if (rc != QMM_OK) return rc;
        if (c.nranks > 1) {
            QMM_CUDA_OK(cudaEventRecord(c.chunk_ready[ci], s));
            QMM_CUDA_OK(cudaStreamWaitEvent(c.stream, c.chunk_ready[ci], 0));
            QMM_NCCL_OK(nccl().AllReduce(ep.out, ep.out, static_cast<size_t>(rows) * N, dt, ncclSum, c.comm,
                                         c.stream));
        }
    }
    if (c.nranks > 1) {
        {
            std::lock_guard<std::mutex> lock(g_comm_mutex);
            auto it = g_comms.find(hcom);
            if (it != g_comms.end()) ++it->second.stat_nccl;
        }
        QMM_CUDA_OK(cudaEventRecord(c.done, c.stream));
        QMM_CUDA_OK(cudaStreamWaitEvent(s, c.done, 0));
        ncclResult_t async = ncclSuccess;
        QMM_NCCL_OK(nccl().CommGetAsyncError(c.comm, &async));
        if (async != ncclSuccess && async != ncclInProgress)
            return fail(QMM_ERR_NCCL, std::string("NCCL asynchronous error: ") + nccl().GetErrorString(async));
    }
    return QMM_OK;
}


// ---------------------------------------------------------------------------------------------------------
// npu_mm_reduce_scatter_base and npu_all_gather_base_mm
// (op_plugin/ops/base_ops/opapi/MatmulReduceScatterBaseKernelNpuOpApi.cpp:22-42,
//  AllGatherBaseMatmulKernelNpuOpApi.cpp:22-60).
// ---------------------------------------------------------------------------------------------------------
namespace qmm {
namespace {

int find_comm(const char *fn, const char *hcom, Comm *out) {
    if (hcom == nullptr || hcom[0] == '\0') return fail(QMM_ERR_INVALID_ARGUMENT, std::string(fn) + ": empty communicator name");
    std::lock_guard<std::mutex> lock(g_comm_mutex);
    auto it = g_comms.find(hcom);
    if (it == g_comms.end()) return fail(QMM_ERR_NOT_FOUND, std::string("communicator '") + hcom + "' is not registered");
    *out = it->second;
    return QMM_OK;
}

int check_dense_operands(const char *fn, const void *x1, int dtype, int64_t ld_x1, const void *x2, int64_t sk, int64_t sn,
                         int64_t M, int64_t N, int64_t K) {
    const std::string f(fn);
    QMM_REQUIRE(M >= 0 && N >= 0 && K >= 0, f + ": negative dimension");
    QMM_REQUIRE(dtype == QMM_DTYPE_BF16 || dtype == QMM_DTYPE_F16, f + ": operands must be bf16 or f16");
    if (M > 0 && N > 0 && K > 0) {
        QMM_REQUIRE(x1 != nullptr && x2 != nullptr, f + ": NULL operand");
        QMM_REQUIRE(ld_x1 >= K, f + ": ld_x1 smaller than K");
        QMM_REQUIRE(sk == 1 || sn == 1, f + ": x2 must have a unit stride along K or N");
    }
    return QMM_OK;
}

// draws the next epoch and the CTA-counter target of a reduce-scatter (which = 0) or all-gather (1) launch
int next_sg_epoch(const char *hcom, int which, uint32_t grid, uint32_t *epoch, uint32_t *done_target) {
    std::lock_guard<std::mutex> lock(g_comm_mutex);
    auto it = g_comms.find(hcom);
    if (it == g_comms.end()) return fail(QMM_ERR_NOT_FOUND, std::string("communicator '") + hcom + "' is not registered");
    *epoch = ++it->second.peer.epoch;
    uint32_t &calls = which == 0 ? it->second.peer.rs_calls : it->second.peer.ag_calls;
    *done_target = ++calls * grid;
    ++it->second.stat_peer;
    return QMM_OK;
}

void fill_sg(PeerSgParams &pp, const Comm &c) {
    for (int r = 0; r < kPeerMaxRanks; ++r) pp.base[r] = c.peer.base[r];
    pp.world = c.nranks;
    pp.rank = c.rank;
    pp.area_off = kPeerFlagBytes;
    pp.status = device_status_word();
    pp.status_at_launch = device_status_peek(false);
}

bool peer_usable(const Comm &c, size_t half_need) {
    return c.nranks > 1 && c.nranks <= kPeerMaxRanks && !peer_path_disabled() && peer_half_bytes(c.peer.bytes) >= half_need;
}

}  // namespace
}  // namespace qmm

extern "C" int qmm_mm_reduce_scatter_workspace_size(int64_t M, int64_t N, int64_t K, int nranks, size_t *bytes) {
    using namespace qmm;
    (void)K;
    QMM_REQUIRE(bytes != nullptr, "qmm_mm_reduce_scatter_workspace_size: bytes is NULL");
    QMM_REQUIRE(M >= 0 && N >= 0 && nranks >= 1, "qmm_mm_reduce_scatter_workspace_size: bad argument");
    // NCCL path: the fp32 partial [M, N] and the fp32 reduced rows [M / nranks, N]
    *bytes = align256(static_cast<size_t>(M) * N * 4) + align256(static_cast<size_t>((M + nranks - 1) / nranks) * N * 4);
    return QMM_OK;
}

extern "C" int qmm_mm_reduce_scatter(const void *x1, int dtype, int64_t ld_x1, const void *x2, int64_t x2_stride_k,
                                     int64_t x2_stride_n, const void *bias, void *out, int64_t ld_out, int64_t M,
                                     int64_t N, int64_t K, const char *hcom, const char *reduce_op, int64_t comm_turn,
                                     void *workspace, size_t workspace_bytes, void *stream) {
    using namespace qmm;
    const char *fn = "qmm_mm_reduce_scatter";
    QMM_REQUIRE(reduce_op != nullptr && std::string(reduce_op) == "sum",
                std::string(fn) + ": reduce_op must be 'sum', got '" + (reduce_op ? reduce_op : "") + "'");
    QMM_REQUIRE(comm_turn >= 0, std::string(fn) + ": comm_turn must be non-negative");
    int rc = check_dense_operands(fn, x1, dtype, ld_x1, x2, x2_stride_k, x2_stride_n, M, N, K);
    if (rc != QMM_OK) return rc;
    Comm c;
    rc = find_comm(fn, hcom, &c);
    if (rc != QMM_OK) return rc;
    QMM_REQUIRE(M % c.nranks == 0, std::string(fn) + ": M must be divisible by the communicator's size");
    if (M == 0 || N == 0) return QMM_OK;
    QMM_REQUIRE(out != nullptr && ld_out >= N, std::string(fn) + ": out is NULL or ld_out smaller than N");
    int dev = 0;
    QMM_CUDA_OK(cudaGetDevice(&dev));
    QMM_REQUIRE(dev == c.device, std::string(fn) + ": communicator belongs to another device");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int64_t rows_per = M / c.nranks;

    DenseParams d;
    memset(&d, 0, sizeof(d));
    d.a = x1;
    d.ld_a = ld_x1;
    d.b = x2;
    d.b_sk = x2_stride_k;
    d.b_sn = x2_stride_n;
    d.dtype = dtype;
    d.M = M;
    d.N = N;
    d.K = K;
    if (c.nranks == 1) {  // nothing to exchange: the matmul alone
        d.mode = kDenseOutCast;
        d.out = out;
        d.ld_out = ld_out;
        d.bias = bias;
        return launch_dense_gemm(d, s);
    }
    if (peer_usable(c, align256(static_cast<size_t>(M) * N * 4))) {
        cudaStreamCaptureStatus capture = cudaStreamCaptureStatusNone;
        QMM_CUDA_OK(cudaStreamIsCapturing(s, &capture));
        if (capture != cudaStreamCaptureStatusNone)
            return fail(QMM_ERR_UNSUPPORTED, std::string(fn) + ": the peer-memory path cannot be captured in a CUDA graph; "
                                                               "set QMM_ALLREDUCE=nccl on every rank");
        // matmul whose epilogue stores the fp32 rows into the owners' regions, then the owner's sum
        d.mode = kDenseOutPush;
        for (int r = 0; r < kPeerMaxRanks; ++r) d.base[r] = c.peer.base[r];
        d.area_off = kPeerFlagBytes;
        d.world = c.nranks;
        d.rank = c.rank;
        d.rows_per = rows_per;
        rc = launch_dense_gemm(d, s);
        if (rc != QMM_OK) return rc;
        PeerSgParams pp;
        fill_sg(pp, c);
        const uint32_t grid = static_cast<uint32_t>(sm_count());
        rc = next_sg_epoch(hcom, 0, grid, &pp.epoch, &pp.done_target);
        if (rc != QMM_OK) return rc;
        pp.flag_off = kPeerSgFlagOffset;
        pp.rows = rows_per;
        pp.cols = N;
        pp.bias = bias;
        pp.out = out;
        pp.ld_out = ld_out;
        if (dtype == QMM_DTYPE_BF16)
            peer_reduce_scatter_kernel<__nv_bfloat16><<<grid, kPeerThreads, 0, s>>>(pp);
        else
            peer_reduce_scatter_kernel<__half><<<grid, kPeerThreads, 0, s>>>(pp);
        QMM_CUDA_OK(cudaGetLastError());
        return QMM_OK;
    }
    // NCCL: fp32 partial -> ncclReduceScatter(sum) -> bias and cast
    rc = nccl_ready();
    if (rc != QMM_OK) return rc;
    size_t need = 0;
    qmm_mm_reduce_scatter_workspace_size(M, N, K, c.nranks, &need);
    if (workspace == nullptr || workspace_bytes < need || (reinterpret_cast<uintptr_t>(workspace) & 255) != 0)
        return fail(QMM_ERR_WORKSPACE, std::string(fn) + ": workspace missing, not 256-byte aligned or smaller than "
                                                         "qmm_mm_reduce_scatter_workspace_size reports");
    float *partial = static_cast<float *>(workspace);
    float *reduced = reinterpret_cast<float *>(static_cast<uint8_t *>(workspace) + align256(static_cast<size_t>(M) * N * 4));
    d.mode = kDenseOutPush;  // with one "owner" spanning all rows this is a plain fp32 [M, N] output
    d.base[0] = reinterpret_cast<uint8_t *>(partial);
    d.area_off = 0;
    d.world = 1;
    d.rank = 0;
    d.rows_per = M;
    rc = launch_dense_gemm(d, s);
    if (rc != QMM_OK) return rc;
    QMM_CUDA_OK(cudaEventRecord(c.chunk_ready[0], s));
    QMM_CUDA_OK(cudaStreamWaitEvent(c.stream, c.chunk_ready[0], 0));
    QMM_NCCL_OK(nccl().ReduceScatter(partial, reduced, static_cast<size_t>(rows_per) * N, ncclFloat32, ncclSum, c.comm,
                                     c.stream));
    QMM_CUDA_OK(cudaEventRecord(c.done, c.stream));
    QMM_CUDA_OK(cudaStreamWaitEvent(s, c.done, 0));
    const int64_t total = rows_per * N;
    if (dtype == QMM_DTYPE_BF16)
        cast_rows_kernel<__nv_bfloat16><<<static_cast<unsigned>((total + 255) / 256), 256, 0, s>>>(
            reduced, static_cast<const __nv_bfloat16 *>(bias), static_cast<__nv_bfloat16 *>(out), ld_out, rows_per, N);
    else
        cast_rows_kernel<__half><<<static_cast<unsigned>((total + 255) / 256), 256, 0, s>>>(
            reduced, static_cast<const __half *>(bias), static_cast<__half *>(out), ld_out, rows_per, N);
    QMM_CUDA_OK(cudaGetLastError());
    {
        std::lock_guard<std::mutex> lock(g_comm_mutex);
        auto it = g_comms.find(hcom);
        if (it != g_comms.end()) ++it->second.stat_nccl;
    }
    return QMM_OK;
}

extern "C" int qmm_all_gather_mm_workspace_size(int64_t M, int64_t N, int64_t K, int nranks, size_t *bytes) {
    using namespace qmm;
    (void)N;
    QMM_REQUIRE(bytes != nullptr, "qmm_all_gather_mm_workspace_size: bytes is NULL");
    QMM_REQUIRE(M >= 0 && K >= 0 && nranks >= 1, "qmm_all_gather_mm_workspace_size: bad argument");
    *bytes = align256(static_cast<size_t>(M) * nranks * K * 2);  // the gathered x1 when the caller does not want it back
    return QMM_OK;
}

extern "C" int qmm_all_gather_mm(const void *x1, int dtype, int64_t ld_x1, const void *x2, int64_t x2_stride_k,
                                 int64_t x2_stride_n, const void *bias, void *out, int64_t ld_out, void *gather_out,
                                 int64_t ld_gather, int64_t M, int64_t N, int64_t K, const char *hcom,
                                 int64_t gather_index, int64_t comm_turn, void *workspace, size_t workspace_bytes,
                                 void *stream) {
    using namespace qmm;
    const char *fn = "qmm_all_gather_mm";
    QMM_REQUIRE(gather_index == 0, std::string(fn) + ": only gather_index == 0 (gather x1 along its rows) is supported");
    QMM_REQUIRE(comm_turn >= 0, std::string(fn) + ": comm_turn must be non-negative");
    int rc = check_dense_operands(fn, x1, dtype, ld_x1, x2, x2_stride_k, x2_stride_n, M, N, K);
    if (rc != QMM_OK) return rc;
    Comm c;
    rc = find_comm(fn, hcom, &c);
    if (rc != QMM_OK) return rc;
    if (M == 0) return QMM_OK;
    QMM_REQUIRE(N == 0 || (out != nullptr && ld_out >= N), std::string(fn) + ": out is NULL or ld_out smaller than N");
    QMM_REQUIRE(gather_out == nullptr || ld_gather >= K, std::string(fn) + ": ld_gather smaller than K");
    int dev = 0;
    QMM_CUDA_OK(cudaGetDevice(&dev));
    QMM_REQUIRE(dev == c.device, std::string(fn) + ": communicator belongs to another device");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int W = c.nranks;

    // where the gathered [W * M, K] matrix lives: the caller's tensor, or the workspace
    uint8_t *gathered = static_cast<uint8_t *>(gather_out);
    int64_t ld_g = ld_gather;
    if (gathered == nullptr && W > 1 && K > 0) {
        size_t need = 0;
        qmm_all_gather_mm_workspace_size(M, N, K, W, &need);
        if (workspace == nullptr || workspace_bytes < need || (reinterpret_cast<uintptr_t>(workspace) & 255) != 0)
            return fail(QMM_ERR_WORKSPACE, std::string(fn) + ": workspace missing, not 256-byte aligned or smaller than "
                                                             "qmm_all_gather_mm_workspace_size reports");
        gathered = static_cast<uint8_t *>(workspace);
        ld_g = K;
    }
    const size_t shard_bytes = static_cast<size_t>(M) * K * 2;
    if (gathered != nullptr && K > 0) {
        // own shard into its slot of the gathered matrix
        QMM_CUDA_OK(cudaMemcpy2DAsync(gathered + static_cast<size_t>(c.rank) * M * ld_g * 2, static_cast<size_t>(ld_g) * 2, x1,
                                      static_cast<size_t>(ld_x1) * 2, static_cast<size_t>(K) * 2, static_cast<size_t>(M),
                                      cudaMemcpyDeviceToDevice, s));
    }
    if (W > 1 && K > 0) {
        if (peer_usable(c, align256(shard_bytes))) {
            cudaStreamCaptureStatus capture = cudaStreamCaptureStatusNone;
            QMM_CUDA_OK(cudaStreamIsCapturing(s, &capture));
            if (capture != cudaStreamCaptureStatusNone)
                return fail(QMM_ERR_UNSUPPORTED, std::string(fn) + ": the peer-memory path cannot be captured in a CUDA "
                                                                   "graph; set QMM_ALLREDUCE=nccl on every rank");
            // own shard, densely packed, into this rank's region for the peers to pull
            QMM_CUDA_OK(cudaMemcpy2DAsync(c.peer.base[c.rank] + kPeerFlagBytes, static_cast<size_t>(K) * 2, x1,
                                          static_cast<size_t>(ld_x1) * 2, static_cast<size_t>(K) * 2,
                                          static_cast<size_t>(M), cudaMemcpyDeviceToDevice, s));
            PeerSgParams pp;
            fill_sg(pp, c);
            const uint32_t grid = static_cast<uint32_t>(sm_count());
            rc = next_sg_epoch(hcom, 1, grid, &pp.epoch, &pp.done_target);
            if (rc != QMM_OK) return rc;
            pp.flag_off = kPeerAgFlagOffset;
            pp.rows = M;
            pp.cols = K;
            pp.bias = nullptr;
            pp.out = gathered;
            pp.ld_out = ld_g;
            peer_all_gather_kernel<<<grid, kPeerThreads, 0, s>>>(pp);
            QMM_CUDA_OK(cudaGetLastError());
        } else {
            rc = nccl_ready();
            if (rc != QMM_OK) return rc;
            QMM_REQUIRE(ld_g == K && ld_x1 == K, std::string(fn) + ": the NCCL path needs contiguous x1 and gather output");
            QMM_CUDA_OK(cudaEventRecord(c.chunk_ready[0], s));
            QMM_CUDA_OK(cudaStreamWaitEvent(c.stream, c.chunk_ready[0], 0));
            QMM_NCCL_OK(nccl().AllGather(x1, gathered, static_cast<size_t>(M) * K,
                                         dtype == QMM_DTYPE_BF16 ? ncclBfloat16 : ncclFloat16, c.comm, c.stream));
            QMM_CUDA_OK(cudaEventRecord(c.done, c.stream));
            QMM_CUDA_OK(cudaStreamWaitEvent(s, c.done, 0));
            std::lock_guard<std::mutex> lock(g_comm_mutex);
            auto it = g_comms.find(hcom);
            if (it != g_comms.end()) ++it->second.stat_nccl;
        }
    }
    if (N == 0) return QMM_OK;
    DenseParams d;
    memset(&d, 0, sizeof(d));
    d.a = (W > 1 && K > 0) ? static_cast<const void *>(gathered) : x1;
    d.ld_a = (W > 1 && K > 0) ? ld_g : ld_x1;
    d.b = x2;
    d.b_sk = x2_stride_k;
    d.b_sn = x2_stride_n;
    d.dtype = dtype;
    d.M = M * W;
    d.N = N;
    d.K = K;
    d.mode = kDenseOutCast;
    d.out = out;
    d.ld_out = ld_out;
    d.bias = bias;
    return launch_dense_gemm(d, s);
}
