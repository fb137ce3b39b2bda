// W8A8 matmul for decode shapes (M <= 128): weight-bandwidth bound.
//
// The weight tile is the MMA's 128-row M operand (rows = output columns n),
// the activations are its N operand (M padded to a multiple of 16), so no
// tensor-core lane is wasted on padding beyond 16 tokens and each accumulator
// lane maps to one output column: stores of a token row are coalesced.
//
// The (n-tile, k-block) space is cut into gridDim.x equal contiguous ranges
// ("stream-K"): every CTA streams the same number of 16 KiB weight tiles
// whatever N and K are.  A CTA whose range covers a whole K extent finishes
// the tile itself; otherwise it adds its int32 partial sums into a scratch
// accumulator with red.global.add (integer addition: the result does not
// depend on arrival order) and the CTA that completes the tile's k-block count
// applies the epilogue and re-zeroes the scratch for the next call.
#include <mutex>

#include "qmm_common.cuh"
#include "w8a8_epilogue.cuh"

namespace qmm {

namespace {

constexpr int kSkTileN = 128;  // output columns per MMA = MMA M
constexpr int kSkHalves = 2;   // MMAs side by side per work unit: a unit is 256 columns wide, so that a
                               // weight row contributes 256 contiguous bytes and the activation tile
                               // is fetched once per two MMAs
constexpr int kSkUnitN = kSkTileN * kSkHalves;
constexpr int kSkBK = 128;     // k elements per stage
constexpr int kSkABytes = kSkUnitN * kSkBK;
constexpr int kSkMaxStages = 8;
constexpr int kSkThreads = 192;
constexpr uint32_t kSkTmemCols = 512;  // two buffers x two accumulators of up to 128 columns
constexpr size_t kSkSmemBudget = 200 * 1024;

struct SkSmemTail {
    uint64_t full[kSkMaxStages];
    uint64_t empty[kSkMaxStages];
    uint64_t tmem_full[2];
    uint64_t tmem_empty[2];
    uint32_t tmem_base;
    uint32_t abort_flag;
    uint32_t is_last;
    uint32_t epi_abort;
    float pertoken[128];  // per-token scales of the (at most 128) rows, staged once per CTA
};

struct SkParams {
    EpilogueParams ep;
    int K;
    int mpad;         // M rounded up to a multiple of 16
    int stages;
    int stage_bytes;  // kSkABytes + mpad * kSkBK
    int tiles_n;          // 256-column work units along N
    int kblocks;
    int32_t *ws_acc;      // [ceil(N/128)][mpad][128] int32, zero between calls
    uint32_t *ws_count;   // one per work unit, zero between calls
    uint32_t *status;
};

__device__ __forceinline__ void epi_bar_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

template <typename OutT, bool A_MN_MAJOR>
__global__ void __launch_bounds__(kSkThreads, 1)
w8a8_streamk_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
                    SkParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *smem_aligned = smem_raw + (smem_base - smem_u32(smem_raw));
    SkSmemTail *tail = reinterpret_cast<SkSmemTail *>(smem_aligned + p.stages * p.stage_bytes);
    volatile uint32_t *abort_flag = &tail->abort_flag;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    // this CTA's contiguous range of (tile, k-block) units
    const int64_t total = static_cast<int64_t>(p.tiles_n) * p.kblocks;
    const int64_t u_begin = total * blockIdx.x / gridDim.x;
    const int64_t u_end = total * (blockIdx.x + 1) / gridDim.x;

    if (threadIdx.x == 0) {
        for (int s = 0; s < p.stages; ++s) {
            mbar_init(smem_u32(&tail->full[s]), 1);
            mbar_init(smem_u32(&tail->empty[s]), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(smem_u32(&tail->tmem_full[b]), 1);
            mbar_init(smem_u32(&tail->tmem_empty[b]), 4);
        }
        tail->abort_flag = 0;
        tail->is_last = 0;
        tail->epi_abort = 0;
        mbar_fence_init();
    }
    if (warp == 0 && lane == 0) {
        tma_prefetch_desc(&tmap_w);
        tma_prefetch_desc(&tmap_x);
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(&tail->tmem_base), kSkTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tail->tmem_base;

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        uint32_t stage = 0, phase = 0;
        int tile = static_cast<int>(u_begin / p.kblocks);
        int kb = static_cast<int>(u_begin - static_cast<int64_t>(tile) * p.kblocks);
        const uint32_t full0 = smem_u32(&tail->full[0]);
        const uint32_t empty0 = smem_u32(&tail->empty[0]);
        for (int64_t u = u_begin; u < u_end; ++u) {
            if (!mbar_wait(empty0 + stage * 8, phase ^ 1, abort_flag, 0x11)) break;
            if (lane == 0) {
                const uint32_t full = full0 + stage * 8;
                const uint32_t sa = smem_base + stage * p.stage_bytes;
                const uint32_t sb = sa + kSkABytes;
                mbar_expect_tx(full, static_cast<uint32_t>(p.stage_bytes));
                if (A_MN_MAJOR) {
                    // two [128 k-rows][128 n-bytes] boxes, one per 128-column half
                    tma_load_2d(sa, &tmap_w, tile * kSkUnitN, kb * kSkBK, full);
                    tma_load_2d(sa + kSkABytes / 2, &tmap_w, tile * kSkUnitN + kSkTileN, kb * kSkBK, full);
                } else {
                    tma_load_2d(sa, &tmap_w, kb * kSkBK, tile * kSkUnitN, full);  // [256 n-rows][128 k-bytes]
                }
                tma_load_2d(sb, &tmap_x, kb * kSkBK, 0, full);                    // [mpad m-rows][128 k-bytes]
            }
            __syncwarp();
            if (++kb == p.kblocks) {
                kb = 0;
                ++tile;
            }
            if (++stage == static_cast<uint32_t>(p.stages)) {
                stage = 0;
                phase ^= 1;
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        // The whole warp runs the loop with warp-uniform operands; elect.sync picks the issuing lane.
        // Descriptors advance by 32-bit adds on their low words (the issue loop is the critical path:
        // with 16 tokens an MMA executes in a few tens of cycles).
        const uint32_t idesc = make_idesc(/*c=s32*/ 2, 1, 1, A_MN_MAJOR ? 1u : 0u, /*b K-major*/ 0, kSkTileN,
                                          static_cast<uint32_t>(p.mpad));
        constexpr uint32_t kDescHi = smem_desc_hi_sw128(1024);
        constexpr uint32_t kAStep = A_MN_MAJOR ? (4096u >> 4) : 2u;  // per 32-element K step
        constexpr uint32_t kAHalf = (kSkABytes / 2) >> 4;
        const uint32_t a_lo0 = smem_desc_lo(smem_base, A_MN_MAJOR ? 1024u : 16u);
        const uint32_t b_lo0 = smem_desc_lo(smem_base + kSkABytes, 16);
        const uint32_t stage_step = static_cast<uint32_t>(p.stage_bytes) >> 4;
        const uint32_t full0 = smem_u32(&tail->full[0]);
        const uint32_t empty0 = smem_u32(&tail->empty[0]);
        uint32_t stage = 0, phase = 0;
        int seg = 0;
        bool ok = true;
        int64_t u = u_begin;
        int64_t tile_end = (u_begin / p.kblocks + 1) * static_cast<int64_t>(p.kblocks);
        while (u < u_end && ok) {
            const int64_t seg_end = tile_end < u_end ? tile_end : u_end;
            const uint32_t buf = seg & 1;
            const uint32_t buf_phase = (seg >> 1) & 1;
            ok = mbar_wait(smem_u32(&tail->tmem_empty[buf]), buf_phase ^ 1, abort_flag, 0x12);
            if (!ok) break;
            tc_fence_after();
            const uint32_t d_tmem = tmem_base + buf * 256;
            uint32_t accumulate = 0;
            for (; u < seg_end; ++u) {
                ok = mbar_wait(full0 + stage * 8, phase, abort_flag, 0x13);
                if (!ok) break;
                tc_fence_after();
                const uint32_t a_lo = a_lo0 + stage * stage_step;
                const uint32_t b_lo = b_lo0 + stage * stage_step;
#pragma unroll
                for (int k = 0; k < kSkBK / 32; ++k) {
                    const uint64_t bdesc = desc64(b_lo + 2 * k, kDescHi);
#pragma unroll
                    for (int h = 0; h < kSkHalves; ++h) {
                        mma_i8_ss_warp(d_tmem + h * kSkTileN, desc64(a_lo + h * kAHalf + kAStep * k, kDescHi), bdesc,
                                       idesc, accumulate);
                    }
                    accumulate = 1;
                }
                tc_commit_warp(empty0 + stage * 8);
                if (++stage == static_cast<uint32_t>(p.stages)) {
                    stage = 0;
                    phase ^= 1;
                }
            }
            if (ok) tc_commit_warp(smem_u32(&tail->tmem_full[buf]));
            tile_end += p.kblocks;
            ++seg;
        }
    } else {
        // ---------------- epilogue warps ----------------
        const int quarter = warp & 3;
        const int row = quarter * 32 + lane;  // accumulator lane = output column within the tile
        const bool leader = (threadIdx.x == 64);
        const EpilogueParams &ep = p.ep;
        const int M = static_cast<int>(ep.M);
        // every thread needs every row's per-token scale: one coalesced fetch per CTA, broadcasts afterwards
        if (ep.pertoken_scale != nullptr && row < M) tail->pertoken[row] = __ldg(ep.pertoken_scale + row);
        epi_bar_sync();
        int seg = 0;
        bool ok = true;
        int64_t u = u_begin;
        while (u < u_end && ok) {
            const int tile = static_cast<int>(u / p.kblocks);
            const int64_t tile_begin = static_cast<int64_t>(tile) * p.kblocks;
            const int64_t tile_end = tile_begin + p.kblocks;
            const int64_t seg_end = tile_end < u_end ? tile_end : u_end;
            const bool whole = (u == tile_begin && seg_end == tile_end);
            const uint32_t units = static_cast<uint32_t>(seg_end - u);
            const uint32_t buf = seg & 1;
            const uint32_t buf_phase = (seg >> 1) & 1;
            ok = mbar_wait(smem_u32(&tail->tmem_full[buf]), buf_phase, abort_flag, 0x14);
            // The four epilogue warps meet at named barriers below, so they must
            // leave the loop together: agree on the outcome of the wait first.
            if (!ok) *reinterpret_cast<volatile uint32_t *>(&tail->epi_abort) = 1;
            epi_bar_sync();
            if (*reinterpret_cast<volatile uint32_t *>(&tail->epi_abort) != 0) break;
            tc_fence_after();

#pragma unroll 1
            for (int h = 0; h < kSkHalves; ++h) {
            const int64_t n = static_cast<int64_t>(tile) * kSkUnitN + h * kSkTileN + row;
            const bool n_ok = n < ep.N;
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + buf * 256 + h * kSkTileN;

            // per-column constants of the dequantization
            float sc = 0.0f, bi = 0.0f;
            int32_t bi32 = 0;
            const bool has_pt = (ep.pertoken_scale != nullptr);
            bool has_bias = false;
            if (n_ok) {
                if constexpr (sizeof(OutT) == 4) {
                    has_bias = (ep.bias != nullptr && ep.bias_dtype == QMM_DTYPE_I32);
                    if (has_bias) bi32 = __ldg(static_cast<const int32_t *>(ep.bias) + n);
                } else {
                    has_bias = (ep.bias != nullptr && ep.bias_dtype != QMM_DTYPE_NONE &&
                                ep.bias_dtype != QMM_DTYPE_I32);
                    sc = ep.scale_is_scalar ? __ldg(ep.scale) : __ldg(ep.scale + n);
                    if (has_bias) bi = load_bias_f32(ep, n);
                }
            }
            auto finish = [&](int m, int32_t acc) {
                OutT *o = static_cast<OutT *>(ep.out) + static_cast<int64_t>(m) * ep.ld_out + n;
                if constexpr (sizeof(OutT) == 4) {
                    *reinterpret_cast<int32_t *>(o) = acc + bi32;
                } else {
                    const float pt = has_pt ? tail->pertoken[m] : 1.0f;
                    *o = from_float<OutT>(dequant_one(acc, sc, pt, has_pt, bi, has_bias));
                }
            };

            int32_t *ws = p.ws_acc + (static_cast<int64_t>(tile * kSkHalves + h) * p.mpad) * kSkTileN + row;
            for (int c = 0; c < p.mpad; c += 16) {
                uint32_t acc[16];
                tmem_ld_32x16(taddr + c, acc);
                tmem_ld_wait();
                if (n_ok) {
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const int m = c + j;
                        if (m < M) {
                            if (whole)
                                finish(m, static_cast<int32_t>(acc[j]));
                            else
                                atomicAdd(ws + static_cast<int64_t>(m) * kSkTileN, static_cast<int32_t>(acc[j]));
                        }
                    }
                }
            }
            }  // halves
            // accumulator buffer can be reused by the MMA warp
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&tail->tmem_empty[buf]));

            if (!whole) {
                // publish the partial sums, then find out whether this CTA completed the tile
                epi_bar_sync();
                if (leader) {
                    __threadfence();
                    const uint32_t old = atomicAdd(p.ws_count + tile, units);
                    tail->is_last = (old + units == static_cast<uint32_t>(p.kblocks)) ? 1u : 0u;
                    __threadfence();
                }
                epi_bar_sync();
                if (tail->is_last) {
                    for (int h = 0; h < kSkHalves; ++h) {
                        const int64_t n = static_cast<int64_t>(tile) * kSkUnitN + h * kSkTileN + row;
                        if (n < ep.N) {
                            int32_t *ws = p.ws_acc + (static_cast<int64_t>(tile * kSkHalves + h) * p.mpad) * kSkTileN + row;
                            // sixteen independent loads at a time: one L2 round trip per batch, not per row
                            for (int m0 = 0; m0 < M; m0 += 16) {
                                int32_t v[16];
#pragma unroll
                                for (int j = 0; j < 16; ++j)
                                    v[j] = (m0 + j < M) ? __ldcg(ws + static_cast<int64_t>(m0 + j) * kSkTileN) : 0;
#pragma unroll
                                for (int j = 0; j < 16; ++j)
                                    if (m0 + j < M) __stcg(ws + static_cast<int64_t>(m0 + j) * kSkTileN, 0);
#pragma unroll
                                for (int j = 0; j < 16; ++j)
                                    if (m0 + j < M) epilogue_one<OutT>(ep, m0 + j, n, v[j]);
                            }
                        }
                    }
                    if (leader) p.ws_count[tile] = 0;
                }
                epi_bar_sync();  // is_last is rewritten by the next split segment
            }
            u = seg_end;
            ++seg;
        }
    }

    // ---------------- teardown ----------------
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && tail->abort_flag != 0 && p.status != nullptr) atomicMax(p.status, tail->abort_flag);
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kSkTmemCols);
    }
}

int mpad_of(int64_t M) { return static_cast<int>((M + 15) / 16 * 16); }

}  // namespace

bool streamk_supported(int64_t M, int64_t N, int64_t K, int64_t x2_sn) {
    (void)x2_sn;
    return M >= 1 && M <= 128 && N >= 1 && K >= 1;
}

size_t streamk_workspace_bytes(int64_t M, int64_t N, int64_t K) {
    (void)K;
    const int64_t tiles_n = (N + kSkTileN - 1) / kSkTileN;
    const size_t acc = static_cast<size_t>(tiles_n) * mpad_of(M) * kSkTileN * sizeof(int32_t);
    const size_t cnt = (static_cast<size_t>(tiles_n) * sizeof(uint32_t) + 255) / 256 * 256;
    return acc + cnt;
}

template <typename OutT>
static int launch_streamk_t(const int8_t *x1, int64_t ld_x1, const int8_t *x2, int64_t x2_sk, int64_t x2_sn,
                            const EpilogueParams &ep, int64_t K, void *workspace, uint32_t *status,
                            cudaStream_t stream) {
    SkParams p;
    p.ep = ep;
    p.K = static_cast<int>(K);
    p.mpad = mpad_of(ep.M);
    p.stage_bytes = kSkABytes + p.mpad * kSkBK;
    int stages = static_cast<int>((kSkSmemBudget - 1024 - sizeof(SkSmemTail)) / p.stage_bytes);
    p.stages = stages > kSkMaxStages ? kSkMaxStages : stages;
    p.tiles_n = static_cast<int>((ep.N + kSkUnitN - 1) / kSkUnitN);
    p.kblocks = static_cast<int>((K + kSkBK - 1) / kSkBK);
    const size_t acc_bytes = static_cast<size_t>((ep.N + kSkTileN - 1) / kSkTileN) * p.mpad * kSkTileN * sizeof(int32_t);
    p.ws_acc = static_cast<int32_t *>(workspace);
    p.ws_count = reinterpret_cast<uint32_t *>(static_cast<uint8_t *>(workspace) + acc_bytes);
    p.status = status;  // where a bounded wait that gives up records its code

    const bool mn_major = (x2_sn == 1);
    CUtensorMap tw, tx;
    int rc;
    if (mn_major)
        rc = make_tmap_2d(&tw, x2, 1, static_cast<uint64_t>(ep.N), static_cast<uint64_t>(K),
                          static_cast<uint64_t>(x2_sk), 128, kSkBK, true);
    else
        rc = make_tmap_2d(&tw, x2, 1, static_cast<uint64_t>(K), static_cast<uint64_t>(ep.N),
                          static_cast<uint64_t>(x2_sn), kSkBK, kSkUnitN, true);
    if (rc != QMM_OK) return rc;
    rc = make_tmap_2d(&tx, x1, 1, static_cast<uint64_t>(K), static_cast<uint64_t>(ep.M),
                      static_cast<uint64_t>(ld_x1), kSkBK, static_cast<uint32_t>(p.mpad), true);
    if (rc != QMM_OK) return rc;

    const int64_t total = static_cast<int64_t>(p.tiles_n) * p.kblocks;
    const int grid = total < sm_count() ? static_cast<int>(total) : sm_count();
    const size_t smem = 1024 + static_cast<size_t>(p.stages) * p.stage_bytes + sizeof(SkSmemTail);
    auto kern = mn_major ? w8a8_streamk_kernel<OutT, true> : w8a8_streamk_kernel<OutT, false>;
    QMM_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     static_cast<int>(kSkSmemBudget)));
    kern<<<grid, kSkThreads, smem, stream>>>(tw, tx, p);
    QMM_CUDA_OK(cudaGetLastError());
    return QMM_OK;
}

int launch_streamk(const int8_t *x1, int64_t ld_x1, const int8_t *x2, int64_t x2_sk, int64_t x2_sn,
                   const EpilogueParams &ep, int out_dtype, int64_t K, void *workspace, size_t workspace_bytes,
                   cudaStream_t stream) {
    if (!streamk_supported(ep.M, ep.N, K, x2_sn))
        return fail(QMM_ERR_UNSUPPORTED, "qmm_quant_matmul: the stream-K kernel handles 1 <= M <= 128 only");
    if (workspace == nullptr || workspace_bytes < streamk_workspace_bytes(ep.M, ep.N, K))
        return fail(QMM_ERR_WORKSPACE, "qmm_quant_matmul: workspace missing or smaller than "
                                       "qmm_quant_matmul_workspace_size reports");
    if (reinterpret_cast<uintptr_t>(workspace) & 15)
        return fail(QMM_ERR_WORKSPACE, "qmm_quant_matmul: workspace must be 16-byte aligned");
    switch (out_dtype) {
        case QMM_DTYPE_BF16:
            return launch_streamk_t<__nv_bfloat16>(x1, ld_x1, x2, x2_sk, x2_sn, ep, K, workspace, device_status_word(), stream);
        case QMM_DTYPE_F16:
            return launch_streamk_t<__half>(x1, ld_x1, x2, x2_sk, x2_sn, ep, K, workspace, device_status_word(), stream);
        default:
            return launch_streamk_t<int32_t>(x1, ld_x1, x2, x2_sk, x2_sn, ep, K, workspace, device_status_word(), stream);
    }
}

}  // namespace qmm

// ---------------------------------------------------------------------------
// Decode matmul for callers that cannot allocate device memory.
//
// Some hosts of this library run where cudaMalloc is off limits: inside a
// serving loop whose memory was carved up at start-up and handed out by the
// host's own arena, in a plugin whose contract forbids allocation after
// initialisation, or on a thread that must never take the allocator's locks.
// The regular entry point needs a scratch buffer from its caller (and the
// operator host code takes that from the framework allocator).  This variant
// brings its own: the split-K partial sums and tile counters live in a
// fixed-size array that is part of the library image, so the call itself
// allocates nothing, on the device or on the host.
// ---------------------------------------------------------------------------
namespace qmm {
namespace {

// Scratch of the no-allocation entry point.  Every device that loads the library
// holds these 16 MiB until the process exits.
static __device__ __align__(256) uint8_t g_noalloc_scratch[QMM_NOALLOC_SCRATCH_BYTES];
// Where a kernel launched through this entry point records a bounded wait that gave up (the process-wide
// status word of the other entry points lives in allocated host memory, which this path must not create).
static __device__ uint32_t g_noalloc_status;
// Codes already acted upon by noalloc_prepare_kernel (kept so that the host can still read them).
static __device__ uint32_t g_noalloc_status_reported;

// What must start at zero: the partial sums and tile counters.  The stream-K kernel hands the array back
// zeroed (every tile's last arriver clears what the tile used), so in the normal case there is nothing to do
// and a memset of up to 16 MiB per call (74 us at M = 128, N = 28672) would be wasted.  Only a call that was cut
// short - a bounded wait gave up, which the kernel records in g_noalloc_status - can leave sums behind; this
// one-CTA kernel, launched in front of every call, clears the whole array when the status word is set, and
// moves the code to a second word for the host to read.  The library loader zero-fills the array, so the first
// call needs no clearing either.
__global__ void __launch_bounds__(1024) noalloc_prepare_kernel() {
    __shared__ uint32_t code;
    if (threadIdx.x == 0) code = g_noalloc_status;
    __syncthreads();
    if (code == 0) return;
    uint4 *p = reinterpret_cast<uint4 *>(g_noalloc_scratch);
    for (uint32_t i = threadIdx.x; i < QMM_NOALLOC_SCRATCH_BYTES / 16; i += blockDim.x) p[i] = make_uint4(0, 0, 0, 0);
    __syncthreads();
    if (threadIdx.x == 0) {
        if (code > g_noalloc_status_reported) g_noalloc_status_reported = code;
        g_noalloc_status = 0;
    }
}

constexpr int kMaxDevices = 64;
std::mutex g_noalloc_mutex;
void *g_noalloc_ptr[kMaxDevices] = {};
uint32_t *g_noalloc_status_ptr[kMaxDevices] = {};

// Device address of g_noalloc_scratch on the current device.  In host code the
// array's name is only a handle for the runtime, not an address a kernel could
// use, so the address is looked up once per device (with that device current).
int noalloc_scratch_address(void **out, uint32_t **status_out) {
    int dev = 0;
    QMM_CUDA_OK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) return fail(QMM_ERR_UNSUPPORTED, "device ordinal beyond 63");
    std::lock_guard<std::mutex> lock(g_noalloc_mutex);
    if (g_noalloc_ptr[dev] == nullptr) {
        void *p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
        if (e != cudaSuccess || p == nullptr)
            return fail(QMM_ERR_CUDA, std::string("cudaGetSymbolAddress(g_noalloc_scratch): ") + cudaGetErrorString(e));
        void *st = nullptr;
        e = cudaGetSymbolAddress(&st, g_noalloc_status);
        if (e != cudaSuccess || st == nullptr)
            return fail(QMM_ERR_CUDA, std::string("cudaGetSymbolAddress(g_noalloc_status): ") + cudaGetErrorString(e));
        g_noalloc_ptr[dev] = p;
        g_noalloc_status_ptr[dev] = static_cast<uint32_t *>(st);
    }
    *out = g_noalloc_ptr[dev];
    *status_out = g_noalloc_status_ptr[dev];
    return QMM_OK;
}

}  // namespace

int validate_quant_matmul(const int8_t *x1, int64_t ld_x1, const int8_t *x2, int64_t x2_sk, int64_t x2_sn,
                          const float *scale, int64_t scale_len, const void *bias, int bias_dtype, void *out,
                          int out_dtype, int64_t ld_out, int64_t M, int64_t N, int64_t K);

}  // namespace qmm

extern "C" int qmm_quant_matmul_decode_noalloc(const int8_t *x1, int64_t ld_x1, const int8_t *x2,
                                               int64_t x2_stride_k, int64_t x2_stride_n, const float *scale,
                                               int64_t scale_len, const float *pertoken_scale, const void *bias,
                                               int bias_dtype, void *out, int out_dtype, int64_t ld_out, int64_t M,
                                               int64_t N, int64_t K, void *stream) {
    using namespace qmm;
    int rc = validate_quant_matmul(x1, ld_x1, x2, x2_stride_k, x2_stride_n, scale, scale_len, bias, bias_dtype, out,
                                   out_dtype, ld_out, M, N, K);
    if (rc != QMM_OK) return rc;
    if (M == 0 || N == 0) return QMM_OK;
    if (!(M >= 1 && M <= 128 && K >= 1))
        return fail(QMM_ERR_UNSUPPORTED, "qmm_quant_matmul_decode_noalloc: needs 1 <= M <= 128 and K >= 1, got M=" +
                                             std::to_string(M) + " K=" + std::to_string(K));
    const size_t need = streamk_workspace_bytes(M, N, K);
    if (need > static_cast<size_t>(QMM_NOALLOC_SCRATCH_BYTES))
        return fail(QMM_ERR_WORKSPACE, "qmm_quant_matmul_decode_noalloc: M=" + std::to_string(M) + ", N=" +
                                           std::to_string(N) + " needs " + std::to_string(need) +
                                           " bytes of scratch, the built-in buffer holds " +
                                           std::to_string(static_cast<size_t>(QMM_NOALLOC_SCRATCH_BYTES)) +
                                           "; use qmm_quant_matmul with a caller-provided workspace");
    const bool aligned = ((reinterpret_cast<uintptr_t>(x1) & 15) == 0) && ((ld_x1 & 15) == 0) &&
                         ((reinterpret_cast<uintptr_t>(x2) & 15) == 0) &&
                         ((x2_stride_n == 1) ? ((x2_stride_k & 15) == 0) : ((x2_stride_n & 15) == 0));
    if (!aligned)
        return fail(QMM_ERR_UNSUPPORTED,
                    "qmm_quant_matmul_decode_noalloc: operands need 16-byte aligned addresses and row pitches");
    void *scratch = nullptr;
    uint32_t *status = nullptr;
    rc = noalloc_scratch_address(&scratch, &status);
    if (rc != QMM_OK) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // The array keeps whatever the previous call left: zeros, unless that call was cut short, in which case
    // the prepare kernel clears it (device code names the array directly; only the launch below needs the
    // address that was looked up).
    noalloc_prepare_kernel<<<1, 1024, 0, s>>>();
    QMM_CUDA_OK(cudaGetLastError());
    EpilogueParams ep;
    ep.scale = scale;
    ep.pertoken_scale = (out_dtype == QMM_DTYPE_I32) ? nullptr : pertoken_scale;
    ep.bias = bias;
    ep.bias_dtype = bias ? bias_dtype : QMM_DTYPE_NONE;
    ep.scale_is_scalar = (scale_len == 1 && N != 1) ? 1 : 0;
    ep.out = out;
    ep.ld_out = ld_out;
    ep.M = M;
    ep.N = N;
    switch (out_dtype) {
        case QMM_DTYPE_BF16:
            return launch_streamk_t<__nv_bfloat16>(x1, ld_x1, x2, x2_stride_k, x2_stride_n, ep, K, scratch, status, s);
        case QMM_DTYPE_F16:
            return launch_streamk_t<__half>(x1, ld_x1, x2, x2_stride_k, x2_stride_n, ep, K, scratch, status, s);
        default:
            return launch_streamk_t<int32_t>(x1, ld_x1, x2, x2_stride_k, x2_stride_n, ep, K, scratch, status, s);
    }
}

extern "C" int qmm_noalloc_status(int reset) {
    using namespace qmm;
    // the live word (a call was cut short and no later call has cleaned up yet) or the word of codes already
    // cleaned up after; only the second one is cleared here, the first one belongs to the prepare kernel
    uint32_t live = 0, reported = 0;
    if (cudaMemcpyFromSymbol(&live, g_noalloc_status, sizeof(live)) != cudaSuccess ||
        cudaMemcpyFromSymbol(&reported, g_noalloc_status_reported, sizeof(reported)) != cudaSuccess) {
        (void)cudaGetLastError();
        return -1;
    }
    if (reset && reported != 0) {
        const uint32_t zero = 0;
        (void)cudaMemcpyToSymbol(g_noalloc_status_reported, &zero, sizeof(zero));
    }
    return static_cast<int>(live > reported ? live : reported);
}
