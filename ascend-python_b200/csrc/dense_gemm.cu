// Dense bf16/f16 matmul, fp32 accumulation: the compute half of npu_mm_reduce_scatter_base and
// npu_all_gather_base_mm (see dense_gemm.cuh).
//
// Same skeleton as the W8A8 tile kernel: warp 0 feeds a ring of [128 x 64] A and [64 x 256] B stages by
// TMA (128-byte swizzle), warp 1 issues four tcgen05.mma.kind::f16 128 x 256 x 16 per stage into one of
// two TMEM accumulators, four epilogue warps drain the other one.  (256 columns per MMA: a 128 x 128 x 16
// MMA reads 8 KiB of operands in the 64 clocks it occupies the pipe, all of an SM's shared-memory
// bandwidth, and the pipe was measured half idle; 128 x 256 x 16 reads 12 KiB in 128 clocks.)  B is
// taken as stored: a row-major
// [K, N] matrix is the MMA's MN-major operand (four 64-column boxes per stage), the transposed view of a
// row-major [N, K] its K-major operand.  The epilogue either casts (+ bias) into a local 16-bit output or
// stores the raw fp32 accumulator rows straight into the peer region of the rank that will reduce them.
#include "dense_gemm.cuh"

#include <type_traits>

namespace qmm {

namespace {

constexpr int kDM = 128, kDN = 256, kDK = 64;        // tile; kDK 16-bit elements = one 128-byte swizzle row
constexpr int kDStages = 4;
constexpr int kDABytes = kDM * kDK * 2;              // 16 KiB
constexpr int kDBBytes = kDN * kDK * 2;              // 32 KiB
constexpr int kDBBoxBytes = 64 * kDK * 2;            // one [64 k-rows][64 n] box of an MN-major B: 8 KiB
constexpr int kDStageBytes = kDABytes + kDBBytes;
constexpr int kDThreads = 192;
constexpr uint32_t kDTmemCols = 512;                 // two accumulators of 256 columns

struct DenseSmemTail {
    uint64_t full[kDStages];
    uint64_t empty[kDStages];
    uint64_t tmem_full[2];
    uint64_t tmem_empty[2];
    uint32_t tmem_base;
    uint32_t abort_flag;
};
constexpr size_t kDenseSmemBytes = 1024 + kDStages * kDStageBytes + sizeof(DenseSmemTail);

struct DenseKernelParams {
    int64_t M, N;
    int K;
    int mode;
    void *out;
    int64_t ld_out;
    const void *bias;
    uint8_t *base[8];
    size_t area_off;
    int rank;
    int64_t rows_per;
    uint32_t *status;
};

template <typename T>
__device__ __forceinline__ void dense_store_row(const DenseKernelParams &p, int64_t m, int64_t n0, const uint32_t (&acc)[32]) {
    if (m >= p.M) return;
    if (p.mode == kDenseOutPush) {
        const int64_t o = m / p.rows_per;
        float *dst = reinterpret_cast<float *>(p.base[o] + p.area_off) +
                     (static_cast<int64_t>(p.rank) * p.rows_per + (m - o * p.rows_per)) * p.N + n0;
        if (n0 + 32 <= p.N && (p.N & 3) == 0) {
#pragma unroll
            for (int j = 0; j < 32; j += 4)
                *reinterpret_cast<uint4 *>(dst + j) = make_uint4(acc[j], acc[j + 1], acc[j + 2], acc[j + 3]);
        } else {
            for (int j = 0; j < 32 && n0 + j < p.N; ++j) dst[j] = __uint_as_float(acc[j]);
        }
        return;
    }
    const T *bias = static_cast<const T *>(p.bias);
    T *dst = static_cast<T *>(p.out) + m * p.ld_out + n0;
    if (n0 + 32 <= p.N && (p.ld_out & 7) == 0 && (reinterpret_cast<uintptr_t>(p.out) & 15) == 0) {
#pragma unroll
        for (int j = 0; j < 32; j += 8) {
            float f[8];
#pragma unroll
            for (int i = 0; i < 8; ++i)
                f[i] = __uint_as_float(acc[j + i]) + (bias != nullptr ? to_float(bias[n0 + j + i]) : 0.0f);
            *reinterpret_cast<uint4 *>(dst + j) =
                make_uint4(pack2<T>(f[0], f[1]), pack2<T>(f[2], f[3]), pack2<T>(f[4], f[5]), pack2<T>(f[6], f[7]));
        }
    } else {
        for (int j = 0; j < 32 && n0 + j < p.N; ++j)
            dst[j] = from_float<T>(__uint_as_float(acc[j]) + (bias != nullptr ? to_float(bias[n0 + j]) : 0.0f));
    }
}

template <typename T, bool B_MN_MAJOR>
__global__ void __launch_bounds__(kDThreads, 1)
dense_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                  DenseKernelParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *smem_aligned = smem_raw + (smem_base - smem_u32(smem_raw));
    DenseSmemTail *tail = reinterpret_cast<DenseSmemTail *>(smem_aligned + kDStages * kDStageBytes);
    volatile uint32_t *abort_flag = &tail->abort_flag;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int tiles_m = static_cast<int>((p.M + kDM - 1) / kDM);
    const int tiles_n = static_cast<int>((p.N + kDN - 1) / kDN);
    const int num_tiles = tiles_m * tiles_n;
    const int num_kb = (p.K + kDK - 1) / kDK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kDStages; ++s) {
            mbar_init(smem_u32(&tail->full[s]), 1);
            mbar_init(smem_u32(&tail->empty[s]), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(smem_u32(&tail->tmem_full[b]), 1);
            mbar_init(smem_u32(&tail->tmem_empty[b]), 4);
        }
        tail->abort_flag = 0;
        mbar_fence_init();
        tma_prefetch_desc(&tmap_a);
        tma_prefetch_desc(&tmap_b);
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(&tail->tmem_base), kDTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tail->tmem_base;

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        uint32_t stage = 0, phase = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
            const int m_blk = tile % tiles_m, n_blk = tile / tiles_m;
            for (int kb = 0; kb < num_kb; ++kb) {
                ok = mbar_wait(smem_u32(&tail->empty[stage]), phase ^ 1, abort_flag, 0x70);
                if (!ok) break;
                if (lane == 0) {
                    const uint32_t full = smem_u32(&tail->full[stage]);
                    const uint32_t sa = smem_base + stage * kDStageBytes;
                    const uint32_t sb = sa + kDABytes;
                    mbar_expect_tx(full, kDStageBytes);
                    tma_load_2d(sa, &tmap_a, kb * kDK, m_blk * kDM, full);  // [128 rows][64 k]
                    if (B_MN_MAJOR) {
                        // four [64 k-rows][64 n] boxes side by side
#pragma unroll
                        for (int bx = 0; bx < kDN / 64; ++bx)
                            tma_load_2d(sb + bx * kDBBoxBytes, &tmap_b, n_blk * kDN + bx * 64, kb * kDK, full);
                    } else {
                        tma_load_2d(sb, &tmap_b, kb * kDK, n_blk * kDN, full);  // [256 n-rows][64 k]
                    }
                }
                __syncwarp();
                if (++stage == kDStages) {
                    stage = 0;
                    phase ^= 1;
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer (warp-uniform, one elected lane) ----------------
        constexpr uint32_t kFmt = sizeof(T) == 2 && std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;
        constexpr uint32_t idesc = make_idesc(/*c=f32*/ 1, kFmt, kFmt, /*a K-major*/ 0, B_MN_MAJOR ? 1u : 0u, kDM, kDN);
        constexpr uint32_t kDescHi = smem_desc_hi_sw128(1024);
        constexpr uint32_t kStageStep = kDStageBytes >> 4;
        // A and K-major B: 16 k = 32 bytes (+2) per MMA.  MN-major B: 16 k-rows of 128 bytes = 2048 bytes (+128)
        // per MMA, the next 64-column box 8 KiB further (leading offset).
        constexpr uint32_t kBStep = B_MN_MAJOR ? (2048u >> 4) : 2u;
        const uint32_t a_lo0 = smem_desc_lo(smem_base, 16);
        const uint32_t b_lo0 = smem_desc_lo(smem_base + kDABytes, B_MN_MAJOR ? kDBBoxBytes : 16);
        uint32_t stage = 0, phase = 0;
        int local = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++local) {
            const uint32_t buf = local & 1, buf_phase = (local >> 1) & 1;
            ok = mbar_wait(smem_u32(&tail->tmem_empty[buf]), buf_phase ^ 1, abort_flag, 0x71);
            if (!ok) break;
            tc_fence_after();
            const uint32_t d_tmem = tmem_base + buf * kDN;
            uint32_t accumulate = 0;
            for (int kb = 0; kb < num_kb; ++kb) {
                ok = mbar_wait(smem_u32(&tail->full[stage]), phase, abort_flag, 0x72);
                if (!ok) break;
                tc_fence_after();
                const uint32_t a_lo = a_lo0 + stage * kStageStep;
                const uint32_t b_lo = b_lo0 + stage * kStageStep;
#pragma unroll
                for (int k = 0; k < kDK / 16; ++k) {
                    mma_f16_ss_warp(d_tmem, desc64(a_lo + 2 * k, kDescHi), desc64(b_lo + kBStep * k, kDescHi), idesc,
                                    accumulate);
                    accumulate = 1;
                }
                tc_commit_warp(smem_u32(&tail->empty[stage]));
                if (++stage == kDStages) {
                    stage = 0;
                    phase ^= 1;
                }
            }
            if (ok) tc_commit_warp(smem_u32(&tail->tmem_full[buf]));
        }
    } else {
        // ---------------- epilogue warps: thread = accumulator lane = one output row ----------------
        const int quarter = warp & 3;
        int local = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++local) {
            const int m_blk = tile % tiles_m, n_blk = tile / tiles_m;
            const uint32_t buf = local & 1, buf_phase = (local >> 1) & 1;
            ok = mbar_wait(smem_u32(&tail->tmem_full[buf]), buf_phase, abort_flag, 0x73);
            if (!ok) break;
            tc_fence_after();
            const int64_t m = static_cast<int64_t>(m_blk) * kDM + quarter * 32 + lane;
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + buf * kDN;
#pragma unroll 1
            for (int c = 0; c < kDN / 32; ++c) {
                uint32_t acc[32];
                tmem_ld_32x32(taddr + c * 32, acc);
                tmem_ld_wait();
                if (p.K == 0) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) acc[j] = 0;
                }
                dense_store_row<T>(p, m, static_cast<int64_t>(n_blk) * kDN + c * 32, acc);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&tail->tmem_empty[buf]));
        }
    }

    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && tail->abort_flag != 0 && p.status != nullptr) atomicMax(p.status, tail->abort_flag);
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kDTmemCols);
    }
}

// Any stride or alignment: one thread per output element, fp32 accumulation in k order.
template <typename T>
__global__ void __launch_bounds__(256)
dense_gemm_simt_kernel(const T *__restrict__ a, int64_t ld_a, const T *__restrict__ b, int64_t b_sk, int64_t b_sn,
                       DenseKernelParams p) {
    const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= p.M * p.N) return;
    const int64_t m = idx / p.N, n = idx - m * p.N;
    float acc = 0.0f;
    for (int64_t k = 0; k < p.K; ++k) acc = fmaf(to_float(a[m * ld_a + k]), to_float(b[k * b_sk + n * b_sn]), acc);
    if (p.mode == kDenseOutPush) {
        const int64_t o = m / p.rows_per;
        reinterpret_cast<float *>(p.base[o] + p.area_off)[(static_cast<int64_t>(p.rank) * p.rows_per + (m - o * p.rows_per)) * p.N + n] = acc;
    } else {
        const T *bias = static_cast<const T *>(p.bias);
        static_cast<T *>(p.out)[m * p.ld_out + n] = from_float<T>(acc + (bias != nullptr ? to_float(bias[n]) : 0.0f));
    }
}

template <typename T>
int launch_dense_t(const DenseParams &d, cudaStream_t stream) {
    DenseKernelParams p;
    p.M = d.M;
    p.N = d.N;
    p.K = static_cast<int>(d.K);
    p.mode = d.mode;
    p.out = d.out;
    p.ld_out = d.ld_out;
    p.bias = d.bias;
    for (int r = 0; r < 8; ++r) p.base[r] = d.base[r];
    p.area_off = d.area_off;
    p.rank = d.rank;
    p.rows_per = d.rows_per > 0 ? d.rows_per : 1;
    p.status = device_status_word();

    const bool mn_major = (d.b_sn == 1);
    const int64_t b_ld = mn_major ? d.b_sk : d.b_sn;
    const bool tma_ok = d.K > 0 && d.K < (1ll << 31) && d.M < (1ll << 31) && d.N < (1ll << 31) &&
                        (reinterpret_cast<uintptr_t>(d.a) & 15) == 0 && (d.ld_a & 7) == 0 &&
                        (reinterpret_cast<uintptr_t>(d.b) & 15) == 0 && (b_ld & 7) == 0 &&
                        (d.b_sk == 1 || d.b_sn == 1);
    if (!tma_ok) {
        const int64_t total = d.M * d.N;
        dense_gemm_simt_kernel<T><<<static_cast<unsigned>((total + 255) / 256), 256, 0, stream>>>(
            static_cast<const T *>(d.a), d.ld_a, static_cast<const T *>(d.b), d.b_sk, d.b_sn, p);
        QMM_CUDA_OK(cudaGetLastError());
        return QMM_OK;
    }
    CUtensorMap ta, tb;
    int rc = make_tmap_2d(&ta, d.a, 2, static_cast<uint64_t>(d.K), static_cast<uint64_t>(d.M),
                          static_cast<uint64_t>(d.ld_a), kDK, kDM, true);
    if (rc != QMM_OK) return rc;
    if (mn_major)
        rc = make_tmap_2d(&tb, d.b, 2, static_cast<uint64_t>(d.N), static_cast<uint64_t>(d.K),
                          static_cast<uint64_t>(d.b_sk), 64, kDK, true);
    else
        rc = make_tmap_2d(&tb, d.b, 2, static_cast<uint64_t>(d.K), static_cast<uint64_t>(d.N),
                          static_cast<uint64_t>(d.b_sn), kDK, kDN, true);
    if (rc != QMM_OK) return rc;
    const int tiles = static_cast<int>(((d.M + kDM - 1) / kDM) * ((d.N + kDN - 1) / kDN));
    const int grid = tiles < sm_count() ? tiles : sm_count();
    auto kern = mn_major ? dense_gemm_kernel<T, true> : dense_gemm_kernel<T, false>;
    QMM_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     static_cast<int>(kDenseSmemBytes)));
    kern<<<grid, kDThreads, kDenseSmemBytes, stream>>>(ta, tb, p);
    QMM_CUDA_OK(cudaGetLastError());
    return QMM_OK;
}

}  // namespace

int launch_dense_gemm(const DenseParams &p, cudaStream_t stream) {
    if (p.M <= 0 || p.N <= 0) return QMM_OK;
    if (p.dtype == QMM_DTYPE_BF16) return launch_dense_t<__nv_bfloat16>(p, stream);
    if (p.dtype == QMM_DTYPE_F16) return launch_dense_t<__half>(p, stream);
    return fail(QMM_ERR_UNSUPPORTED, "dense matmul: operands must be bf16 or f16");
}

}  // namespace qmm
