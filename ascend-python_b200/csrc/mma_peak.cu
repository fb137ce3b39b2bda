// Issue-rate ceiling of the int8 tensor pipe, measured: the denominator for the roofline fraction of the
// W8A8 prefill kernels (no published or driver-measured int8 figure exists for this part).
//
// One CTA per SM; operands stay resident in shared memory (no global traffic), one warp issues
// tcgen05.mma.kind::i8 128 x 256 x 32 back to back into two alternating TMEM accumulators and commits
// every 64 MMAs.  The result is what the tensor pipe sustains when nothing but the MMA stream limits it:
// operations per clock and SM (from the SMs' own cycle counters) and TOPS (from CUDA events), at whatever
// clock the board holds during the run.
#include <vector>

#include "qmm_common.cuh"

namespace qmm {
namespace {

constexpr int kPeakM = 128, kPeakN = 256, kPeakK = 32;
constexpr int kPeakBatch = 64;                       // MMAs per commit
constexpr uint32_t kPeakSmem = 1024 + 16384 + 32768;  // A [128][128 B] + B [256][128 B], 128-byte swizzle

__global__ void __launch_bounds__(128, 1) int8_mma_peak_kernel(int batches, long long *cycles, uint32_t *status) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t bar;
    __shared__ uint32_t tbase, abort_flag;
    const uint32_t sb = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // any bit pattern is a valid int8 operand; fill with a fixed non-trivial one (data toggling costs power)
    uint32_t *w = reinterpret_cast<uint32_t *>(smem_raw + (sb - smem_u32(smem_raw)));
    for (uint32_t i = threadIdx.x; i < (16384 + 32768) / 4; i += blockDim.x) w[i] = 0x9e3779b9u * (i + 1u);
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&bar), 1);
        abort_flag = 0;
        mbar_fence_init();
    }
    fence_proxy_async_smem();
    if (warp == 0) {
        tmem_alloc(smem_u32(&tbase), 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tb = tbase;
    if (warp == 0) {
        const uint32_t idesc = make_idesc(/*c=s32*/ 2, 1, 1, 0, 0, kPeakM, kPeakN);
        constexpr uint32_t kHi = smem_desc_hi_sw128(1024);
        const uint32_t a_lo = smem_desc_lo(sb, 16), b_lo = smem_desc_lo(sb + 16384, 16);
        uint32_t phase = 0;
        long long t0 = 0;
        bool ok = true;
        for (int it = 0; it <= batches && ok; ++it) {
            if (it == 1) t0 = clock64();  // the first batch warms up
#pragma unroll 8
            for (int m = 0; m < kPeakBatch; ++m)
                mma_i8_ss_warp(tb + (m & 1) * 256, desc64(a_lo + (m & 3) * 2, kHi), desc64(b_lo + (m & 3) * 2, kHi), idesc, 1);
            tc_commit_warp(smem_u32(&bar));
            ok = mbar_wait(smem_u32(&bar), phase, &abort_flag, 0x60);
            phase ^= 1;
        }
        if (lane == 0) cycles[blockIdx.x] = ok ? clock64() - t0 : -1;
        if (!ok && lane == 0 && status != nullptr) atomicMax(status, abort_flag);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        tmem_dealloc(tb, 512);
    }
}

}  // namespace
}  // namespace qmm

extern "C" int qmm_int8_mma_peak(int batches, double *ops_per_clk_per_sm, double *tops, double *sm_mhz) {
    using namespace qmm;
    QMM_REQUIRE(batches >= 1 && batches <= (1 << 20), "qmm_int8_mma_peak: batches must be in [1, 2^20]");
    const int grid = sm_count();
    long long *d_cycles = nullptr;
    QMM_CUDA_OK(cudaMalloc(&d_cycles, sizeof(long long) * grid));
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    QMM_CUDA_OK(cudaEventCreate(&e0));
    QMM_CUDA_OK(cudaEventCreate(&e1));
    QMM_CUDA_OK(cudaFuncSetAttribute(int8_mma_peak_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     static_cast<int>(kPeakSmem)));
    QMM_CUDA_OK(cudaEventRecord(e0, nullptr));
    int8_mma_peak_kernel<<<grid, 128, kPeakSmem, nullptr>>>(batches, d_cycles, device_status_word());
    QMM_CUDA_OK(cudaEventRecord(e1, nullptr));
    cudaError_t err = cudaEventSynchronize(e1);
    std::vector<long long> h(grid, 0);
    if (err == cudaSuccess) err = cudaMemcpy(h.data(), d_cycles, sizeof(long long) * grid, cudaMemcpyDeviceToHost);
    float ms = 0.0f;
    if (err == cudaSuccess) err = cudaEventElapsedTime(&ms, e0, e1);
    cudaFree(d_cycles);
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    if (err != cudaSuccess) return fail(QMM_ERR_CUDA, std::string("qmm_int8_mma_peak: ") + cudaGetErrorString(err));
    long long worst = 0;
    for (long long c : h) {
        if (c < 0) return fail(QMM_ERR_DEVICE_TIMEOUT, "qmm_int8_mma_peak: a bounded wait gave up");
        if (c > worst) worst = c;
    }
    const double ops_cta = static_cast<double>(batches) * kPeakBatch * 2.0 * kPeakM * kPeakN * kPeakK;  // timed batches
    if (ops_per_clk_per_sm) *ops_per_clk_per_sm = worst > 0 ? ops_cta / static_cast<double>(worst) : 0.0;
    // the event interval also holds the untimed warm-up batch and the launch: scale by (batches + 1) / batches
    if (tops) *tops = ms > 0 ? ops_cta * (batches + 1.0) / batches * grid / (ms * 1e-3) / 1e12 : 0.0;
    if (sm_mhz) *sm_mhz = ms > 0 ? static_cast<double>(worst) * (batches + 1.0) / batches / (ms * 1e-3) / 1e6 : 0.0;
    return QMM_OK;
}
