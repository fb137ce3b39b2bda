// W4A16 matmul, CUDA-core kernel: any M, any alignment; deterministic.
// Each thread owns one packed weight word column (8 output columns) and four
// token rows, walks a slice of K, and the K slices of a block are summed in a
// fixed order through shared memory.
#pragma once

#include "qmm_common.cuh"

namespace qmm {

constexpr int kW4SimtRows = 4;     // token rows per thread
constexpr int kW4SimtSlices = 8;   // K slices per block
constexpr int kW4SimtWords = 32;   // packed words (x8 columns) per block

struct W4Params {
    const void *x;
    int64_t ld_x;
    const int32_t *w;
    int64_t ld_w;
    const void *scale;
    const void *offset;  // may be nullptr
    int64_t group;
    const void *bias;    // may be nullptr
    void *out;
    int64_t ld_out;
    int64_t M, N, K;
};

// signed value of nibble j of a packed word
__device__ __forceinline__ float nibble_value(uint32_t word, int j) {
    return static_cast<float>(static_cast<int32_t>(word << (28 - 4 * j)) >> 28);
}

template <typename T>
__global__ void __launch_bounds__(kW4SimtWords * kW4SimtSlices)
w4a16_simt_kernel(W4Params p) {
    __shared__ float red[kW4SimtSlices][kW4SimtRows][8][kW4SimtWords + 1];
    const int wl = threadIdx.x % kW4SimtWords;
    const int slice = threadIdx.x / kW4SimtWords;
    const int64_t word = static_cast<int64_t>(blockIdx.x) * kW4SimtWords + wl;
    const int64_t n0 = word * 8;
    const int64_t m0 = static_cast<int64_t>(blockIdx.y) * kW4SimtRows;
    const bool word_ok = n0 < p.N;
    const T *x = static_cast<const T *>(p.x);
    const T *sc = static_cast<const T *>(p.scale);
    const T *of = static_cast<const T *>(p.offset);

    float acc[kW4SimtRows][8];
#pragma unroll
    for (int r = 0; r < kW4SimtRows; ++r)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[r][j] = 0.0f;

    // groups are dealt to the K slices round-robin so that a slice never splits a group
    const int64_t ngroups = (p.K + p.group - 1) / p.group;
    if (word_ok) {
        for (int64_t g = slice; g < ngroups; g += kW4SimtSlices) {
            float s[8], o[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const bool ok = n0 + j < p.N;
                s[j] = ok ? to_float(sc[g * p.N + n0 + j]) : 0.0f;
                o[j] = (ok && of != nullptr) ? to_float(of[g * p.N + n0 + j]) : 0.0f;
            }
            const int64_t k_end = min(p.K, (g + 1) * p.group);
            for (int64_t k = g * p.group; k < k_end; ++k) {
                const uint32_t wv = static_cast<uint32_t>(__ldg(p.w + k * p.ld_w + word));
                float wf[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) wf[j] = (nibble_value(wv, j) + o[j]) * s[j];
#pragma unroll
                for (int r = 0; r < kW4SimtRows; ++r) {
                    const int64_t m = m0 + r;
                    const float xv = m < p.M ? to_float(x[m * p.ld_x + k]) : 0.0f;
#pragma unroll
                    for (int j = 0; j < 8; ++j) acc[r][j] = fmaf(xv, wf[j], acc[r][j]);
                }
            }
        }
    }
#pragma unroll
    for (int r = 0; r < kW4SimtRows; ++r)
#pragma unroll
        for (int j = 0; j < 8; ++j) red[slice][r][j][wl] = acc[r][j];
    __syncthreads();
    if (slice == 0 && word_ok) {
        const T *bias = static_cast<const T *>(p.bias);
        T *out = static_cast<T *>(p.out);
#pragma unroll
        for (int r = 0; r < kW4SimtRows; ++r) {
            const int64_t m = m0 + r;
            if (m >= p.M) continue;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                if (n0 + j >= p.N) continue;
                float v = 0.0f;
#pragma unroll
                for (int sl = 0; sl < kW4SimtSlices; ++sl) v += red[sl][r][j][wl];
                if (bias != nullptr) v += to_float(bias[n0 + j]);
                out[m * p.ld_out + n0 + j] = from_float<T>(v);
            }
        }
    }
}

template <typename T>
int launch_w4a16_simt(const W4Params &p, cudaStream_t stream) {
    const int64_t words = (p.N + 7) / 8;
    dim3 grid(static_cast<unsigned>((words + kW4SimtWords - 1) / kW4SimtWords),
              static_cast<unsigned>((p.M + kW4SimtRows - 1) / kW4SimtRows));
    if (grid.y > 65535) return fail(QMM_ERR_UNSUPPORTED, "qmm_weight_quant_batchmatmul: M too large");
    w4a16_simt_kernel<T><<<grid, kW4SimtWords * kW4SimtSlices, 0, stream>>>(p);
    QMM_CUDA_OK(cudaGetLastError());
    return QMM_OK;
}

}  // namespace qmm
