// Per-token dynamic quantization (npu_dynamic_quant).
//
// One pass over HBM: a row (token) is held in registers as 128-bit vectors,
// its absmax is reduced with warp shuffles (plus one shared-memory hop when a
// row spans several warps), then the same registers are scaled, rounded
// half-to-even, packed to int8 and stored.  Algorithmic traffic is
// 2*cols (read) + cols (write) + 4 (scale) bytes per row.
//
// Numerics (bit-exact contract with the CPU oracle):
//   scale = amax / 127            IEEE fp32 division
//   q     = rint(x / scale)       IEEE fp32 division, round half to even
// The division x / scale runs on the FMA pipe: with y = RN(1/scale), q0 = RN(x*y) (within two ulps
// of the quotient), r = fma(-q0, scale, x) (the remainder, one rounding at most) and
// q1 = RN(q0 + r*y).  q0 + r*y differs from the exact quotient by less than 2^-21 ulp, so q1 is the
// IEEE quotient unless x/scale lies that close to a rounding boundary without being on it; the
// integer rint(q1) could differ from rint(x/scale) only if, in addition, that boundary neighbours a
// half-integer.  The tests compare against IEEE division for every pair of bf16 significands and of
// f16 significands (quotient significands do not depend on exponents), which covers the inputs this
// operator accepts.  Rows whose scale is tiny, not finite, or has an all-ones significand take
// true divisions.  A row that holds an infinity has an infinite scale (finite elements quantize to 0);
// a row that holds a NaN has a NaN scale; a quotient that is NaN (Inf / Inf, anything / NaN)
// quantizes to 0.
// bf16/f16 inputs make EXACT ties (x / scale = n + 1/2) common - x and amax are short-significand
// numbers - so a scheme that falls back to a division near ties would fall back all the time.
#include "dynamic_quant.cuh"

namespace qmm {

namespace {

using namespace dq;

// Vector kernel: `tpr` threads per row, each holding VPT 16-byte vectors.
template <typename T, int VPT>
__global__ void __launch_bounds__(512)
dynamic_quant_vec_kernel(const T *__restrict__ x, int64_t rows, int cols, int64_t ld_x, int8_t *__restrict__ q,
                         int64_t ld_q, float *__restrict__ scale, int tpr) {
    __shared__ float s_part[16];
    const int tpr_shift = __ffs(tpr) - 1;  // tpr is a power of two
    const int rows_per_cta = blockDim.x >> tpr_shift;
    const int row_in_cta = threadIdx.x >> tpr_shift;
    const int t = threadIdx.x & (tpr - 1);
    const int64_t row = static_cast<int64_t>(blockIdx.x) * rows_per_cta + row_in_cta;
    const bool row_ok = row < rows;
    const int nvec = cols >> 3;

    uint4 v[VPT];
    float amax = 0.0f;
    if (row_ok) {
        const uint4 *src = reinterpret_cast<const uint4 *>(x + row * ld_x);
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            const int idx = t + i * tpr;
            v[i] = idx < nvec ? __ldg(src + idx) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int i = 0; i < VPT; ++i) amax = max_nan(amax, absmax8<T>(v[i]));
    }
    amax = warp_max(amax);
    if (tpr > 32) {
        const int warp = threadIdx.x >> 5;
        const int warps_per_row = tpr >> 5;
        if ((threadIdx.x & 31) == 0) s_part[warp] = amax;
        __syncthreads();
        const int w0 = row_in_cta * warps_per_row;
        float m = 0.0f;
        for (int w = 0; w < warps_per_row; ++w) m = max_nan(m, s_part[w0 + w]);
        amax = m;
    }
    if (!row_ok) return;
    const RowQuant rq = make_row_quant(amax);
    if (t == 0) scale[row] = rq.scale;
    const bool fast = !rq.exact_only && rq.scale != 0.0f;

    uint2 *dst = reinterpret_cast<uint2 *>(q + row * ld_q);
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int idx = t + i * tpr;
        if (idx < nvec) {
            float f[8];
            unpack8<T>(v[i], f);
            dst[idx] = quantize8(f, rq, fast);
        }
    }
}

// Generic kernel: any column count, stride or alignment; one CTA per row, the
// row is read twice (second read is served by L2).
template <typename T>
__global__ void __launch_bounds__(256)
dynamic_quant_generic_kernel(const T *__restrict__ x, int64_t rows, int64_t cols, int64_t ld_x,
                             int8_t *__restrict__ q, int64_t ld_q, float *__restrict__ scale) {
    __shared__ float s_part[8];
    const int64_t row = blockIdx.x;
    if (row >= rows) return;
    const T *src = x + row * ld_x;
    float amax = 0.0f;
    for (int64_t c = threadIdx.x; c < cols; c += blockDim.x) amax = max_nan(amax, fabsf(to_float(src[c])));
    amax = warp_max(amax);
    if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = amax;
    __syncthreads();
    float m = 0.0f;
    for (int w = 0; w < static_cast<int>(blockDim.x >> 5); ++w) m = max_nan(m, s_part[w]);
    const RowQuant rq = make_row_quant(m);
    if (threadIdx.x == 0) scale[row] = rq.scale;
    int8_t *dst = q + row * ld_q;
    for (int64_t c = threadIdx.x; c < cols; c += blockDim.x)
        dst[c] = static_cast<int8_t>(quant_one(to_float(src[c]), rq));
}

template <typename T>
int launch_dynamic_quant(const T *x, int64_t rows, int64_t cols, int64_t ld_x, int8_t *q, int64_t ld_q, float *scale,
                         cudaStream_t stream) {
    const bool vec_ok = (cols % 8 == 0) && (ld_x % 8 == 0) && (ld_q % 8 == 0) &&
                        ((reinterpret_cast<uintptr_t>(x) & 15) == 0) && ((reinterpret_cast<uintptr_t>(q) & 7) == 0) &&
                        cols <= 32768;
    if (vec_ok) {
        const int nvec = static_cast<int>(cols / 8);
        int tpr = 32;
        // eight vectors per thread where the row is long enough: the kernels are bound by instruction issue, and
        // the per-thread fixed cost (row scale, reductions, index arithmetic) is then spread over more elements
        while (tpr < 512 && tpr * 8 < nvec) tpr <<= 1;
        const int need = (nvec + tpr - 1) / tpr;
        const int vpt = need <= 1 ? 1 : need <= 2 ? 2 : need <= 4 ? 4 : 8;
        const int threads = tpr > 128 ? tpr : 128;  // small CTAs: the tail of the grid is one CTA long
        const int rows_per_cta = threads / tpr;
        const int64_t grid = (rows + rows_per_cta - 1) / rows_per_cta;
        const int icols = static_cast<int>(cols);
        switch (vpt) {
            case 1:
                dynamic_quant_vec_kernel<T, 1><<<grid, threads, 0, stream>>>(x, rows, icols, ld_x, q, ld_q, scale, tpr);
                break;
            case 2:
                dynamic_quant_vec_kernel<T, 2><<<grid, threads, 0, stream>>>(x, rows, icols, ld_x, q, ld_q, scale, tpr);
                break;
            case 4:
                dynamic_quant_vec_kernel<T, 4><<<grid, threads, 0, stream>>>(x, rows, icols, ld_x, q, ld_q, scale, tpr);
                break;
            default:
                dynamic_quant_vec_kernel<T, 8><<<grid, threads, 0, stream>>>(x, rows, icols, ld_x, q, ld_q, scale, tpr);
                break;
        }
    } else {
        dynamic_quant_generic_kernel<T><<<rows, 256, 0, stream>>>(x, rows, cols, ld_x, q, ld_q, scale);
    }
    QMM_CUDA_OK(cudaGetLastError());
    return QMM_OK;
}

}  // namespace

}  // namespace qmm

extern "C" int qmm_dynamic_quant(const void *x, int x_dtype, int64_t rows, int64_t cols, int64_t ld_x, int8_t *q,
                                 int64_t ld_q, float *scale, void *stream) {
    using namespace qmm;
    QMM_REQUIRE(rows >= 0 && cols >= 0, "qmm_dynamic_quant: rows and cols must be non-negative");
    if (rows == 0) return QMM_OK;
    QMM_REQUIRE(scale != nullptr, "qmm_dynamic_quant: scale output is NULL");
    QMM_REQUIRE(rows < (1ll << 31), "qmm_dynamic_quant: more than 2^31-1 rows");
    if (cols == 0) {
        QMM_CUDA_OK(cudaMemsetAsync(scale, 0, sizeof(float) * rows, static_cast<cudaStream_t>(stream)));
        return QMM_OK;
    }
    QMM_REQUIRE(x != nullptr && q != nullptr, "qmm_dynamic_quant: NULL input or output");
    QMM_REQUIRE(ld_x >= cols && ld_q >= cols, "qmm_dynamic_quant: row stride smaller than the row length");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    switch (x_dtype) {
        case QMM_DTYPE_BF16:
            return launch_dynamic_quant(static_cast<const __nv_bfloat16 *>(x), rows, cols, ld_x, q, ld_q, scale, s);
        case QMM_DTYPE_F16:
            return launch_dynamic_quant(static_cast<const __half *>(x), rows, cols, ld_x, q, ld_q, scale, s);
        default:
            return fail(QMM_ERR_UNSUPPORTED, "qmm_dynamic_quant: input dtype must be bf16 or f16");
    }
}
