// RMS normalisation (npu_rms_norm) and its fusion with the per-token dynamic quantization that
// follows it in a decoder block (npu_rms_norm_dynamic_quant).
//
// Reference: op_plugin/ops/base_ops/opapi/RmsNormKernelOpApi.cpp:24-35 (host function: outputs y with
// the input's dtype and rstd in fp32) and the numpy golden of
// test/test_custom_ops/test_npu_rms_norm.py:10-18:
//     variance = mean(x^2, axis=-1);  rstd = 1 / sqrt(variance + epsilon);  y = (x * rstd) * gamma
// All arithmetic is fp32 with one rounding per operation in that order; y is rounded once to the
// input dtype.  The sum of squares is taken per thread over its elements in index order, then over
// the lanes of a warp by an xor-shuffle tree, then over the warps of a row in warp order, so it does
// not depend on timing.
//
// One pass over HBM: a row stays in registers as 128-bit vectors between the reduction and the
// scaling.  The fused kernel goes on in the same registers: absmax of the ROUNDED y, scale =
// amax / 127, q = rint(y / scale), exactly the arithmetic of qmm_dynamic_quant applied to the y that
// qmm_rms_norm would have stored, so fused and unfused results are identical bit for bit while y
// never travels to HBM and back (2 * cols bytes written + 2 * cols bytes read per row saved).
#include "dynamic_quant.cuh"

namespace qmm {

namespace {

using dq::max_nan;

template <typename T>
struct VecOf {
    static constexpr int kElems = 16 / sizeof(T);
};

template <typename T>
__device__ __forceinline__ void unpack_vec(const uint4 &v, float (&f)[VecOf<T>::kElems]);
template <>
__device__ __forceinline__ void unpack_vec<float>(const uint4 &v, float (&f)[4]) {
    f[0] = __uint_as_float(v.x);
    f[1] = __uint_as_float(v.y);
    f[2] = __uint_as_float(v.z);
    f[3] = __uint_as_float(v.w);
}
template <>
__device__ __forceinline__ void unpack_vec<__nv_bfloat16>(const uint4 &v, float (&f)[8]) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        f[2 * i] = __uint_as_float(w[i] << 16);
        f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}
template <>
__device__ __forceinline__ void unpack_vec<__half>(const uint4 &v, float (&f)[8]) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 p = __half22float2(*reinterpret_cast<const __half2 *>(&w[i]));
        f[2 * i] = p.x;
        f[2 * i + 1] = p.y;
    }
}

template <typename T>
__device__ __forceinline__ uint4 pack_vec(const float (&f)[VecOf<T>::kElems]);
template <>
__device__ __forceinline__ uint4 pack_vec<float>(const float (&f)[4]) {
    return make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]), __float_as_uint(f[3]));
}
template <>
__device__ __forceinline__ uint4 pack_vec<__nv_bfloat16>(const float (&f)[8]) {
    return make_uint4(pack2<__nv_bfloat16>(f[0], f[1]), pack2<__nv_bfloat16>(f[2], f[3]),
                      pack2<__nv_bfloat16>(f[4], f[5]), pack2<__nv_bfloat16>(f[6], f[7]));
}
template <>
__device__ __forceinline__ uint4 pack_vec<__half>(const float (&f)[8]) {
    return make_uint4(pack2<__half>(f[0], f[1]), pack2<__half>(f[2], f[3]), pack2<__half>(f[4], f[5]),
                      pack2<__half>(f[6], f[7]));
}

__device__ __forceinline__ float rstd_of(float sumsq, int cols, float eps) {
    const float variance = __fdiv_rn(sumsq, static_cast<float>(cols));
    return __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(variance, eps)));
}

// `tpr` threads per row, each holding VPT 16-byte vectors.  QUANT: write int8 + scale instead of y.
template <typename T, int VPT, bool QUANT>
__global__ void __launch_bounds__(512)
rms_norm_vec_kernel(const T *__restrict__ x, int64_t rows, int cols, int64_t ld_x, const T *__restrict__ gamma,
                    float eps, T *__restrict__ y, int64_t ld_y, int8_t *__restrict__ q, int64_t ld_q,
                    float *__restrict__ scale, float *__restrict__ rstd_out, int tpr) {
    constexpr int E = VecOf<T>::kElems;
    __shared__ float s_part[2][16];
    const int tpr_shift = __ffs(tpr) - 1;  // tpr is a power of two
    const int rows_per_cta = blockDim.x >> tpr_shift;
    const int row_in_cta = threadIdx.x >> tpr_shift;
    const int t = threadIdx.x & (tpr - 1);
    const int64_t row = static_cast<int64_t>(blockIdx.x) * rows_per_cta + row_in_cta;
    const bool row_ok = row < rows;
    const int nvec = cols / E;
    const int warp = threadIdx.x >> 5;
    const int warps_per_row = tpr >> 5;
    const int w0 = row_in_cta * warps_per_row;

    uint4 v[VPT];
    float sumsq = 0.0f;
    if (row_ok) {
        const uint4 *src = reinterpret_cast<const uint4 *>(x + row * ld_x);
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            const int idx = t + i * tpr;
            v[i] = idx < nvec ? __ldg(src + idx) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            float f[E];
            unpack_vec<T>(v[i], f);
#pragma unroll
            for (int j = 0; j < E; ++j) sumsq = fmaf(f[j], f[j], sumsq);
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sumsq += __shfl_xor_sync(0xffffffffu, sumsq, o);
    if (tpr > 32) {
        if ((threadIdx.x & 31) == 0) s_part[0][warp] = sumsq;
        __syncthreads();
        float s = 0.0f;
        for (int w = 0; w < warps_per_row; ++w) s += s_part[0][w0 + w];
        sumsq = s;
    }
    const float rstd = rstd_of(sumsq, cols, eps);
    if (row_ok && t == 0) rstd_out[row] = rstd;

    // y = (x * rstd) * gamma, rounded once to T; kept in the same registers
    float amax = 0.0f;
    if (row_ok) {
        const uint4 *gsrc = reinterpret_cast<const uint4 *>(gamma);
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            const int idx = t + i * tpr;
            if (idx < nvec) {
                float f[E], g[E];
                unpack_vec<T>(v[i], f);
                unpack_vec<T>(__ldg(gsrc + idx), g);
#pragma unroll
                for (int j = 0; j < E; ++j) f[j] = __fmul_rn(__fmul_rn(f[j], rstd), g[j]);
                v[i] = pack_vec<T>(f);
                if constexpr (QUANT) {
                    amax = max_nan(amax, dq::absmax8<T>(v[i]));  // of the rounded values
                } else {
                    reinterpret_cast<uint4 *>(y + row * ld_y)[idx] = v[i];
                }
            }
        }
    }
    if constexpr (QUANT) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) amax = max_nan(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        if (tpr > 32) {
            if ((threadIdx.x & 31) == 0) s_part[1][warp] = amax;
            __syncthreads();
            float m = 0.0f;
            for (int w = 0; w < warps_per_row; ++w) m = max_nan(m, s_part[1][w0 + w]);
            amax = m;
        }
        if (!row_ok) return;
        const dq::RowQuant rq = dq::make_row_quant(amax);
        if (t == 0) scale[row] = rq.scale;
        const bool fast = !rq.exact_only && rq.scale != 0.0f;
        uint2 *dst = reinterpret_cast<uint2 *>(q + row * ld_q);
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            const int idx = t + i * tpr;
            if (idx < nvec) {
                float f[8];
                dq::unpack8<T>(v[i], f);
                dst[idx] = dq::quantize8(f, rq, fast);
            }
        }
    }
}

// Any column count, stride or alignment: one CTA per row, the row is read again from L2 for each pass.
template <typename T, bool QUANT>
__global__ void __launch_bounds__(256)
rms_norm_generic_kernel(const T *__restrict__ x, int64_t rows, int64_t cols, int64_t ld_x, const T *__restrict__ gamma,
                        float eps, T *__restrict__ y, int64_t ld_y, int8_t *__restrict__ q, int64_t ld_q,
                        float *__restrict__ scale, float *__restrict__ rstd_out) {
    __shared__ float s_part[8];
    __shared__ float s_bcast;
    const int64_t row = blockIdx.x;
    const T *src = x + row * ld_x;
    float sumsq = 0.0f;
    for (int64_t c = threadIdx.x; c < cols; c += blockDim.x) {
        const float f = to_float(src[c]);
        sumsq = fmaf(f, f, sumsq);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sumsq += __shfl_xor_sync(0xffffffffu, sumsq, o);
    if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = sumsq;
    __syncthreads();
    if (threadIdx.x == 0) {
        float s = 0.0f;
        for (int w = 0; w < 8; ++w) s += s_part[w];
        s_bcast = rstd_of(s, static_cast<int>(cols), eps);
        rstd_out[row] = s_bcast;
    }
    __syncthreads();
    const float rstd = s_bcast;
    auto y_of = [&](int64_t c) {
        return to_float(from_float<T>(__fmul_rn(__fmul_rn(to_float(src[c]), rstd), to_float(gamma[c]))));
    };
    if constexpr (!QUANT) {
        for (int64_t c = threadIdx.x; c < cols; c += blockDim.x) y[row * ld_y + c] = from_float<T>(y_of(c));
    } else {
        float amax = 0.0f;
        for (int64_t c = threadIdx.x; c < cols; c += blockDim.x) amax = max_nan(amax, fabsf(y_of(c)));
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) amax = max_nan(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        __syncthreads();
        if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = amax;
        __syncthreads();
        float m = 0.0f;
        for (int w = 0; w < 8; ++w) m = max_nan(m, s_part[w]);
        const dq::RowQuant rq = dq::make_row_quant(m);
        if (threadIdx.x == 0) scale[row] = rq.scale;
        for (int64_t c = threadIdx.x; c < cols; c += blockDim.x)
            q[row * ld_q + c] = static_cast<int8_t>(dq::quant_one(y_of(c), rq));
    }
}

template <typename T, bool QUANT>
int launch_rms_norm(const T *x, int64_t rows, int64_t cols, int64_t ld_x, const T *gamma, float eps, T *y, int64_t ld_y,
                    int8_t *q, int64_t ld_q, float *scale, float *rstd, cudaStream_t stream) {
    constexpr int E = VecOf<T>::kElems;
    const bool out_ok = QUANT ? ((ld_q % 8 == 0) && (reinterpret_cast<uintptr_t>(q) & 7) == 0)
                              : ((ld_y % E == 0) && (reinterpret_cast<uintptr_t>(y) & 15) == 0);
    const bool vec_ok = (cols % E == 0) && (ld_x % E == 0) && out_ok && (reinterpret_cast<uintptr_t>(x) & 15) == 0 &&
                        (reinterpret_cast<uintptr_t>(gamma) & 15) == 0 && cols / E <= 512 * 8;
    if (vec_ok) {
        const int nvec = static_cast<int>(cols / E);
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
#define QMM_RMS_LAUNCH(V)                                                                                        \
    rms_norm_vec_kernel<T, V, QUANT><<<grid, threads, 0, stream>>>(x, rows, icols, ld_x, gamma, eps, y, ld_y, q, ld_q, \
                                                                   scale, rstd, tpr)
        switch (vpt) {
            case 1: QMM_RMS_LAUNCH(1); break;
            case 2: QMM_RMS_LAUNCH(2); break;
            case 4: QMM_RMS_LAUNCH(4); break;
            default: QMM_RMS_LAUNCH(8); break;
        }
#undef QMM_RMS_LAUNCH
    } else {
        rms_norm_generic_kernel<T, QUANT><<<rows, 256, 0, stream>>>(x, rows, cols, ld_x, gamma, eps, y, ld_y, q, ld_q,
                                                                    scale, rstd);
    }
    QMM_CUDA_OK(cudaGetLastError());
    return QMM_OK;
}

}  // namespace
}  // namespace qmm

extern "C" int qmm_rms_norm(const void *x, int x_dtype, int64_t rows, int64_t cols, int64_t ld_x, const void *gamma,
                            double epsilon, void *y, int64_t ld_y, float *rstd, void *stream) {
    using namespace qmm;
    QMM_REQUIRE(rows >= 0 && cols > 0, "qmm_rms_norm: rows must be non-negative and cols positive");
    if (rows == 0) return QMM_OK;
    QMM_REQUIRE(x != nullptr && gamma != nullptr && y != nullptr && rstd != nullptr, "qmm_rms_norm: NULL operand");
    QMM_REQUIRE(ld_x >= cols && ld_y >= cols, "qmm_rms_norm: row stride smaller than the row length");
    QMM_REQUIRE(rows < (1ll << 31), "qmm_rms_norm: more than 2^31-1 rows");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const float eps = static_cast<float>(epsilon);
    switch (x_dtype) {
        case QMM_DTYPE_BF16:
            return launch_rms_norm<__nv_bfloat16, false>(static_cast<const __nv_bfloat16 *>(x), rows, cols, ld_x,
                                                         static_cast<const __nv_bfloat16 *>(gamma), eps,
                                                         static_cast<__nv_bfloat16 *>(y), ld_y, nullptr, 0, nullptr, rstd, s);
        case QMM_DTYPE_F16:
            return launch_rms_norm<__half, false>(static_cast<const __half *>(x), rows, cols, ld_x,
                                                  static_cast<const __half *>(gamma), eps, static_cast<__half *>(y), ld_y,
                                                  nullptr, 0, nullptr, rstd, s);
        case QMM_DTYPE_F32:
            return launch_rms_norm<float, false>(static_cast<const float *>(x), rows, cols, ld_x,
                                                 static_cast<const float *>(gamma), eps, static_cast<float *>(y), ld_y,
                                                 nullptr, 0, nullptr, rstd, s);
        default:
            return fail(QMM_ERR_UNSUPPORTED, "qmm_rms_norm: dtype must be bf16, f16 or f32");
    }
}

extern "C" int qmm_rms_norm_dynamic_quant(const void *x, int x_dtype, int64_t rows, int64_t cols, int64_t ld_x,
                                          const void *gamma, double epsilon, int8_t *q, int64_t ld_q, float *scale,
                                          float *rstd, void *stream) {
    using namespace qmm;
    QMM_REQUIRE(rows >= 0 && cols > 0, "qmm_rms_norm_dynamic_quant: rows must be non-negative and cols positive");
    if (rows == 0) return QMM_OK;
    QMM_REQUIRE(x != nullptr && gamma != nullptr && q != nullptr && scale != nullptr && rstd != nullptr,
                "qmm_rms_norm_dynamic_quant: NULL operand");
    QMM_REQUIRE(ld_x >= cols && ld_q >= cols, "qmm_rms_norm_dynamic_quant: row stride smaller than the row length");
    QMM_REQUIRE(rows < (1ll << 31), "qmm_rms_norm_dynamic_quant: more than 2^31-1 rows");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const float eps = static_cast<float>(epsilon);
    switch (x_dtype) {
        case QMM_DTYPE_BF16:
            return launch_rms_norm<__nv_bfloat16, true>(static_cast<const __nv_bfloat16 *>(x), rows, cols, ld_x,
                                                        static_cast<const __nv_bfloat16 *>(gamma), eps, nullptr, 0, q, ld_q,
                                                        scale, rstd, s);
        case QMM_DTYPE_F16:
            return launch_rms_norm<__half, true>(static_cast<const __half *>(x), rows, cols, ld_x,
                                                 static_cast<const __half *>(gamma), eps, nullptr, 0, q, ld_q, scale, rstd,
                                                 s);
        default:
            return fail(QMM_ERR_UNSUPPORTED, "qmm_rms_norm_dynamic_quant: dtype must be bf16 or f16");
    }
}
