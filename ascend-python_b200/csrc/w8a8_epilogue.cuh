// Fused dequantization epilogue shared by every W8A8 kernel.
//
//   out_dtype int32 : out = acc (+ int32 bias)
//   otherwise       : out = cast(float(acc) * scale[n] * pertoken_scale[m] + float(bias[n]))
// evaluated in fp32 with one rounding per operation in exactly this order, so
// that the result equals the CPU oracle's fp32 epilogue bit for bit before the
// final round-to-nearest-even conversion to bf16/f16.
#pragma once

#include "qmm_common.cuh"

namespace qmm {

struct EpilogueParams {
    const float *scale;           // [N] or [1]
    const float *pertoken_scale;  // [M] or nullptr
    const void *bias;             // [N] or nullptr
    int bias_dtype;               // QMM_DTYPE_* or QMM_DTYPE_NONE
    int scale_is_scalar;          // scale has a single element
    void *out;
    int64_t ld_out;
    int64_t M;
    int64_t N;
};

__device__ __forceinline__ float load_bias_f32(const EpilogueParams &p, int64_t n) {
    switch (p.bias_dtype) {
        case QMM_DTYPE_BF16:
            return __bfloat162float(static_cast<const __nv_bfloat16 *>(p.bias)[n]);
        case QMM_DTYPE_F16:
            return __half2float(static_cast<const __half *>(p.bias)[n]);
        case QMM_DTYPE_F32:
            return static_cast<const float *>(p.bias)[n];
        default:
            return 0.0f;
    }
}

__device__ __forceinline__ float dequant_one(int32_t acc, float scale_n, float pertoken_m, bool has_pertoken,
                                             float bias_n, bool has_bias) {
    float v = __fmul_rn(static_cast<float>(acc), scale_n);
    if (has_pertoken) v = __fmul_rn(v, pertoken_m);
    if (has_bias) v = __fadd_rn(v, bias_n);
    return v;
}

// One thread finishes `COUNT` consecutive columns [n0, n0+COUNT) of row m
// (COUNT a multiple of 8).  OutT is __nv_bfloat16, __half or int32_t.
template <typename OutT, int COUNT>
__device__ __forceinline__ void epilogue_row_segment(const EpilogueParams &p, int64_t m, int64_t n0,
                                                     const uint32_t (&acc)[COUNT]) {
    if (m >= p.M || n0 >= p.N) return;
    OutT *orow = static_cast<OutT *>(p.out) + m * p.ld_out + n0;
    const bool full = (n0 + COUNT <= p.N);
    if constexpr (sizeof(OutT) == 4) {
        const bool has_bias = (p.bias != nullptr && p.bias_dtype == QMM_DTYPE_I32);
        const int32_t *b = static_cast<const int32_t *>(p.bias);
        const bool vec = full && ((reinterpret_cast<uintptr_t>(orow) & 15) == 0);
        if (vec) {
#pragma unroll
            for (int j = 0; j < COUNT; j += 4) {
                int32_t v[4];
#pragma unroll
                for (int t = 0; t < 4; ++t)
                    v[t] = static_cast<int32_t>(acc[j + t]) + (has_bias ? __ldg(b + n0 + j + t) : 0);
                *reinterpret_cast<int4 *>(orow + j) = make_int4(v[0], v[1], v[2], v[3]);
            }
        } else {
            for (int j = 0; j < COUNT; ++j) {
                if (n0 + j < p.N)
                    reinterpret_cast<int32_t *>(orow)[j] =
                        static_cast<int32_t>(acc[j]) + (has_bias ? __ldg(b + n0 + j) : 0);
            }
        }
    } else {
        const bool has_bias = (p.bias != nullptr && p.bias_dtype != QMM_DTYPE_NONE && p.bias_dtype != QMM_DTYPE_I32);
        const bool has_pt = (p.pertoken_scale != nullptr);
        const float pt = has_pt ? __ldg(p.pertoken_scale + m) : 1.0f;
        const float s0 = __ldg(p.scale);
        const bool vec = full && ((reinterpret_cast<uintptr_t>(orow) & 15) == 0);
        if (vec) {
#pragma unroll
            for (int j = 0; j < COUNT; j += 8) {
                float f[8];
#pragma unroll
                for (int t = 0; t < 8; ++t) {
                    const int64_t n = n0 + j + t;
                    const float sc = p.scale_is_scalar ? s0 : __ldg(p.scale + n);
                    const float bi = has_bias ? load_bias_f32(p, n) : 0.0f;
                    f[t] = dequant_one(static_cast<int32_t>(acc[j + t]), sc, pt, has_pt, bi, has_bias);
                }
                uint4 w;
                w.x = pack2<OutT>(f[0], f[1]);
                w.y = pack2<OutT>(f[2], f[3]);
                w.z = pack2<OutT>(f[4], f[5]);
                w.w = pack2<OutT>(f[6], f[7]);
                *reinterpret_cast<uint4 *>(orow + j) = w;
            }
        } else {
            for (int j = 0; j < COUNT; ++j) {
                const int64_t n = n0 + j;
                if (n < p.N) {
                    const float sc = p.scale_is_scalar ? s0 : __ldg(p.scale + n);
                    const float bi = has_bias ? load_bias_f32(p, n) : 0.0f;
                    orow[j] = from_float<OutT>(dequant_one(static_cast<int32_t>(acc[j]), sc, pt, has_pt, bi, has_bias));
                }
            }
        }
    }
}

// One element (used by kernels whose threads own a column of the accumulator).
template <typename OutT>
__device__ __forceinline__ void epilogue_one(const EpilogueParams &p, int64_t m, int64_t n, int32_t acc) {
    if (m >= p.M || n >= p.N) return;
    OutT *o = static_cast<OutT *>(p.out) + m * p.ld_out + n;
    if constexpr (sizeof(OutT) == 4) {
        const bool has_bias = (p.bias != nullptr && p.bias_dtype == QMM_DTYPE_I32);
        *reinterpret_cast<int32_t *>(o) = acc + (has_bias ? __ldg(static_cast<const int32_t *>(p.bias) + n) : 0);
    } else {
        const bool has_bias = (p.bias != nullptr && p.bias_dtype != QMM_DTYPE_NONE && p.bias_dtype != QMM_DTYPE_I32);
        const bool has_pt = (p.pertoken_scale != nullptr);
        const float pt = has_pt ? __ldg(p.pertoken_scale + m) : 1.0f;
        const float sc = p.scale_is_scalar ? __ldg(p.scale) : __ldg(p.scale + n);
        const float bi = has_bias ? load_bias_f32(p, n) : 0.0f;
        *o = from_float<OutT>(dequant_one(acc, sc, pt, has_pt, bi, has_bias));
    }
}

}  // namespace qmm
