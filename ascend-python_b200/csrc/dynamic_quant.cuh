// Device helpers shared by the per-token quantization kernels (dynamic_quant.cu, rms_norm.cu): the
// row scale, the division on the FMA pipe and the packing of eight results.  See dynamic_quant.cu
// for the numerical contract.
#pragma once

#include "qmm_common.cuh"

namespace qmm {
namespace dq {

template <typename T>
__device__ __forceinline__ void unpack8(const uint4 &v, float (&f)[8]);

template <>
__device__ __forceinline__ void unpack8<__nv_bfloat16>(const uint4 &v, float (&f)[8]) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        f[2 * i] = __uint_as_float(w[i] << 16);
        f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}

template <>
__device__ __forceinline__ void unpack8<__half>(const uint4 &v, float (&f)[8]) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        __half2 h = *reinterpret_cast<const __half2 *>(&w[i]);
        float2 p = __half22float2(h);
        f[2 * i] = p.x;
        f[2 * i + 1] = p.y;
    }
}

// max that keeps a NaN (fmaxf and the plain packed maximum would drop it): a row that holds a NaN gets a
// NaN scale, and every quotient by a NaN or infinite scale that is itself NaN quantizes to 0
__device__ __forceinline__ float max_nan(float a, float b) {
    float r;
    asm("max.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
    return r;
}

struct RowQuant {
    float scale;
    float inv;
    bool exact_only;  // reciprocal unusable (zero, denormal or non-finite scale)
};

__device__ __forceinline__ RowQuant make_row_quant(float amax) {
    RowQuant r;
    r.scale = __fdiv_rn(amax, 127.0f);
    r.inv = __frcp_rn(r.scale);
    // preconditions of the FMA division: no underflow in the remainder, a finite reciprocal, and a
    // divisor whose significand is not all ones
    r.exact_only = !(r.scale >= 1e-25f) || !(r.scale <= 3.0e38f) || !(r.inv <= 3.0e38f) ||
                   (__float_as_uint(r.scale) & 0x007fffffu) == 0x007fffffu;
    return r;
}

__device__ __forceinline__ int quant_one(float x, const RowQuant &rq) {
    if (rq.scale == 0.0f) return 0;
    float t;
    if (rq.exact_only) {
        t = __fdiv_rn(x, rq.scale);
    } else {
        const float q0 = x * rq.inv;
        t = fmaf(fmaf(-q0, rq.scale, x), rq.inv, q0);
    }
    return max(-128, min(127, __float2int_rn(t)));
}

// absmax of the eight 16-bit floats of a 128-bit vector, packed two at a time
template <typename T>
__device__ __forceinline__ float absmax8(const uint4 &v);
template <>
__device__ __forceinline__ float absmax8<__nv_bfloat16>(const uint4 &v) {
    const uint32_t w[4] = {v.x & 0x7fff7fffu, v.y & 0x7fff7fffu, v.z & 0x7fff7fffu, v.w & 0x7fff7fffu};
    __nv_bfloat162 m = __hmax2_nan(__hmax2_nan(*reinterpret_cast<const __nv_bfloat162 *>(&w[0]),
                                       *reinterpret_cast<const __nv_bfloat162 *>(&w[1])),
                               __hmax2_nan(*reinterpret_cast<const __nv_bfloat162 *>(&w[2]),
                                       *reinterpret_cast<const __nv_bfloat162 *>(&w[3])));
    return max_nan(__low2float(m), __high2float(m));
}
template <>
__device__ __forceinline__ float absmax8<__half>(const uint4 &v) {
    const uint32_t w[4] = {v.x & 0x7fff7fffu, v.y & 0x7fff7fffu, v.z & 0x7fff7fffu, v.w & 0x7fff7fffu};
    __half2 m = __hmax2_nan(__hmax2_nan(*reinterpret_cast<const __half2 *>(&w[0]), *reinterpret_cast<const __half2 *>(&w[1])),
                        __hmax2_nan(*reinterpret_cast<const __half2 *>(&w[2]), *reinterpret_cast<const __half2 *>(&w[3])));
    return max_nan(__low2float(m), __high2float(m));
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = max_nan(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// int8 values of eight row elements, packed (elements 0..3 in .x, 4..7 in .y).  `fast`: the row's scale
// meets the preconditions of the FMA-pipe division (uniform over the row).
__device__ __forceinline__ uint2 quantize8(const float (&f)[8], const RowQuant &rq, bool fast) {
    uint32_t lo = 0, hi = 0;
    if (fast) {
        // FMA pipe only: product, exact remainder, corrected quotient, magic-number rounding
        constexpr float kMagic = 12582912.0f;  // 1.5 * 2^23: adding it rounds to an integer, ties to even
        uint32_t b[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float q0 = f[j] * rq.inv;
            const float rem = fmaf(-q0, rq.scale, f[j]);
            const float q1 = fmaf(rem, rq.inv, q0);  // the IEEE quotient f / scale
            b[j] = __float_as_uint(q1 + kMagic);
        }
        // the int8 results are the low bytes of the biased floats: gather (b0..b3) and (b4..b7)
        lo = __byte_perm(__byte_perm(b[0], b[1], 0x0040), __byte_perm(b[2], b[3], 0x0040), 0x5410);
        hi = __byte_perm(__byte_perm(b[4], b[5], 0x0040), __byte_perm(b[6], b[7], 0x0040), 0x5410);
    } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            lo |= (static_cast<uint32_t>(quant_one(f[j], rq)) & 0xffu) << (8 * j);
            hi |= (static_cast<uint32_t>(quant_one(f[4 + j], rq)) & 0xffu) << (8 * j);
        }
    }
    return make_uint2(lo, hi);
}


}  // namespace dq
}  // namespace qmm
