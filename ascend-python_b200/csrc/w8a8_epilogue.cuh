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

// Row-parallel matmul whose output tiles go straight to the rank that will reduce them: rank o owns the
// rows [o * rows_per, (o+1) * rows_per) and receives them from rank s at
// base[o] + area_off + s * rows_per * N * element size.  Host-side description (see LaunchOptions).
struct PushSpec {
    uint8_t *base[8];
    size_t area_off;
    int world, rank;
    int64_t rows_per;  // a multiple of 32, so the 32 rows of an epilogue warp have one owner
};
struct FusedComm;  // peer_fused.cuh
// What a caller of quant_matmul_dispatch may ask of the launch beyond the problem itself.
struct LaunchOptions {
    int sm_reserve = 0;              // SMs the persistent kernels leave idle (a collective runs beside them)
    const PushSpec *push = nullptr;  // owners' receive areas for the output tiles (CTA-pair kernel only)
    bool push_applied = false;       // out: the launch did deliver its tiles to the owners
    const FusedComm *fused = nullptr;  // allreduce inside the CTA-pair kernel (needs push)
    bool fused_applied = false;      // out: the launch reduces and gathers the output itself
};
// Kernel-side form: one output tensor map per owner.
struct PushMaps {
    CUtensorMap m[8];
    int64_t rows_per;
    int enabled;
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

// ---------------------------------------------------------------------------
// Epilogue of one warp through shared memory and TMA stores.
//
// The warp owns 32 accumulator rows (TMEM lanes) of a tile that is TILE_N
// columns wide.  It walks the tile in chunks whose rows are 128 bytes of
// output (64 columns of bf16/f16, 32 of int32): TMEM -> registers -> fp32
// dequantization -> a 4 KiB staging buffer laid out with the 128-byte swizzle
// (bank-conflict free 16-byte stores) -> one TMA store per chunk.  Two staging
// buffers alternate so that the store of chunk c overlaps the math of c+1.
// Per-column scale and bias of a chunk are fetched once per warp (coalesced)
// into a small shared array and read back as broadcasts.
//
// `stage` points to this warp's 8 KiB staging area (1024-byte aligned),
// `colbuf` to its 2*64 floats.  `chunk_counter` persists across tiles: it
// numbers the warp's TMA stores so that buffer reuse can be fenced.
// ---------------------------------------------------------------------------
template <typename OutT>
struct EpiChunk {
    static constexpr int kCols = 128 / static_cast<int>(sizeof(OutT));  // columns per 128-byte row
};

template <typename OutT, int TILE_N>
__device__ __forceinline__ void epilogue_warp_tile_tma(const EpilogueParams &p, const CUtensorMap *tmap_out,
                                                       uint32_t taddr_warp, int64_t m_warp0, int64_t n_tile0,
                                                       uint8_t *stage, float *colbuf, uint32_t &chunk_counter,
                                                       int64_t store_row0 = -1) {
    // store_row0: row coordinate of the warp's first row in tmap_out when that map does not start at
    // row 0 of the output (tiles pushed into another rank's receive area); -1: same as m_warp0
    constexpr int CC = EpiChunk<OutT>::kCols;
    const int lane = threadIdx.x & 31;
    const int64_t m = m_warp0 + lane;
    const bool is_int = (sizeof(OutT) == 4);
    const bool has_pt = !is_int && (p.pertoken_scale != nullptr);
    const bool has_bias = (p.bias != nullptr) && (is_int ? p.bias_dtype == QMM_DTYPE_I32
                                                         : (p.bias_dtype != QMM_DTYPE_NONE &&
                                                            p.bias_dtype != QMM_DTYPE_I32));
    const float pt = (has_pt && m < p.M) ? __ldg(p.pertoken_scale + m) : 1.0f;
    const uint32_t stage_u32 = smem_u32(stage);
    if (m_warp0 >= p.M) return;  // the warp's rows are all padding

#pragma unroll 1
    for (int c = 0; c < TILE_N / CC; ++c) {
        const int64_t n0 = n_tile0 + static_cast<int64_t>(c) * CC;
        if (n0 >= p.N) break;
        const uint32_t buf = chunk_counter & 1;
        // the TMA store that last read this buffer (two chunks ago) must have finished reading it
        if (lane == 0) tma_store_wait_read<1>();
        __syncwarp();

        // per-column constants of this chunk -> shared (coalesced), as fp32 bit patterns
#pragma unroll
        for (int i = lane; i < CC; i += 32) {
            const int64_t n = n0 + i;
            float sc = 1.0f, bi = 0.0f;
            if (n < p.N) {
                if (is_int) {
                    if (has_bias) bi = __int_as_float(__ldg(static_cast<const int32_t *>(p.bias) + n));
                } else {
                    sc = p.scale_is_scalar ? __ldg(p.scale) : __ldg(p.scale + n);
                    if (has_bias) bi = load_bias_f32(p, n);
                }
            }
            colbuf[i] = sc;
            colbuf[64 + i] = bi;
        }
        __syncwarp();

        uint8_t *dst_row = stage + buf * 4096 + lane * 128;
#pragma unroll
        for (int h = 0; h < CC / 32; ++h) {
            uint32_t acc[32];
            tmem_ld_32x32(taddr_warp + c * CC + h * 32, acc);
            tmem_ld_wait();
            if constexpr (sizeof(OutT) == 4) {
#pragma unroll
                for (int j = 0; j < 32; j += 4) {
                    const float4 b4 = *reinterpret_cast<const float4 *>(colbuf + 64 + h * 32 + j);
                    int4 v;
                    v.x = static_cast<int32_t>(acc[j + 0]) + __float_as_int(b4.x);
                    v.y = static_cast<int32_t>(acc[j + 1]) + __float_as_int(b4.y);
                    v.z = static_cast<int32_t>(acc[j + 2]) + __float_as_int(b4.z);
                    v.w = static_cast<int32_t>(acc[j + 3]) + __float_as_int(b4.w);
                    const int chunk16 = (h * 32 + j) / 4;  // 16-byte chunk index within the 128-byte row
                    *reinterpret_cast<int4 *>(dst_row + ((chunk16 ^ (lane & 7)) << 4)) = v;
                }
            } else {
#pragma unroll
                for (int j = 0; j < 32; j += 8) {
                    float f[8];
#pragma unroll
                    for (int q4 = 0; q4 < 2; ++q4) {
                        const float4 s4 = *reinterpret_cast<const float4 *>(colbuf + h * 32 + j + q4 * 4);
                        const float4 b4 = *reinterpret_cast<const float4 *>(colbuf + 64 + h * 32 + j + q4 * 4);
                        f[q4 * 4 + 0] = dequant_one(static_cast<int32_t>(acc[j + q4 * 4 + 0]), s4.x, pt, has_pt, b4.x, has_bias);
                        f[q4 * 4 + 1] = dequant_one(static_cast<int32_t>(acc[j + q4 * 4 + 1]), s4.y, pt, has_pt, b4.y, has_bias);
                        f[q4 * 4 + 2] = dequant_one(static_cast<int32_t>(acc[j + q4 * 4 + 2]), s4.z, pt, has_pt, b4.z, has_bias);
                        f[q4 * 4 + 3] = dequant_one(static_cast<int32_t>(acc[j + q4 * 4 + 3]), s4.w, pt, has_pt, b4.w, has_bias);
                    }
                    uint4 w;
                    w.x = pack2<OutT>(f[0], f[1]);
                    w.y = pack2<OutT>(f[2], f[3]);
                    w.z = pack2<OutT>(f[4], f[5]);
                    w.w = pack2<OutT>(f[6], f[7]);
                    const int chunk16 = (h * 32 + j) / 8;
                    *reinterpret_cast<uint4 *>(dst_row + ((chunk16 ^ (lane & 7)) << 4)) = w;
                }
            }
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
            tma_store_2d(tmap_out, stage_u32 + buf * 4096, static_cast<int32_t>(n0),
                         static_cast<int32_t>(store_row0 >= 0 ? store_row0 : m_warp0));
            tma_store_commit();
        }
        ++chunk_counter;
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
