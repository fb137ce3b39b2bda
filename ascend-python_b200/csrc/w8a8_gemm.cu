// W8A8 matmul with fused dequantization (npu_quant_matmul) for sm_100a.
//
// Three kernels:
//  * w8a8_tile_kernel   — prefill shapes.  Persistent CTAs, one 128x256 output
//    tile at a time: TMA -> 4-stage shared-memory ring -> tcgen05.mma kind::i8
//    (128x256x32 per instruction) -> int32 accumulator in TMEM (two buffers, so
//    the epilogue of tile i overlaps the main loop of tile i+1) -> fused
//    dequantization epilogue straight from TMEM to global memory.
//    Warp roles: warp 0 TMA producer, warp 1 MMA issuer + TMEM owner,
//    warps 2-5 epilogue (each owns the 32 TMEM lanes of its warp_id % 4).
//  * w8a8_streamk_kernel — decode shapes (M <= 128), weight-bandwidth bound.
//    (see below)
//  * w8a8_simt_kernel   — dp4a kernel for operands whose addresses or strides
//    do not meet the 16-byte rules of TMA.
//
// x2 is taken as stored: a row-major [K,N] weight is the MMA's MN-major B
// operand, the transposed view of a row-major [N,K] weight is its K-major B
// operand; no repacking pass.
#include "qmm_common.cuh"
#include "w8a8_epilogue.cuh"

namespace qmm {

// Implemented in w8a8_gemm_pair.cu
int launch_pair(const int8_t *x1, int64_t ld_x1, const int8_t *x2, int64_t x2_sk, int64_t x2_sn,
                const struct EpilogueParams &ep, int out_dtype, int64_t K, struct LaunchOptions *opts,
                cudaStream_t stream);

namespace {

// ---------------------------------------------------------------------------
// Tile kernel
// ---------------------------------------------------------------------------
constexpr int kBM = 128;
constexpr int kBN = 256;
constexpr int kBK = 128;  // int8 elements = bytes: one 128-byte swizzle row
constexpr int kStages = 4;
constexpr int kAStageBytes = kBM * kBK;
constexpr int kBStageBytes = kBN * kBK;
constexpr int kStageBytes = kAStageBytes + kBStageBytes;
constexpr int kTileThreads = 192;
constexpr int kGroupM = 16;  // m-tiles per rasterization group
constexpr uint32_t kTmemCols = 512;

struct TileSmemTail {
    uint64_t full[kStages];
    uint64_t empty[kStages];
    uint64_t tmem_full[2];
    uint64_t tmem_empty[2];
    uint32_t tmem_base;
    uint32_t abort_flag;
};

constexpr int kEpiWarps = 4;
constexpr int kEpiStageBytes = 2 * 4096;  // per warp: two 32-row x 128-byte staging buffers
constexpr int kEpiColFloats = 128;        // per warp: 64 scales + 64 biases

// dynamic shared memory: [operand ring][epilogue staging][per-column constants][barriers]
constexpr size_t kTileSmemBytes = kStages * kStageBytes + kEpiWarps * kEpiStageBytes +
                                  kEpiWarps * kEpiColFloats * sizeof(float) + sizeof(TileSmemTail);
static_assert(kTileSmemBytes <= 232448, "tile kernel exceeds the 227 KiB of shared memory a CTA may use");

__device__ __forceinline__ void tile_coords(int tile, int tiles_m, int tiles_n, int &m_blk, int &n_blk) {
    const int per_group = kGroupM * tiles_n;
    const int g = tile / per_group;
    const int first_m = g * kGroupM;
    const int rows = min(kGroupM, tiles_m - first_m);
    const int r = tile - g * per_group;
    m_blk = first_m + r % rows;
    n_blk = r / rows;
}

template <typename OutT, bool B_MN_MAJOR>
__global__ void __launch_bounds__(kTileThreads, 1)
w8a8_tile_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                 const __grid_constant__ CUtensorMap tmap_out, EpilogueParams ep, int K, int use_tma_store,
                 int slices, int slice_rows, uint32_t *status) {
    // slices > 1: split-K.  Work item w = slice * tiles + tile multiplies the slice's share of the k
    // blocks and stores raw int32 sums at row slice * slice_rows + m of tmap_out (a scratch array
    // [slices][slice_rows][N]); a second kernel adds the slices and applies the epilogue.
    // The 128-byte swizzle of TMA and of the MMA descriptors needs 1024-byte aligned tiles.
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    const uint32_t smem_base = smem_u32(smem_raw);
    if ((smem_base & 1023u) != 0) {
        if (threadIdx.x == 0 && status != nullptr) atomicMax(status, DEV_STATUS_SMEM_MISALIGNED);
        return;
    }
    uint8_t *smem_aligned = smem_raw;
    uint8_t *epi_stage = smem_aligned + kStages * kStageBytes;
    float *epi_cols = reinterpret_cast<float *>(epi_stage + kEpiWarps * kEpiStageBytes);
    TileSmemTail *tail = reinterpret_cast<TileSmemTail *>(epi_cols + kEpiWarps * kEpiColFloats);
    volatile uint32_t *abort_flag = &tail->abort_flag;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int tiles_m = static_cast<int>((ep.M + kBM - 1) / kBM);
    const int tiles_n = static_cast<int>((ep.N + kBN - 1) / kBN);
    const int num_tiles = tiles_m * tiles_n;
    const int num_kb = (K + kBK - 1) / kBK;
    const int num_items = num_tiles * slices;
    const int kb_per_slice = (num_kb + slices - 1) / slices;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(smem_u32(&tail->full[s]), 1);
            mbar_init(smem_u32(&tail->empty[s]), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(smem_u32(&tail->tmem_full[b]), 1);
            mbar_init(smem_u32(&tail->tmem_empty[b]), 4);
        }
        tail->abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == 0 && lane == 0) {
        tma_prefetch_desc(&tmap_a);
        tma_prefetch_desc(&tmap_b);
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(&tail->tmem_base), kTmemCols);
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
        for (int item = blockIdx.x; item < num_items && ok; item += gridDim.x) {
            int m_blk, n_blk;
            tile_coords(item % num_tiles, tiles_m, tiles_n, m_blk, n_blk);
            const int kb0 = (item / num_tiles) * kb_per_slice;
            const int kb1 = min(num_kb, kb0 + kb_per_slice);
            for (int kb = kb0; kb < kb1; ++kb) {
                ok = mbar_wait(smem_u32(&tail->empty[stage]), phase ^ 1, abort_flag, 1);
                if (!ok) break;
                if (lane == 0) {
                    const uint32_t full = smem_u32(&tail->full[stage]);
                    const uint32_t sa = smem_base + stage * kStageBytes;
                    const uint32_t sb = sa + kAStageBytes;
                    mbar_expect_tx(full, kStageBytes);
                    tma_load_2d(sa, &tmap_a, kb * kBK, m_blk * kBM, full);
                    if (B_MN_MAJOR) {
                        // two [128 k-rows x 128 n-bytes] boxes side by side
                        tma_load_2d(sb, &tmap_b, n_blk * kBN, kb * kBK, full);
                        tma_load_2d(sb + kBStageBytes / 2, &tmap_b, n_blk * kBN + 128, kb * kBK, full);
                    } else {
                        // one [256 n-rows x 128 k-bytes] box
                        tma_load_2d(sb, &tmap_b, kb * kBK, n_blk * kBN, full);
                    }
                }
                __syncwarp();
                if (++stage == kStages) {
                    stage = 0;
                    phase ^= 1;
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        // The whole warp runs the loop with warp-uniform operands; elect.sync picks the issuing lane.
        constexpr uint32_t idesc = make_idesc(/*c=s32*/ 2, /*a=s8*/ 1, /*b=s8*/ 1, /*a K-major*/ 0,
                                              B_MN_MAJOR ? 1u : 0u, kBM, kBN);
        constexpr uint32_t kDescHi = smem_desc_hi_sw128(1024);  // 8-row groups are 1024 bytes apart
        constexpr uint32_t kStageStep = kStageBytes >> 4;
        // A: K-major, 32 bytes (+2) per K step.  B: MN-major (second 128-column half 16 KiB further)
        // 32 k-rows = 4096 bytes (+256) per K step; K-major +2.
        constexpr uint32_t kBStep = B_MN_MAJOR ? (4096u >> 4) : 2u;
        const uint32_t a_lo0 = smem_desc_lo(smem_base, 16);
        const uint32_t b_lo0 = smem_desc_lo(smem_base + kAStageBytes, B_MN_MAJOR ? kBStageBytes / 2 : 16);
        const uint32_t full0 = smem_u32(&tail->full[0]);
        const uint32_t empty0 = smem_u32(&tail->empty[0]);
        uint32_t stage = 0, phase = 0;
        int local = 0;
        bool ok = true;
        for (int item = blockIdx.x; item < num_items && ok; item += gridDim.x, ++local) {
            const uint32_t buf = local & 1;
            const uint32_t buf_phase = (local >> 1) & 1;
            ok = mbar_wait(smem_u32(&tail->tmem_empty[buf]), buf_phase ^ 1, abort_flag, 2);
            if (!ok) break;
            tc_fence_after();
            const uint32_t d_tmem = tmem_base + buf * kBN;
            uint32_t accumulate = 0;
            const int kb0 = (item / num_tiles) * kb_per_slice;
            const int kb1 = min(num_kb, kb0 + kb_per_slice);
            for (int kb = kb0; kb < kb1; ++kb) {
                ok = mbar_wait(full0 + stage * 8, phase, abort_flag, 3);
                if (!ok) break;
                tc_fence_after();
                const uint32_t a_lo = a_lo0 + stage * kStageStep;
                const uint32_t b_lo = b_lo0 + stage * kStageStep;
#pragma unroll
                for (int k = 0; k < kBK / 32; ++k) {
                    mma_i8_ss_warp(d_tmem, desc64(a_lo + 2 * k, kDescHi), desc64(b_lo + kBStep * k, kDescHi), idesc,
                                   accumulate);
                    accumulate = 1;
                }
                tc_commit_warp(empty0 + stage * 8);
                if (++stage == kStages) {
                    stage = 0;
                    phase ^= 1;
                }
            }
            if (ok) tc_commit_warp(smem_u32(&tail->tmem_full[buf]));
        }
    } else {
        // ---------------- epilogue warps ----------------
        const int quarter = warp & 3;  // TMEM lanes [32*quarter, 32*quarter+32)
        uint8_t *my_stage = epi_stage + quarter * kEpiStageBytes;
        float *my_cols = epi_cols + quarter * kEpiColFloats;
        uint32_t chunk_counter = 0;
        int local = 0;
        bool ok = true;
        if (lane == 0 && use_tma_store) tma_prefetch_desc(&tmap_out);
        for (int item = blockIdx.x; item < num_items && ok; item += gridDim.x, ++local) {
            int m_blk, n_blk;
            tile_coords(item % num_tiles, tiles_m, tiles_n, m_blk, n_blk);
            const int slice = item / num_tiles;
            const uint32_t buf = local & 1;
            const uint32_t buf_phase = (local >> 1) & 1;
            ok = mbar_wait(smem_u32(&tail->tmem_full[buf]), buf_phase, abort_flag, 4);
            if (!ok) break;
            tc_fence_after();
            const int64_t m_warp0 = static_cast<int64_t>(m_blk) * kBM + quarter * 32;
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + buf * kBN;
            if (use_tma_store) {
                epilogue_warp_tile_tma<OutT, kBN>(ep, &tmap_out, taddr, m_warp0, static_cast<int64_t>(n_blk) * kBN,
                                                  my_stage, my_cols, chunk_counter,
                                                  slices > 1 ? static_cast<int64_t>(slice) * slice_rows + m_warp0 : -1);
            } else {
#pragma unroll 1
                for (int c = 0; c < kBN / 32; ++c) {
                    uint32_t acc[32];
                    tmem_ld_32x32(taddr + c * 32, acc);
                    tmem_ld_wait();
                    epilogue_row_segment<OutT, 32>(ep, m_warp0 + lane, static_cast<int64_t>(n_blk) * kBN + c * 32, acc);
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&tail->tmem_empty[buf]));
        }
        // all of this warp's TMA stores must have left shared memory before the CTA exits
        if (lane == 0) tma_store_wait_all<0>();
        __syncwarp();
    }

    // ---------------- teardown ----------------
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && tail->abort_flag != 0 && status != nullptr) atomicMax(status, tail->abort_flag);
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

// ---------------------------------------------------------------------------
// SIMT kernel (any stride / alignment): 64x64 tile, 256 threads, 4x4 per thread,
// int8 operands staged in shared memory with K contiguous, dp4a inner product.
// ---------------------------------------------------------------------------
constexpr int kSimtTile = 64;
constexpr int kSimtK = 64;

template <typename OutT>
__global__ void __launch_bounds__(256)
w8a8_simt_kernel(const int8_t *__restrict__ x1, int64_t ld_x1, const int8_t *__restrict__ x2, int64_t x2_sk,
                 int64_t x2_sn, EpilogueParams ep, int64_t K) {
    __shared__ int32_t As[kSimtTile][kSimtK / 4 + 1];
    __shared__ int32_t Bs[kSimtTile][kSimtK / 4 + 1];
    int8_t *As8 = reinterpret_cast<int8_t *>(&As[0][0]);
    int8_t *Bs8 = reinterpret_cast<int8_t *>(&Bs[0][0]);
    constexpr int kRowBytes = (kSimtK / 4 + 1) * 4;

    const int64_t m0 = static_cast<int64_t>(blockIdx.y) * kSimtTile;
    const int64_t n0 = static_cast<int64_t>(blockIdx.x) * kSimtTile;
    const int tx = threadIdx.x & 15;  // n direction
    const int ty = threadIdx.x >> 4;  // m direction
    int32_t acc[4][4] = {};

    for (int64_t k0 = 0; k0 < K; k0 += kSimtK) {
        for (int i = threadIdx.x; i < kSimtTile * kSimtK; i += 256) {
            const int r = i / kSimtK, c = i % kSimtK;  // A: r = m, c = k (k contiguous in memory)
            const int64_t m = m0 + r, k = k0 + c;
            As8[r * kRowBytes + c] = (m < ep.M && k < K) ? x1[m * ld_x1 + k] : int8_t(0);
        }
        if (x2_sn == 1) {
            for (int i = threadIdx.x; i < kSimtTile * kSimtK; i += 256) {
                const int c = i / kSimtTile, r = i % kSimtTile;  // r = n (contiguous in memory), c = k
                const int64_t n = n0 + r, k = k0 + c;
                Bs8[r * kRowBytes + c] = (n < ep.N && k < K) ? x2[k * x2_sk + n] : int8_t(0);
            }
        } else {
            for (int i = threadIdx.x; i < kSimtTile * kSimtK; i += 256) {
                const int r = i / kSimtK, c = i % kSimtK;  // r = n, c = k (k contiguous in memory)
                const int64_t n = n0 + r, k = k0 + c;
                Bs8[r * kRowBytes + c] = (n < ep.N && k < K) ? x2[k * x2_sk + n * x2_sn] : int8_t(0);
            }
        }
        __syncthreads();
#pragma unroll 4
        for (int kk = 0; kk < kSimtK / 4; ++kk) {
            int32_t a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[ty * 4 + i][kk];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = Bs[tx * 4 + j][kk];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = __dp4a(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) epilogue_one<OutT>(ep, m0 + ty * 4 + i, n0 + tx * 4 + j, acc[i][j]);
}

// ---------------------------------------------------------------------------
// Host launchers
// ---------------------------------------------------------------------------
template <typename OutT>
int launch_tile(const int8_t *x1, int64_t ld_x1, const int8_t *x2, int64_t x2_sk, int64_t x2_sn,
                const EpilogueParams &ep, int64_t K, int sm_reserve, cudaStream_t stream) {
    CUtensorMap ta, tb;
    int rc = make_tmap_2d(&ta, x1, 1, static_cast<uint64_t>(K), static_cast<uint64_t>(ep.M),
                          static_cast<uint64_t>(ld_x1), kBK, kBM, true);
    if (rc != QMM_OK) return rc;
    const bool mn_major = (x2_sn == 1);
    if (mn_major) {
        rc = make_tmap_2d(&tb, x2, 1, static_cast<uint64_t>(ep.N), static_cast<uint64_t>(K),
                          static_cast<uint64_t>(x2_sk), 128, kBK, true);
    } else {
        rc = make_tmap_2d(&tb, x2, 1, static_cast<uint64_t>(K), static_cast<uint64_t>(ep.N),
                          static_cast<uint64_t>(x2_sn), kBK, kBN, true);
    }
    if (rc != QMM_OK) return rc;
    // The epilogue stores through TMA when the output meets the 16-byte rules; it writes
    // straight from registers otherwise.
    constexpr int kElt = static_cast<int>(sizeof(OutT));
    CUtensorMap tout = ta;
    int use_tma_store = 0;
    if ((reinterpret_cast<uintptr_t>(ep.out) & 15) == 0 && ((ep.ld_out * kElt) & 15) == 0) {
        rc = make_tmap_2d(&tout, ep.out, kElt, static_cast<uint64_t>(ep.N), static_cast<uint64_t>(ep.M),
                          static_cast<uint64_t>(ep.ld_out), 128 / kElt, 32, true);
        if (rc != QMM_OK) return rc;
        use_tma_store = 1;
    }
    const int tiles = static_cast<int>(((ep.M + kBM - 1) / kBM) * ((ep.N + kBN - 1) / kBN));
    int ctas = sm_count() - sm_reserve;
    if (ctas < 1) ctas = 1;
    const int grid = tiles < ctas ? tiles : ctas;
    uint32_t *status = device_status_word();
    auto kern = mn_major ? w8a8_tile_kernel<OutT, true> : w8a8_tile_kernel<OutT, false>;
    QMM_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     static_cast<int>(kTileSmemBytes)));
    kern<<<grid, kTileThreads, kTileSmemBytes, stream>>>(ta, tb, tout, ep, static_cast<int>(K), use_tma_store, 1, 0,
                                                         status);
    QMM_CUDA_OK(cudaGetLastError());
    return QMM_OK;
}

// ---- split-K for shapes whose tiles leave most SMs idle (decode with a narrow N and a long K) ----

// Adds the slices' int32 sums, applies the epilogue and zeroes what it read (the scratch is shared with
// the stream-K kernel, which relies on finding zeros).
// Eight columns per thread, one row per blockIdx.y step: the slices' loads of a thread are all in flight at once,
// the per-column constants are loaded once per thread and the 16-bit results leave as one 16-byte store.
// Needs N % 8 == 0, a 16-bit output with 16-byte aligned rows, fp32 per-column scale and no int32 output.
template <typename OutT, int SLICES>
__global__ void __launch_bounds__(256)
splitk_reduce_vec8_kernel(int32_t *__restrict__ scratch, int64_t slice_elems, EpilogueParams ep) {
    const int64_t n = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) * 8;
    if (n >= ep.N) return;
    const bool has_pt = ep.pertoken_scale != nullptr;
    const bool has_bias = ep.bias != nullptr && ep.bias_dtype != QMM_DTYPE_NONE && ep.bias_dtype != QMM_DTYPE_I32;
    float sc[8], bi[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        sc[j] = ep.scale_is_scalar ? __ldg(ep.scale) : __ldg(ep.scale + n + j);
        bi[j] = has_bias ? load_bias_f32(ep, n + j) : 0.0f;
    }
    for (int64_t m = blockIdx.y; m < ep.M; m += gridDim.y) {
        int4 a[SLICES][2];
#pragma unroll
        for (int s = 0; s < SLICES; ++s) {
            int4 *src = reinterpret_cast<int4 *>(scratch + s * slice_elems + m * ep.N + n);
            a[s][0] = __ldcg(src);
            a[s][1] = __ldcg(src + 1);
        }
        int32_t acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
        for (int s = 0; s < SLICES; ++s) {
            acc[0] += a[s][0].x, acc[1] += a[s][0].y, acc[2] += a[s][0].z, acc[3] += a[s][0].w;
            acc[4] += a[s][1].x, acc[5] += a[s][1].y, acc[6] += a[s][1].z, acc[7] += a[s][1].w;
            int4 *src = reinterpret_cast<int4 *>(scratch + s * slice_elems + m * ep.N + n);
            __stcg(src, make_int4(0, 0, 0, 0));
            __stcg(src + 1, make_int4(0, 0, 0, 0));
        }
        const float pt = has_pt ? __ldg(ep.pertoken_scale + m) : 1.0f;
        float f[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] = dequant_one(acc[j], sc[j], pt, has_pt, bi[j], has_bias);
        *reinterpret_cast<uint4 *>(static_cast<OutT *>(ep.out) + m * ep.ld_out + n) =
            make_uint4(pack2<OutT>(f[0], f[1]), pack2<OutT>(f[2], f[3]), pack2<OutT>(f[4], f[5]), pack2<OutT>(f[6], f[7]));
    }
}

template <typename OutT>
__global__ void __launch_bounds__(256)
splitk_reduce_kernel(int32_t *__restrict__ scratch, int slices, int64_t slice_elems, EpilogueParams ep) {
    const int64_t vecs = ep.M * ep.N / 4;  // N is a multiple of 4
    for (int64_t v = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; v < vecs;
         v += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        int4 acc = make_int4(0, 0, 0, 0);
        for (int s = 0; s < slices; ++s) {
            int4 *src = reinterpret_cast<int4 *>(scratch + s * slice_elems) + v;
            const int4 a = __ldcg(src);
            acc.x += a.x;
            acc.y += a.y;
            acc.z += a.z;
            acc.w += a.w;
            __stcg(src, make_int4(0, 0, 0, 0));
        }
        const int64_t e = v * 4;
        const int64_t m = e / ep.N, n = e - m * ep.N;
        epilogue_one<OutT>(ep, m, n, acc.x);
        epilogue_one<OutT>(ep, m, n + 1, acc.y);
        epilogue_one<OutT>(ep, m, n + 2, acc.z);
        epilogue_one<OutT>(ep, m, n + 3, acc.w);
    }
}

// Slices for a decode shape: enough to occupy the SMs, at least eight k blocks each.
int splitk_slices(int64_t M, int64_t N, int64_t K) {
    if (M <= 0 || N <= 0 || K <= 0) return 1;
    const int64_t tiles = ((M + kBM - 1) / kBM) * ((N + kBN - 1) / kBN);
    const int64_t num_kb = (K + kBK - 1) / kBK;
    int64_t s = sm_count() / tiles;
    if (s > num_kb / 8) s = num_kb / 8;
    if (s > 8) s = 8;
    return s < 2 ? 1 : static_cast<int>(s);
}

size_t splitk_scratch_bytes(int64_t M, int64_t N, int64_t K) {
    const int s = splitk_slices(M, N, K);
    if (s < 2 || N % 4 != 0) return 0;
    return static_cast<size_t>(s) * ((M + kBM - 1) / kBM * kBM) * N * sizeof(int32_t);
}

template <typename OutT>
int launch_tile_splitk(const int8_t *x1, int64_t ld_x1, const int8_t *x2, int64_t x2_sk, int64_t x2_sn,
                       const EpilogueParams &ep, int64_t K, void *workspace, int sm_reserve, cudaStream_t stream) {
    const int slices = splitk_slices(ep.M, ep.N, K);
    const int64_t slice_rows = (ep.M + kBM - 1) / kBM * kBM;
    CUtensorMap ta, tb, tout;
    int rc = make_tmap_2d(&ta, x1, 1, static_cast<uint64_t>(K), static_cast<uint64_t>(ep.M),
                          static_cast<uint64_t>(ld_x1), kBK, kBM, true);
    if (rc != QMM_OK) return rc;
    const bool mn_major = (x2_sn == 1);
    if (mn_major) {
        rc = make_tmap_2d(&tb, x2, 1, static_cast<uint64_t>(ep.N), static_cast<uint64_t>(K),
                          static_cast<uint64_t>(x2_sk), 128, kBK, true);
    } else {
        rc = make_tmap_2d(&tb, x2, 1, static_cast<uint64_t>(K), static_cast<uint64_t>(ep.N),
                          static_cast<uint64_t>(x2_sn), kBK, kBN, true);
    }
    if (rc != QMM_OK) return rc;
    rc = make_tmap_2d(&tout, workspace, 4, static_cast<uint64_t>(ep.N), static_cast<uint64_t>(slices * slice_rows),
                      static_cast<uint64_t>(ep.N), 32, 32, true);
    if (rc != QMM_OK) return rc;
    EpilogueParams raw;  // first pass: raw int32 sums, no scale, no bias
    raw.scale = nullptr;
    raw.pertoken_scale = nullptr;
    raw.bias = nullptr;
    raw.bias_dtype = QMM_DTYPE_NONE;
    raw.scale_is_scalar = 1;
    raw.out = workspace;
    raw.ld_out = ep.N;
    raw.M = ep.M;
    raw.N = ep.N;
    const int items = static_cast<int>(((ep.M + kBM - 1) / kBM) * ((ep.N + kBN - 1) / kBN)) * slices;
    int ctas = sm_count() - sm_reserve;
    if (ctas < 1) ctas = 1;
    const int grid = items < ctas ? items : ctas;
    auto kern = mn_major ? w8a8_tile_kernel<int32_t, true> : w8a8_tile_kernel<int32_t, false>;
    QMM_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     static_cast<int>(kTileSmemBytes)));
    kern<<<grid, kTileThreads, kTileSmemBytes, stream>>>(ta, tb, tout, raw, static_cast<int>(K), 1, slices,
                                                         static_cast<int>(slice_rows), device_status_word());
    QMM_CUDA_OK(cudaGetLastError());
    if constexpr (sizeof(OutT) == 2) {
        if ((ep.N & 7) == 0 && (ep.ld_out & 7) == 0 && (reinterpret_cast<uintptr_t>(ep.out) & 15) == 0 && slices <= 8) {
            const unsigned gx = static_cast<unsigned>((ep.N / 8 + 255) / 256);
            int64_t gy = static_cast<int64_t>(sm_count()) * 8 / gx;
            if (gy > ep.M) gy = ep.M;
            if (gy < 1) gy = 1;
            const dim3 rg(gx, static_cast<unsigned>(gy));
            int32_t *sp = static_cast<int32_t *>(workspace);
            const int64_t se = slice_rows * ep.N;
            switch (slices) {
                case 2: splitk_reduce_vec8_kernel<OutT, 2><<<rg, 256, 0, stream>>>(sp, se, ep); break;
                case 3: splitk_reduce_vec8_kernel<OutT, 3><<<rg, 256, 0, stream>>>(sp, se, ep); break;
                case 4: splitk_reduce_vec8_kernel<OutT, 4><<<rg, 256, 0, stream>>>(sp, se, ep); break;
                case 5: splitk_reduce_vec8_kernel<OutT, 5><<<rg, 256, 0, stream>>>(sp, se, ep); break;
                case 6: splitk_reduce_vec8_kernel<OutT, 6><<<rg, 256, 0, stream>>>(sp, se, ep); break;
                case 7: splitk_reduce_vec8_kernel<OutT, 7><<<rg, 256, 0, stream>>>(sp, se, ep); break;
                default: splitk_reduce_vec8_kernel<OutT, 8><<<rg, 256, 0, stream>>>(sp, se, ep); break;
            }
            QMM_CUDA_OK(cudaGetLastError());
            return QMM_OK;
        }
    }
    const int64_t vecs = ep.M * ep.N / 4;
    const int rgrid = static_cast<int>(vecs / 256 + 1 < 4 * sm_count() ? vecs / 256 + 1 : 4 * sm_count());
    splitk_reduce_kernel<OutT><<<rgrid, 256, 0, stream>>>(static_cast<int32_t *>(workspace), slices,
                                                          slice_rows * ep.N, ep);
    QMM_CUDA_OK(cudaGetLastError());
    return QMM_OK;
}

template <typename OutT>
int launch_simt(const int8_t *x1, int64_t ld_x1, const int8_t *x2, int64_t x2_sk, int64_t x2_sn,
                const EpilogueParams &ep, int64_t K, cudaStream_t stream) {
    dim3 grid(static_cast<unsigned>((ep.N + kSimtTile - 1) / kSimtTile),
              static_cast<unsigned>((ep.M + kSimtTile - 1) / kSimtTile));
    if (grid.y > 65535) return fail(QMM_ERR_UNSUPPORTED, "qmm_quant_matmul: M too large for the SIMT kernel");
    w8a8_simt_kernel<OutT><<<grid, 256, 0, stream>>>(x1, ld_x1, x2, x2_sk, x2_sn, ep, K);
    QMM_CUDA_OK(cudaGetLastError());
    return QMM_OK;
}

// Decode shapes (M <= 128): stream-K keeps every SM streaming weights whatever N is, but its split
// tiles pay for the int32 scratch traffic, which grows with M.  Measured on B200 (graph replay):
// K x N = 8192 x 28672: M = 1 stream-K 46.9 us, tile kernel 54.2 us; M = 8 49.8 / 52.8 us; M = 32
// 59 / 44 us; M = 128 110 / 46 us.  So up to 16 tokens stream-K wins everywhere; beyond that the
// one-CTA tile kernel is ahead as soon as its 128 x 256 tiles occupy most SMs.  Shapes with few tiles
// and a long K (28672 x 8192) go to the tile kernel over K slices before this function is asked
// (M = 32 47 us, M = 128 61 us against 59 / 85 us for the better of the other two).
bool prefer_streamk(int64_t M, int64_t N) {
    if (M <= 16) return true;
    const int64_t tiles = (N + kBN - 1) / kBN;
    if (tiles * 10 >= static_cast<int64_t>(sm_count()) * 7) return false;
    return M <= 64;
}

bool tma_compatible(const int8_t *x1, int64_t ld_x1, const int8_t *x2, int64_t x2_sk, int64_t x2_sn) {
    if ((reinterpret_cast<uintptr_t>(x1) & 15) || (ld_x1 & 15)) return false;
    if (reinterpret_cast<uintptr_t>(x2) & 15) return false;
    if (x2_sn == 1) return (x2_sk & 15) == 0;
    if (x2_sk == 1) return (x2_sn & 15) == 0;
    return false;
}

}  // namespace

// Implemented in w8a8_streamk.cu
int launch_streamk(const int8_t *x1, int64_t ld_x1, const int8_t *x2, int64_t x2_sk, int64_t x2_sn,
                   const EpilogueParams &ep, int out_dtype, int64_t K, void *workspace, size_t workspace_bytes,
                   cudaStream_t stream);
size_t streamk_workspace_bytes(int64_t M, int64_t N, int64_t K);
bool streamk_supported(int64_t M, int64_t N, int64_t K, int64_t x2_sn);

int quant_matmul_dispatch(const int8_t *x1, int64_t ld_x1, const int8_t *x2, int64_t x2_sk, int64_t x2_sn,
                          const EpilogueParams &ep, int out_dtype, int64_t K, int algo, void *workspace,
                          size_t workspace_bytes, cudaStream_t stream, LaunchOptions *opts) {
    const int sm_reserve = (opts != nullptr && opts->sm_reserve > 0) ? opts->sm_reserve : 0;
    const bool tma_ok = tma_compatible(x1, ld_x1, x2, x2_sk, x2_sn) && K < (1ll << 31) && ep.M < (1ll << 31) &&
                        ep.N < (1ll << 31);
    if (algo == QMM_ALGO_AUTO) {
        if (!tma_ok)
            algo = QMM_ALGO_SIMT;
        else if (ep.M > 16 && ep.M <= 128 && workspace != nullptr && splitk_scratch_bytes(ep.M, ep.N, K) > 0 &&
                 workspace_bytes >= splitk_scratch_bytes(ep.M, ep.N, K) &&
                 (reinterpret_cast<uintptr_t>(workspace) & 15) == 0)
            algo = QMM_ALGO_TCGEN05_SPLITK;  // few tiles, long K: the slices fill the SMs
        else if (streamk_supported(ep.M, ep.N, K, x2_sn) && workspace != nullptr &&
                 workspace_bytes >= streamk_workspace_bytes(ep.M, ep.N, K) && prefer_streamk(ep.M, ep.N))
            algo = QMM_ALGO_TCGEN05_STREAMK;
        else if (ep.M > 128)
            algo = QMM_ALGO_TCGEN05_PAIR;  // a few percent ahead of the one-CTA kernel under the power cap
        else
            algo = QMM_ALGO_TCGEN05_TILE;
    }
    if ((algo == QMM_ALGO_TCGEN05_TILE || algo == QMM_ALGO_TCGEN05_STREAMK || algo == QMM_ALGO_TCGEN05_PAIR ||
         algo == QMM_ALGO_TCGEN05_SPLITK) && !tma_ok)
        return fail(QMM_ERR_UNSUPPORTED,
                    "qmm_quant_matmul: tcgen05 kernels need 16-byte aligned operands and row pitches");
    switch (algo) {
        case QMM_ALGO_TCGEN05_TILE:
            switch (out_dtype) {
                case QMM_DTYPE_BF16:
                    return launch_tile<__nv_bfloat16>(x1, ld_x1, x2, x2_sk, x2_sn, ep, K, sm_reserve, stream);
                case QMM_DTYPE_F16:
                    return launch_tile<__half>(x1, ld_x1, x2, x2_sk, x2_sn, ep, K, sm_reserve, stream);
                default:
                    return launch_tile<int32_t>(x1, ld_x1, x2, x2_sk, x2_sn, ep, K, sm_reserve, stream);
            }
        case QMM_ALGO_TCGEN05_PAIR:
            return launch_pair(x1, ld_x1, x2, x2_sk, x2_sn, ep, out_dtype, K, opts, stream);
        case QMM_ALGO_TCGEN05_SPLITK:
            if (workspace == nullptr || splitk_scratch_bytes(ep.M, ep.N, K) == 0 ||
                workspace_bytes < splitk_scratch_bytes(ep.M, ep.N, K) ||
                (reinterpret_cast<uintptr_t>(workspace) & 15) != 0)
                return fail(QMM_ERR_UNSUPPORTED,
                            "qmm_quant_matmul: split-K needs at least two slices of eight k blocks, N a multiple of "
                            "4 and the scratch qmm_quant_matmul_workspace_size reports");
            switch (out_dtype) {
                case QMM_DTYPE_BF16:
                    return launch_tile_splitk<__nv_bfloat16>(x1, ld_x1, x2, x2_sk, x2_sn, ep, K, workspace, sm_reserve, stream);
                case QMM_DTYPE_F16:
                    return launch_tile_splitk<__half>(x1, ld_x1, x2, x2_sk, x2_sn, ep, K, workspace, sm_reserve, stream);
                default:
                    return launch_tile_splitk<int32_t>(x1, ld_x1, x2, x2_sk, x2_sn, ep, K, workspace, sm_reserve, stream);
            }
        case QMM_ALGO_TCGEN05_STREAMK:
            return launch_streamk(x1, ld_x1, x2, x2_sk, x2_sn, ep, out_dtype, K, workspace, workspace_bytes, stream);
        case QMM_ALGO_SIMT:
            switch (out_dtype) {
                case QMM_DTYPE_BF16:
                    return launch_simt<__nv_bfloat16>(x1, ld_x1, x2, x2_sk, x2_sn, ep, K, stream);
                case QMM_DTYPE_F16:
                    return launch_simt<__half>(x1, ld_x1, x2, x2_sk, x2_sn, ep, K, stream);
                default:
                    return launch_simt<int32_t>(x1, ld_x1, x2, x2_sk, x2_sn, ep, K, stream);
            }
        default:
            return fail(QMM_ERR_INVALID_ARGUMENT, "qmm_quant_matmul: unknown algo");
    }
}

int validate_quant_matmul(const int8_t *x1, int64_t ld_x1, const int8_t *x2, int64_t x2_sk, int64_t x2_sn,
                          const float *scale, int64_t scale_len, const void *bias, int bias_dtype, void *out,
                          int out_dtype, int64_t ld_out, int64_t M, int64_t N, int64_t K) {
    QMM_REQUIRE(M >= 0 && N >= 0 && K >= 0, "qmm_quant_matmul: negative dimension");
    QMM_REQUIRE(out_dtype == QMM_DTYPE_BF16 || out_dtype == QMM_DTYPE_F16 || out_dtype == QMM_DTYPE_I32,
                "qmm_quant_matmul: output dtype must be bf16, f16 or int32");
    if (M == 0 || N == 0) return QMM_OK;
    QMM_REQUIRE(out != nullptr, "qmm_quant_matmul: out is NULL");
    QMM_REQUIRE(ld_out >= N, "qmm_quant_matmul: ld_out smaller than N");
    if (K > 0) {
        QMM_REQUIRE(x1 != nullptr && x2 != nullptr, "qmm_quant_matmul: NULL operand");
        QMM_REQUIRE(ld_x1 >= K, "qmm_quant_matmul: ld_x1 smaller than K");
        QMM_REQUIRE(x2_sk == 1 || x2_sn == 1, "qmm_quant_matmul: x2 must have a unit stride along K or N");
        QMM_REQUIRE((x2_sn == 1 && (x2_sk >= N || K == 1)) || (x2_sk == 1 && (x2_sn >= K || N == 1)),
                    "qmm_quant_matmul: x2 strides overlap");
    }
    if (out_dtype != QMM_DTYPE_I32) {
        QMM_REQUIRE(scale != nullptr, "qmm_quant_matmul: scale is NULL");
        QMM_REQUIRE(scale_len == N || scale_len == 1, "qmm_quant_matmul: scale must have N elements or one");
        QMM_REQUIRE(bias == nullptr || bias_dtype == QMM_DTYPE_BF16 || bias_dtype == QMM_DTYPE_F16 ||
                        bias_dtype == QMM_DTYPE_F32,
                    "qmm_quant_matmul: bias must be bf16, f16 or f32 for a floating-point output");
    } else {
        QMM_REQUIRE(bias == nullptr || bias_dtype == QMM_DTYPE_I32,
                    "qmm_quant_matmul: bias must be int32 for an int32 output");
    }
    return QMM_OK;
}

}  // namespace qmm

extern "C" int qmm_quant_matmul_workspace_size(int64_t M, int64_t N, int64_t K, int algo, size_t *bytes) {
    using namespace qmm;
    QMM_REQUIRE(bytes != nullptr, "qmm_quant_matmul_workspace_size: bytes is NULL");
    QMM_REQUIRE(M >= 0 && N >= 0 && K >= 0, "qmm_quant_matmul_workspace_size: negative dimension");
    *bytes = 0;
    if ((algo == QMM_ALGO_AUTO || algo == QMM_ALGO_TCGEN05_STREAMK) && streamk_supported(M, N, K, 1))
        *bytes = streamk_workspace_bytes(M, N, K);
    if ((algo == QMM_ALGO_AUTO || algo == QMM_ALGO_TCGEN05_SPLITK) && M <= 128) {
        const size_t sk = splitk_scratch_bytes(M, N, K);
        if (sk > *bytes) *bytes = sk;
    }
    return QMM_OK;
}

extern "C" int qmm_quant_matmul(const int8_t *x1, int64_t ld_x1, const int8_t *x2, int64_t x2_stride_k,
                                int64_t x2_stride_n, const float *scale, int64_t scale_len,
                                const float *pertoken_scale, const void *bias, int bias_dtype, void *out,
                                int out_dtype, int64_t ld_out, int64_t M, int64_t N, int64_t K, int algo,
                                void *workspace, size_t workspace_bytes, void *stream) {
    using namespace qmm;
    int rc = validate_quant_matmul(x1, ld_x1, x2, x2_stride_k, x2_stride_n, scale, scale_len, bias, bias_dtype, out,
                                   out_dtype, ld_out, M, N, K);
    if (rc != QMM_OK) return rc;
    if (M == 0 || N == 0) return QMM_OK;
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
    if (K == 0) algo = QMM_ALGO_SIMT;  // empty reduction: epilogue of zeros
    return quant_matmul_dispatch(x1, ld_x1, x2, x2_stride_k, x2_stride_n, ep, out_dtype, K, algo, workspace,
                                 workspace_bytes, static_cast<cudaStream_t>(stream), nullptr);
}
