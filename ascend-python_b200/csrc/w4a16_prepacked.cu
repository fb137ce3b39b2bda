// W4A16 matmul over PREPACKED weights (npu_weight_quant_batchmatmul after a one-time layout pass).
//
// The stock layout, int32 [K, N/8] with eight neighbouring COLUMNS per word, is the wrong way round
// for every tensor-core operand format (they keep consecutive k of ONE column together), and pairing
// the rows at run time costs more integer instructions than the HBM stream leaves time for.  The
// reference has the same notion of a private matmul weight format: it casts operands from the plain
// "ND" layout to the fractal "NZ" layout around its matmul
// (op_plugin/ops/base_ops/aclops/MmKernelNpu.cpp:80-94, :301-316).  Here the format is:
//
//   block (t, c) = output columns [128 t, 128 t + 128) x k rows [128 c, 128 c + 128), 8704 bytes,
//   blocks ordered [t][c] so that a CTA's share of the work is one contiguous byte stream:
//     bytes [0, 8192)     four sub-steps of 32 k; sub-step s holds, for column r = 0..127, one
//                         16-byte vector at (s * 128 + r) * 16: word i of the vector covers
//                         k = 32 s + 8 i .. + 7 of that column, nibble j (j < 4) = k + 2 j,
//                         nibble j + 4 = k + 2 j + 1  (two's complement, as in the stock layout)
//     bytes [8192, 8448)  scale[g, n]            as 16-bit floats, g = group of the block's k rows
//     bytes [8448, 8704)  offset[g, n] * scale[g, n], rounded once to the 16-bit type
//   Columns beyond N are stored as zeros, and the number of blocks along K is rounded up to an even
//   count with an all-zero block (a stage of the kernel is a PAIR of blocks).  Requires K % 128 == 0
//   and group % 128 == 0.
//
// With that order `(word >> 4 j) & 0x000f000f` IS a tensor-memory operand column: two consecutive
// k of one output column as two 16-bit floats (after OR-ing exponent bits).  One thread owns one
// output column, so its scale and offset are scalars, and the weight
//     W = (w + offset) * scale = fma(w, scale, offset * scale)
// is finished in registers (one exact subtraction of the exponent constant, one fused multiply-add
// per pair, rounded once to the 16-bit type) and written to TENSOR MEMORY with tcgen05.st.  The MMA
// (kind::f16, 128 x Mpad x 16) takes that operand from tensor memory and the activations from
// shared memory, so the expanded weights never touch shared memory and the accumulator stays in
// tensor memory over the whole K range: no per-group pass over the accumulator, whatever M is.
//
// Warp roles (736 threads): warp 0 streams the packed weights (a stage is a pair of blocks = 17408
// contiguous bytes, one bulk copy); warp 1 streams the matching [Mpad][256 k] activation tiles by TMA
// into a ring of their own; warp 2 issues the MMAs (eight per block under one election: the issue
// rate of these small MMAs, about 45 clocks each, is one of the kernel's limits); warps 3-18 unpack
// (four teams of four warps; team s converts sub-step s of both blocks of a stage; a warp touches the
// 32 tensor-memory lanes 32 * (warp % 4)); warps 19-22 are the epilogue.  The operand ring in tensor
// memory holds three stages.  An unpack warp announces the operand columns of stage i only after it
// has converted stage i+1, so the latency of its tensor-memory stores hides behind the next stage's
// arithmetic.  Work is cut stream-K style into equal contiguous ranges of (column tile, block pair);
// a tile shared by several CTAs is summed from per-CTA slots in slot order by the CTA that arrives
// last, so results do not depend on arrival order.
//
// Measured bounds (B200, M = 16, K = 8192, N = 28672, per 256-k stage and SM): the conversion costs
// about 670 clocks per unpack warp - the packed 16-bit subtract and multiply-add issue at half rate on
// this part (64 lanes per clock and SM) - and the issue of the stage's 16 MMAs about 730 clocks.
#include "qmm_common.cuh"
#include "w4a16_simt.cuh"

namespace qmm {

namespace {

constexpr int kPTileN = 128;                          // output columns per tile = rows of the MMA
constexpr int kPChunkK = 128;                         // k rows per block
constexpr int kPSubK = 32;                            // k rows per sub-step (one 16-byte vector per column)
constexpr int kPSubs = kPChunkK / kPSubK;             // 4
constexpr int kPWBytes = kPTileN * kPChunkK / 2;      // 8192
constexpr int kPSOBytes = 2 * kPTileN * 2;            // 512: scale, offset * scale
constexpr int kPBlockBytes = kPWBytes + kPSOBytes;    // 8704
constexpr int kPMaxM = 64;                            // token rows per launch
constexpr int kPPair = 2;                             // blocks per stage
constexpr int kPStageK = kPPair * kPChunkK;           // 256 k rows per stage
constexpr int kPStageWBytes = kPPair * kPBlockBytes;  // 17408 bytes of packed weights per stage
constexpr int kPTeams = kPSubs;
constexpr int kPUnpackWarps = 4 * kPTeams;            // 16
constexpr int kPEpiWarps = 4;
constexpr int kPMmaWarp = 2;
constexpr int kPFirstUnpackWarp = 3;
constexpr int kPFirstEpiWarp = kPFirstUnpackWarp + kPUnpackWarps;
constexpr int kPThreads = (kPFirstEpiWarp + kPEpiWarps) * 32;  // 736
constexpr int kPRing = 3;                             // stages of the operand ring in tensor memory
constexpr int kPMaxXStages = 8;                       // activation tiles in shared memory
constexpr uint32_t kPRingCols = kPStageK / 2;         // 128 columns per stage: two 16-bit k per column
constexpr uint32_t kPDBufs = 2;
constexpr uint32_t kPACol0 = kPDBufs * kPMaxM;        // accumulators in columns [0, 128), the ring behind: [128, 512)
constexpr uint32_t kPTmemCols = 512;
constexpr int kPMaxStages = 8;
constexpr size_t kPCounterBytes = 64 * 1024;          // tile counters: a fixed area at the start of the scratch
constexpr size_t kPSmemBudget = 200 * 1024;

struct PSmemTail {
    uint64_t w_full[kPMaxStages];   // packed weights of a stage have landed
    uint64_t w_empty[kPMaxStages];  // ... and have been read into registers by all unpack warps
    uint64_t x_full[kPMaxXStages];  // activation tile of a stage has landed
    uint64_t x_empty[kPMaxXStages]; // ... and the MMAs that read it are complete
    uint64_t a_full[kPRing];        // operand columns of a ring slot are written (16 unpack warps)
    uint64_t mma_done[kPRing];      // the MMAs of a ring slot are complete: its columns are free
    uint64_t tmem_full[kPDBufs];
    uint64_t tmem_empty[kPDBufs];
    uint32_t tmem_base;
    uint32_t abort_flag;
    uint32_t is_last;
    uint32_t epi_abort;
};

struct PParams {
    const uint8_t *packed;
    const void *bias;
    void *out;
    int64_t ld_out;
    int M, N;
    int mpad;         // M rounded up to 16
    int x_box_bytes;  // mpad * 128: one [mpad][64 k] activation box
    int nstages;      // packed-weight stages in shared memory
    int nxstages;     // activation tiles in shared memory
    int tiles_n;
    int nchunks;      // block PAIRS along K
    int max_slots;
    float *slots;        // [tiles_n][max_slots][mpad][128]
    uint32_t *counters;  // [tiles_n], zero between calls
    uint32_t *status;
};

__device__ __forceinline__ int p_cta_of_item(int64_t u, int64_t total, int64_t G) {
    return static_cast<int>((u * G + G - 1) / total);
}
__device__ __forceinline__ void pepi_bar_sync() { asm volatile("bar.sync 3, 128;" ::: "memory"); }

// (a & b) ^ c in one logic instruction
__device__ __forceinline__ uint32_t p_and_xor(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("lop3.b32 %0, %1, %2, %3, 0x6a;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

// (nibble ^ 8) | exponent bits = kRaw0 + 8 + w as a 16-bit float; subtracting the constant is exact.
template <typename T>
struct PMagic;
template <>
struct PMagic<__nv_bfloat16> {
    using T2 = __nv_bfloat162;
    static constexpr uint32_t kFlip = 0x43084308u;  // 128.0 | 8
    static constexpr uint32_t kFmt = 1;
    static __device__ __forceinline__ T2 bias2() { return __floats2bfloat162_rn(136.0f, 136.0f); }
};
template <>
struct PMagic<__half> {
    using T2 = __half2;
    static constexpr uint32_t kFlip = 0x64086408u;  // 1024.0 | 8
    static constexpr uint32_t kFmt = 0;
    static __device__ __forceinline__ T2 bias2() { return __floats2half2_rn(1032.0f, 1032.0f); }
};

template <typename T>
__global__ void __launch_bounds__(kPThreads, 1)
w4a16_prepacked_kernel(const __grid_constant__ CUtensorMap tmap_x, PParams p) {
    using T2 = typename PMagic<T>::T2;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *smem_aligned = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t nstages = static_cast<uint32_t>(p.nstages);
    const uint32_t x_box = static_cast<uint32_t>(p.x_box_bytes);
    const uint32_t x_slot = 4u * x_box;           // [mpad][256 k] as four boxes
    const uint32_t nxstages = static_cast<uint32_t>(p.nxstages);
    const uint32_t w_off = nxstages * x_slot;     // the packed-weight stages sit behind the activation tiles
    PSmemTail *tail = reinterpret_cast<PSmemTail *>(smem_aligned + w_off + nstages * kPStageWBytes);
    volatile uint32_t *abort_flag = &tail->abort_flag;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int64_t total = static_cast<int64_t>(p.tiles_n) * p.nchunks;
    const int64_t G = gridDim.x;
    const int64_t u_begin = total * blockIdx.x / G;
    const int64_t u_end = total * (blockIdx.x + 1) / G;

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < nstages; ++s) {
            mbar_init(smem_u32(&tail->w_full[s]), 1);
            mbar_init(smem_u32(&tail->w_empty[s]), kPUnpackWarps);
        }
        for (uint32_t a = 0; a < nxstages; ++a) {
            mbar_init(smem_u32(&tail->x_full[a]), 1);
            mbar_init(smem_u32(&tail->x_empty[a]), 1);
        }
        for (int a = 0; a < kPRing; ++a) {
            mbar_init(smem_u32(&tail->a_full[a]), kPUnpackWarps);
            mbar_init(smem_u32(&tail->mma_done[a]), 1);
        }
        for (uint32_t b = 0; b < kPDBufs; ++b) {
            mbar_init(smem_u32(&tail->tmem_full[b]), 1);
            mbar_init(smem_u32(&tail->tmem_empty[b]), kPEpiWarps);
        }
        tail->abort_flag = 0;
        tail->is_last = 0;
        tail->epi_abort = 0;
        mbar_fence_init();
        tma_prefetch_desc(&tmap_x);
    }
    if (warp == kPMmaWarp) {
        tmem_alloc(smem_u32(&tail->tmem_base), kPTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tail->tmem_base;

    if (warp == 0) {
        // ---------------- weight producer: one bulk copy of 17408 contiguous bytes per stage ----------------
        const uint8_t *src = p.packed + u_begin * kPStageWBytes;  // items are consecutive in [tile][pair] order
        uint32_t st = 0, ph = 0;
        const uint32_t full0 = smem_u32(&tail->w_full[0]), empty0 = smem_u32(&tail->w_empty[0]);
        for (int64_t it = u_begin; it < u_end; ++it, src += kPStageWBytes) {
            if (!mbar_wait(empty0 + st * 8, ph ^ 1, abort_flag, 0x50)) break;
            if (lane == 0) {
                mbar_expect_tx(full0 + st * 8, kPStageWBytes);
                bulk_load_1d(smem_base + w_off + st * kPStageWBytes, src, kPStageWBytes, full0 + st * 8);
            }
            __syncwarp();
            if (++st == nstages) {
                st = 0;
                ph ^= 1;
            }
        }
    } else if (warp == 1) {
        // ---------------- activation producer: one [mpad][256 k] tile per stage ----------------
        int c = static_cast<int>(u_begin % p.nchunks);
        uint32_t rs = 0, rph = 0;
        for (int64_t it = u_begin; it < u_end; ++it) {
            if (!mbar_wait(smem_u32(&tail->x_empty[rs]), rph ^ 1, abort_flag, 0x57)) break;
            if (lane == 0) {
                const uint32_t bar = smem_u32(&tail->x_full[rs]);
                const uint32_t dst = smem_base + rs * x_slot;
                mbar_expect_tx(bar, x_slot);
#pragma unroll
                for (int b = 0; b < 4; ++b)  // rows beyond M and k beyond K arrive as zeros
                    tma_load_2d(dst + b * x_box, &tmap_x, c * kPStageK + b * 64, 0, bar);
            }
            __syncwarp();
            if (++rs == nxstages) {
                rs = 0;
                rph ^= 1;
            }
            if (++c == p.nchunks) c = 0;
        }
    } else if (warp == kPMmaWarp) {
        // ---------------- MMA issuer (whole warp, one elected lane issues) ----------------
        const uint32_t idesc = make_idesc(/*c=f32*/ 1, PMagic<T>::kFmt, PMagic<T>::kFmt, /*a*/ 0, /*b K-major*/ 0,
                                          kPTileN, static_cast<uint32_t>(p.mpad));
        constexpr uint32_t kDescHi = smem_desc_hi_sw128(1024);
        int c = static_cast<int>(u_begin % p.nchunks);
        uint32_t rs = 0, rph = 0, xs = 0, xph = 0, pb = 0, pb_phase = 0, accumulate = 0;
        bool ok = true;
        for (int64_t it = u_begin; it < u_end && ok; ++it) {
            const bool first = (it == u_begin) || (c == 0);
            const bool last = (it + 1 == u_end) || (c + 1 == p.nchunks);
            if (first) {
                ok = mbar_wait(smem_u32(&tail->tmem_empty[pb]), pb_phase ^ 1, abort_flag, 0x51);
                if (!ok) break;
                accumulate = 0;
            }
            ok = mbar_wait(smem_u32(&tail->x_full[xs]), xph, abort_flag, 0x52) &&
                 mbar_wait(smem_u32(&tail->a_full[rs]), rph, abort_flag, 0x53);
            if (!ok) break;
            tc_fence_after();
            const uint32_t d = tmem_base + pb * kPMaxM;
            const uint32_t a = tmem_base + kPACol0 + rs * kPRingCols;
            const uint32_t x_lo = smem_desc_lo(smem_base + xs * x_slot, 16);
            const uint32_t box = x_box >> 4;
            mma_f16_ts_warp_x8(d, a, x_lo, x_lo + box, kDescHi, idesc, accumulate);
            mma_f16_ts_warp_x8(d, a + 64, x_lo + 2 * box, x_lo + 3 * box, kDescHi, idesc, 1);
            accumulate = 1;
            tc_commit_warp(smem_u32(&tail->mma_done[rs]));
            tc_commit_warp(smem_u32(&tail->x_empty[xs]));
            if (++xs == nxstages) {
                xs = 0;
                xph ^= 1;
            }
            if (last) {
                tc_commit_warp(smem_u32(&tail->tmem_full[pb]));
                if (++pb == kPDBufs) {
                    pb = 0;
                    pb_phase ^= 1;
                }
            }
            if (++rs == kPRing) {
                rs = 0;
                rph ^= 1;
            }
            if (++c == p.nchunks) c = 0;
        }
    } else if (warp < kPFirstEpiWarp) {
        // ---------------- unpack warps ----------------
        const int team = (warp - kPFirstUnpackWarp) >> 2;  // sub-step of both blocks of a stage this warp converts
        const int quarter = warp & 3;                      // tensor-memory lanes [32 quarter, +32)
        const int r = quarter * 32 + lane;                 // output column within the tile
        const uint32_t nib_mask = 0x000f000fu;
        const uint32_t flip = PMagic<T>::kFlip;
        const T2 bias2 = PMagic<T>::bias2();
        // this warp's 16 columns of sub-step `team` of block 0; block 1 is 64 columns further
        const uint32_t lane_taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + kPACol0 + team * 16;
        uint32_t st = 0, ph = 0, rs = 0, rph = 0;
        int pending = -1;  // ring slot whose stores are in flight
        for (int64_t it = u_begin; it < u_end; ++it) {
            if (!mbar_wait(smem_u32(&tail->w_full[st]), ph, abort_flag, 0x54)) break;
            const uint8_t *blk = smem_aligned + w_off + st * kPStageWBytes;
            uint4 wv[kPPair];
            uint32_t s32[kPPair], t32[kPPair];
#pragma unroll
            for (int b = 0; b < kPPair; ++b) {
                const uint8_t *bb = blk + b * kPBlockBytes;
                wv[b] = *reinterpret_cast<const uint4 *>(bb + (team * kPTileN + r) * 16);
                const uint32_t s16 = *reinterpret_cast<const uint16_t *>(bb + kPWBytes + r * 2);
                const uint32_t t16 = *reinterpret_cast<const uint16_t *>(bb + kPWBytes + kPTileN * 2 + r * 2);
                s32[b] = s16 * 0x10001u;
                t32[b] = t16 * 0x10001u;
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&tail->w_empty[st]));
            uint32_t v[kPPair][16];
#pragma unroll
            for (int b = 0; b < kPPair; ++b) {
                const T2 s2 = *reinterpret_cast<const T2 *>(&s32[b]);
                const T2 t2 = *reinterpret_cast<const T2 *>(&t32[b]);
                const uint32_t words[4] = {wv[b].x, wv[b].y, wv[b].z, wv[b].w};
#pragma unroll
                for (int i = 0; i < 4; ++i)
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const uint32_t raw = p_and_xor(words[i] >> (4 * j), nib_mask, flip);
                        const T2 wq = __hsub2(*reinterpret_cast<const T2 *>(&raw), bias2);  // exact: w itself
                        const T2 wf = __hfma2(wq, s2, t2);                                  // (w + offset) * scale
                        v[b][4 * i + j] = *reinterpret_cast<const uint32_t *>(&wf);
                    }
            }
            // the previous stage's stores have had this stage's arithmetic to complete: announce them
            if (pending >= 0) {
                tmem_st_wait();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&tail->a_full[pending]));
            }
            if (!mbar_wait(smem_u32(&tail->mma_done[rs]), rph ^ 1, abort_flag, 0x55)) break;
            tc_fence_after();
            tmem_st_32x16(lane_taddr + rs * kPRingCols, v[0]);
            tmem_st_32x16(lane_taddr + rs * kPRingCols + 64, v[1]);
            pending = static_cast<int>(rs);
            if (++rs == kPRing) {
                rs = 0;
                rph ^= 1;
            }
            if (++st == nstages) {
                st = 0;
                ph ^= 1;
            }
        }
        if (pending >= 0) {
            tmem_st_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&tail->a_full[pending]));
        }
    } else {
        // ---------------- epilogue warps: thread = tensor-memory lane = one output column ----------------
        const int quarter = warp & 3;
        const int row = quarter * 32 + lane;
        const bool leader_thread = (threadIdx.x == kPFirstEpiWarp * 32);
        const T *bias = static_cast<const T *>(p.bias);
        T *out = static_cast<T *>(p.out);
        const int M = p.M;
        int64_t u = u_begin;
        uint32_t pb = 0, pb_phase = 0;
        while (u < u_end) {
            const int tile = static_cast<int>(u / p.nchunks);
            const int64_t tile_begin = static_cast<int64_t>(tile) * p.nchunks;
            const int64_t tile_end = tile_begin + p.nchunks;
            const int64_t seg_end = tile_end < u_end ? tile_end : u_end;
            const bool whole = (u == tile_begin && seg_end == tile_end);
            const int64_t n = static_cast<int64_t>(tile) * kPTileN + row;
            const bool n_ok = n < p.N;
            const float b = (n_ok && bias != nullptr) ? to_float(bias[n]) : 0.0f;

            if (!mbar_wait(smem_u32(&tail->tmem_full[pb]), pb_phase, abort_flag, 0x56))
                *reinterpret_cast<volatile uint32_t *>(&tail->epi_abort) = 1;
            // the four warps meet at named barriers below, so they leave together or not at all
            pepi_bar_sync();
            if (*reinterpret_cast<volatile uint32_t *>(&tail->epi_abort) != 0) break;
            tc_fence_after();
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + pb * kPMaxM;

            const int first_cta = p_cta_of_item(tile_begin, total, G);
            const int last_cta = p_cta_of_item(tile_end - 1, total, G);
            const int nslots = last_cta - first_cta + 1;
            const int64_t slot_elems = static_cast<int64_t>(p.mpad) * kPTileN;
            float *tile_slots = p.slots + static_cast<int64_t>(tile) * p.max_slots * slot_elems;
            float *mine = tile_slots + (static_cast<int>(blockIdx.x) - first_cta) * slot_elems + row;
            for (int c0 = 0; c0 < p.mpad; c0 += 16) {
                uint32_t v[16];
                tmem_ld_32x16(taddr + c0, v);
                tmem_ld_wait();
                if (whole) {
                    if (n_ok) {
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            if (c0 + j < M)
                                out[static_cast<int64_t>(c0 + j) * p.ld_out + n] = from_float<T>(__uint_as_float(v[j]) + b);
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 16; ++j)
                        if (c0 + j < M) __stcg(mine + (c0 + j) * kPTileN, __uint_as_float(v[j]));
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&tail->tmem_empty[pb]));
            if (++pb == kPDBufs) {
                pb = 0;
                pb_phase ^= 1;
            }
            if (!whole) {
                __threadfence();
                pepi_bar_sync();
                if (leader_thread) {
                    const uint32_t old = atomicAdd(p.counters + tile, 1u);
                    const bool is_last = (old + 1 == static_cast<uint32_t>(nslots));
                    if (is_last) p.counters[tile] = 0;
                    tail->is_last = is_last ? 1u : 0u;
                    __threadfence();
                }
                pepi_bar_sync();
                if (*reinterpret_cast<volatile uint32_t *>(&tail->is_last) != 0 && n_ok) {
                    for (int m0 = 0; m0 < M; m0 += 16) {
                        float v[16];
#pragma unroll
                        for (int j = 0; j < 16; ++j) v[j] = 0.0f;
                        for (int sl = 0; sl < nslots; ++sl) {
#pragma unroll
                            for (int j = 0; j < 16; ++j)
                                if (m0 + j < M) v[j] += __ldcg(tile_slots + sl * slot_elems + row + (m0 + j) * kPTileN);
                        }
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            if (m0 + j < M) out[static_cast<int64_t>(m0 + j) * p.ld_out + n] = from_float<T>(v[j] + b);
                    }
                }
                pepi_bar_sync();  // is_last is rewritten by the next shared tile
            }
            u = seg_end;
        }
    }

    // ---------------- teardown ----------------
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && tail->abort_flag != 0 && p.status != nullptr) atomicMax(p.status, tail->abort_flag);
    if (warp == kPMmaWarp) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kPTmemCols);
    }
}

// ---- layout pass and its inverse ----------------------------------------------------------------------

// one CTA per block (tile, chunk): 512 threads write the 512 vectors, the first 128 also scale and offset*scale
template <typename T>
__global__ void __launch_bounds__(512)
w4a16_prepack_kernel(const int32_t *__restrict__ w, int64_t ld_w, const T *__restrict__ scale,
                     const T *__restrict__ offset, int64_t group, int64_t N, int64_t K, int nchunks,
                     uint8_t *__restrict__ out) {
    const int tile = blockIdx.y, c = blockIdx.x;  // c runs over the padded (even) number of blocks
    uint8_t *blk = out + (static_cast<int64_t>(tile) * nchunks + c) * kPBlockBytes;
    const int s = threadIdx.x >> 7, r = threadIdx.x & 127;
    const int64_t n = static_cast<int64_t>(tile) * kPTileN + r;
    const int64_t k0 = static_cast<int64_t>(c) * kPChunkK + s * kPSubK;
    const bool real = n < N && k0 < K;  // the padding block and the padding columns are zeros
    uint32_t words[4] = {0, 0, 0, 0};
    if (real) {
        const int64_t word_col = n >> 3;
        const int sh = static_cast<int>(n & 7) * 4;
#pragma unroll
        for (int kk = 0; kk < kPSubK; ++kk) {
            const uint32_t nib = (static_cast<uint32_t>(w[(k0 + kk) * ld_w + word_col]) >> sh) & 15u;
            const int e = kk & 7;
            words[kk >> 3] |= nib << (4 * ((e >> 1) + (e & 1) * 4));
        }
    }
    *reinterpret_cast<uint4 *>(blk + (s * kPTileN + r) * 16) = make_uint4(words[0], words[1], words[2], words[3]);
    if (threadIdx.x < kPTileN) {
        const int64_t g = (static_cast<int64_t>(c) * kPChunkK) / group;
        T sv = from_float<T>(0.0f), tv = from_float<T>(0.0f);
        if (real) {
            sv = scale[g * N + n];
            if (offset != nullptr) tv = from_float<T>(to_float(offset[g * N + n]) * to_float(sv));
        }
        reinterpret_cast<T *>(blk + kPWBytes)[r] = sv;
        reinterpret_cast<T *>(blk + kPWBytes + kPTileN * 2)[r] = tv;
    }
}

// inverse of the weight part: one thread per stock word (k, i)
__global__ void __launch_bounds__(256)
w4a16_unpack_kernel(const uint8_t *__restrict__ packed, int64_t N, int64_t K, int nchunks, int32_t *__restrict__ w,
                    int64_t ld_w) {
    const int64_t words_n = N >> 3;
    const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= K * words_n) return;
    const int64_t k = idx / words_n, i = idx - k * words_n;
    const int c = static_cast<int>(k / kPChunkK), kc = static_cast<int>(k % kPChunkK);
    const int s = kc / kPSubK, kk = kc % kPSubK, e = kk & 7;
    const int pos = (e >> 1) + (e & 1) * 4;
    uint32_t word = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const int64_t n = i * 8 + j;
        const int tile = static_cast<int>(n / kPTileN), r = static_cast<int>(n % kPTileN);
        const uint8_t *blk = packed + (static_cast<int64_t>(tile) * nchunks + c) * kPBlockBytes;
        const uint32_t pw = reinterpret_cast<const uint32_t *>(blk + (s * kPTileN + r) * 16)[kk >> 3];
        word |= ((pw >> (4 * pos)) & 15u) << (4 * j);
    }
    w[k * ld_w + i] = static_cast<int32_t>(word);
}

struct PPlan {
    int mpad, tiles_n, nchunks, grid, max_slots, nstages, nxstages;
    size_t slots_bytes;
};

PPlan p_make_plan(int64_t M, int64_t N, int64_t K) {
    PPlan pl;
    const int64_t m = M < kPMaxM ? M : kPMaxM;
    pl.mpad = static_cast<int>((m + 15) / 16 * 16);
    pl.tiles_n = static_cast<int>((N + kPTileN - 1) / kPTileN);
    pl.nchunks = static_cast<int>((K + kPStageK - 1) / kPStageK);  // block pairs
    const int64_t total = static_cast<int64_t>(pl.tiles_n) * pl.nchunks;
    pl.grid = static_cast<int>(total < sm_count() ? total : sm_count());
    const int64_t ipc = total / pl.grid;  // items per CTA, rounded down (>= 1)
    pl.max_slots = static_cast<int>((pl.nchunks + ipc - 1) / ipc + 1);
    // activation tiles: enough to cover the L2 latency of their loads; the rest of the budget holds weights
    pl.nxstages = pl.mpad <= 16 ? 8 : (pl.mpad <= 32 ? 6 : 4);
    pl.nstages = static_cast<int>((kPSmemBudget - static_cast<size_t>(pl.nxstages) * pl.mpad * 512) / kPStageWBytes);
    if (pl.nstages > kPMaxStages) pl.nstages = kPMaxStages;
    pl.slots_bytes = static_cast<size_t>(pl.tiles_n) * pl.max_slots * pl.mpad * kPTileN * sizeof(float);
    return pl;
}

bool p_shape_ok(int64_t N, int64_t K, int64_t group) {
    return N > 0 && K > 0 && N % 8 == 0 && K % kPChunkK == 0 && group > 0 && group % kPChunkK == 0 && K % group == 0 &&
           K < (1ll << 31) && N < (1ll << 31) && (N + kPTileN - 1) / kPTileN <= static_cast<int64_t>(kPCounterBytes / 4);
}

// blocks along K, rounded up to an even count
int p_blocks_k(int64_t K) { return static_cast<int>((K + kPStageK - 1) / kPStageK) * kPPair; }

size_t p_packed_bytes(int64_t N, int64_t K) {
    return static_cast<size_t>((N + kPTileN - 1) / kPTileN) * static_cast<size_t>(p_blocks_k(K)) * kPBlockBytes;
}

// ---- one or two tokens: integer dot products on the CUDA cores --------------------------------------------
//
// For a handful of tokens the tensor cores have nothing to add: a thread owns one output column, reads its
// 64 bytes of a block straight from global memory (a warp's loads are 512 contiguous bytes), splits each
// packed word into two words of four unsigned bytes - `w ^ 0x88888888` turns the two's complement nibbles into
// w + 8, `& 0x0f0f0f0f` and `>> 4 & 0x0f0f0f0f` are bytes (k, k+4, k+1, k+5) and (k+2, k+6, k+3, k+7) of a
// group of eight k - and multiplies them with dp4a by the activations, which a small kernel in front has
// turned into two int8 digits of a block floating-point form, in that byte order: per token and block of
// 128 k, with e the exponent of the block's absmax,
//     X = rint(x * 2^(14 - e))  (|X| <= 2^14),   X = 128 * d1 + d2,  d1 in [-128, 127], d2 in [0, 127].
// An activation within 2^-6 of its block's absmax is represented exactly (16-bit floats carry 8 or 11
// significant bits); smaller ones are rounded to 2^-14 of the absmax, far below the 2^-9 / 2^-12 of the
// output's own rounding.  Per block the exact integers D1 = sum u*d1 and D2 = sum u*d2 (u = w + 8) give
//     y[m, n] += scale * esc[m] * (128 D1 + D2) + (offset*scale - 8 scale) * xs[m],
// esc = 2^(e - 14), xs = esc * sum X; the weight itself is never rounded.  About 1.3 instructions per weight
// for one token; every further token adds 64 dp4a per block and thread, which at the rate dp4a issues here costs
// 7-8 us per token, so beyond two tokens the tensor-core kernels are faster (the kernel itself is written for up
// to four).  A form with four columns per lane, which needs a quarter of the broadcast loads of digits, was
// measured slower still (37 us against 33 us at two tokens): the loads are not the limit.  Making the digits inside this kernel (every
// CTA for its own blocks) instead of in a kernel in front was measured slower: 30 us against 26 us for one token;
// so was pulling lines of later blocks into L2 with prefetch instructions (29.6 us).
// Two mma.sync forms of the same idea (the split words as register operands of m16n8k32.s8 on these digits, or
// pairs (k, k+1) as 16-bit operands of m16n8k16) were built and measured for 3..16 tokens: correct, but the legacy
// MMA instructions cost 10-19 clocks each per SM on this part (41 / 63 us at 8 tokens, 63 / 116 us at 16), slower
// than the kernels those sizes already have.  Work is cut into equal contiguous
// runs of blocks, many CTAs per SM; a tile's partial sums go to per-CTA slots that the last arriver adds in
// slot order, as in the tensor-core kernel.
constexpr int kGvMaxM = 2;            // measured (K=8192, N=28672): 26 / 33 us for 1 / 2 tokens, 41 / 51 us for 3 / 4
constexpr int kGvThreads = kPTileN;  // one output column per thread
constexpr int kGvCtasPerSm = 5;       // resident CTAs per SM (three blocks of weights in flight per thread; best of 4..8)

struct GvParams {
    const uint8_t *packed;
    const void *bias;
    void *out;
    int64_t ld_out;
    int N, tiles_n, nblocks, max_slots;
    int max_run;         // most blocks of one tile a CTA works on in a row (sizes the shared-memory copy of the digits)
    const uint4 *xd;     // digits [nblocks][M][2][8 x 16 bytes], bytes in the order the split words have
    const float *esc;    // [nblocks][M]
    const float *xs;     // [nblocks][M]
    float *slots;        // [tiles_n][max_slots][M][128]
    uint32_t *counters;  // [tiles_n], zero between calls
};

__device__ __forceinline__ uint4 ldg_stream(const uint8_t *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

template <typename T, int M>
__global__ void __launch_bounds__(kGvThreads, kGvCtasPerSm)
w4a16_gemv_kernel(GvParams p) {
    extern __shared__ uint4 gv_smem[];  // digits of a run of blocks [nb][M][2][8], then esc [nb][M], xs [nb][M]
    __shared__ uint32_t s_is_last;
    const int r = threadIdx.x;
    const int64_t total = static_cast<int64_t>(p.tiles_n) * p.nblocks;
    const int64_t G = gridDim.x;
    const int64_t u_begin = total * blockIdx.x / G;
    const int64_t u_end = total * (blockIdx.x + 1) / G;
    const T *bias = static_cast<const T *>(p.bias);
    T *out = static_cast<T *>(p.out);
    bool waited = false;
    int64_t u = u_begin;
    while (u < u_end) {
        const int tile = static_cast<int>(u / p.nblocks);
        const int64_t tile_begin = static_cast<int64_t>(tile) * p.nblocks;
        const int64_t tile_end = tile_begin + p.nblocks;
        const int64_t seg_end = tile_end < u_end ? tile_end : u_end;
        const bool whole = (u == tile_begin && seg_end == tile_end);
        const int64_t n = static_cast<int64_t>(tile) * kPTileN + r;
        const bool n_ok = n < p.N;
        const int nb = static_cast<int>(seg_end - u), b_first = static_cast<int>(u - tile_begin);
        // the first two blocks' weights are on their way before anything else happens
        const uint8_t *blk = p.packed + u * kPBlockBytes;
        uint4 wv[kPSubs], n1[kPSubs], n2[kPSubs];
#pragma unroll
        for (int s = 0; s < kPSubs; ++s) {
            wv[s] = ldg_stream(blk + (s * kPTileN + r) * 16);
            n1[s] = nb > 1 ? ldg_stream(blk + kPBlockBytes + (s * kPTileN + r) * 16) : make_uint4(0, 0, 0, 0);
        }
        T s_raw = *reinterpret_cast<const T *>(blk + kPWBytes + r * 2);
        T t_raw = *reinterpret_cast<const T *>(blk + kPWBytes + kPTileN * 2 + r * 2);
        // the digits come from the kernel launched just before this one (programmatic dependent launch: this
        // kernel may start while that one still runs)
        if (!waited) {
            asm volatile("griddepcontrol.wait;" ::: "memory");
            waited = true;
        }
        __syncthreads();  // the previous segment's digits are no longer read
        {
            const int nvec = nb * M * 16;
            const uint4 *src = p.xd + static_cast<int64_t>(b_first) * M * 16;
            for (int i = r; i < nvec; i += kGvThreads) gv_smem[i] = __ldg(src + i);
            float *tab = reinterpret_cast<float *>(gv_smem + p.max_run * M * 16);
            for (int i = r; i < nb * M; i += kGvThreads) {
                tab[i] = __ldg(p.esc + b_first * M + i);
                tab[p.max_run * M + i] = __ldg(p.xs + b_first * M + i);
            }
        }
        __syncthreads();
        const float *esc_s = reinterpret_cast<const float *>(gv_smem + p.max_run * M * 16);
        const float *xs_s = esc_s + p.max_run * M;
        float y[M];
#pragma unroll
        for (int m = 0; m < M; ++m) y[m] = 0.0f;
        for (int lb = 0; lb < nb; ++lb, blk += kPBlockBytes) {
            // the weights of the block after the next one are requested before this block is worked on
            if (lb + 2 < nb) {
#pragma unroll
                for (int s = 0; s < kPSubs; ++s) n2[s] = ldg_stream(blk + 2 * kPBlockBytes + (s * kPTileN + r) * 16);
            }
            T s_next = s_raw, t_next = t_raw;
            if (lb + 1 < nb) {
                s_next = *reinterpret_cast<const T *>(blk + kPBlockBytes + kPWBytes + r * 2);
                t_next = *reinterpret_cast<const T *>(blk + kPBlockBytes + kPWBytes + kPTileN * 2 + r * 2);
            }
            int d1[M], d2[M];
#pragma unroll
            for (int m = 0; m < M; ++m) d1[m] = d2[m] = 0;
            const uint4 *xd = gv_smem + lb * M * 16;
#pragma unroll
            for (int s = 0; s < kPSubs; ++s) {
                const uint32_t words[4] = {wv[s].x, wv[s].y, wv[s].z, wv[s].w};
#pragma unroll
                for (int h = 0; h < 2; ++h) {  // words 2h and 2h + 1 of the sub-step share one 16-byte digit vector
                    const uint32_t w0 = words[2 * h] ^ 0x88888888u, w1 = words[2 * h + 1] ^ 0x88888888u;
                    const int a0 = static_cast<int>(w0 & 0x0f0f0f0fu), b0 = static_cast<int>((w0 >> 4) & 0x0f0f0f0fu);
                    const int a1 = static_cast<int>(w1 & 0x0f0f0f0fu), b1 = static_cast<int>((w1 >> 4) & 0x0f0f0f0fu);
#pragma unroll
                    for (int m = 0; m < M; ++m) {
                        const uint4 x1 = xd[(m * 2 + 0) * 8 + s * 2 + h];  // the same address in every lane: a broadcast
                        const uint4 x2 = xd[(m * 2 + 1) * 8 + s * 2 + h];
                        d1[m] = __dp4a(a0, static_cast<int>(x1.x), d1[m]);
                        d1[m] = __dp4a(b0, static_cast<int>(x1.y), d1[m]);
                        d1[m] = __dp4a(a1, static_cast<int>(x1.z), d1[m]);
                        d1[m] = __dp4a(b1, static_cast<int>(x1.w), d1[m]);
                        d2[m] = __dp4a(a0, static_cast<int>(x2.x), d2[m]);
                        d2[m] = __dp4a(b0, static_cast<int>(x2.y), d2[m]);
                        d2[m] = __dp4a(a1, static_cast<int>(x2.z), d2[m]);
                        d2[m] = __dp4a(b1, static_cast<int>(x2.w), d2[m]);
                    }
                }
            }
            const float sc = to_float(s_raw), tc = to_float(t_raw) - 8.0f * sc;
#pragma unroll
            for (int m = 0; m < M; ++m) {
                const float v = fmaf(static_cast<float>(d1[m]), 128.0f, static_cast<float>(d2[m]));
                y[m] = fmaf(sc * esc_s[lb * M + m], v, y[m]);
                y[m] = fmaf(tc, xs_s[lb * M + m], y[m]);
            }
#pragma unroll
            for (int s = 0; s < kPSubs; ++s) {
                wv[s] = n1[s];
                n1[s] = n2[s];
            }
            s_raw = s_next;
            t_raw = t_next;
        }
        const float bv = (n_ok && bias != nullptr) ? to_float(bias[n]) : 0.0f;
        if (whole) {
            if (n_ok) {
#pragma unroll
                for (int m = 0; m < M; ++m) out[static_cast<int64_t>(m) * p.ld_out + n] = from_float<T>(y[m] + bv);
            }
        } else {
            const int first_cta = p_cta_of_item(tile_begin, total, G);
            const int last_cta = p_cta_of_item(tile_end - 1, total, G);
            const int nslots = last_cta - first_cta + 1;
            const int64_t slot_elems = static_cast<int64_t>(M) * kPTileN;
            float *tile_slots = p.slots + static_cast<int64_t>(tile) * p.max_slots * slot_elems;
            float *mine = tile_slots + (static_cast<int>(blockIdx.x) - first_cta) * slot_elems + r;
#pragma unroll
            for (int m = 0; m < M; ++m) __stcg(mine + m * kPTileN, y[m]);
            __threadfence();
            __syncthreads();
            if (threadIdx.x == 0) {
                const uint32_t old = atomicAdd(p.counters + tile, 1u);
                const bool is_last = (old + 1 == static_cast<uint32_t>(nslots));
                if (is_last) p.counters[tile] = 0;
                s_is_last = is_last ? 1u : 0u;
                __threadfence();
            }
            __syncthreads();
            if (s_is_last != 0 && n_ok) {
                float v[M];
#pragma unroll
                for (int m = 0; m < M; ++m) v[m] = 0.0f;
                for (int sl = 0; sl < nslots; ++sl) {
#pragma unroll
                    for (int m = 0; m < M; ++m) v[m] += __ldcg(tile_slots + sl * slot_elems + m * kPTileN + r);
                }
#pragma unroll
                for (int m = 0; m < M; ++m) out[static_cast<int64_t>(m) * p.ld_out + n] = from_float<T>(v[m] + bv);
            }
        }
        u = seg_end;
    }
}

// activations -> two int8 digits per element.  One warp per (block of 128 k, token): a lane takes four consecutive
// k (one 8-byte load), the block's absmax and sum are warp shuffles, no shared memory and no CTA barrier; the
// kernel is a few microseconds of latency in front of the matmul, so every step of it counts.
// grid (ceil(blocks / 4), M), 128 threads.
template <typename T>
__global__ void __launch_bounds__(128)
w4a16_gemv_digits_kernel(const T *__restrict__ x, int64_t ld_x, int M, int64_t K, int nblocks, int8_t *__restrict__ xd,
                         float *__restrict__ esc, float *__restrict__ xs) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");  // the matmul may start its weight loads
    const int lane = threadIdx.x & 31;
    const int blk = blockIdx.x * 4 + (threadIdx.x >> 5), m = blockIdx.y;
    if (blk >= nblocks) return;
    const int64_t k0 = static_cast<int64_t>(blk) * kPChunkK + lane * 4;
    float v[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    if (k0 < K) {  // K is a multiple of 128: a block is inside or a padding block
        const uint2 raw = __ldg(reinterpret_cast<const uint2 *>(x + static_cast<int64_t>(m) * ld_x + k0));
        const T *h = reinterpret_cast<const T *>(&raw);
#pragma unroll
        for (int j = 0; j < 4; ++j) v[j] = to_float(h[j]);
    }
    float a = 0.0f;
    int bad = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float av = fabsf(v[j]);
        if (av <= 3.0e38f) a = fmaxf(a, av); else bad = 1;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, o));
        bad |= __shfl_xor_sync(0xffffffffu, bad, o);
    }
    int e = 0, sum = 0;
    float e_scale = 0.0f;
    if (a > 0.0f) {
        (void)frexpf(a, &e);  // a = f * 2^e, f in [0.5, 1): |x| < 2^e; X = rint(x * 2^(14 - e))
        e_scale = ldexpf(1.0f, e - 14);
    }
    // byte positions inside the block's two 128-byte records (see the kernel's header for the order): the four k
    // of a lane lie in one group of eight, whose two words are bytes [8 g, 8 g + 8) of the sub-step's 32
    int8_t *rec = xd + (static_cast<int64_t>(blk) * M + m) * 256;
    const int s = lane >> 3, i = (lane >> 1) & 3;
    uint32_t d1w[2] = {0, 0}, d2w[2] = {0, 0};  // this lane's bytes of word A ([0]) and word B ([1]) of its group
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        int X = 0;
        if (a > 0.0f) {
            float q = rintf(ldexpf(v[j], 14 - e));
            q = fminf(fmaxf(q, -16384.0f), 16383.0f);
            X = (q == q) ? static_cast<int>(q) : 0;
        }
        sum += X;
        const int e8 = (lane & 1) * 4 + j;                     // k within its group of eight
        const int pos = (e8 & 1) ? 4 + (e8 >> 1) : (e8 >> 1);  // nibble position of that k in the packed word
        const int word = pos & 1, byte = pos >> 1;
        d1w[word] |= (static_cast<uint32_t>(X >> 7) & 0xffu) << (8 * byte);
        d2w[word] |= (static_cast<uint32_t>(X & 127)) << (8 * byte);
    }
    // the two lanes of a group hold disjoint bytes of the same two words: merge them and let the even lane store
#pragma unroll
    for (int w = 0; w < 2; ++w) {
        d1w[w] |= __shfl_xor_sync(0xffffffffu, d1w[w], 1);
        d2w[w] |= __shfl_xor_sync(0xffffffffu, d2w[w], 1);
    }
    if ((lane & 1) == 0) {
        *reinterpret_cast<uint2 *>(rec + s * 32 + i * 8) = make_uint2(d1w[0], d1w[1]);
        *reinterpret_cast<uint2 *>(rec + 128 + s * 32 + i * 8) = make_uint2(d2w[0], d2w[1]);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    if (lane == 0) {
        // a block that holds a NaN or an infinity poisons the token's outputs, as the plain arithmetic would
        esc[blk * M + m] = bad ? __int_as_float(0x7fc00000) : e_scale;
        xs[blk * M + m] = e_scale * static_cast<float>(sum);  // |sum| < 2^21: exact
    }
}

struct GvPlan {
    int tiles_n, nblocks, grid, max_slots, max_run;
    size_t slots_bytes, xd_bytes, tab_bytes;
};

size_t gv_align256(size_t v) { return (v + 255) / 256 * 256; }

GvPlan gv_make_plan(int64_t M, int64_t N, int64_t K) {
    GvPlan pl;
    pl.tiles_n = static_cast<int>((N + kPTileN - 1) / kPTileN);
    pl.nblocks = p_blocks_k(K);
    const int64_t total = static_cast<int64_t>(pl.tiles_n) * pl.nblocks;
    const int64_t cap = static_cast<int64_t>(sm_count()) * kGvCtasPerSm;
    pl.grid = static_cast<int>(total < cap ? total : cap);
    const int64_t ipc = total / pl.grid;  // blocks per CTA, rounded down (>= 1)
    pl.max_slots = static_cast<int>((pl.nblocks + ipc - 1) / ipc + 1);
    pl.max_run = static_cast<int>(ipc + 1 < pl.nblocks ? ipc + 1 : pl.nblocks);
    pl.slots_bytes = gv_align256(static_cast<size_t>(pl.tiles_n) * pl.max_slots * M * kPTileN * sizeof(float));
    pl.xd_bytes = gv_align256(static_cast<size_t>(pl.nblocks) * M * 256);
    pl.tab_bytes = gv_align256(static_cast<size_t>(pl.nblocks) * M * sizeof(float));
    return pl;
}

size_t gv_workspace_bytes(int64_t M, int64_t N, int64_t K) {
    const GvPlan pl = gv_make_plan(M, N, K);
    return kPCounterBytes + pl.slots_bytes + pl.xd_bytes + 2 * pl.tab_bytes;
}

template <typename T>
int launch_gemv_t(const uint8_t *packed, const void *x, int64_t ld_x, const void *bias, void *out, int64_t ld_out,
                  int64_t M, int64_t N, int64_t K, void *workspace, cudaStream_t stream) {
    const GvPlan pl = gv_make_plan(M, N, K);
    uint8_t *ws = static_cast<uint8_t *>(workspace);
    int8_t *xd = reinterpret_cast<int8_t *>(ws + kPCounterBytes + pl.slots_bytes);
    float *esc = reinterpret_cast<float *>(ws + kPCounterBytes + pl.slots_bytes + pl.xd_bytes);
    float *xs = reinterpret_cast<float *>(ws + kPCounterBytes + pl.slots_bytes + pl.xd_bytes + pl.tab_bytes);
    w4a16_gemv_digits_kernel<T><<<dim3(static_cast<unsigned>((pl.nblocks + 3) / 4), static_cast<unsigned>(M)), 128, 0,
                                  stream>>>(static_cast<const T *>(x), ld_x, static_cast<int>(M), K, pl.nblocks, xd, esc, xs);
    QMM_CUDA_OK(cudaGetLastError());
    GvParams p;
    p.packed = packed;
    p.bias = bias;
    p.out = out;
    p.ld_out = ld_out;
    p.N = static_cast<int>(N);
    p.tiles_n = pl.tiles_n;
    p.nblocks = pl.nblocks;
    p.max_slots = pl.max_slots;
    p.max_run = pl.max_run;
    p.xd = reinterpret_cast<const uint4 *>(xd);
    p.esc = esc;
    p.xs = xs;
    p.counters = reinterpret_cast<uint32_t *>(ws);
    p.slots = reinterpret_cast<float *>(ws + kPCounterBytes);
    // programmatic dependent launch: the kernel starts (and requests its first weights) while the digits
    // kernel still runs, and waits for it (griddepcontrol.wait) before it reads the digits
    const size_t smem = static_cast<size_t>(pl.max_run) * M * (256 + 8);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(pl.grid));
    cfg.blockDim = dim3(kGvThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    auto launch = [&](auto kern) -> int {
        if (smem > 48 * 1024)
            QMM_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
        QMM_CUDA_OK(cudaLaunchKernelEx(&cfg, kern, p));
        return QMM_OK;
    };
    switch (M) {
        case 1: return launch(w4a16_gemv_kernel<T, 1>);
        case 2: return launch(w4a16_gemv_kernel<T, 2>);
        case 3: return launch(w4a16_gemv_kernel<T, 3>);
        default: return launch(w4a16_gemv_kernel<T, 4>);
    }
}

template <typename T>
int launch_prepacked_t(const uint8_t *packed, const void *x, int64_t ld_x, const void *bias, void *out, int64_t ld_out,
                       int64_t M, int64_t N, int64_t K, void *workspace, cudaStream_t stream) {
    const PPlan pl = p_make_plan(M, N, K);
    PParams p;
    p.packed = packed;
    p.bias = bias;
    p.out = out;
    p.ld_out = ld_out;
    p.M = static_cast<int>(M);
    p.N = static_cast<int>(N);
    p.mpad = pl.mpad;
    p.x_box_bytes = pl.mpad * 128;
    p.nstages = pl.nstages;
    p.nxstages = pl.nxstages;
    p.tiles_n = pl.tiles_n;
    p.nchunks = pl.nchunks;
    p.max_slots = pl.max_slots;
    uint8_t *ws = static_cast<uint8_t *>(workspace);
    p.counters = reinterpret_cast<uint32_t *>(ws);
    p.slots = reinterpret_cast<float *>(ws + kPCounterBytes);
    p.status = device_status_word();

    CUtensorMap tx;
    int rc = make_tmap_2d(&tx, x, 2, static_cast<uint64_t>(K), static_cast<uint64_t>(M), static_cast<uint64_t>(ld_x), 64,
                          static_cast<uint32_t>(pl.mpad), true);
    if (rc != QMM_OK) return rc;
    static_assert(sizeof(PSmemTail) <= 1024, "the tail has 1 KiB");
    const size_t smem = 1024 + static_cast<size_t>(pl.nxstages) * pl.mpad * 512 +
                        static_cast<size_t>(pl.nstages) * kPStageWBytes + 1024;
    auto kern = w4a16_prepacked_kernel<T>;
    QMM_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    kern<<<pl.grid, kPThreads, smem, stream>>>(tx, p);
    QMM_CUDA_OK(cudaGetLastError());
    return QMM_OK;
}

}  // namespace
}  // namespace qmm

extern "C" int qmm_w4a16_prepack_size(int64_t N, int64_t K, int64_t group, size_t *bytes) {
    using namespace qmm;
    QMM_REQUIRE(bytes != nullptr, "qmm_w4a16_prepack_size: bytes is NULL");
    *bytes = p_shape_ok(N, K, group > 0 ? group : K) ? p_packed_bytes(N, K) : 0;
    return QMM_OK;
}

extern "C" int qmm_w4a16_prepack(const int32_t *weight, int64_t ld_w, const void *antiquant_scale,
                                 const void *antiquant_offset, int sdtype, int64_t group, int64_t N, int64_t K,
                                 void *packed, size_t packed_bytes, void *stream) {
    using namespace qmm;
    if (group <= 0) group = K;
    QMM_REQUIRE(sdtype == QMM_DTYPE_BF16 || sdtype == QMM_DTYPE_F16, "qmm_w4a16_prepack: scale must be bf16 or f16");
    if (!p_shape_ok(N, K, group))
        return fail(QMM_ERR_UNSUPPORTED,
                    "qmm_w4a16_prepack: needs N % 8 == 0, K % 128 == 0 and a group that is a multiple of 128 dividing K");
    QMM_REQUIRE(weight != nullptr && antiquant_scale != nullptr && packed != nullptr, "qmm_w4a16_prepack: NULL operand");
    QMM_REQUIRE(ld_w >= N / 8, "qmm_w4a16_prepack: ld_w smaller than N/8");
    QMM_REQUIRE((reinterpret_cast<uintptr_t>(packed) & 15) == 0, "qmm_w4a16_prepack: packed must be 16-byte aligned");
    if (packed_bytes < p_packed_bytes(N, K))
        return fail(QMM_ERR_WORKSPACE, "qmm_w4a16_prepack: packed buffer smaller than qmm_w4a16_prepack_size");
    const int nchunks = p_blocks_k(K);
    const int64_t tiles = (N + kPTileN - 1) / kPTileN;
    QMM_REQUIRE(tiles <= 65535, "qmm_w4a16_prepack: N too large");
    const dim3 grid(static_cast<unsigned>(nchunks), static_cast<unsigned>(tiles));
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (sdtype == QMM_DTYPE_BF16)
        w4a16_prepack_kernel<__nv_bfloat16><<<grid, 512, 0, s>>>(
            weight, ld_w, static_cast<const __nv_bfloat16 *>(antiquant_scale),
            static_cast<const __nv_bfloat16 *>(antiquant_offset), group, N, K, nchunks, static_cast<uint8_t *>(packed));
    else
        w4a16_prepack_kernel<__half><<<grid, 512, 0, s>>>(weight, ld_w, static_cast<const __half *>(antiquant_scale),
                                                          static_cast<const __half *>(antiquant_offset), group, N, K,
                                                          nchunks, static_cast<uint8_t *>(packed));
    QMM_CUDA_OK(cudaGetLastError());
    return QMM_OK;
}

extern "C" int qmm_w4a16_unpack_weight(const void *packed, int64_t N, int64_t K, int32_t *weight, int64_t ld_w,
                                       void *stream) {
    using namespace qmm;
    if (!p_shape_ok(N, K, K)) return fail(QMM_ERR_UNSUPPORTED, "qmm_w4a16_unpack_weight: needs N % 8 == 0 and K % 128 == 0");
    QMM_REQUIRE(packed != nullptr && weight != nullptr, "qmm_w4a16_unpack_weight: NULL operand");
    QMM_REQUIRE(ld_w >= N / 8, "qmm_w4a16_unpack_weight: ld_w smaller than N/8");
    const int64_t total = K * (N / 8);
    w4a16_unpack_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint8_t *>(packed), N, K, p_blocks_k(K), weight, ld_w);
    QMM_CUDA_OK(cudaGetLastError());
    return QMM_OK;
}

extern "C" int qmm_weight_quant_batchmatmul_prepacked_workspace_size(int64_t M, int64_t N, int64_t K, size_t *bytes) {
    using namespace qmm;
    QMM_REQUIRE(bytes != nullptr, "qmm_weight_quant_batchmatmul_prepacked_workspace_size: bytes is NULL");
    QMM_REQUIRE(M >= 0 && N >= 0 && K >= 0, "qmm_weight_quant_batchmatmul_prepacked_workspace_size: negative argument");
    *bytes = 0;
    if (M > 0 && p_shape_ok(N, K, K)) {
        *bytes = kPCounterBytes + p_make_plan(M, N, K).slots_bytes;
        if (M <= kGvMaxM && gv_workspace_bytes(M, N, K) > *bytes) *bytes = gv_workspace_bytes(M, N, K);
    }
    return QMM_OK;
}

extern "C" int qmm_weight_quant_batchmatmul_prepacked(const void *x, int x_dtype, int64_t ld_x, const void *packed,
                                                      size_t packed_bytes, const void *bias, void *out,
                                                      int64_t ld_out, int64_t M, int64_t N, int64_t K,
                                                      void *workspace, size_t workspace_bytes, void *stream) {
    using namespace qmm;
    QMM_REQUIRE(M >= 0, "qmm_weight_quant_batchmatmul_prepacked: negative M");
    QMM_REQUIRE(x_dtype == QMM_DTYPE_BF16 || x_dtype == QMM_DTYPE_F16,
                "qmm_weight_quant_batchmatmul_prepacked: x must be bf16 or f16");
    if (!p_shape_ok(N, K, K))
        return fail(QMM_ERR_UNSUPPORTED, "qmm_weight_quant_batchmatmul_prepacked: needs N % 8 == 0 and K % 128 == 0");
    if (M == 0) return QMM_OK;
    QMM_REQUIRE(x != nullptr && packed != nullptr && out != nullptr, "qmm_weight_quant_batchmatmul_prepacked: NULL operand");
    QMM_REQUIRE(ld_x >= K && ld_out >= N, "qmm_weight_quant_batchmatmul_prepacked: row pitch smaller than the row");
    QMM_REQUIRE(packed_bytes >= p_packed_bytes(N, K),
                "qmm_weight_quant_batchmatmul_prepacked: packed buffer smaller than qmm_w4a16_prepack_size");
    if ((reinterpret_cast<uintptr_t>(x) & 15) || (ld_x & 7) || (reinterpret_cast<uintptr_t>(packed) & 15))
        return fail(QMM_ERR_UNSUPPORTED,
                    "qmm_weight_quant_batchmatmul_prepacked: x and packed need 16-byte aligned addresses and row pitch");
    size_t need = 0;
    qmm_weight_quant_batchmatmul_prepacked_workspace_size(M, N, K, &need);
    if (workspace == nullptr || (reinterpret_cast<uintptr_t>(workspace) & 255) != 0 || workspace_bytes < need)
        return fail(QMM_ERR_WORKSPACE,
                    "qmm_weight_quant_batchmatmul_prepacked: workspace missing, not 256-byte aligned or too small");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (M <= kGvMaxM)  // a handful of tokens: dp4a on the CUDA cores, at the speed of the weight stream
        return (x_dtype == QMM_DTYPE_BF16)
                   ? launch_gemv_t<__nv_bfloat16>(static_cast<const uint8_t *>(packed), x, ld_x, bias, out, ld_out, M, N, K,
                                                  workspace, s)
                   : launch_gemv_t<__half>(static_cast<const uint8_t *>(packed), x, ld_x, bias, out, ld_out, M, N, K,
                                           workspace, s);
    const size_t elt = 2;
    for (int64_t m0 = 0; m0 < M; m0 += kPMaxM) {  // 64 token rows per launch (the accumulator's columns)
        const int64_t mc = (M - m0) < kPMaxM ? (M - m0) : kPMaxM;
        const void *xc = static_cast<const uint8_t *>(x) + static_cast<size_t>(m0) * ld_x * elt;
        void *oc = static_cast<uint8_t *>(out) + static_cast<size_t>(m0) * ld_out * elt;
        const int rc = (x_dtype == QMM_DTYPE_BF16)
                           ? launch_prepacked_t<__nv_bfloat16>(static_cast<const uint8_t *>(packed), xc, ld_x, bias, oc,
                                                               ld_out, mc, N, K, workspace, s)
                           : launch_prepacked_t<__half>(static_cast<const uint8_t *>(packed), xc, ld_x, bias, oc, ld_out,
                                                        mc, N, K, workspace, s);
        if (rc != QMM_OK) return rc;
    }
    return QMM_OK;
}
