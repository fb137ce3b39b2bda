// W4A16 matmul on the tensor cores (npu_weight_quant_batchmatmul, M <= 64 per launch).
//
//   y[m,n] = sum_g scale[g,n] * ( sum_{k in g} x[m,k] * w[k,n]  +  offset[g,n] * sum_{k in g} x[m,k] )
//
// The inner sums run on tcgen05 (kind::f16, fp32 accumulator in TMEM) over the RAW 4-bit
// integers, which are exact in bf16/f16; scale and offset are applied once per group to the
// accumulator, not once per weight.
//
// A work unit is 512 output columns x one quantization group.  512 columns are 256 contiguous
// bytes of a packed weight row: narrower strips (the 64 bytes of a 128-column tile) leave HBM
// with one short burst per DRAM page.  Per 32 k-rows (one step) a CTA
//   1. receives the packed words [32 k][512 n / 8] (8 KiB) by TMA (the activations [M16][64 k]
//      arrive once per 64 k-rows through their own ring),
//   2. turns every packed word into eight 16-bit floats with a handful of logic operations
//      (nibble | exponent bits = BIAS + w; for bf16 BIAS = 136 stays in the operand and is folded
//      into the offset term, for f16 the constant 1032 is subtracted on the spot) and stores
//      them as one 16-byte vector into the MN-major, 128-byte-swizzled A tiles,
//   3. issues eight 128 x M16 x 16 MMAs, two per 128-column sub-tile: weights are the M operand
//      (TMEM lane = output column, so row stores are coalesced), tokens padded to a multiple of
//      16 are the N operand.
// Within a 16-byte vector the columns appear in the order 0,4,1,5,2,6,3,7 (what the logic
// operations produce without a shuffle); the epilogue maps lanes back to columns.
//
// The nibbles of a packed word belong to eight different output columns, while every tensor-core
// operand format keeps consecutive k of ONE column together; the MN-major shared-memory layout is
// what bridges the two.  Its price is shared-memory bandwidth: each weight is written as 2 bytes
// and read back as 2 bytes by the MMA, next to the 0.5 byte that came from HBM, so the kernel is
// bounded by the shared-memory pipe (about 5 bytes per weight at 128 bytes per clock and SM), not
// by HBM.
//
// Warp roles (864 threads): warp 0 TMA producer; warps 1-2 MMA issuers (two sub-tiles each; warp 1
// owns the TMEM allocation); warps 3-10 dequantization (two groups of four warps taking alternate
// steps); warps 11-26 per-group scaling and epilogue (four warps per sub-tile).  Work is cut
// stream-K style into equal contiguous ranges of (column unit, group); a unit shared by several
// CTAs is summed from per-CTA slots in slot order by the last arriver, so results do not depend on
// arrival order.
#include "qmm_common.cuh"
#include "w4a16_simt.cuh"

namespace qmm {

namespace {

constexpr int kWTileN = 128;                 // columns per MMA (its M dimension)
constexpr int kWSub = 4;                     // MMAs side by side
constexpr int kWUnitN = kWTileN * kWSub;     // 512 columns per work unit
constexpr int kWBK = 64;                     // k rows per activation tile: one 128-byte swizzle row
constexpr int kWMmaK = 16;                   // k rows of one MMA
constexpr int kWStepK = 32;                  // k rows per weight stage = two MMAs per sub-tile
constexpr int kWPackedBytes = kWStepK * (kWUnitN / 8) * 4;  // 8 KiB of packed words per step
constexpr int kWAHalfBytes = kWMmaK * kWUnitN * 2;          // 16 KiB of dequantized A per 16 k rows
constexpr int kWABytes = (kWStepK / kWMmaK) * kWAHalfBytes; // 32 KiB per step
constexpr int kWASubBytes = kWAHalfBytes / kWSub;           // 4 KiB per sub-tile and 16 k rows
constexpr int kWABufs = 3;
constexpr int kWStages = 8;                  // packed-weight stages (64 KiB in flight)
constexpr int kWXStages = 4;                 // activation tiles
constexpr int kWMmaWarps = 2;                // each issues the MMAs of kWSub / kWMmaWarps sub-tiles
constexpr int kWSubPerMma = kWSub / kWMmaWarps;
constexpr int kWDeqGroups = 2;               // groups of dequantization warps taking alternate steps
constexpr int kWDeqWarpsPerStep = 4;         // eight k rows of a step each
constexpr int kWDeqWarps = kWDeqGroups * kWDeqWarpsPerStep;
constexpr int kWEpiWarps = 16;
constexpr int kWDeqFirstWarp = 1 + kWMmaWarps;
constexpr int kWEpiFirstWarp = kWDeqFirstWarp + kWDeqWarps;
constexpr int kWThreads = (kWEpiFirstWarp + kWEpiWarps) * 32;  // 864
constexpr int kWMaxM = 64;
constexpr int kWAccBufs = 2;                 // group accumulators in flight
constexpr uint32_t kWTmemCols = 512;        // 2 buffers x 4 sub-tiles x up to 64 columns
constexpr size_t kWXsSmemBytes = 16 * 1024;  // shared copy of the group sums of x
constexpr size_t kWCounterBytes = 64 * 1024;  // unit counters: a fixed area at the start of the scratch

struct WSmemTail {
    uint64_t full[kWStages];
    uint64_t empty[kWStages];
    uint64_t x_full[kWXStages];
    uint64_t x_empty[kWXStages];
    uint64_t a_full[kWABufs];
    uint64_t a_empty[kWABufs];
    uint64_t tmem_full[kWAccBufs];
    uint64_t tmem_empty[kWAccBufs];
    uint32_t tmem_base;
    uint32_t abort_flag;
    uint32_t is_last;
    uint32_t epi_abort;
};

struct WTcParams {
    W4Params w;
    int mpad;            // M rounded up to 16
    int x_bytes;         // mpad * 128: one activation tile
    int units_n;         // 512-column units along N
    int ngroups;
    int steps_per_group; // group / 32
    int max_slots;
    int xs_in_smem;      // the group sums fit the shared-memory area reserved for them
    const float *xsum;   // [ngroups][64]: sum over the group's k of x[m,k]
    float *slots;        // [units_n][max_slots][4][mpad][128]
    uint32_t *counters;  // [units_n], zero between calls
    uint32_t *status;
};

__device__ __forceinline__ void wepi_bar_sync() { asm volatile("bar.sync 2, 512;" ::: "memory"); }

// CTA whose contiguous unit range [total*b/G, total*(b+1)/G) contains unit u
__device__ __forceinline__ int cta_of_unit(int64_t u, int64_t total, int64_t G) {
    return static_cast<int>((u * G + G - 1) / total);
}

template <typename T>
struct W4Magic;
template <>
struct W4Magic<__nv_bfloat16> {
    static constexpr uint32_t kExp = 0x43004300u;  // 128.0 in both halves: 128 + nibble
    static constexpr float kBias = 136.0f;         // 128 + 8 (nibbles are offset-binary after ^8)
    static constexpr uint32_t kFmt = 1;            // instruction-descriptor format code: bf16
    // the operand keeps the constant: BIAS + w; the epilogue's offset term removes it
    static __device__ __forceinline__ uint32_t finish(uint32_t v) { return v; }
};
template <>
struct W4Magic<__half> {
    static constexpr uint32_t kExp = 0x64006400u;  // 1024.0: 1024 + nibble
    static constexpr float kBias = 0.0f;           // removed right away (below): the operand is w itself
    static constexpr uint32_t kFmt = 0;            // f16
    // f16 outputs are held to 2^-11: a constant of 1032 in the operand would cost accuracy through
    // cancellation in long groups, so it is subtracted exactly (1024 + u - 1032 is representable)
    static __device__ __forceinline__ uint32_t finish(uint32_t v) {
        const __half2 r = __hsub2(*reinterpret_cast<const __half2 *>(&v), __floats2half2_rn(1032.0f, 1032.0f));
        return *reinterpret_cast<const uint32_t *>(&r);
    }
};

// Sum over each group's k of x[m,k], fp32, fixed order: xsum[g][m] (row pitch 64).
template <typename T>
__global__ void __launch_bounds__(128)
w4a16_xsum_kernel(const T *__restrict__ x, int64_t ld_x, int M, int64_t group, float *__restrict__ xsum) {
    const int g = blockIdx.x;
    const int m = blockIdx.y;
    __shared__ float part[4];
    float s = 0.0f;
    const T *row = x + static_cast<int64_t>(m) * ld_x + static_cast<int64_t>(g) * group;
    for (int64_t k = threadIdx.x; k < group; k += 128) s += to_float(row[k]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = s;
    __syncthreads();
    if (threadIdx.x == 0 && m < M) xsum[g * kWMaxM + m] = (part[0] + part[1]) + (part[2] + part[3]);
}

}  // namespace
}  // namespace qmm

#include "w4a16_tc_kernel.inl"

namespace qmm {

namespace {

struct WTcPlan {
    int mpad, units_n, ngroups, steps_per_group, grid, max_slots;
    size_t counters_bytes, xsum_bytes, slots_bytes;
};

WTcPlan make_plan(int64_t M, int64_t N, int64_t K, int64_t group) {
    WTcPlan pl;
    const int64_t m = M < kWMaxM ? M : kWMaxM;
    pl.mpad = static_cast<int>((m + 15) / 16 * 16);
    pl.units_n = static_cast<int>((N + kWUnitN - 1) / kWUnitN);
    pl.ngroups = static_cast<int>(K / group);
    pl.steps_per_group = static_cast<int>(group / kWStepK);
    const int64_t total = static_cast<int64_t>(pl.units_n) * pl.ngroups;
    pl.grid = static_cast<int>(total < sm_count() ? total : sm_count());
    const int64_t upc = total / pl.grid;  // units per CTA, rounded down (>= 1)
    pl.max_slots = static_cast<int>((pl.ngroups + upc - 1) / upc + 1);
    // The counters are the only part that must be zero between calls.  They own a fixed area at the
    // start of the scratch, so that no other shape's sums ever land where a later call expects zeros.
    pl.counters_bytes = kWCounterBytes;
    pl.xsum_bytes = static_cast<size_t>(pl.ngroups) * kWMaxM * sizeof(float);
    pl.slots_bytes = static_cast<size_t>(pl.units_n) * pl.max_slots * kWSub * pl.mpad * kWTileN * sizeof(float);
    return pl;
}

template <typename T>
int launch_w4a16_tc_t(const W4Params &w, void *workspace, cudaStream_t stream) {
    const WTcPlan pl = make_plan(w.M, w.N, w.K, w.group);
    WTcParams p;
    p.w = w;
    p.mpad = pl.mpad;
    p.x_bytes = pl.mpad * 128;
    p.xs_in_smem = (static_cast<size_t>(pl.ngroups) * pl.mpad * sizeof(float) <= kWXsSmemBytes) ? 1 : 0;
    p.units_n = pl.units_n;
    p.ngroups = pl.ngroups;
    p.steps_per_group = pl.steps_per_group;
    p.max_slots = pl.max_slots;
    uint8_t *ws = static_cast<uint8_t *>(workspace);
    p.counters = reinterpret_cast<uint32_t *>(ws);
    float *xsum = reinterpret_cast<float *>(ws + pl.counters_bytes);
    p.xsum = xsum;
    p.slots = reinterpret_cast<float *>(ws + pl.counters_bytes + pl.xsum_bytes);
    p.status = device_status_word();

    CUtensorMap tw, tx;
    int rc = make_tmap_2d(&tw, w.w, 4, static_cast<uint64_t>(w.N / 8), static_cast<uint64_t>(w.K),
                          static_cast<uint64_t>(w.ld_w), kWUnitN / 8, kWStepK, false);
    if (rc != QMM_OK) return rc;
    rc = make_tmap_2d(&tx, w.x, 2, static_cast<uint64_t>(w.K), static_cast<uint64_t>(w.M),
                      static_cast<uint64_t>(w.ld_x), kWBK, static_cast<uint32_t>(pl.mpad), true);
    if (rc != QMM_OK) return rc;

    w4a16_xsum_kernel<T><<<dim3(pl.ngroups, static_cast<unsigned>(w.M)), 128, 0, stream>>>(
        static_cast<const T *>(w.x), w.ld_x, static_cast<int>(w.M), w.group, xsum);
    QMM_CUDA_OK(cudaGetLastError());

    const size_t smem = 1024 + kWABufs * kWABytes + kWStages * kWPackedBytes +
                        static_cast<size_t>(kWXStages) * p.x_bytes + sizeof(WSmemTail) + kWXsSmemBytes;
    auto kern = pl.mpad <= 32 ? w4a16_tc_kernel<T, 32> : w4a16_tc_kernel<T, 64>;
    QMM_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    kern<<<pl.grid, kWThreads, smem, stream>>>(tw, tx, p);
    QMM_CUDA_OK(cudaGetLastError());
    return QMM_OK;
}

}  // namespace

bool w4a16_tc_supported(const W4Params &p, int x_dtype) {
    (void)x_dtype;
    if (p.K <= 0 || p.M <= 0) return false;
    if (p.group % kWBK != 0) return false;
    if ((reinterpret_cast<uintptr_t>(p.x) & 15) || (p.ld_x & 7)) return false;
    if ((reinterpret_cast<uintptr_t>(p.w) & 15) || (p.ld_w & 3)) return false;
    if ((p.N + kWUnitN - 1) / kWUnitN > static_cast<int64_t>(kWCounterBytes / 4)) return false;
    return p.K < (1ll << 31) && p.N < (1ll << 31);
}

size_t w4a16_tc_workspace_bytes(int64_t M, int64_t N, int64_t K, int64_t group) {
    if (M <= 0 || N <= 0 || K <= 0 || group <= 0 || group % kWBK != 0 || K % group != 0) return 0;
    const WTcPlan pl = make_plan(M, N, K, group);
    return pl.counters_bytes + pl.xsum_bytes + pl.slots_bytes;
}

// M is processed in chunks of 64 token rows (the accumulator of one launch holds 64 columns).
int launch_w4a16_tc(const W4Params &p, int x_dtype, void *workspace, cudaStream_t stream) {
    const size_t elt = 2;
    for (int64_t m0 = 0; m0 < p.M; m0 += kWMaxM) {
        W4Params c = p;
        c.M = (p.M - m0) < kWMaxM ? (p.M - m0) : kWMaxM;
        c.x = static_cast<const uint8_t *>(p.x) + static_cast<size_t>(m0) * p.ld_x * elt;
        c.out = static_cast<uint8_t *>(p.out) + static_cast<size_t>(m0) * p.ld_out * elt;
        int rc = (x_dtype == QMM_DTYPE_BF16) ? launch_w4a16_tc_t<__nv_bfloat16>(c, workspace, stream)
                                             : launch_w4a16_tc_t<__half>(c, workspace, stream);
        if (rc != QMM_OK) return rc;
    }
    return QMM_OK;
}

}  // namespace qmm
