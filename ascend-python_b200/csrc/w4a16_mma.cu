// W4A16 matmul for decode (npu_weight_quant_batchmatmul, M <= 16): the int4 weights are unpacked
// in registers and never expanded in shared memory.
//
//   y[m,n] = sum_g scale[g,n] * ( sum_{k in g} x[m,k] * w[k,n]  +  offset[g,n] * sum_{k in g} x[m,k] )
//
// A packed word holds one k row of EIGHT neighbouring columns, while a tensor-core operand register
// holds TWO neighbouring k of ONE column.  The kernel bridges the two without moving data between
// threads: a thread that holds the words of rows k, k+1 (and k+8, k+9) of word column c feeds
// nibble j of those words to the j-th of eight register-operand MMAs (mma.sync m16n8k16, weights as
// the 16-row operand, up to 8 token rows as the 8-column operand).  MMA j of a warp therefore
// computes the output columns {8 * (c0 + i) + j : i = 0..15} of the warp's sixteen word columns; all
// 8 x 16 = 128 columns of the warp are covered by the eight MMAs, every loaded word is used in full
// and every thread loads distinct words.  Two logic operations extract a pair of nibbles as two
// 16-bit floats (nibble | exponent bits = BIAS + w), one byte permute pairs them along k.
//
// The group sums of x that the offset term needs come from one more MMA per k block whose weight
// operand is all ones, so they see exactly the rows (and the accumulation order) of the main sums.
//
// Roles: warp 0 feeds a ring of 64-row stages by TMA (packed words as two 128-byte-swizzled boxes
// of 32 words, plus the activation tile [8 or 16 tokens][64 k]); the consumer warps form sets of
// four (128 columns per warp) that take the quantization groups of the CTA's range in turn, apply
// scale and offset to the group's accumulator in registers and keep the running output in fp32
// (registers for up to 8 token rows with three sets; one private shared-memory column per thread
// for 9..16 rows with two sets, which is what the register file allows).  Work is cut stream-K
// style into equal contiguous ranges of (512-column unit, group).  Every (CTA, set) writes its
// share of a unit to its own slot; the one that arrives last adds the slots in slot order, so
// results do not depend on arrival order.
//
// The kernel is bounded by the integer/logic pipe (half rate): about one logic operation per weight
// (pairing permutes, shifts, mask-and-flip), not by HBM and not by the tensor pipe.
// QMM_W4_SETS and QMM_W4_YSMEM (1 = registers, 2 = shared memory) override the two choices above
// for tuning.
#include "qmm_common.cuh"
#include "w4a16_simt.cuh"

#include <cstdlib>

namespace qmm {

namespace {

constexpr int kGUnitN = 512;                    // columns per work unit: 64 packed words = 256 B per k row
constexpr int kGStageK = 64;                    // k rows per stage
constexpr int kGStages = 8;
constexpr int kGMaxSets = 4;                    // consumer sets (four warps each) taking the groups in turn
constexpr int kGColWarps = 4;                   // warps side by side, 128 columns each
constexpr int kGBoxBytes = kGStageK * 128;      // 8 KiB: [64 rows][32 words]
constexpr int kGPackedBytes = 2 * kGBoxBytes;   // 16 KiB per stage
constexpr int kGXBytesMax = 2048;               // [16 tokens][64 k] of 16-bit values
constexpr int kGStageBytes = kGPackedBytes + kGXBytesMax;  // 18 KiB, a multiple of 1 KiB
constexpr int kGMaxM = 16;
constexpr size_t kGCounterBytes = 64 * 1024;    // unit counters: a fixed area at the start of the scratch

struct GSmemTail {
    uint64_t full[kGStages];
    uint64_t empty[kGStages];
    uint32_t abort_flag;
    uint32_t is_last[kGMaxSets];
};

struct GParams {
    W4Params w;
    int units_n;
    int ngroups;
    int stages_per_group;  // group / 64
    int max_slots;         // slots per unit (CTAs sharing a unit x sets)
    int nstages;           // stages of the ring actually used (shared memory permitting)
    float *slots;          // [units_n][max_slots][8 * MT][512]
    uint32_t *counters;    // [units_n], zero between calls
    uint32_t *status;
};

__device__ __forceinline__ int g_cta_of_item(int64_t u, int64_t total, int64_t G) {
    return static_cast<int>((u * G + G - 1) / total);
}

__device__ __forceinline__ void set_bar_sync(int set) {
    asm volatile("bar.sync %0, %1;" ::"r"(1 + set), "r"(kGColWarps * 32) : "memory");
}

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
    return r;
}
// (a & b) ^ c in one logic instruction
__device__ __forceinline__ uint32_t and_xor(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("lop3.b32 %0, %1, %2, %3, 0x6a;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

// a constant the compiler cannot fold into immediates
__device__ __forceinline__ uint32_t opaque_u32(uint32_t v) {
    uint32_t r;
    asm volatile("mov.u32 %0, %1;" : "=r"(r) : "r"(v));
    return r;
}

template <typename T>
struct GMagic;
template <>
struct GMagic<__nv_bfloat16> {
    static constexpr uint32_t kExp = 0x43004300u;   // 128.0 in both halves: 128 + nibble
    static constexpr float kBias = 136.0f;          // 128 + 8 (nibbles are offset-binary after ^8)
    static constexpr uint32_t kOnes = 0x3F803F80u;  // 1.0, 1.0
    static __device__ __forceinline__ uint32_t finish(uint32_t v) { return v; }
    static __device__ __forceinline__ void mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
        asm(
            "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
            "{%0,%1,%2,%3};"
            : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
            : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    }
};
template <>
struct GMagic<__half> {
    static constexpr uint32_t kExp = 0x64006400u;   // 1024.0: 1024 + nibble
    static constexpr float kBias = 0.0f;            // removed on the spot: the operand is w itself
    static constexpr uint32_t kOnes = 0x3C003C00u;
    // 1024 + u - 1032 is exact in f16; keeping the constant would cost accuracy in long groups
    static __device__ __forceinline__ uint32_t finish(uint32_t v) {
        const __half2 r = __hsub2(*reinterpret_cast<const __half2 *>(&v), __floats2half2_rn(1032.0f, 1032.0f));
        return *reinterpret_cast<const uint32_t *>(&r);
    }
    static __device__ __forceinline__ void mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
        asm(
            "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
            "{%0,%1,%2,%3};"
            : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
            : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    }
};

// eight 16-bit values of a row of scale / offset as floats
template <typename T>
__device__ __forceinline__ void unpack8(const uint4 &v, float (&f)[8]) {
    const T *h = reinterpret_cast<const T *>(&v);
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] = to_float(h[j]);
}

}  // namespace
}  // namespace qmm

#include "w4a16_mma_kernel.inl"

namespace qmm {

namespace {

struct GPlan {
    int mt, sets, units_n, ngroups, stages_per_group, grid, max_slots;
    size_t slots_bytes;
};

int g_env_int(const char *name) {
    const char *e = std::getenv(name);
    return e ? std::atoi(e) : 0;
}

// Whether the running outputs are kept in shared memory (frees 32 registers per token tile).
bool g_outputs_in_smem(int mt) {
    static const int forced = g_env_int("QMM_W4_YSMEM");  // 1: registers, 2: shared memory
    if (forced == 1) return false;
    if (forced == 2) return true;
    return mt == 2;
}

// Consumer sets per CTA: as many as the register file allows.
int g_sets_for(int mt) {
    static const int forced = g_env_int("QMM_W4_SETS");
    const bool ys = g_outputs_in_smem(mt);
    const int lo = 2, hi = mt == 1 ? (ys ? 4 : 3) : (ys ? 3 : 2);  // bounded by registers and by shared memory
    if (forced >= lo && forced <= hi) return forced;
    return mt == 1 ? 3 : 2;
}

GPlan g_make_plan(int64_t M, int64_t N, int64_t K, int64_t group) {
    GPlan pl;
    pl.mt = M <= 8 ? 1 : 2;
    pl.sets = g_sets_for(pl.mt);
    pl.units_n = static_cast<int>((N + kGUnitN - 1) / kGUnitN);
    pl.ngroups = static_cast<int>(K / group);
    pl.stages_per_group = static_cast<int>(group / kGStageK);
    const int64_t total = static_cast<int64_t>(pl.units_n) * pl.ngroups;
    pl.grid = static_cast<int>(total < sm_count() ? total : sm_count());
    const int64_t ipc = total / pl.grid;  // items per CTA, rounded down (>= 1)
    pl.max_slots = static_cast<int>(((pl.ngroups + ipc - 1) / ipc + 1) * pl.sets);
    pl.slots_bytes = static_cast<size_t>(pl.units_n) * pl.max_slots * (8 * pl.mt) * kGUnitN * sizeof(float);
    return pl;
}

template <typename T>
int launch_w4a16_mma_t(const W4Params &w, void *workspace, cudaStream_t stream) {
    const GPlan pl = g_make_plan(w.M, w.N, w.K, w.group);
    GParams p;
    p.w = w;
    p.units_n = pl.units_n;
    p.ngroups = pl.ngroups;
    p.stages_per_group = pl.stages_per_group;
    p.max_slots = pl.max_slots;
    uint8_t *ws = static_cast<uint8_t *>(workspace);
    p.counters = reinterpret_cast<uint32_t *>(ws);
    p.slots = reinterpret_cast<float *>(ws + kGCounterBytes);
    p.status = device_status_word();

    CUtensorMap tw, tx;
    int rc = make_tmap_2d(&tw, w.w, 4, static_cast<uint64_t>(w.N / 8), static_cast<uint64_t>(w.K),
                          static_cast<uint64_t>(w.ld_w), 32, kGStageK, true);
    if (rc != QMM_OK) return rc;
    rc = make_tmap_2d(&tx, w.x, 2, static_cast<uint64_t>(w.K), static_cast<uint64_t>(w.M),
                      static_cast<uint64_t>(w.ld_x), kGStageK, static_cast<uint32_t>(8 * pl.mt), true);
    if (rc != QMM_OK) return rc;

    // stages, 1 KiB for the barriers, then (optionally) the running outputs of every consumer thread;
    // the ring gives up stages when the outputs need the room
    const bool ys = g_outputs_in_smem(pl.mt);
    static_assert(sizeof(GSmemTail) <= 1024, "the tail has 1 KiB");
    const size_t ys_bytes = ys ? static_cast<size_t>(32 * pl.mt) * pl.sets * kGColWarps * 32 * sizeof(float) : 0;
    int nstages = kGStages;
    while (nstages > 4 && 1024 + static_cast<size_t>(nstages) * kGStageBytes + 1024 + ys_bytes > 232448) --nstages;
    p.nstages = nstages;
    const size_t smem = 1024 + static_cast<size_t>(nstages) * kGStageBytes + 1024 + ys_bytes;
    void (*kern)(CUtensorMap, CUtensorMap, GParams) = nullptr;
    if (pl.mt == 1) {
        if (ys)
            kern = pl.sets == 4 ? w4a16_mma_kernel<T, 1, 4, true> : pl.sets == 3 ? w4a16_mma_kernel<T, 1, 3, true>
                                                                                 : w4a16_mma_kernel<T, 1, 2, true>;
        else
            kern = pl.sets == 3 ? w4a16_mma_kernel<T, 1, 3, false> : w4a16_mma_kernel<T, 1, 2, false>;
    } else {
        if (ys)
            kern = pl.sets == 3 ? w4a16_mma_kernel<T, 2, 3, true> : w4a16_mma_kernel<T, 2, 2, true>;
        else
            kern = w4a16_mma_kernel<T, 2, 2, false>;
    }
    QMM_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    kern<<<pl.grid, (1 + pl.sets * kGColWarps) * 32, smem, stream>>>(tw, tx, p);
    QMM_CUDA_OK(cudaGetLastError());
    return QMM_OK;
}

}  // namespace

bool w4a16_mma_supported(const W4Params &p, int x_dtype) {
    (void)x_dtype;
    if (p.K <= 0 || p.M <= 0 || p.M > kGMaxM) return false;
    if (p.group % kGStageK != 0) return false;
    if ((reinterpret_cast<uintptr_t>(p.x) & 15) || (p.ld_x & 7)) return false;
    if ((reinterpret_cast<uintptr_t>(p.w) & 15) || (p.ld_w & 3)) return false;
    if ((reinterpret_cast<uintptr_t>(p.scale) & 15) || (reinterpret_cast<uintptr_t>(p.offset) & 15)) return false;
    if ((reinterpret_cast<uintptr_t>(p.out) & 15) || (p.ld_out & 7)) return false;
    if ((p.N + kGUnitN - 1) / kGUnitN > static_cast<int64_t>(kGCounterBytes / 4)) return false;
    return p.K < (1ll << 31) && p.N < (1ll << 31);
}

size_t w4a16_mma_workspace_bytes(int64_t M, int64_t N, int64_t K, int64_t group) {
    if (M <= 0 || M > kGMaxM || N <= 0 || K <= 0 || group <= 0 || group % kGStageK != 0 || K % group != 0) return 0;
    return kGCounterBytes + g_make_plan(M, N, K, group).slots_bytes;
}

int launch_w4a16_mma(const W4Params &p, int x_dtype, void *workspace, cudaStream_t stream) {
    return (x_dtype == QMM_DTYPE_BF16) ? launch_w4a16_mma_t<__nv_bfloat16>(p, workspace, stream)
                                       : launch_w4a16_mma_t<__half>(p, workspace, stream);
}

}  // namespace qmm
