// Shared device helpers for the sm_100a kernels: mbarrier, TMA, tcgen05/TMEM
// wrappers (inline PTX), bounded waits and the host-side error plumbing.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>

#include "qmm_b200.h"

namespace qmm {

// ---------------------------------------------------------------------------
// Host side: error text + status helpers
// ---------------------------------------------------------------------------
void set_last_error(const std::string &msg);
int fail(int code, const std::string &msg);

#define QMM_CUDA_OK(expr)                                                                   \
    do {                                                                                    \
        cudaError_t _e = (expr);                                                            \
        if (_e != cudaSuccess) {                                                            \
            return ::qmm::fail(QMM_ERR_CUDA, std::string(#expr) + ": " + cudaGetErrorString(_e)); \
        }                                                                                   \
    } while (0)

#define QMM_REQUIRE(cond, msg)                                              \
    do {                                                                    \
        if (!(cond)) return ::qmm::fail(QMM_ERR_INVALID_ARGUMENT, (msg));   \
    } while (0)

// Device-visible status word (host-mapped, one per process). Kernels write a
// non-zero code when a bounded wait gives up; see qmm_device_status().
uint32_t *device_status_word();
// Host-side view of that word without creating it (0 if it does not exist yet); `clear` resets it.
uint32_t device_status_peek(bool clear);
// moves whenever a non-zero status word is cleared (see qmm_runtime.cu)
uint64_t device_status_generation();

// Number of SMs of the current device (cached per device).
int sm_count();

// Encode a 2-D tiled tensor map for a row-major byte matrix.
//   inner: contiguous extent (elements), outer: number of rows, ld: row pitch in elements,
//   elem_bytes: 1 or 2 or 4; box_inner/box_outer: tile extents in elements/rows;
//   swizzle128: CU_TENSOR_MAP_SWIZZLE_128B when true (box_inner*elem_bytes must be 128).
int make_tmap_2d(CUtensorMap *map, const void *base, int elem_bytes, uint64_t inner, uint64_t outer,
                 uint64_t ld, uint32_t box_inner, uint32_t box_outer, bool swizzle128);

// ---------------------------------------------------------------------------
// Device side
// ---------------------------------------------------------------------------
#if defined(__CUDACC__)

enum : uint32_t {
    DEV_STATUS_OK = 0,
    DEV_STATUS_WAIT_TIMEOUT = 0x10000,  // low 16 bits: which wait gave up
    DEV_STATUS_SMEM_MISALIGNED = 0x20000,  // dynamic shared memory not 1024-byte aligned: kernel did nothing
};

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint64_t globaltimer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_fence_init() {
    // make the inits visible to the async proxy (TMA, tcgen05.commit)
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

// Wait limit for every device-side spin: two seconds of wall clock.
constexpr uint64_t kWaitLimitNs = 2000000000ull;

// Bounded wait on an mbarrier phase.  Returns false when the wait gave up or
// when another thread of the CTA already did (abort flag in shared memory);
// the caller then leaves its loop and falls through to the common teardown.
// The slow path is kept out of line so that the hot loops carry one try_wait and one branch.
static __device__ __noinline__ bool mbar_wait_slow(uint32_t bar, uint32_t parity, volatile uint32_t *abort_flag,
                                            uint32_t where) {
    const uint64_t t0 = globaltimer_ns();
    uint32_t spins = 0;
    while (true) {
        if (mbar_try_wait(bar, parity)) return true;
        if (((++spins) & 0xffu) == 0) {
            if (*abort_flag != 0) return false;
            if (globaltimer_ns() - t0 > kWaitLimitNs) {
                *abort_flag = DEV_STATUS_WAIT_TIMEOUT | where;
                return false;
            }
        }
    }
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile uint32_t *abort_flag,
                                          uint32_t where) {
    if (mbar_try_wait(bar, parity)) return true;
    return mbar_wait_slow(bar, parity, abort_flag, where);
}

// ---- TMA ------------------------------------------------------------------
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap *m) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}

// 2-D tiled load global -> shared (this CTA), completion on an mbarrier.
// c0 is the innermost coordinate: c0 * element size must be a multiple of 16.
__device__ __forceinline__ void tma_load_2d(uint32_t smem_dst, const CUtensorMap *m, int32_t c0, int32_t c1,
                                            uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar), "r"(c0), "r"(c1)
        : "memory");
}

// 2-D tiled store shared (this CTA) -> global, tracked by the thread's bulk async-group.
// Out-of-range parts of the box are clipped.  c0 * element size must be a multiple of 16
// and no coordinate may be negative.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap *m, uint32_t smem_src, int32_t c0, int32_t c1) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(
                     reinterpret_cast<uint64_t>(m)),
                 "r"(smem_src), "r"(c0), "r"(c1)
                 : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Wait until at most N of this thread's bulk groups still read their shared-memory source.
template <int N>
__device__ __forceinline__ void tma_store_wait_read() {
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N>
__device__ __forceinline__ void tma_store_wait_all() {
    asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}
// Make generic-proxy writes to shared memory visible to the async proxy (TMA).
__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ---- tcgen05 / TMEM ---------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t smem_result, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_result), "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// Arrive on an mbarrier once all tcgen05.mma issued so far by this thread are done.
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
                 : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// D[tmem] (+)= A[smem desc] * B[smem desc], int8 x int8 -> int32.
__device__ __forceinline__ void mma_i8_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t"
        "}\n" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// D[tmem] (+)= A * B, bf16/f16 x bf16/f16 -> fp32.
__device__ __forceinline__ void mma_f16_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                           uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
        "}\n" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// 32 lanes x 32 consecutive 32-bit columns: thread i of the warp receives
// lane (base_lane + i), registers r[0..31] = columns col..col+31.
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_32x16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}

// 32 lanes x 16 consecutive 32-bit columns, registers -> TMEM: thread i of the warp writes lane
// (base_lane + i), r[0..15] = columns col..col+15.  Complete (for this thread) after tmem_st_wait().
__device__ __forceinline__ void tmem_st_32x16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
        "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
__device__ __forceinline__ void tmem_st_wait() {
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// D[tmem] (+)= A[tmem] * B[smem desc], bf16/f16 -> fp32, issued by one elected lane of a converged
// warp.  A lives in tensor memory: row i of the 128-row operand in lane i, two consecutive k per
// 32-bit column (low half = even k), so a K=16 MMA reads eight columns starting at `a_tmem`.
__device__ __forceinline__ void mma_f16_ts_warp(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                                uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p, e;\n\t"
        "elect.sync _|e, 0xffffffff;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "@e tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t"
        "}\n" ::"r"(d_tmem),
        "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// Eight K=16 MMAs of one 128-row block under one election: A = 64 consecutive tensor-memory columns
// starting at `a_tmem` (eight columns per MMA), B = two K-major 128-byte-swizzled boxes of 64 k each
// (`b_lo0`, `b_lo1`: low descriptor halves of the boxes; 32 bytes = +2 per MMA within a box).  The first
// MMA accumulates only if `accumulate` is set, the others always.
__device__ __forceinline__ void mma_f16_ts_warp_x8(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo0, uint32_t b_lo1,
                                                   uint32_t b_hi, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p, e, t;\n\t"
        ".reg .b64 bd;\n\t"
        ".reg .b32 a, bl;\n\t"
        "elect.sync _|e, 0xffffffff;\n\t"
        "setp.ne.b32 p, %6, 0;\n\t"
        "setp.eq.b32 t, 0, 0;\n\t"
        "mov.b64 bd, {%2, %4};\n\t"
        "@e tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], bd, %5, p;\n\t"
        "add.u32 a, %1, 8;\n\t"
        "add.u32 bl, %2, 2;\n\t"
        "mov.b64 bd, {bl, %4};\n\t"
        "@e tcgen05.mma.cta_group::1.kind::f16 [%0], [a], bd, %5, t;\n\t"
        "add.u32 a, %1, 16;\n\t"
        "add.u32 bl, %2, 4;\n\t"
        "mov.b64 bd, {bl, %4};\n\t"
        "@e tcgen05.mma.cta_group::1.kind::f16 [%0], [a], bd, %5, t;\n\t"
        "add.u32 a, %1, 24;\n\t"
        "add.u32 bl, %2, 6;\n\t"
        "mov.b64 bd, {bl, %4};\n\t"
        "@e tcgen05.mma.cta_group::1.kind::f16 [%0], [a], bd, %5, t;\n\t"
        "add.u32 a, %1, 32;\n\t"
        "mov.b64 bd, {%3, %4};\n\t"
        "@e tcgen05.mma.cta_group::1.kind::f16 [%0], [a], bd, %5, t;\n\t"
        "add.u32 a, %1, 40;\n\t"
        "add.u32 bl, %3, 2;\n\t"
        "mov.b64 bd, {bl, %4};\n\t"
        "@e tcgen05.mma.cta_group::1.kind::f16 [%0], [a], bd, %5, t;\n\t"
        "add.u32 a, %1, 48;\n\t"
        "add.u32 bl, %3, 4;\n\t"
        "mov.b64 bd, {bl, %4};\n\t"
        "@e tcgen05.mma.cta_group::1.kind::f16 [%0], [a], bd, %5, t;\n\t"
        "add.u32 a, %1, 56;\n\t"
        "add.u32 bl, %3, 6;\n\t"
        "mov.b64 bd, {bl, %4};\n\t"
        "@e tcgen05.mma.cta_group::1.kind::f16 [%0], [a], bd, %5, t;\n\t"
        "}\n" ::"r"(d_tmem),
        "r"(a_tmem), "r"(b_lo0), "r"(b_lo1), "r"(b_hi), "r"(idesc), "r"(accumulate)
        : "memory");
}

// Untiled bulk copy global -> shared (this CTA), completion bytes counted on an mbarrier.
// Both addresses 16-byte aligned, `bytes` a multiple of 16.
__device__ __forceinline__ void bulk_load_1d(uint32_t smem_dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_dst),
                 "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(bar)
                 : "memory");
}

// ---- CTA pairs (cluster of 2, tcgen05 cta_group::2) ---------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of `local_smem_addr` as seen in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local_smem_addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_smem_addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_bar_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar_addr) : "memory");
}
// TMA load into this CTA's shared memory whose completion bytes are counted on an
// mbarrier of the pair's leader CTA (`cluster_bar_addr`).  No multicast.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t smem_dst, const CUtensorMap *m, int32_t c0, int32_t c1,
                                                 uint32_t cluster_bar_addr) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%3, %4}], [%2];" ::"r"(smem_dst),
        "l"(reinterpret_cast<uint64_t>(m)), "r"(cluster_bar_addr), "r"(c0), "r"(c1)
        : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t smem_result, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_result), "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// 256 x N x 32 MMA over the CTA pair: each CTA supplies 128 rows of A and N/2 columns of B
// from its own shared memory (same offsets in both) and receives 128 rows of D in its TMEM.
__device__ __forceinline__ void mma_i8_ss_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                               uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t"
        "}\n" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Arrive on the mbarrier at this shared-memory offset in every CTA of `cta_mask`
// once all MMAs issued so far by this thread are done.
__device__ __forceinline__ void tc_commit_pair(uint32_t bar, uint16_t cta_mask) {
    asm volatile(
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar),
        "h"(cta_mask)
        : "memory");
}

// Shared-memory matrix descriptor (tcgen05 "version 1").
//   start address, leading and stride byte offsets are stored without their
//   4 LSBs; bits 46-47 = 0b01 (descriptor version of this architecture);
//   bits 61-63 = swizzle mode (2 = 128-byte swizzle).
__host__ __device__ __forceinline__ uint64_t make_smem_desc_sw128(uint32_t smem_addr, uint32_t lbo_bytes,
                                                                  uint32_t sbo_bytes) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr >> 4) & 0x3fff);
    d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3fff) << 16;
    d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3fff) << 32;
    d |= 1ull << 46;
    d |= 2ull << 61;
    return d;
}

// The same descriptor split into its two 32-bit halves.  The high half is a constant of the
// kernel; the low half is (address >> 4) | (lbo >> 4) << 16, so stepping through a tile is one
// 32-bit add.  (Shared-memory addresses are below 256 KiB: address >> 4 fits the 14-bit field.)
__host__ __device__ constexpr uint32_t smem_desc_hi_sw128(uint32_t sbo_bytes) {
    return ((sbo_bytes >> 4) & 0x3fffu) | (1u << 14) | (2u << 29);
}
__host__ __device__ constexpr uint32_t smem_desc_lo(uint32_t smem_addr, uint32_t lbo_bytes) {
    return (smem_addr >> 4) | (((lbo_bytes >> 4) & 0x3fffu) << 16);
}
__device__ __forceinline__ uint64_t desc64(uint32_t lo, uint32_t hi) {
    uint64_t d;
    asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "r"(lo), "r"(hi));
    return d;
}

// Issue forms for a whole, converged warp: every lane executes the call with the same operands and
// elect.sync lets one lane (always the same one) issue.  Operands stay warp-uniform, which keeps the
// issue loop short: a single thread can otherwise spend ~200 cycles per MMA on scalar bookkeeping,
// more than a 128x256x32 MMA takes to execute.
__device__ __forceinline__ void mma_i8_ss_warp(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                               uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p, e;\n\t"
        "elect.sync _|e, 0xffffffff;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "@e tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t"
        "}\n" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void mma_f16_ss_warp(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                                uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p, e;\n\t"
        "elect.sync _|e, 0xffffffff;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "@e tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
        "}\n" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// One 32-row step of two side-by-side accumulators: four MMAs (two k halves for each of d0, d1) and
// the commit that releases the operands, all under one election.  The second k half always accumulates.
__device__ __forceinline__ void mma_f16_ss_warp_2x2_commit(uint32_t d0, uint32_t d1, uint64_t a00, uint64_t a01,
                                                           uint64_t a10, uint64_t a11, uint64_t b0, uint64_t b1,
                                                           uint32_t idesc, uint32_t accumulate, uint32_t bar) {
    asm volatile(
        "{\n\t"
        ".reg .pred p, e, t;\n\t"
        "elect.sync _|e, 0xffffffff;\n\t"
        "setp.ne.b32 p, %9, 0;\n\t"
        "setp.eq.b32 t, 0, 0;\n\t"
        "@e tcgen05.mma.cta_group::1.kind::f16 [%0], %2, %6, %8, p;\n\t"
        "@e tcgen05.mma.cta_group::1.kind::f16 [%1], %4, %6, %8, p;\n\t"
        "@e tcgen05.mma.cta_group::1.kind::f16 [%0], %3, %7, %8, t;\n\t"
        "@e tcgen05.mma.cta_group::1.kind::f16 [%1], %5, %7, %8, t;\n\t"
        "@e tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%10];\n\t"
        "}\n" ::"r"(d0),
        "r"(d1), "l"(a00), "l"(a01), "l"(a10), "l"(a11), "l"(b0), "l"(b1), "r"(idesc), "r"(accumulate), "r"(bar)
        : "memory");
}
__device__ __forceinline__ void mma_i8_ss_pair_warp(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                                    uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p, e;\n\t"
        "elect.sync _|e, 0xffffffff;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "@e tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t"
        "}\n" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void tc_commit_warp(uint32_t bar) {
    asm volatile(
        "{\n\t"
        ".reg .pred e;\n\t"
        "elect.sync _|e, 0xffffffff;\n\t"
        "@e tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t"
        "}\n" ::"r"(bar)
        : "memory");
}
__device__ __forceinline__ void tc_commit_pair_warp(uint32_t bar, uint16_t cta_mask) {
    asm volatile(
        "{\n\t"
        ".reg .pred e;\n\t"
        "elect.sync _|e, 0xffffffff;\n\t"
        "@e tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;\n\t"
        "}\n" ::"r"(bar),
        "h"(cta_mask)
        : "memory");
}

// Instruction descriptor for kind::i8 / kind::f16 (dense, no negate, no saturate).
//   c_format: 1 = f32, 2 = s32;  ab_format: i8 -> 1 (signed); f16 kind -> 0 f16, 1 bf16
//   a_mn_major / b_mn_major: 0 = K-major operand, 1 = MN-major operand
__host__ __device__ constexpr uint32_t make_idesc(uint32_t c_format, uint32_t a_format, uint32_t b_format,
                                                  uint32_t a_mn_major, uint32_t b_mn_major, uint32_t mma_m,
                                                  uint32_t mma_n) {
    return (c_format << 4) | (a_format << 7) | (b_format << 10) | (a_mn_major << 15) | (b_mn_major << 16) |
           ((mma_n >> 3) << 17) | ((mma_m >> 4) << 24);
}

// Typed 2-byte float helpers used by epilogues.
template <typename T>
struct Half2Of;
template <>
struct Half2Of<__nv_bfloat16> {
    using type = __nv_bfloat162;
};
template <>
struct Half2Of<__half> {
    using type = __half2;
};

__device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ float to_float(__half v) { return __half2float(v); }
__device__ __forceinline__ float to_float(float v) { return v; }

template <typename T>
__device__ __forceinline__ T from_float(float v);
template <>
__device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) {
    return __float2bfloat16_rn(v);
}
template <>
__device__ __forceinline__ __half from_float<__half>(float v) {
    return __float2half_rn(v);
}
template <>
__device__ __forceinline__ float from_float<float>(float v) {
    return v;
}

// pack two floats into one 32-bit word of two 16-bit floats (lo = a, hi = b)
template <typename T>
__device__ __forceinline__ uint32_t pack2(float a, float b);
template <>
__device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float a, float b) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t *>(&v);
}
template <>
__device__ __forceinline__ uint32_t pack2<__half>(float a, float b) {
    __half2 v = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t *>(&v);
}

#endif  // __CUDACC__

}  // namespace qmm
