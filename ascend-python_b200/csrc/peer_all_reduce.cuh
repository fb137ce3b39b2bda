// Allreduce over peer memory for the row-parallel matmul (npu_mm_all_reduce_base): one kernel per
// rank that reduce-scatters and all-gathers the ranks' partial outputs through NVLink loads.
//
// Every rank owns a region of the same size that all ranks of the node have mapped (peer
// pointers).  Layout of a region: 64 KiB of flags, the rank's partial output [M][N] (written by the
// matmul kernel that ran just before on the same stream), the reduced output [M][N] (a rank fills
// the rows it owns; with multicast, everybody's rows).
//
// The CTA-pair matmul can deliver its output tiles straight into the owners' regions (TMA stores to
// peer memory from its epilogue), which moves the reduce-scatter traffic under the matmul; step 2
// then reads local memory only.  Otherwise the partial stays in the producing rank's region.
//
//   1. the kernel tells every peer "my partial is complete" (flag A) and waits for theirs;
//   2. rank r owns rows [r * rows_per, (r+1) * rows_per): it loads those rows of all W partials
//      (its own from HBM, the others over NVLink), adds them in fp32 in rank order - so the result
//      does not depend on timing - rounds once, writes them to the output and to its region, and
//      raises flag B[chunk] at every peer chunk by chunk;
//   3. every rank copies the other ranks' reduced rows into its output as their flags arrive.
//
// Where the regions are also mapped through an NVLink multicast object (NVSwitch), step 2 loads the
// sum of the W partials with one multimem.ld_reduce (added inside the switch, fp32 accumulation) and
// broadcasts the reduced rows into every rank's region with one multimem.st, so step 3 copies from
// the rank's own region: each byte then crosses a link once per direction instead of twice.
//
// The kernels of different ranks wait on one another only across GPUs; within a GPU no CTA waits on
// another CTA, and the grid is one CTA per SM, so every CTA is resident.  Every wait is
// bounded (2 s): on expiry the kernel records a status code and leaves without touching peer data
// again.  Flags carry the call's epoch, which only grows, so they are never reset.
//
// Buffer reuse across calls needs no extra synchronisation: a rank finishes step 3 only after all
// peers have raised all their B flags, i.e. after they are done reading the partial halves (its own, or
// - with pushed tiles - the one its next matmul will write into); and it overwrites the reduced half in
// the next call only after all peers have raised the next A flag, i.e. after their previous kernel,
// which read that half, has ended.  Partial data never lands in a reduced half or the other way round,
// whatever M and N the next call has.
#pragma once

#include "qmm_common.cuh"

namespace qmm {

constexpr int kPeerMaxRanks = 8;
constexpr int kPeerChunks = 592;                  // most chunks a rank's rows are cut into (size of a flag row)
constexpr size_t kPeerChunkBytes = 64 * 1024;     // aimed-at chunk size: enough loads in flight per CTA to hide
                                                  // the NVLink round trip, few enough flag operations
constexpr size_t kPeerFlagBytes = 64 * 1024;      // flag A: [W] at 0; flag B: [W][kPeerChunks] at 1 KiB
constexpr size_t kPeerFlagBOffset = 1024;
constexpr int kPeerThreads = 512;
constexpr uint32_t DEV_STATUS_PEER_TIMEOUT = 0x30000;

struct PeerParams {
    uint8_t *base[kPeerMaxRanks];  // every rank's region as mapped here (own region included)
    uint8_t *mc_base;              // the regions through the multicast mapping, or nullptr
    int world, rank;
    uint32_t epoch;
    int64_t M, N;
    int64_t rows_per;              // rows owned by a rank (the last owner may hold fewer)
    int nchunks;                   // chunks a rank's rows are cut into (<= kPeerChunks)
    int pushed;                    // the matmul already delivered every rank's share of the rows this rank owns
                                   // into this rank's region: [source rank][rows_per][N] in the partial area
    size_t partial_off, red_off;   // byte offsets of the two data areas inside a region
    void *out;                     // [M][N], this rank's result
    uint32_t *status;
    uint32_t status_at_launch;     // value of *status when the host launched this kernel: only a CHANGE aborts a wait
};

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t *p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t *p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Waits until *flag has reached `epoch` (epochs only grow; the difference is taken modulo 2^32).
// The poll backs off with nanosleep: hundreds of CTAs polling at full speed (system-scope loads, plus
// reads of the host-mapped status word) were measured to slow the very transfers they wait for by
// several times.
// A wait also gives up when the process-wide status word changes while it polls (some kernel of this process
// recorded a timeout): compared with the value at launch, so that an old, unread code does not abort later calls.
static __device__ __noinline__ bool peer_wait_flag(const uint32_t *flag, uint32_t epoch, uint32_t *status, uint32_t status0,
                                            uint32_t where) {
    if (static_cast<int32_t>(ld_acquire_sys(flag) - epoch) >= 0) return true;
    const uint64_t t0 = globaltimer_ns();
    uint32_t spins = 0;
    while (true) {
        __nanosleep(spins < 16 ? 100 : 400);
        if (static_cast<int32_t>(ld_acquire_sys(flag) - epoch) >= 0) return true;
        if (((++spins) & 0xfffu) == 0) {  // every millisecond or two
            if (status != nullptr && *reinterpret_cast<volatile uint32_t *>(status) != status0) return false;
            if (globaltimer_ns() - t0 > kWaitLimitNs) {
                if (status != nullptr) atomicMax(status, DEV_STATUS_PEER_TIMEOUT | where);
                return false;
            }
        }
    }
}

// sum over all ranks of the 16 bytes at the same offset of every region (fp32 accumulation in the switch)
template <typename T>
__device__ __forceinline__ uint4 multimem_ld_reduce(const uint8_t *mc_addr);
template <>
__device__ __forceinline__ uint4 multimem_ld_reduce<__nv_bfloat16>(const uint8_t *mc_addr) {
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(mc_addr)
                 : "memory");
    return v;
}
template <>
__device__ __forceinline__ uint4 multimem_ld_reduce<__half>(const uint8_t *mc_addr) {
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(mc_addr)
                 : "memory");
    return v;
}
// 16 bytes to the same offset of every region
__device__ __forceinline__ void multimem_st(uint8_t *mc_addr, const uint4 &v) {
    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(mc_addr), "r"(v.x), "r"(v.y),
                 "r"(v.z), "r"(v.w)
                 : "memory");
}

template <typename T>
__device__ __forceinline__ void accumulate8(const uint4 &v, float (&acc)[8]) {
    const T *h = reinterpret_cast<const T *>(&v);
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] += to_float(h[j]);
}

// vectors (16 bytes = 8 elements) of chunk c of a range of `total` vectors
__device__ __forceinline__ void chunk_bounds(int64_t total, int c, int nchunks, int64_t &lo, int64_t &hi) {
    lo = total * c / nchunks;
    hi = total * (c + 1) / nchunks;
}

// Sum of the ranks' shares of the vectors [lo, hi) of this rank's rows, in rank order; WW: ranks rounded
// up (2, 4, 8), U: vectors per thread and pass.
template <typename T, bool MC, int WW, int U>
__device__ __forceinline__ void reduce_chunk(const PeerParams &p, int64_t lo, int64_t hi, size_t own_byte0, uint4 *red,
                                             uint4 *out_own) {
    const int W = p.world;
    for (int64_t v0 = lo + threadIdx.x; v0 < hi; v0 += U * kPeerThreads) {
        uint4 part[U][WW];
#pragma unroll
        for (int u = 0; u < U; ++u)
#pragma unroll
            for (int r = 0; r < WW; ++r)
                if (r < W && v0 + u * kPeerThreads < hi) {
                    const uint8_t *src = p.pushed ? p.base[p.rank] + p.partial_off +
                                                        static_cast<size_t>(r) * p.rows_per * p.N * sizeof(T)
                                                  : p.base[r] + p.partial_off + own_byte0;
                    part[u][r] = __ldcg(reinterpret_cast<const uint4 *>(src) + v0 + u * kPeerThreads);
                }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int64_t v = v0 + u * kPeerThreads;
            if (v < hi) {
                float acc[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[j] = 0.0f;
#pragma unroll
                for (int r = 0; r < WW; ++r)
                    if (r < W) accumulate8<T>(part[u][r], acc);
                uint4 o;
                o.x = pack2<T>(acc[0], acc[1]);
                o.y = pack2<T>(acc[2], acc[3]);
                o.z = pack2<T>(acc[4], acc[5]);
                o.w = pack2<T>(acc[6], acc[7]);
                if constexpr (MC)
                    multimem_st(p.mc_base + p.red_off + own_byte0 + v * 16, o);
                else
                    red[v] = o;
                out_own[v] = o;
            }
        }
    }
}

// MC: the regions have a multicast mapping (p.mc_base)
template <typename T, bool MC>
__global__ void __launch_bounds__(kPeerThreads, 1) peer_all_reduce_kernel(PeerParams p) {
    __shared__ int s_ok;
    const int W = p.world;
    uint32_t *my_flags = reinterpret_cast<uint32_t *>(p.base[p.rank]);

    // ---- 1. partials complete: tell every rank, wait for every rank ----
    if (blockIdx.x == 0 && threadIdx.x < W) {
        __threadfence_system();
        st_release_sys(reinterpret_cast<uint32_t *>(p.base[threadIdx.x]) + p.rank, p.epoch);
    }
    if (threadIdx.x == 0) s_ok = 1;
    __syncthreads();
    if (threadIdx.x < W) {
        if (!peer_wait_flag(my_flags + threadIdx.x, p.epoch, p.status, p.status_at_launch, 0x01)) s_ok = 0;
    }
    __syncthreads();
    if (!s_ok) return;

    // ---- 2. reduce the rows this rank owns ----
    const int64_t vec_per_row = p.N / 8;
    const int64_t r0 = static_cast<int64_t>(p.rank) * p.rows_per;
    const int64_t r1 = (r0 + p.rows_per < p.M) ? r0 + p.rows_per : p.M;
    const int64_t own_vecs = (r1 > r0 ? (r1 - r0) : 0) * vec_per_row;
    const size_t own_byte0 = static_cast<size_t>(r0) * p.N * sizeof(T);
    uint4 *red = reinterpret_cast<uint4 *>(p.base[p.rank] + p.red_off + own_byte0);
    uint4 *out_own = reinterpret_cast<uint4 *>(static_cast<uint8_t *>(p.out) + own_byte0);
    for (int c = blockIdx.x; c < p.nchunks; c += gridDim.x) {
        int64_t lo, hi;
        chunk_bounds(own_vecs, c, p.nchunks, lo, hi);
        if (MC && !p.pushed) {
            const uint8_t *mc_part = p.mc_base + p.partial_off + own_byte0;
            uint8_t *mc_red = p.mc_base + p.red_off + own_byte0;
            // four vectors per thread and pass, so that enough loads are in flight for the link latency
            for (int64_t v0 = lo + threadIdx.x; v0 < hi; v0 += 4 * kPeerThreads) {
                uint4 o[4];
#pragma unroll
                for (int u = 0; u < 4; ++u)
                    if (v0 + u * kPeerThreads < hi) o[u] = multimem_ld_reduce<T>(mc_part + (v0 + u * kPeerThreads) * 16);
#pragma unroll
                for (int u = 0; u < 4; ++u)
                    if (v0 + u * kPeerThreads < hi) {
                        out_own[v0 + u * kPeerThreads] = o[u];
                        multimem_st(mc_red + (v0 + u * kPeerThreads) * 16, o[u]);
                    }
            }
        } else {
            // eight 16-byte loads per thread are in flight: U vectors x W ranks
            if (W <= 2)
                reduce_chunk<T, MC, 2, 4>(p, lo, hi, own_byte0, red, out_own);
            else if (W <= 4)
                reduce_chunk<T, MC, 4, 2>(p, lo, hi, own_byte0, red, out_own);
            else
                reduce_chunk<T, MC, 8, 1>(p, lo, hi, own_byte0, red, out_own);
        }
        __syncthreads();
        if (threadIdx.x < W && static_cast<int>(threadIdx.x) != p.rank) {
            __threadfence_system();
            uint32_t *peer_b = reinterpret_cast<uint32_t *>(p.base[threadIdx.x] + kPeerFlagBOffset);
            st_release_sys(peer_b + static_cast<size_t>(p.rank) * kPeerChunks + c, p.epoch);
        }
    }

    // ---- 3. gather the other ranks' rows as they become ready ----
    const uint32_t *my_b = reinterpret_cast<const uint32_t *>(p.base[p.rank] + kPeerFlagBOffset);
    const int items = (W - 1) * p.nchunks;
    for (int i = blockIdx.x; i < items; i += gridDim.x) {
        // consecutive CTAs read from different ranks, every rank starting with its right-hand neighbour
        const int src = (p.rank + 1 + i % (W - 1)) % W;
        const int c = i / (W - 1);
        const int64_t s0 = static_cast<int64_t>(src) * p.rows_per;
        const int64_t s1 = (s0 + p.rows_per < p.M) ? s0 + p.rows_per : p.M;
        const int64_t src_vecs = (s1 > s0 ? (s1 - s0) : 0) * vec_per_row;
        int64_t lo, hi;
        chunk_bounds(src_vecs, c, p.nchunks, lo, hi);
        __syncthreads();  // s_ok of the previous item has been read by everyone
        if (threadIdx.x == 0)
            s_ok = peer_wait_flag(my_b + static_cast<size_t>(src) * kPeerChunks + c, p.epoch, p.status, p.status_at_launch,
                                  0x02) ? 1 : 0;
        __syncthreads();
        if (!s_ok) return;
        // reduced rows of `src`: in its region, or (multicast) already in this rank's own region
        const size_t src_byte0 = static_cast<size_t>(s0) * p.N * sizeof(T);
        const uint4 *from = reinterpret_cast<const uint4 *>(p.base[MC ? p.rank : src] + p.red_off + src_byte0);
        uint4 *to = reinterpret_cast<uint4 *>(static_cast<uint8_t *>(p.out) + src_byte0);
        for (int64_t v0 = lo + threadIdx.x; v0 < hi; v0 += 4 * kPeerThreads) {
            uint4 tmp[4];
#pragma unroll
            for (int u = 0; u < 4; ++u)
                if (v0 + u * kPeerThreads < hi) tmp[u] = __ldcg(from + v0 + u * kPeerThreads);
#pragma unroll
            for (int u = 0; u < 4; ++u)
                if (v0 + u * kPeerThreads < hi) to[v0 + u * kPeerThreads] = tmp[u];
        }
    }
}

}  // namespace qmm
