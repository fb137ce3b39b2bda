// Allreduce inside the row-parallel matmul (npu_mm_all_reduce_base): the CTA-pair kernel carries four
// more warps per CTA that reduce and gather finished column chunks over peer memory while the tensor
// pipe works on the next ones, so that only the last chunk's exchange is left when the matmul ends.
//
// The output's tile columns are cut into `chunks` column chunks, and every rank multiplies them in that
// order.  For chunk c:
//   1. the epilogue warps store the chunk's tiles straight into the owners' regions (TMA stores to peer
//      memory, slot [source rank] of the partial area).  An epilogue warp that leaves a chunk waits for
//      its own stores to complete, and the last warp of the GPU to do so raises pushed[c][rank] at
//      every rank;
//   2. a rank's communication warps wait for pushed[c][*], add the W shares of the rows the rank owns
//      in rank order (fp32, one rounding: the result does not depend on timing and is the same on
//      every rank), write them to the rank's output and to the reduced area of its region; the last
//      CTA to finish raises reduced[c][rank] at every peer;
//   3. then they copy the other owners' rows of chunk c from those owners' regions into this rank's
//      output (peer loads), each CTA from one owner, starting with the right-hand neighbour; the owners
//      reduce chunk c at the same time, so their flags follow shortly.
//
// The matmul roles never wait for the communication warps, and communication warps wait for flags
// only, so there is no cycle: pushed[c] needs matmul progress alone, reduced[c] needs pushed[c].
// The counters that elect "the last one" count CTAs of the one grid they belong to, which is resident as a
// whole (one CTA per SM, grid <= SM count).  Every wait is bounded; a wait that gives up records a status
// code, and the communication warps of that CTA stop touching peer data.
//
// Flags carry the communicator's epoch (only grows, never reset).  The counters return to zero when they
// complete; after a call that was cut short the host clears them (fused_counter_bytes at kFusedPushCountOffset).
//
// Buffer reuse across calls: a rank leaves the kernel only after it has seen reduced[last][o] of every
// peer o, i.e. after every peer has finished reading the partial area that this rank's next matmul
// pushes into; and a rank overwrites its reduced area in the next call only after pushed[0] of that call
// has arrived from every peer, i.e. after their previous kernel, which read that area, has ended.
#pragma once

#include "peer_all_reduce.cuh"

namespace qmm {

constexpr int kFusedMaxChunks = 8;
constexpr int kFusedThreads = 192;                 // communication threads per CTA
constexpr size_t kFusedFlagOffset = 40 * 1024;     // pushed [8][8] u32, reduced [8][8] u32 at +256,
constexpr size_t kFusedReducedOffset = 256;        // push counters [8] at +512, reduce counters [8] at +576
constexpr size_t kFusedPushCountOffset = 512;
constexpr size_t kFusedReduceCountOffset = 576;
constexpr size_t kFusedCounterBytes = 128;         // both counter rows
constexpr int kFusedTileCols = 256;                // width of the matmul's output tile

struct FusedComm {
    uint8_t *base[kPeerMaxRanks];  // every rank's region as mapped here (own region included)
    int world, rank;
    uint32_t epoch;
    int chunks;                    // column chunks, 1..kFusedMaxChunks
    int first[kFusedMaxChunks + 1];  // chunk c covers the tile columns [first[c], first[c + 1]); none is empty
    int64_t M, N;
    int64_t rows_per;              // rows owned by a rank, a multiple of 32
    size_t partial_off, red_off;   // byte offsets of the two data areas inside a region
    void *out;                     // [M][N], this rank's result
    uint32_t *status;
    uint32_t status_at_launch;
    int enabled;
};

// Cuts `tiles_n` tile columns into `chunks` (<= tiles_n) chunks whose widths fall off quadratically: what is
// still to be exchanged when the matmul ends is the last chunk, so that one is the narrowest, while the wide
// early chunks keep the number of flag rounds small.  No chunk is empty.
inline void fused_chunk_bounds(int tiles_n, int chunks, int (&first)[kFusedMaxChunks + 1]) {
    for (int c = 0; c <= kFusedMaxChunks; ++c) first[c] = tiles_n;
    for (int c = 0; c <= chunks; ++c) {
        const int64_t left = static_cast<int64_t>(chunks - c) * (chunks - c);
        first[c] = tiles_n - static_cast<int>(tiles_n * left / (static_cast<int64_t>(chunks) * chunks));
    }
    for (int c = chunks - 1; c >= 1; --c)  // every chunk at least one column wide, from the back
        if (first[c] > first[c + 1] - 1) first[c] = first[c + 1] - 1;
    for (int c = 1; c <= chunks; ++c)
        if (first[c] < first[c - 1] + 1) first[c] = first[c - 1] + 1;
    first[0] = 0;
    first[chunks] = tiles_n;
}

// Adds `add` to an arrival counter; true for the arrival that completes `expected`, which also puts the
// counter back to zero for the next call.  One atomic per arrival: hundreds of warps arrive at the same moment
// when the matmul ends (a compare-and-swap loop was measured to cost 150 us there).  A call that is cut short
// leaves its counters dirty; the host clears them before the next launch (it sees the status word).
__device__ __forceinline__ bool counter_arrive(uint32_t *ctr, uint32_t add, uint32_t expected) {
    const uint32_t old = atomicAdd(ctr, add);
    if (old + add != expected) return false;
    atomicExch(ctr, 0u);
    return true;
}

__device__ __forceinline__ void fused_bar_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kFusedThreads) : "memory"); }

// Called by an epilogue warp's lane 0 when the warp has issued the stores of `units` tiles of chunk c and
// moves on: waits for the stores, counts them, and tells every rank once the whole GPU is done with c.
__device__ __forceinline__ void fused_chunk_pushed(const FusedComm &f, int c, uint32_t units, uint32_t expected) {
    tma_store_wait_all<0>();
    // device scope is enough for the count; the one arrival that completes it orders everything it has
    // observed before the flags with a system-scope fence.  (A system-scope fence per warp was measured to cost
    // 150 us per call on two GPUs: hundreds of them queue up behind one another.)
    __threadfence();
    uint8_t *mine = f.base[f.rank] + kFusedFlagOffset;
    if (counter_arrive(reinterpret_cast<uint32_t *>(mine + kFusedPushCountOffset) + c, units, expected)) {
        __threadfence_system();
        for (int r = 0; r < f.world; ++r)
            st_release_sys(reinterpret_cast<uint32_t *>(f.base[r] + kFusedFlagOffset) + c * kPeerMaxRanks + f.rank,
                           f.epoch);
    }
}

// Sum of the ranks' shares of `total` vectors (rows x vps 16-byte vectors of a column chunk) in rank order;
// WW: ranks rounded up, U: vectors per thread and pass (U * WW loads in flight per thread).
template <typename T, int WW, int U>
__device__ __forceinline__ void fused_reduce_chunk(int W, int ct, uint32_t total, uint32_t vps, size_t row_bytes,
                                                   size_t share_bytes, const uint8_t *part0, uint8_t *red0,
                                                   uint8_t *out0) {
    // 32-bit indices: a rank's rows of a chunk are far fewer than 2^31 vectors (checked by the launcher)
    const uint32_t stride = gridDim.x * kFusedThreads;
    for (uint32_t v = blockIdx.x * kFusedThreads + ct; v < total; v += U * stride) {
        uint4 part[U][WW];
        uint32_t off[U];  // a rank's share of the rows stays far below 4 GiB
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const uint32_t vv = v + u * stride;
            if (vv < total) {
                const uint32_t row = vv / vps;
                off[u] = static_cast<uint32_t>(static_cast<size_t>(row) * row_bytes + static_cast<size_t>(vv - row * vps) * 16);
#pragma unroll
                for (int r = 0; r < WW; ++r)
                    if (r < W) part[u][r] = __ldcg(reinterpret_cast<const uint4 *>(part0 + r * share_bytes + off[u]));
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            if (v + u * stride < total) {
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
                *reinterpret_cast<uint4 *>(red0 + off[u]) = o;
                *reinterpret_cast<uint4 *>(out0 + off[u]) = o;
            }
        }
    }
}

// The communication warps' loop; `ct` = 0..kFusedThreads-1, s_ok = a shared word of the CTA (set to 1 here).
template <typename T>
__device__ __forceinline__ void fused_comm_role(const FusedComm &f, int ct, volatile uint32_t *s_ok) {
    const int W = f.world;
    uint8_t *my_flags = f.base[f.rank] + kFusedFlagOffset;
    const uint32_t *pushed = reinterpret_cast<const uint32_t *>(my_flags);
    const uint32_t *reduced = reinterpret_cast<const uint32_t *>(my_flags + kFusedReducedOffset);
    const int64_t own_r0 = static_cast<int64_t>(f.rank) * f.rows_per;
    const int64_t own_r1 = (own_r0 + f.rows_per < f.M) ? own_r0 + f.rows_per : f.M;
    const int64_t own_rows = own_r1 > own_r0 ? own_r1 - own_r0 : 0;
    const size_t row_bytes = static_cast<size_t>(f.N) * sizeof(T);
    const size_t share_bytes = static_cast<size_t>(f.rows_per) * row_bytes;
    // gather: this CTA copies slice `gs` of `gn` from owner `gsrc`
    const int gn = static_cast<int>(gridDim.x) / (W - 1);
    const int gs = static_cast<int>(blockIdx.x) / (W - 1);
    const int gsrc = (f.rank + 1 + static_cast<int>(blockIdx.x) % (W - 1)) % W;
    const int64_t src_r0 = static_cast<int64_t>(gsrc) * f.rows_per;
    const int64_t src_r1 = (src_r0 + f.rows_per < f.M) ? src_r0 + f.rows_per : f.M;
    const int64_t src_rows = src_r1 > src_r0 ? src_r1 - src_r0 : 0;
    if (ct == 0) *s_ok = 1;
    fused_bar_sync();

    for (int c = 0; c < f.chunks; ++c) {
        {
            // ---- reduce chunk c of the rows this rank owns ----
            if (ct < W && !peer_wait_flag(pushed + c * kPeerMaxRanks + ct, f.epoch, f.status, f.status_at_launch, 0x11))
                *s_ok = 0;
            fused_bar_sync();
            if (*s_ok == 0) return;
            const int64_t col0 = static_cast<int64_t>(f.first[c]) * kFusedTileCols;
            int64_t col1 = static_cast<int64_t>(f.first[c + 1]) * kFusedTileCols;
            if (col1 > f.N) col1 = f.N;
            const uint32_t vps = static_cast<uint32_t>((col1 - col0) / 8);  // 16-byte vectors per row segment
            const uint32_t total = static_cast<uint32_t>(own_rows) * vps;
            const uint8_t *part0 = f.base[f.rank] + f.partial_off + static_cast<size_t>(col0) * sizeof(T);
            const size_t own_byte0 = static_cast<size_t>(own_r0) * row_bytes + static_cast<size_t>(col0) * sizeof(T);
            uint8_t *red0 = f.base[f.rank] + f.red_off + own_byte0;
            uint8_t *out0 = static_cast<uint8_t *>(f.out) + own_byte0;
            if (W <= 2)
                fused_reduce_chunk<T, 2, 4>(W, ct, total, vps, row_bytes, share_bytes, part0, red0, out0);
            else if (W <= 4)
                fused_reduce_chunk<T, 4, 2>(W, ct, total, vps, row_bytes, share_bytes, part0, red0, out0);
            else
                fused_reduce_chunk<T, 8, 1>(W, ct, total, vps, row_bytes, share_bytes, part0, red0, out0);
            fused_bar_sync();
            if (ct == 0) {
                __threadfence();
                if (counter_arrive(reinterpret_cast<uint32_t *>(my_flags + kFusedReduceCountOffset) + c, 1, gridDim.x)) {
                    __threadfence_system();
                    for (int r = 0; r < W; ++r)
                        if (r != f.rank)
                            st_release_sys(reinterpret_cast<uint32_t *>(f.base[r] + kFusedFlagOffset + kFusedReducedOffset) +
                                               c * kPeerMaxRanks + f.rank,
                                           f.epoch);
                }
            }
        }
        {
            // ---- gather chunk c of one other owner's rows (its reduce ran at the same time as this rank's) ----
            const int g = c;
            // every CTA waits, also the ones without a slice: a rank may leave only after all peers are done reducing
            if (ct == 0 && !peer_wait_flag(reduced + g * kPeerMaxRanks + gsrc, f.epoch, f.status, f.status_at_launch, 0x12))
                *s_ok = 0;
            fused_bar_sync();
            if (*s_ok == 0) return;
            if (gs < gn) {
                const int64_t col0 = static_cast<int64_t>(f.first[g]) * kFusedTileCols;
                int64_t col1 = static_cast<int64_t>(f.first[g + 1]) * kFusedTileCols;
                if (col1 > f.N) col1 = f.N;
                const uint32_t vps = static_cast<uint32_t>((col1 - col0) / 8);
                const uint32_t total = static_cast<uint32_t>(src_rows) * vps;
                const uint32_t lo = static_cast<uint32_t>(static_cast<uint64_t>(total) * gs / gn);
                const uint32_t hi = static_cast<uint32_t>(static_cast<uint64_t>(total) * (gs + 1) / gn);
                const size_t src_byte0 = static_cast<size_t>(src_r0) * row_bytes + static_cast<size_t>(col0) * sizeof(T);
                const uint8_t *from = f.base[gsrc] + f.red_off + src_byte0;
                uint8_t *to = static_cast<uint8_t *>(f.out) + src_byte0;
                for (uint32_t v0 = lo + ct; v0 < hi; v0 += 8 * kFusedThreads) {
                    uint4 tmp[8];
                    uint32_t off[8];
#pragma unroll
                    for (int u = 0; u < 8; ++u) {
                        const uint32_t vv = v0 + u * kFusedThreads;
                        if (vv < hi) {
                            const uint32_t row = vv / vps;
                            off[u] = static_cast<uint32_t>(static_cast<size_t>(row) * row_bytes +
                                                           static_cast<size_t>(vv - row * vps) * 16);
                            tmp[u] = __ldcg(reinterpret_cast<const uint4 *>(from + off[u]));
                        }
                    }
#pragma unroll
                    for (int u = 0; u < 8; ++u)
                        if (v0 + u * kFusedThreads < hi) *reinterpret_cast<uint4 *>(to + off[u]) = tmp[u];
                }
            }
        }
    }
}

}  // namespace qmm
