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
//   2. five of a CTA's communication warps wait for pushed[c][*], add the W shares of the rows the rank
//      owns in rank order (fp32, one rounding: the result does not depend on timing and is the same on
//      every rank), write them to the rank's output and to the reduced area of its region; the last
//      CTA to finish raises reduced[c][rank] at every peer;
//   3. one thread of the sixth warp waits for reduced[c] of one other owner and copies that owner's rows
//      of chunk c into this rank's output with bulk copies through two 16 KiB staging buffers (peer
//      region -> shared memory -> output): the copy engine moves the data, no warp does.
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
constexpr int kFusedReduceThreads = kFusedThreads - 32;  // five warps reduce, one drives the gather
constexpr uint32_t kFusedStageBytes = 16 * 1024;   // one of the two staging buffers of the gather

// Development builds (-DQMM_FUSED_TRACE): CTA 0 records %globaltimer at the steps of the exchange into the flag
// area of its rank's region (64-bit slots at 48 KiB: 0 start, 1+c epilogue left chunk c, 9+c pushed[c] seen,
// 17+c reduce of c done, 25+c reduced[c] seen, 33+c gather of c done, 41 matmul end, 42 gather end).
#ifdef QMM_FUSED_TRACE
constexpr size_t kFusedTraceOffset = 48 * 1024;
#define QMM_TRACE(f, idx)                                                                                  \
    do {                                                                                                   \
        if (blockIdx.x == 0)                                                                               \
            reinterpret_cast<unsigned long long *>((f).base[(f).rank] + kFusedTraceOffset)[idx] = globaltimer_ns(); \
    } while (0)
#else
#define QMM_TRACE(f, idx) do { } while (0)
#endif

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
    const uint32_t stride = gridDim.x * kFusedReduceThreads;
    for (uint32_t v = blockIdx.x * kFusedReduceThreads + ct; v < total; v += U * stride) {
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

// Bulk copy shared -> global as a bulk group of the issuing thread (both addresses 16-byte aligned,
// `bytes` a multiple of 16).
__device__ __forceinline__ void bulk_store_1d(void *dst, uint32_t smem_src, uint32_t bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(reinterpret_cast<uint64_t>(dst)),
                 "r"(smem_src), "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ void fused_reduce_bar_sync() {
    asm volatile("bar.sync 1, %0;" ::"n"(kFusedReduceThreads) : "memory");
}

// The reduce warps' loop (communication warps 1..5); `rt` = 0..kFusedReduceThreads-1, s_ok = a shared word.
template <typename T>
__device__ __forceinline__ void fused_reduce_role(const FusedComm &f, int rt, volatile uint32_t *s_ok) {
    const int W = f.world;
    uint8_t *my_flags = f.base[f.rank] + kFusedFlagOffset;
    const uint32_t *pushed = reinterpret_cast<const uint32_t *>(my_flags);
    const int64_t own_r0 = static_cast<int64_t>(f.rank) * f.rows_per;
    const int64_t own_r1 = (own_r0 + f.rows_per < f.M) ? own_r0 + f.rows_per : f.M;
    const int64_t own_rows = own_r1 > own_r0 ? own_r1 - own_r0 : 0;
    const size_t row_bytes = static_cast<size_t>(f.N) * sizeof(T);
    const size_t share_bytes = static_cast<size_t>(f.rows_per) * row_bytes;
    if (rt == 0) *s_ok = 1;
    fused_reduce_bar_sync();
    for (int c = 0; c < f.chunks; ++c) {
        if (rt < W && !peer_wait_flag(pushed + c * kPeerMaxRanks + rt, f.epoch, f.status, f.status_at_launch, 0x11))
            *s_ok = 0;
        fused_reduce_bar_sync();
        if (*s_ok == 0) return;
        if (rt == 0) QMM_TRACE(f, 9 + c);
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
            fused_reduce_chunk<T, 2, 4>(W, rt, total, vps, row_bytes, share_bytes, part0, red0, out0);
        else if (W <= 4)
            fused_reduce_chunk<T, 4, 2>(W, rt, total, vps, row_bytes, share_bytes, part0, red0, out0);
        else
            fused_reduce_chunk<T, 8, 1>(W, rt, total, vps, row_bytes, share_bytes, part0, red0, out0);
        fused_reduce_bar_sync();
        if (rt == 0) {
            QMM_TRACE(f, 17 + c);
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
}

// The gather, driven by ONE thread per CTA (lane 0 of communication warp 0) with bulk copies: the reduced rows
// of one other owner travel peer region -> 16 KiB staging buffer in shared memory -> this rank's output,
// two buffers in flight, so the copy engine moves the data and no warp spends registers or issue slots on
// it.  `stage` = shared-memory address of the two staging buffers, `bar` = of their two mbarriers.
template <typename T>
__device__ __forceinline__ void fused_gather_role(const FusedComm &f, uint32_t stage, uint32_t bar,
                                                  volatile uint32_t *abort_flag) {
    const int W = f.world;
    const uint32_t *reduced =
        reinterpret_cast<const uint32_t *>(f.base[f.rank] + kFusedFlagOffset + kFusedReducedOffset);
    const size_t row_bytes = static_cast<size_t>(f.N) * sizeof(T);
    // this CTA copies row slice `gs` of `gn` of owner `gsrc` (consecutive CTAs read from different owners,
    // every rank starting with its right-hand neighbour)
    const int gn = static_cast<int>(gridDim.x) / (W - 1);
    const int gs = static_cast<int>(blockIdx.x) / (W - 1);
    const int gsrc = (f.rank + 1 + static_cast<int>(blockIdx.x) % (W - 1)) % W;
    const int64_t src_r0 = static_cast<int64_t>(gsrc) * f.rows_per;
    const int64_t src_r1 = (src_r0 + f.rows_per < f.M) ? src_r0 + f.rows_per : f.M;
    const int64_t src_rows = src_r1 > src_r0 ? src_r1 - src_r0 : 0;
    const int64_t row_lo = gs < gn ? src_rows * gs / gn : 0, row_hi = gs < gn ? src_rows * (gs + 1) / gn : 0;
    uint32_t phase[2] = {0, 0};
    bool gave_up = false;
    for (int c = 0; c < f.chunks && !gave_up; ++c) {
        // every CTA waits, also the ones without a slice: a rank may leave only after all peers are done reducing
        if (!peer_wait_flag(reduced + c * kPeerMaxRanks + gsrc, f.epoch, f.status, f.status_at_launch, 0x12)) break;
        QMM_TRACE(f, 25 + c);
        const int64_t col0 = static_cast<int64_t>(f.first[c]) * kFusedTileCols;
        int64_t col1 = static_cast<int64_t>(f.first[c + 1]) * kFusedTileCols;
        if (col1 > f.N) col1 = f.N;
        const uint32_t seg = static_cast<uint32_t>((col1 - col0) * sizeof(T));  // bytes of a row's share of the chunk
        const uint32_t piece = seg <= kFusedStageBytes ? seg : 8192u;             // bytes per bulk copy
        const uint32_t ppr = (seg + piece - 1) / piece;                           // pieces per row
        const uint32_t per_batch = kFusedStageBytes / piece;                      // pieces per staging buffer
        const size_t byte0 = static_cast<size_t>(src_r0) * row_bytes + static_cast<size_t>(col0) * sizeof(T);
        const uint8_t *from = f.base[gsrc] + f.red_off + byte0;
        uint8_t *to = static_cast<uint8_t *>(f.out) + byte0;
        const uint32_t npieces = static_cast<uint32_t>(row_hi - row_lo) * ppr;
        // batch j = pieces [j * per_batch, ...): load batch j + 1 while batch j lands, then store batch j
        int prev_buf = -1;
        uint32_t prev_first = 0, prev_count = 0;
        int buf = 0;
        for (uint32_t first = 0; (first < npieces || prev_buf >= 0) && !gave_up; first += per_batch) {
            const uint32_t count = first < npieces ? (npieces - first < per_batch ? npieces - first : per_batch) : 0;
            if (count > 0) {
                // the bulk stores that last read this buffer (two batches ago) are all committed: wait for their reads
                tma_store_wait_read<0>();
                uint32_t bytes = 0;
                for (uint32_t i = 0; i < count; ++i) {
                    const uint32_t pi = first + i, off = (pi % ppr) * piece;
                    bytes += (seg - off < piece) ? seg - off : piece;
                }
                mbar_expect_tx(bar + buf * 8, bytes);
                uint32_t at = 0;
                for (uint32_t i = 0; i < count; ++i) {
                    const uint32_t pi = first + i, off = (pi % ppr) * piece;
                    const uint32_t n = (seg - off < piece) ? seg - off : piece;
                    bulk_load_1d(stage + buf * kFusedStageBytes + at,
                                 from + static_cast<size_t>(row_lo + pi / ppr) * row_bytes + off, n, bar + buf * 8);
                    at += n;
                }
            }
            if (prev_buf >= 0) {
                if (!mbar_wait(bar + prev_buf * 8, phase[prev_buf], abort_flag, 0x13)) {
                    gave_up = true;  // a load that has not landed after the wait limit: nothing more to copy
                    break;
                }
                phase[prev_buf] ^= 1;
                fence_proxy_async_smem();
                uint32_t at = 0;
                for (uint32_t i = 0; i < prev_count; ++i) {
                    const uint32_t pi = prev_first + i, off = (pi % ppr) * piece;
                    const uint32_t n = (seg - off < piece) ? seg - off : piece;
                    bulk_store_1d(to + static_cast<size_t>(row_lo + pi / ppr) * row_bytes + off,
                                  stage + prev_buf * kFusedStageBytes + at, n);
                    at += n;
                }
                tma_store_commit();
            }
            if (count > 0) {
                prev_buf = buf;
                prev_first = first;
                prev_count = count;
                buf ^= 1;
            } else {
                prev_buf = -1;
            }
        }
        QMM_TRACE(f, 33 + c);
    }
    // also on the way out after a wait that gave up: the bulk stores already issued read shared memory
    tma_store_wait_all<0>();
    QMM_TRACE(f, 42);
}

}  // namespace qmm
