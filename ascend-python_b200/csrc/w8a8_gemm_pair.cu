// W8A8 prefill matmul on CTA pairs (tcgen05 cta_group::2).
//
// Two CTAs of a cluster, on the two SMs of a TPC, share one 256x256 output
// tile: each loads its own 128 rows of A and one 128-column half of B per
// k-block (32 KiB per stage and CTA instead of 48 KiB for a 128x256 tile of its
// own), the leader CTA issues one 256x256x32 MMA for the pair, and each CTA
// receives its 128 rows of the int32 accumulator in its own TMEM.  Per output
// element the pair moves a third less data from L2 to shared memory and keeps
// six stages in flight instead of four, which is what the int8 MMA rate needs.
//
// Synchronisation (s = stage, b = accumulator buffer):
//   full[s]       leader's barrier; both CTAs' TMA loads count their bytes on it
//   empty[s]      one per CTA; the leader's tcgen05.commit arrives on both
//   tmem_full[b]  one per CTA; the leader's tcgen05.commit arrives on both
//   tmem_empty[b] leader's barrier; the 4+4 epilogue warps of the pair arrive on it
// No TMA load uses multicast; every wait is bounded (see mbar_wait).
//
// FUSED (the row-parallel matmul + allreduce): four more warps per CTA reduce and gather finished column
// chunks over peer memory while the matmul goes on; tiles are then visited chunk by chunk, and within a
// chunk every rank starts with the rows of its right-hand neighbour so that the owners' links fill evenly.
#include <cstring>

#include "peer_fused.cuh"
#include "qmm_common.cuh"
#include "w8a8_epilogue.cuh"

namespace qmm {


namespace {

constexpr int kPM = 128;   // rows per CTA
constexpr int kPN = 256;   // columns of the pair's tile
constexpr int kPK = 128;   // k elements per stage
constexpr int kPStages = 6;
constexpr int kPAStageBytes = kPM * kPK;
constexpr int kPBStageBytes = (kPN / 2) * kPK;
constexpr int kPStageBytes = kPAStageBytes + kPBStageBytes;  // per CTA
constexpr int kPThreads = 192;
constexpr int kPFusedThreads = kPThreads + kFusedThreads;
static_assert(kPN == kFusedTileCols, "the communication warps cut the output into the matmul's tile columns");
constexpr uint32_t kPTmemCols = 512;
constexpr int kPEpiWarps = 4;
constexpr int kPEpiStageBytes = 2 * 4096;
constexpr int kPEpiColFloats = 128;

struct PairSmemTail {
    uint64_t full[kPStages];
    uint64_t empty[kPStages];
    uint64_t tmem_full[2];
    uint64_t tmem_empty[2];
    uint32_t tmem_base;
    uint32_t abort_flag;
    uint32_t comm_ok;
    uint64_t comm_full[2];  // fused kernel: the gather's two staging buffers have landed
};

constexpr size_t kPairSmemBytes = kPStages * kPStageBytes + kPEpiWarps * kPEpiStageBytes +
                                  kPEpiWarps * kPEpiColFloats * sizeof(float) + sizeof(PairSmemTail);
static_assert(kPairSmemBytes <= 232448, "pair kernel exceeds the 227 KiB of shared memory a CTA may use");

// Tile order.  raster > 0: groups of `raster` tile rows, each swept across all tile columns with the
// rows running fastest, so the group's rows of A stay in L2 while B streams through once per group;
// raster < 0: the same with the roles of rows and columns exchanged (-raster tile columns of B stay).
__device__ __forceinline__ void pair_tile_coords(int tile, int tiles_m, int tiles_n, int raster, int &m_blk,
                                                 int &n_blk) {
    if (raster > 0) {
        const int per_group = raster * tiles_n;
        const int g = tile / per_group;
        const int first_m = g * raster;
        const int rows = min(raster, tiles_m - first_m);
        const int r = tile - g * per_group;
        m_blk = first_m + r % rows;
        n_blk = r / rows;
    } else {
        const int gc = -raster;
        const int per_group = gc * tiles_m;
        const int g = tile / per_group;
        const int first_n = g * gc;
        const int cols = min(gc, tiles_n - first_n);
        const int r = tile - g * per_group;
        n_blk = first_n + r % cols;
        m_blk = r / cols;
    }
}

// Tile order of the fused kernel: column chunk by column chunk; inside a chunk the order above (`raster`
// chosen for a chunk's width), with the tile rows rotated by m_rot (the first tile row of the right-hand
// neighbour's rows) so that the ranks do not all push to the same owner at the same time.
__device__ __forceinline__ void fused_tile_coords(int tile, int tiles_m, const FusedComm &fc, int raster, int m_rot,
                                                  int &m_blk, int &n_blk, int &chunk) {
    int c = 0;
    while (c + 1 < fc.chunks && tile >= fc.first[c + 1] * tiles_m) ++c;
    const int nb0 = fc.first[c];
    const int ncols = fc.first[c + 1] - nb0;
    int m, n;
    pair_tile_coords(tile - nb0 * tiles_m, tiles_m, ncols, raster, m, n);
    n_blk = nb0 + n;
    m_blk = (m_rot + m) % tiles_m;
    chunk = c;
}

// Chooses the order that moves fewer bytes from DRAM.  With g tile rows (or columns) per group the
// group's share of one operand stays in L2 while the other streams through once per group.  That
// only works while the resident share, the part of the streaming operand that one wave of tiles
// touches and the wave's outputs fit the L2 capacity seen by data that every SM reads (about half of
// the 126 MB: each die keeps its own copy); when no group size fits, the smallest footprint wins.
int pair_choose_raster(int64_t M, int64_t N, int64_t K, int64_t out_elt, int wave_tiles) {
    const int64_t tiles_m = (M + 2 * kPM - 1) / (2 * kPM), tiles_n = (N + kPN - 1) / kPN;
    const int64_t row_bytes = 2ll * kPM * K, col_bytes = static_cast<int64_t>(kPN) * K;
    const int64_t out_bytes = static_cast<int64_t>(wave_tiles) * 2 * kPM * kPN * out_elt;
    const int64_t capacity = 60ll << 20;
    const int64_t a_total = M * K, b_total = N * K;
    int best = 1;
    int64_t best_traffic = -1, best_foot = -1;
    bool best_fits = false;
    auto consider = [&](int64_t g, bool rows) {
        const int64_t tiles_g = rows ? tiles_m : tiles_n;
        const int64_t across = (wave_tiles + g - 1) / g;  // tiles of the streaming operand per wave
        const int64_t foot = g * (rows ? row_bytes : col_bytes) + across * (rows ? col_bytes : row_bytes) + out_bytes;
        const int64_t traffic = rows ? a_total + (tiles_g + g - 1) / g * b_total
                                     : b_total + (tiles_g + g - 1) / g * a_total;
        const bool fits = foot <= capacity;
        const bool better = best_traffic < 0 || (fits && !best_fits) ||
                            (fits == best_fits && (fits ? traffic < best_traffic : foot < best_foot));
        if (better) {
            best = rows ? static_cast<int>(g) : -static_cast<int>(g);
            best_traffic = traffic;
            best_foot = foot;
            best_fits = fits;
        }
    };
    for (int64_t g = 1; g <= tiles_m; ++g) consider(g, true);
    for (int64_t g = 1; g <= tiles_n; ++g) consider(g, false);
    return best;
}

template <typename OutT, bool B_MN_MAJOR, bool FUSED>
__global__ void __launch_bounds__(FUSED ? kPFusedThreads : kPThreads, 1)
w8a8_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                 const __grid_constant__ CUtensorMap tmap_out, const __grid_constant__ PushMaps push,
                 const __grid_constant__ FusedComm fc, EpilogueParams ep, int K, int use_tma_store, int raster,
                 uint32_t *status) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    const uint32_t smem_base = smem_u32(smem_raw);
    const uint32_t cta_rank = cluster_ctarank();  // 0 = leader
    const bool leader = (cta_rank == 0);
    uint8_t *epi_stage = smem_raw + kPStages * kPStageBytes;
    float *epi_cols = reinterpret_cast<float *>(epi_stage + kPEpiWarps * kPEpiStageBytes);
    PairSmemTail *tail = reinterpret_cast<PairSmemTail *>(epi_cols + kPEpiWarps * kPEpiColFloats);
    volatile uint32_t *abort_flag = &tail->abort_flag;
    // both CTAs of a pair see the same alignment, so this exit is taken by both or by none
    if ((smem_base & 1023u) != 0) {
        if (threadIdx.x == 0 && status != nullptr) atomicMax(status, DEV_STATUS_SMEM_MISALIGNED);
        return;
    }

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int tiles_m = static_cast<int>((ep.M + 2 * kPM - 1) / (2 * kPM));
    const int tiles_n = static_cast<int>((ep.N + kPN - 1) / kPN);
    const int num_tiles = tiles_m * tiles_n;
    const int num_kb = (K + kPK - 1) / kPK;
    const int pair_id = blockIdx.x >> 1;
    const int num_pairs = gridDim.x >> 1;
    // the fused kernel gives its last stage (32 KiB) to the gather's staging buffers
    constexpr int kStages = FUSED ? kPStages - 1 : kPStages;
    static_assert(2 * kFusedStageBytes <= kPStageBytes, "the gather's staging buffers take one stage");
    // fused: first tile row of the right-hand neighbour's rows
    const int m_rot = FUSED ? static_cast<int>((static_cast<int64_t>((fc.rank + 1) % fc.world) * fc.rows_per / (2 * kPM)) %
                                               tiles_m)
                            : 0;
    auto tile_coords = [&](int tile, int &m_blk, int &n_blk, int &chunk) {
        if constexpr (FUSED) {
            fused_tile_coords(tile, tiles_m, fc, raster, m_rot, m_blk, n_blk, chunk);
        } else {
            pair_tile_coords(tile, tiles_m, tiles_n, raster, m_blk, n_blk);
            chunk = 0;
        }
    };

    if (threadIdx.x == 0) {
        for (int s = 0; s < kPStages; ++s) {
            mbar_init(smem_u32(&tail->full[s]), 1);
            mbar_init(smem_u32(&tail->empty[s]), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(smem_u32(&tail->tmem_full[b]), 1);
            mbar_init(smem_u32(&tail->tmem_empty[b]), 2 * kPEpiWarps);
        }
        mbar_init(smem_u32(&tail->comm_full[0]), 1);
        mbar_init(smem_u32(&tail->comm_full[1]), 1);
        tail->abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == 0 && lane == 0) {
        tma_prefetch_desc(&tmap_a);
        tma_prefetch_desc(&tmap_b);
    }
    if (warp == 1) {
        tmem_alloc_pair(smem_u32(&tail->tmem_base), kPTmemCols);
        tmem_relinquish_pair();
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();  // the peer's barriers are initialised before anything signals them
    tc_fence_after();
    const uint32_t tmem_base = tail->tmem_base;

    if (warp == 0) {
        // ---------------- TMA producer (both CTAs) ----------------
        uint32_t stage = 0, phase = 0;
        bool ok = true;
        for (int tile = pair_id; tile < num_tiles && ok; tile += num_pairs) {
            int m_blk, n_blk, chunk;
            tile_coords(tile, m_blk, n_blk, chunk);
            const int m0 = m_blk * 2 * kPM + static_cast<int>(cta_rank) * kPM;
            const int n0 = n_blk * kPN + static_cast<int>(cta_rank) * (kPN / 2);
            for (int kb = 0; kb < num_kb; ++kb) {
                ok = mbar_wait(smem_u32(&tail->empty[stage]), phase ^ 1, abort_flag, 0x21);
                if (!ok) break;
                if (lane == 0) {
                    const uint32_t full_local = smem_u32(&tail->full[stage]);
                    const uint32_t full_leader = map_to_cta(full_local, 0);
                    const uint32_t sa = smem_base + stage * kPStageBytes;
                    const uint32_t sb = sa + kPAStageBytes;
                    if (leader) mbar_expect_tx(full_local, 2 * kPStageBytes);
                    tma_load_2d_pair(sa, &tmap_a, kb * kPK, m0, full_leader);
                    if (B_MN_MAJOR)
                        tma_load_2d_pair(sb, &tmap_b, n0, kb * kPK, full_leader);  // [128 k-rows][128 n-bytes]
                    else
                        tma_load_2d_pair(sb, &tmap_b, kb * kPK, n0, full_leader);  // [128 n-rows][128 k-bytes]
                }
                __syncwarp();
                if (++stage == kStages) {
                    stage = 0;
                    phase ^= 1;
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer (leader CTA only) ----------------
        // The whole warp runs the loop with warp-uniform operands; elect.sync picks the issuing lane.
        if (leader) {
            constexpr uint32_t idesc = make_idesc(/*c=s32*/ 2, 1, 1, /*a K-major*/ 0, B_MN_MAJOR ? 1u : 0u, 2 * kPM, kPN);
            constexpr uint32_t kDescHi = smem_desc_hi_sw128(1024);  // 8-row groups are 1024 bytes apart
            constexpr uint32_t kStageStep = kPStageBytes >> 4;
            // A: K-major, 32 bytes (+2) per K step.  B: MN-major 4096 bytes (+256) per K step, K-major +2.
            constexpr uint32_t kBStep = B_MN_MAJOR ? (4096u >> 4) : 2u;
            const uint32_t a_lo0 = smem_desc_lo(smem_base, 16);
            const uint32_t b_lo0 = smem_desc_lo(smem_base + kPAStageBytes, B_MN_MAJOR ? 1024u : 16u);
            const uint32_t full0 = smem_u32(&tail->full[0]);
            const uint32_t empty0 = smem_u32(&tail->empty[0]);
            uint32_t stage = 0, phase = 0;
            int local = 0;
            bool ok = true;
            for (int tile = pair_id; tile < num_tiles && ok; tile += num_pairs, ++local) {
                const uint32_t buf = local & 1;
                const uint32_t buf_phase = (local >> 1) & 1;
                ok = mbar_wait(smem_u32(&tail->tmem_empty[buf]), buf_phase ^ 1, abort_flag, 0x22);
                if (!ok) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + buf * kPN;
                uint32_t accumulate = 0;
                for (int kb = 0; kb < num_kb; ++kb) {
                    ok = mbar_wait(full0 + stage * 8, phase, abort_flag, 0x23);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t a_lo = a_lo0 + stage * kStageStep;
                    const uint32_t b_lo = b_lo0 + stage * kStageStep;
#pragma unroll
                    for (int k = 0; k < kPK / 32; ++k) {
                        mma_i8_ss_pair_warp(d_tmem, desc64(a_lo + 2 * k, kDescHi), desc64(b_lo + kBStep * k, kDescHi),
                                            idesc, accumulate);
                        accumulate = 1;
                    }
                    tc_commit_pair_warp(empty0 + stage * 8, 0x3);
                    if (++stage == kStages) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
                if (ok) tc_commit_pair_warp(smem_u32(&tail->tmem_full[buf]), 0x3);
            }
        }
    } else if (FUSED && warp >= kPThreads / 32) {
        // ---------------- communication warps (both CTAs; fused kernel only) ----------------
        if constexpr (FUSED) {
            if (warp == kPThreads / 32) {
                if (lane == 0)
                    fused_gather_role<OutT>(fc, smem_base + kStages * kPStageBytes, smem_u32(&tail->comm_full[0]),
                                            abort_flag);
                __syncwarp();
            } else {
                fused_reduce_role<OutT>(fc, static_cast<int>(threadIdx.x) - kPThreads - 32, &tail->comm_ok);
            }
        }
    } else {
        // ---------------- epilogue warps (both CTAs) ----------------
        const int quarter = warp & 3;
        uint8_t *my_stage = epi_stage + quarter * kPEpiStageBytes;
        float *my_cols = epi_cols + quarter * kPEpiColFloats;
        uint32_t chunk_counter = 0;
        int local = 0;
        bool ok = true;
        if (lane == 0 && use_tma_store) tma_prefetch_desc(&tmap_out);
        // fused: tiles of the chunk this warp is in whose stores it has issued
        int cur_chunk = -1;
        uint32_t units = 0;
        auto chunk_expected = [&](int c) {
            return static_cast<uint32_t>((fc.first[c + 1] - fc.first[c]) * tiles_m * 2 * kPEpiWarps);
        };
        for (int tile = pair_id; tile < num_tiles && ok; tile += num_pairs, ++local) {
            int m_blk, n_blk, chunk;
            tile_coords(tile, m_blk, n_blk, chunk);
            if (FUSED && chunk != cur_chunk) {
                if (cur_chunk >= 0 && lane == 0) fused_chunk_pushed(fc, cur_chunk, units, chunk_expected(cur_chunk));
                if (FUSED && cur_chunk >= 0 && warp == 2 && lane == 0) QMM_TRACE(fc, 1 + cur_chunk);
                if (FUSED && cur_chunk < 0 && warp == 2 && lane == 0) QMM_TRACE(fc, 0);
                cur_chunk = chunk;
                units = 0;
            }
            const uint32_t buf = local & 1;
            const uint32_t buf_phase = (local >> 1) & 1;
            ok = mbar_wait(smem_u32(&tail->tmem_full[buf]), buf_phase, abort_flag, 0x24);
            if (!ok) break;
            tc_fence_after();
            const int64_t m_warp0 = static_cast<int64_t>(m_blk) * 2 * kPM + cta_rank * kPM + quarter * 32;
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + buf * kPN;
            if (use_tma_store) {
                // with push targets the tile goes to the receive area of the rank that owns its rows
                const CUtensorMap *omap = &tmap_out;
                int64_t store_row0 = -1;
                if (push.enabled) {
                    const int owner = static_cast<int>(m_warp0 / push.rows_per);
                    omap = &push.m[owner];
                    store_row0 = m_warp0 - owner * push.rows_per;
                }
                epilogue_warp_tile_tma<OutT, kPN>(ep, omap, taddr, m_warp0, static_cast<int64_t>(n_blk) * kPN,
                                                  my_stage, my_cols, chunk_counter, store_row0);
            } else {
#pragma unroll 1
                for (int c = 0; c < kPN / 32; ++c) {
                    uint32_t acc[32];
                    tmem_ld_32x32(taddr + c * 32, acc);
                    tmem_ld_wait();
                    epilogue_row_segment<OutT, 32>(ep, m_warp0 + lane, static_cast<int64_t>(n_blk) * kPN + c * 32, acc);
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&tail->tmem_empty[buf]), 0));
            ++units;
        }
        if (lane == 0) tma_store_wait_all<0>();
        // a warp that was cut short reports nothing: the peers' bounded waits then run out
        if (FUSED && ok && cur_chunk >= 0 && lane == 0) fused_chunk_pushed(fc, cur_chunk, units, chunk_expected(cur_chunk));
        if (FUSED && cur_chunk >= 0 && warp == 2 && lane == 0) QMM_TRACE(fc, 1 + cur_chunk);
        if (FUSED && warp == 2 && lane == 0) QMM_TRACE(fc, 41);
        __syncwarp();
    }

    // ---------------- teardown ----------------
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && tail->abort_flag != 0 && status != nullptr) atomicMax(status, tail->abort_flag);
    cluster_sync_all();  // nobody signals a CTA that already left; both are done with TMEM
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc_pair(tmem_base, kPTmemCols);
    }
}

template <typename OutT>
int launch_pair_t(const int8_t *x1, int64_t ld_x1, const int8_t *x2, int64_t x2_sk, int64_t x2_sn,
                  const EpilogueParams &ep, int64_t K, LaunchOptions *opts, cudaStream_t stream) {
    CUtensorMap ta, tb;
    int rc = make_tmap_2d(&ta, x1, 1, static_cast<uint64_t>(K), static_cast<uint64_t>(ep.M),
                          static_cast<uint64_t>(ld_x1), kPK, kPM, true);
    if (rc != QMM_OK) return rc;
    const bool mn_major = (x2_sn == 1);
    if (mn_major)
        rc = make_tmap_2d(&tb, x2, 1, static_cast<uint64_t>(ep.N), static_cast<uint64_t>(K),
                          static_cast<uint64_t>(x2_sk), 128, kPK, true);
    else
        rc = make_tmap_2d(&tb, x2, 1, static_cast<uint64_t>(K), static_cast<uint64_t>(ep.N),
                          static_cast<uint64_t>(x2_sn), kPK, kPN / 2, true);
    if (rc != QMM_OK) return rc;
    constexpr int kElt = static_cast<int>(sizeof(OutT));
    CUtensorMap tout = ta;
    int use_tma_store = 0;
    if ((reinterpret_cast<uintptr_t>(ep.out) & 15) == 0 && ((ep.ld_out * kElt) & 15) == 0) {
        rc = make_tmap_2d(&tout, ep.out, kElt, static_cast<uint64_t>(ep.N), static_cast<uint64_t>(ep.M),
                          static_cast<uint64_t>(ep.ld_out), 128 / kElt, 32, true);
        if (rc != QMM_OK) return rc;
        use_tma_store = 1;
    }
    const int tiles = static_cast<int>(((ep.M + 2 * kPM - 1) / (2 * kPM)) * ((ep.N + kPN - 1) / kPN));
    int pairs = (sm_count() - (opts != nullptr && opts->sm_reserve > 0 ? opts->sm_reserve : 0)) / 2;
    if (pairs < 1) pairs = 1;
    const int pairs_all = pairs;
    if (tiles < pairs) pairs = tiles;
    uint32_t *status = device_status_word();
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(2 * pairs));
    cfg.blockDim = dim3(kPThreads);
    cfg.dynamicSmemBytes = kPairSmemBytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int raster = pair_choose_raster(ep.M, ep.N, K, static_cast<int64_t>(sizeof(OutT)), pairs);
    PushMaps push;
    memset(&push, 0, sizeof(push));
    if (const PushSpec *ps = (opts != nullptr ? opts->push : nullptr)) {
        if (use_tma_store && sizeof(OutT) == 2 && ps->rows_per % 32 == 0 && ep.ld_out == ep.N) {
            for (int o = 0; o < ps->world; ++o) {
                const int64_t row0 = static_cast<int64_t>(o) * ps->rows_per;
                int64_t rows_o = ep.M - row0;
                if (rows_o > ps->rows_per) rows_o = ps->rows_per;
                if (rows_o <= 0) {  // this owner holds no rows: never addressed, keep a valid map
                    push.m[o] = tout;
                    continue;
                }
                uint8_t *dst = ps->base[o] + ps->area_off +
                               static_cast<size_t>(ps->rank) * ps->rows_per * ep.N * sizeof(OutT);
                rc = make_tmap_2d(&push.m[o], dst, kElt, static_cast<uint64_t>(ep.N), static_cast<uint64_t>(rows_o),
                                  static_cast<uint64_t>(ep.N), 128 / kElt, 32, true);
                if (rc != QMM_OK) return rc;
            }
            push.rows_per = ps->rows_per;
            push.enabled = 1;
            opts->push_applied = true;
        }
    }
    // The allreduce inside the kernel: only when the tiles are pushed, the whole GPU is one resident wave of
    // CTAs (the communication warps of different CTAs count one another) and 32-bit vector indices suffice.
    FusedComm fc;
    memset(&fc, 0, sizeof(fc));
    bool fused = false;
    if constexpr (sizeof(OutT) == 2) {
        if (opts != nullptr && opts->fused != nullptr && push.enabled && opts->sm_reserve == 0 &&
            2 * pairs_all <= sm_count() && 2 * pairs_all >= 2 * (opts->fused->world - 1) && ep.N % 8 == 0) {
            fc = *opts->fused;
            const int tiles_m = static_cast<int>((ep.M + 2 * kPM - 1) / (2 * kPM));
            const int tiles_n = static_cast<int>((ep.N + kPN - 1) / kPN);
            if (fc.chunks > tiles_n) fc.chunks = tiles_n;
            if (fc.chunks > kFusedMaxChunks) fc.chunks = kFusedMaxChunks;
            if (fc.chunks < 1) fc.chunks = 1;
            if (fc.rows_per * ep.N * static_cast<int64_t>(sizeof(OutT)) < (1ll << 32)) {  // 32-bit offsets inside a share
                fused_chunk_bounds(tiles_n, fc.chunks, fc.first);
                // the order inside a chunk: as for a matmul of the widest chunk's width
                const int64_t chunk_cols = static_cast<int64_t>(fc.first[1]) * kPN;
                raster = pair_choose_raster(ep.M, chunk_cols < ep.N ? chunk_cols : ep.N, K,
                                            static_cast<int64_t>(sizeof(OutT)), pairs_all);
                fc.enabled = 1;
                fused = true;
                opts->fused_applied = true;
            }
        }
    }
    if (fused) {
        if constexpr (sizeof(OutT) == 2) {
            auto kern = mn_major ? w8a8_pair_kernel<OutT, true, true> : w8a8_pair_kernel<OutT, false, true>;
            QMM_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             static_cast<int>(kPairSmemBytes)));
            cfg.blockDim = dim3(kPFusedThreads);
            cfg.gridDim = dim3(static_cast<unsigned>(2 * pairs_all));  // also the CTAs without a tile communicate
            QMM_CUDA_OK(cudaLaunchKernelEx(&cfg, kern, ta, tb, tout, push, fc, ep, static_cast<int>(K), use_tma_store,
                                           raster, status));
        }
    } else {
        auto kern = mn_major ? w8a8_pair_kernel<OutT, true, false> : w8a8_pair_kernel<OutT, false, false>;
        QMM_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(kPairSmemBytes)));
        QMM_CUDA_OK(cudaLaunchKernelEx(&cfg, kern, ta, tb, tout, push, fc, ep, static_cast<int>(K), use_tma_store, raster,
                                       status));
    }
    return QMM_OK;
}

}  // namespace

int launch_pair(const int8_t *x1, int64_t ld_x1, const int8_t *x2, int64_t x2_sk, int64_t x2_sn,
                const EpilogueParams &ep, int out_dtype, int64_t K, LaunchOptions *opts, cudaStream_t stream) {
    switch (out_dtype) {
        case QMM_DTYPE_BF16:
            return launch_pair_t<__nv_bfloat16>(x1, ld_x1, x2, x2_sk, x2_sn, ep, K, opts, stream);
        case QMM_DTYPE_F16:
            return launch_pair_t<__half>(x1, ld_x1, x2, x2_sk, x2_sn, ep, K, opts, stream);
        default:
            return launch_pair_t<int32_t>(x1, ld_x1, x2, x2_sk, x2_sn, ep, K, opts, stream);
    }
}

}  // namespace qmm
