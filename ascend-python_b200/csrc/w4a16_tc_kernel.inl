// Body of the W4A16 tensor-core kernel; included by w4a16_tc.cu only.
namespace qmm {
namespace {

template <typename T>
__global__ void __launch_bounds__(kWThreads, 1)
w4a16_tc_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
                WTcParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *smem_aligned = smem_raw + (smem_base - smem_u32(smem_raw));
    // [A tiles][stages: packed words + activations][barriers]
    const uint32_t a_base = smem_base;
    const uint32_t st_base = smem_base + kWABufs * kWABytes;
    WSmemTail *tail = reinterpret_cast<WSmemTail *>(smem_aligned + kWABufs * kWABytes + p.stages * p.stage_bytes);
    float *xs_smem = reinterpret_cast<float *>(tail + 1);  // [ngroups][mpad] when p.xs_in_smem
    volatile uint32_t *abort_flag = &tail->abort_flag;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int64_t total = static_cast<int64_t>(p.tiles_n) * p.ngroups;
    const int64_t G = gridDim.x;
    const int64_t u_begin = total * blockIdx.x / G;
    const int64_t u_end = total * (blockIdx.x + 1) / G;
    const int kbg = p.kb_per_group;

    if (threadIdx.x == 0) {
        for (int s = 0; s < p.stages; ++s) {
            mbar_init(smem_u32(&tail->full[s]), 1);
            mbar_init(smem_u32(&tail->empty[s]), 1);
        }
        for (int a = 0; a < kWABufs; ++a) {
            mbar_init(smem_u32(&tail->a_full[a]), 1);
            mbar_init(smem_u32(&tail->a_empty[a]), 1);
        }
        for (int b = 0; b < kWAccBufs; ++b) {
            mbar_init(smem_u32(&tail->tmem_full[b]), 1);
            mbar_init(smem_u32(&tail->tmem_empty[b]), 4);
        }
        tail->abort_flag = 0;
        tail->is_last = 0;
        tail->epi_abort = 0;
        mbar_fence_init();
    }
    if (warp == 0 && lane == 0) {
        tma_prefetch_desc(&tmap_w);
        tma_prefetch_desc(&tmap_x);
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(&tail->tmem_base), kWTmemCols);
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
        for (int64_t u = u_begin; u < u_end && ok; ++u) {
            const int tile = static_cast<int>(u / p.ngroups);
            const int g = static_cast<int>(u - static_cast<int64_t>(tile) * p.ngroups);
            for (int kb = 0; kb < kbg; ++kb) {
                ok = mbar_wait(smem_u32(&tail->empty[stage]), phase ^ 1, abort_flag, 0x31);
                if (!ok) break;
                if (lane == 0) {
                    const uint32_t full = smem_u32(&tail->full[stage]);
                    const uint32_t sw = st_base + stage * p.stage_bytes;
                    const uint32_t sx = sw + kWPackedBytes;
                    const int k0 = (g * kbg + kb) * kWBK;
                    mbar_expect_tx(full, static_cast<uint32_t>(p.stage_bytes));
                    tma_load_2d(sw, &tmap_w, tile * (kWTileN / 8), k0, full);  // [64 k][16 words]
                    tma_load_2d(sx, &tmap_x, k0, 0, full);                      // [mpad m][64 k]
                }
                __syncwarp();
                if (++stage == static_cast<uint32_t>(p.stages)) {
                    stage = 0;
                    phase ^= 1;
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        const uint32_t idesc = make_idesc(/*c=f32*/ 1, W4Magic<T>::kFmt, W4Magic<T>::kFmt, /*a MN-major*/ 1,
                                          /*b K-major*/ 0, kWTileN, static_cast<uint32_t>(p.mpad));
        uint32_t stage = 0, phase = 0, abuf = 0, aphase = 0;
        int local = 0;
        bool ok = true;
        for (int64_t u = u_begin; u < u_end && ok; ++u, ++local) {
            const uint32_t pb = local % kWAccBufs;
            const uint32_t pb_phase = (local / kWAccBufs) & 1;
            ok = mbar_wait(smem_u32(&tail->tmem_empty[pb]), pb_phase ^ 1, abort_flag, 0x32);
            if (!ok) break;
            tc_fence_after();
            const uint32_t d_tmem = tmem_base + pb * kWMaxM;
            for (int kb = 0; kb < kbg; ++kb) {
                // the activations arrive with the stage, the dequantized weights with the A tile
                ok = mbar_wait(smem_u32(&tail->full[stage]), phase, abort_flag, 0x33) &&
                     mbar_wait(smem_u32(&tail->a_full[abuf]), aphase, abort_flag, 0x34);
                if (!ok) break;
                tc_fence_after();
                if (lane == 0) {
                    const uint32_t sa = a_base + abuf * kWABytes;
                    const uint32_t sx = st_base + stage * p.stage_bytes + kWPackedBytes;
#pragma unroll
                    for (int k = 0; k < kWBK / 16; ++k) {
                        // A: MN-major; 64 columns (128 bytes) per row, 8-k-row groups 1024 bytes apart,
                        // second 64-column half 8 KiB further; 16 k rows = 2048 bytes per MMA
                        const uint64_t adesc = make_smem_desc_sw128(sa + k * 2048, kWABytes / 2, 1024);
                        // B: K-major; 16 k elements = 32 bytes per MMA
                        const uint64_t bdesc = make_smem_desc_sw128(sx + k * 32, 16, 1024);
                        mma_f16_ss(d_tmem, adesc, bdesc, idesc, (kb > 0 || k > 0) ? 1u : 0u);
                    }
                    tc_commit(smem_u32(&tail->empty[stage]));
                    tc_commit(smem_u32(&tail->a_empty[abuf]));
                }
                __syncwarp();
                if (++stage == static_cast<uint32_t>(p.stages)) {
                    stage = 0;
                    phase ^= 1;
                }
                if (++abuf == kWABufs) {
                    abuf = 0;
                    aphase ^= 1;
                }
            }
            if (ok && lane == 0) tc_commit(smem_u32(&tail->tmem_full[pb]));
            __syncwarp();
        }
    } else if (warp < 6) {
        // ---------------- dequantization warps ----------------
        // Warp w converts the k-blocks i = w, w+4, ... of this CTA into A buffer w, so four k-blocks
        // are in flight and the fixed costs (barrier wake-up, proxy fence) are paid once per 8 KiB of
        // packed words and warp.  Per step a warp reads two packed rows (lane -> word, conflict-free)
        // and writes 32 vectors of 16 bytes (conflict-free under the 128-byte swizzle).
        const int wq = warp - 2;
        const int wd = lane & 15;      // packed word within the row: columns 8*wd .. 8*wd+7 of the tile
        const int half = wd >> 3;      // which 64-column half of the tile
        const int j = wd & 7;          // 16-byte chunk within the 128-byte row of that half
        const int64_t kblocks = (u_end - u_begin) * kbg;
        for (int64_t i = wq; i < kblocks; i += kWABufs) {
            const uint32_t stage = static_cast<uint32_t>(i % p.stages);
            const uint32_t phase = static_cast<uint32_t>((i / p.stages) & 1);
            const uint32_t aphase = static_cast<uint32_t>((i / kWABufs) & 1);
            if (!(mbar_wait(smem_u32(&tail->full[stage]), phase, abort_flag, 0x35) &&
                  mbar_wait(smem_u32(&tail->a_empty[wq]), aphase ^ 1, abort_flag, 0x36)))
                break;
            const uint8_t *packed = smem_aligned + kWABufs * kWABytes + stage * p.stage_bytes + wd * 4;
            uint8_t *dst_half = smem_aligned + wq * kWABytes + half * (kWABytes / 2);
#pragma unroll 8
            for (int it = 0; it < kWBK / 2; ++it) {
                const int r = it * 2 + (lane >> 4);
                const uint32_t u = *reinterpret_cast<const uint32_t *>(packed + r * 64) ^ 0x88888888u;
                uint4 v;  // two's complement nibble -> offset binary -> BIAS + w in a 16-bit float
                v.x = W4Magic<T>::finish((u & 0x000f000fu) | W4Magic<T>::kExp);          // columns 0 and 4
                v.y = W4Magic<T>::finish(((u >> 4) & 0x000f000fu) | W4Magic<T>::kExp);   // columns 1 and 5
                v.z = W4Magic<T>::finish(((u >> 8) & 0x000f000fu) | W4Magic<T>::kExp);   // columns 2 and 6
                v.w = W4Magic<T>::finish(((u >> 12) & 0x000f000fu) | W4Magic<T>::kExp);  // columns 3 and 7
                *reinterpret_cast<uint4 *>(dst_half + (r >> 3) * 1024 + (r & 7) * 128 + ((j ^ (r & 7)) << 4)) = v;
            }
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&tail->a_full[wq]));
        }
    } else {
#include "w4a16_tc_epilogue.inl"
    }

    // ---------------- teardown ----------------
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && tail->abort_flag != 0 && p.status != nullptr) atomicMax(p.status, tail->abort_flag);
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kWTmemCols);
    }
}

}  // namespace
}  // namespace qmm
