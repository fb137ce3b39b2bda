// Body of the W4A16 tensor-core kernel; included by w4a16_tc.cu only.
namespace qmm {
namespace {

// ACC_M: accumulator registers per epilogue thread (32 or 64 token rows)
template <typename T, int ACC_M>
__global__ void __launch_bounds__(kWThreads, 1)
w4a16_tc_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
                WTcParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *smem_aligned = smem_raw + (smem_base - smem_u32(smem_raw));
    // [A tiles][activation tiles][packed-weight stages][barriers][group sums of x]
    constexpr uint32_t kAOff = 0;
    constexpr uint32_t kXOff = kWABufs * kWABytes;
    const uint32_t kWOff = kXOff + kWXStages * p.x_bytes;
    WSmemTail *tail = reinterpret_cast<WSmemTail *>(smem_aligned + kWOff + kWStages * kWPackedBytes);
    float *xs_smem = reinterpret_cast<float *>(tail + 1);  // [ngroups][mpad] when p.xs_in_smem
    volatile uint32_t *abort_flag = &tail->abort_flag;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int64_t total = static_cast<int64_t>(p.units_n) * p.ngroups;
    const int64_t G = gridDim.x;
    const int64_t u_begin = total * blockIdx.x / G;
    const int64_t u_end = total * (blockIdx.x + 1) / G;
    const int spg = p.steps_per_group;  // 32-row steps per group (even: groups are multiples of 64 rows)
    const int64_t nsteps = (u_end - u_begin) * spg;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kWStages; ++s) {
            mbar_init(smem_u32(&tail->full[s]), 1);
            mbar_init(smem_u32(&tail->empty[s]), kWDeqWarpsPerStep);
        }
        for (int s = 0; s < kWXStages; ++s) {
            mbar_init(smem_u32(&tail->x_full[s]), 1);
            mbar_init(smem_u32(&tail->x_empty[s]), kWMmaWarps);
        }
        for (int a = 0; a < kWABufs; ++a) {
            mbar_init(smem_u32(&tail->a_full[a]), kWDeqWarpsPerStep);
            mbar_init(smem_u32(&tail->a_empty[a]), kWMmaWarps);
        }
        for (int b = 0; b < kWAccBufs; ++b) {
            mbar_init(smem_u32(&tail->tmem_full[b]), kWMmaWarps);
            mbar_init(smem_u32(&tail->tmem_empty[b]), kWEpiWarps);
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
        // step i of this CTA belongs to unit u_begin + i / spg and covers rows k0 .. k0+31 of it;
        // all counters advance incrementally (no divisions in the loop)
        int unit = static_cast<int>(u_begin / p.ngroups);
        int g = static_cast<int>(u_begin - static_cast<int64_t>(unit) * p.ngroups);
        int s_in_g = 0;
        uint32_t st = 0, ph = 0, xs = 0, xph = 0;
        const uint32_t full0 = smem_u32(&tail->full[0]), empty0 = smem_u32(&tail->empty[0]);
        const uint32_t xfull0 = smem_u32(&tail->x_full[0]), xempty0 = smem_u32(&tail->x_empty[0]);
        for (int64_t i = 0; i < nsteps; ++i) {
            const int k0 = (g * spg + s_in_g) * kWStepK;
            if ((s_in_g & 1) == 0) {
                // a fresh 64-row activation tile every other step
                if (!mbar_wait(xempty0 + xs * 8, xph ^ 1, abort_flag, 0x30)) break;
                if (lane == 0) {
                    mbar_expect_tx(xfull0 + xs * 8, static_cast<uint32_t>(p.x_bytes));
                    tma_load_2d(smem_base + kXOff + xs * p.x_bytes, &tmap_x, k0, 0, xfull0 + xs * 8);  // [mpad m][64 k]
                }
                if (++xs == kWXStages) {
                    xs = 0;
                    xph ^= 1;
                }
            }
            if (!mbar_wait(empty0 + st * 8, ph ^ 1, abort_flag, 0x31)) break;
            if (lane == 0) {
                mbar_expect_tx(full0 + st * 8, kWPackedBytes);
                tma_load_2d(smem_base + kWOff + st * kWPackedBytes, &tmap_w, unit * (kWUnitN / 8), k0, full0 + st * 8);
            }
            __syncwarp();
            if (++st == kWStages) {
                st = 0;
                ph ^= 1;
            }
            if (++s_in_g == spg) {
                s_in_g = 0;
                if (++g == p.ngroups) {
                    g = 0;
                    ++unit;
                }
            }
        }
    } else if (warp < kWDeqFirstWarp) {
        // ---------------- MMA issuers ----------------
        // Issuer mi owns the sub-tiles 2*mi and 2*mi+1 (their accumulators are disjoint TMEM columns, so
        // the two issuers never touch the same data and each accumulator still sees its MMAs in k
        // order).  The whole warp runs the loop with warp-uniform operands; one election per step
        // covers the four MMAs and the commit.
        const int mi = warp - 1;
        const uint32_t idesc = make_idesc(/*c=f32*/ 1, W4Magic<T>::kFmt, W4Magic<T>::kFmt, /*a MN-major*/ 1,
                                          /*b K-major*/ 0, kWTileN, static_cast<uint32_t>(p.mpad));
        constexpr uint32_t kDescHi = smem_desc_hi_sw128(1024);
        // A sub-tile: MN-major; two 64-column halves 2 KiB apart (leading offset), 8-row groups 1 KiB apart
        const uint32_t a_lo0 = smem_desc_lo(smem_base + kAOff + mi * kWSubPerMma * kWASubBytes, kWASubBytes / 2);
        // B: K-major activations; 16 k elements = 32 bytes (+2) per MMA within the 64-k tile
        const uint32_t b_lo0 = smem_desc_lo(smem_base + kXOff, 16);
        const uint32_t x_step = static_cast<uint32_t>(p.x_bytes) >> 4;
        const uint32_t afull0 = smem_u32(&tail->a_full[0]), aempty0 = smem_u32(&tail->a_empty[0]);
        const uint32_t xfull0 = smem_u32(&tail->x_full[0]), xempty0 = smem_u32(&tail->x_empty[0]);
        static_assert(kWSubPerMma == 2, "the fused issue helper covers two sub-tiles");
        bool ok = true;
        uint32_t ab = 0, aph = 0, xs = 0, xph = 0, pb = 0, pb_phase = 0;
        const int64_t nunits = u_end - u_begin;
        for (int64_t local = 0; local < nunits && ok; ++local) {
            ok = mbar_wait(smem_u32(&tail->tmem_empty[pb]), pb_phase ^ 1, abort_flag, 0x32);
            if (!ok) break;
            tc_fence_after();
            const uint32_t d0 = tmem_base + pb * (kWSub * kWMaxM) + (mi * kWSubPerMma) * kWMaxM;
            uint32_t accumulate = 0;
            for (int s = 0; s < spg; ++s) {
                ok = mbar_wait(afull0 + ab * 8, aph, abort_flag, 0x34);
                if (ok && (s & 1) == 0) ok = mbar_wait(xfull0 + xs * 8, xph, abort_flag, 0x33);
                if (!ok) break;
                tc_fence_after();
                const uint32_t b_lo = b_lo0 + xs * x_step + 4 * (s & 1);
                const uint32_t a_lo = a_lo0 + ab * (kWABytes >> 4);
                mma_f16_ss_warp_2x2_commit(d0, d0 + kWMaxM,
                                           desc64(a_lo, kDescHi), desc64(a_lo + (kWAHalfBytes >> 4), kDescHi),
                                           desc64(a_lo + (kWASubBytes >> 4), kDescHi),
                                           desc64(a_lo + ((kWAHalfBytes + kWASubBytes) >> 4), kDescHi),
                                           desc64(b_lo, kDescHi), desc64(b_lo + 2, kDescHi), idesc, accumulate,
                                           aempty0 + ab * 8);
                accumulate = 1;
                if (++ab == kWABufs) {
                    ab = 0;
                    aph ^= 1;
                }
                if (s & 1) {
                    tc_commit_warp(xempty0 + xs * 8);
                    if (++xs == kWXStages) {
                        xs = 0;
                        xph ^= 1;
                    }
                }
            }
            if (ok) tc_commit_warp(smem_u32(&tail->tmem_full[pb]));
            if (++pb == kWAccBufs) {
                pb = 0;
                pb_phase ^= 1;
            }
        }
    } else if (warp < kWEpiFirstWarp) {
        // ---------------- dequantization warps ----------------
        // Two groups of four warps take alternate steps, so that one group's loads and barrier waits
        // overlap the other's stores; within a step every warp converts eight of the 32 k rows.  Per
        // row a warp reads 2 x 32 consecutive words (conflict-free) and writes 2 x 32 vectors of 16
        // bytes (conflict-free under the swizzle).  The packed words of a step are in registers before
        // the first store, so the stage is handed back to the producer early.
        const int w8 = warp - kWDeqFirstWarp;
        const int grp = w8 / kWDeqWarpsPerStep;  // steps grp, grp + kWDeqGroups, ...
        const int w4 = w8 % kWDeqWarpsPerStep;   // rows 8*w4 .. 8*w4+7 of the step
        const int kk = w4 >> 1;                  // which 16-row half of the step
        const int hr = w4 & 1;                   // which eight k rows of that half
        // lane-dependent parts of the destination address, for words 0..31 and 32..63 of a row
        uint32_t base[2], j16[2];
#pragma unroll
        for (int par = 0; par < 2; ++par) {
            const int wd = (par << 5) + lane;  // word within the row: columns 8*wd .. 8*wd+7
            base[par] = kk * kWAHalfBytes + (wd >> 4) * kWASubBytes + ((wd >> 3) & 1) * (kWASubBytes / 2) + hr * 1024;
            j16[par] = (wd & 7) << 4;          // 16-byte chunk within the 128-byte row
        }
        static_assert(kWStages % kWDeqGroups == 0, "a group revisits the same stages");
        uint32_t st = grp, ph = 0;
        for (int64_t i = grp; i < nsteps; i += kWDeqGroups) {
            const uint32_t ab = static_cast<uint32_t>(i % kWABufs);
            const uint32_t aph = static_cast<uint32_t>((i / kWABufs) & 1);
            if (!mbar_wait(smem_u32(&tail->full[st]), ph, abort_flag, 0x35)) break;
            const uint32_t *packed =
                reinterpret_cast<const uint32_t *>(smem_aligned + kWOff + st * kWPackedBytes) + w4 * 512 + lane;
            uint32_t words[16];
#pragma unroll
            for (int it = 0; it < 16; ++it) words[it] = packed[it * 32];
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&tail->empty[st]));
            if (!mbar_wait(smem_u32(&tail->a_empty[ab]), aph ^ 1, abort_flag, 0x36)) break;
            uint8_t *abuf = smem_aligned + kAOff + ab * kWABytes;
#pragma unroll
            for (int it = 0; it < 16; ++it) {
                const int r7 = it >> 1;      // k row within this warp's eight rows
                const int par = it & 1;
                const uint32_t u = words[it] ^ 0x88888888u;  // two's complement nibble -> offset binary
                uint4 v;                                     // -> BIAS + w in a 16-bit float
                v.x = W4Magic<T>::finish((u & 0x000f000fu) | W4Magic<T>::kExp);          // columns 0 and 4
                v.y = W4Magic<T>::finish(((u >> 4) & 0x000f000fu) | W4Magic<T>::kExp);   // columns 1 and 5
                v.z = W4Magic<T>::finish(((u >> 8) & 0x000f000fu) | W4Magic<T>::kExp);   // columns 2 and 6
                v.w = W4Magic<T>::finish(((u >> 12) & 0x000f000fu) | W4Magic<T>::kExp);  // columns 3 and 7
                *reinterpret_cast<uint4 *>(abuf + base[par] + r7 * 128 + (j16[par] ^ (r7 << 4))) = v;
            }
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&tail->a_full[ab]));
            st += kWDeqGroups;
            if (st >= kWStages) {
                st -= kWStages;
                ph ^= 1;
            }
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
