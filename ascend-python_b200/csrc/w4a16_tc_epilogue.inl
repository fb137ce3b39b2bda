        // ---------------- scaling / epilogue warps (included inside w4a16_tc_kernel) ----------------
        // Four warps per 128-column sub-tile; thread = TMEM lane = one output column.  acc[m] collects,
        // group by group,  scale[g,n] * (P'[n,m] + (offset[g,n] - BIAS) * xsum[g,m]),  P' = sum_k (w + BIAS) * x.
        const int sub = (warp - kWEpiFirstWarp) >> 2;                               // sub-tile of the 512-column unit
        const int quarter = warp & 3;                                  // TMEM lanes [32*quarter, +32)
        const int row = quarter * 32 + lane;                           // lane of the accumulator
        const int n_local = (row & ~7) + ((row & 1) << 2) + ((row & 7) >> 1);  // undo the 0,4,1,5,2,6,3,7 order
        const bool leader_thread = (threadIdx.x == kWEpiFirstWarp * 32);
        const W4Params &w = p.w;
        const T *scale = static_cast<const T *>(w.scale);
        const T *offset = static_cast<const T *>(w.offset);
        const T *bias = static_cast<const T *>(w.bias);
        T *out = static_cast<T *>(w.out);
        const int M = static_cast<int>(w.M);
        float acc[ACC_M];
        int64_t local = 0;
        int64_t u = u_begin;
        // the group sums of x are read once per CTA into shared memory (broadcast reads afterwards)
        if (p.xs_in_smem) {
            for (int i = threadIdx.x - kWEpiFirstWarp * 32; i < p.ngroups * p.mpad; i += kWEpiWarps * 32)
                xs_smem[i] = __ldg(p.xsum + (i / p.mpad) * kWMaxM + (i % p.mpad));
            wepi_bar_sync();
        }
        // scale and offset of a unit are fetched one unit ahead, so that their latency hides
        // behind the wait for the accumulator
        auto load_so = [&](int64_t unit_idx, float &s_out, float &o_out) {
            s_out = 0.0f;
            o_out = 0.0f;
            if (unit_idx < u_end) {
                const int t2 = static_cast<int>(unit_idx / p.ngroups);
                const int g2 = static_cast<int>(unit_idx - static_cast<int64_t>(t2) * p.ngroups);
                const int64_t n2 = static_cast<int64_t>(t2) * kWUnitN + sub * kWTileN + n_local;
                if (n2 < w.N) {
                    s_out = to_float(scale[static_cast<int64_t>(g2) * w.N + n2]);
                    o_out = (offset != nullptr ? to_float(offset[static_cast<int64_t>(g2) * w.N + n2]) : 0.0f) -
                            W4Magic<T>::kBias;
                }
            }
        };
        float s_next, o_next;
        load_so(u, s_next, o_next);
        while (u < u_end) {
            const int unit = static_cast<int>(u / p.ngroups);
            const int64_t unit_begin = static_cast<int64_t>(unit) * p.ngroups;
            const int64_t unit_end = unit_begin + p.ngroups;
            const int64_t seg_end = unit_end < u_end ? unit_end : u_end;
            const bool whole = (u == unit_begin && seg_end == unit_end);
            const int64_t n = static_cast<int64_t>(unit) * kWUnitN + sub * kWTileN + n_local;
            const bool n_ok = n < w.N;
#pragma unroll
            for (int m = 0; m < ACC_M; ++m) acc[m] = 0.0f;

            for (; u < seg_end; ++u, ++local) {
                const int g = static_cast<int>(u - unit_begin);
                const uint32_t pb = static_cast<uint32_t>(local % kWAccBufs);
                const uint32_t pb_phase = static_cast<uint32_t>((local / kWAccBufs) & 1);
                const float s = s_next, o = o_next;
                load_so(u + 1, s_next, o_next);
                if (!mbar_wait(smem_u32(&tail->tmem_full[pb]), pb_phase, abort_flag, 0x37)) {
                    *reinterpret_cast<volatile uint32_t *>(&tail->epi_abort) = 1;
                    break;
                }
                tc_fence_after();
                const float *xs = p.xs_in_smem ? (xs_smem + g * p.mpad) : (p.xsum + g * kWMaxM);
                const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                                       pb * (kWSub * kWMaxM) + sub * kWMaxM;
#pragma unroll
                for (int c = 0; c < ACC_M; c += 16) {
                    if (c < p.mpad) {
                        uint32_t v[16];
                        tmem_ld_32x16(taddr + c, v);
                        tmem_ld_wait();
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            acc[c + j] = fmaf(s, fmaf(o, xs[c + j], __uint_as_float(v[j])), acc[c + j]);
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&tail->tmem_empty[pb]));
            }
            // The sixteen warps meet at named barriers below, so they leave the loop together or not
            // at all: every warp reaches this barrier (its waits are bounded), then reads the verdict.
            wepi_bar_sync();
            if (*reinterpret_cast<volatile uint32_t *>(&tail->epi_abort) != 0) break;

            const float b = (n_ok && bias != nullptr) ? to_float(bias[n]) : 0.0f;
            if (whole) {
                if (n_ok) {
#pragma unroll
                    for (int m = 0; m < ACC_M; ++m)
                        if (m < M) out[static_cast<int64_t>(m) * w.ld_out + n] = from_float<T>(acc[m] + b);
                }
            } else {
                // this CTA's share of the unit goes to its slot; the CTA that arrives last adds the
                // slots in slot order, so the sum does not depend on who arrives when
                const int first_cta = cta_of_unit(unit_begin, total, G);
                const int last_cta = cta_of_unit(unit_end - 1, total, G);
                const int nslots = last_cta - first_cta + 1;
                const int slot = static_cast<int>(blockIdx.x) - first_cta;
                const int64_t slot_elems = static_cast<int64_t>(kWSub) * p.mpad * kWTileN;
                float *unit_slots = p.slots + static_cast<int64_t>(unit) * p.max_slots * slot_elems;
                const int64_t my_off = static_cast<int64_t>(sub) * p.mpad * kWTileN + row;
                float *mine = unit_slots + slot * slot_elems + my_off;
#pragma unroll
                for (int m = 0; m < ACC_M; ++m)
                    if (m < M) __stcg(mine + m * kWTileN, acc[m]);
                wepi_bar_sync();
                if (leader_thread) {
                    __threadfence();
                    const uint32_t old = atomicAdd(p.counters + unit, 1u);
                    tail->is_last = (old + 1 == static_cast<uint32_t>(nslots)) ? 1u : 0u;
                    if (old + 1 == static_cast<uint32_t>(nslots)) p.counters[unit] = 0;
                    __threadfence();
                }
                wepi_bar_sync();
                if (tail->is_last && n_ok) {
                    // slot sums, sixteen rows at a time so that the loads of a batch overlap
                    for (int m0 = 0; m0 < M; m0 += 16) {
                        float v[16];
#pragma unroll
                        for (int j = 0; j < 16; ++j) v[j] = 0.0f;
                        for (int sl = 0; sl < nslots; ++sl) {
#pragma unroll
                            for (int j = 0; j < 16; ++j)
                                if (m0 + j < M)
                                    v[j] += __ldcg(unit_slots + sl * slot_elems + my_off + (m0 + j) * kWTileN);
                        }
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            if (m0 + j < M) out[static_cast<int64_t>(m0 + j) * w.ld_out + n] = from_float<T>(v[j] + b);
                    }
                }
                wepi_bar_sync();  // is_last is rewritten by the next shared unit
            }
        }
