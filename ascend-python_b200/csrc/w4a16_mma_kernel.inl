// Body of the register-operand W4A16 kernel; included by w4a16_mma.cu only.
namespace qmm {
namespace {

// MT: token tiles of eight rows (1: M <= 8, 2: M <= 16); SETS: consumer sets taking the groups in turn;
// YS: the running outputs live in shared memory (one private column per thread) instead of registers
template <typename T, int MT, int SETS, bool YS>
__global__ void __launch_bounds__((1 + SETS * kGColWarps) * 32, 1)
w4a16_mma_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x, GParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *smem_aligned = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t nstages = static_cast<uint32_t>(p.nstages);  // ring length actually used
    GSmemTail *tail = reinterpret_cast<GSmemTail *>(smem_aligned + nstages * kGStageBytes);
    volatile uint32_t *abort_flag = &tail->abort_flag;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int64_t total = static_cast<int64_t>(p.units_n) * p.ngroups;
    const int64_t G = gridDim.x;
    const int64_t u_begin = total * blockIdx.x / G;
    const int64_t u_end = total * (blockIdx.x + 1) / G;
    const int spg = p.stages_per_group;
    const W4Params &w = p.w;

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < nstages; ++s) {
            mbar_init(smem_u32(&tail->full[s]), 1);
            mbar_init(smem_u32(&tail->empty[s]), kGColWarps);
        }
        tail->abort_flag = 0;
        for (int s = 0; s < SETS; ++s) tail->is_last[s] = 0;
        mbar_fence_init();
        tma_prefetch_desc(&tmap_w);
        tma_prefetch_desc(&tmap_x);
    }
    __syncthreads();

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        int unit = static_cast<int>(u_begin / p.ngroups);
        int g = static_cast<int>(u_begin - static_cast<int64_t>(unit) * p.ngroups);
        uint32_t st = 0, ph = 0;
        const uint32_t full0 = smem_u32(&tail->full[0]), empty0 = smem_u32(&tail->empty[0]);
        constexpr uint32_t kTx = kGPackedBytes + MT * 1024;
        bool ok = true;
        for (int64_t it = u_begin; it < u_end && ok; ++it) {
            for (int s = 0; s < spg; ++s) {
                const int k0 = (g * spg + s) * kGStageK;
                if (!mbar_wait(empty0 + st * 8, ph ^ 1, abort_flag, 0x40)) {
                    ok = false;
                    break;
                }
                if (lane == 0) {
                    const uint32_t dst = smem_base + st * kGStageBytes;
                    mbar_expect_tx(full0 + st * 8, kTx);
                    tma_load_2d(dst, &tmap_w, unit * (kGUnitN / 8), k0, full0 + st * 8);
                    tma_load_2d(dst + kGBoxBytes, &tmap_w, unit * (kGUnitN / 8) + 32, k0, full0 + st * 8);
                    tma_load_2d(dst + kGPackedBytes, &tmap_x, k0, 0, full0 + st * 8);  // [8 MT tokens][64 k]
                }
                __syncwarp();
                if (++st == nstages) {
                    st = 0;
                    ph ^= 1;
                }
            }
            if (++g == p.ngroups) {
                g = 0;
                ++unit;
            }
        }
    } else {
        // ---------------- consumer warps ----------------
        const int cwid = warp - 1;
        const int set = cwid / kGColWarps;  // takes the items whose index within this CTA is set mod SETS
        const int cw = cwid % kGColWarps;   // columns [128 cw, 128 cw + 128) of the unit
        const int q = lane & 3;             // k pair within a k block / token pair of the accumulator
        const int gi = lane >> 2;           // word column within the warp's first eight / token of the x operand
        const T *scale = static_cast<const T *>(w.scale);
        const T *offset = static_cast<const T *>(w.offset);
        const T *bias = static_cast<const T *>(w.bias);
        T *out = static_cast<T *>(w.out);
        const int M = static_cast<int>(w.M);

        // Shared-memory offsets of this lane's words inside a stage.  A box row is 128 bytes; the
        // 16-byte chunk index is XORed with (row & 7).  The lane reads rows 2q, 2q+1 (+8) of each k
        // block, from word column gi (chunk ca) and gi + 8 (chunk ca + 2) of the warp's sixteen.
        const uint32_t box = static_cast<uint32_t>(cw >> 1) * kGBoxBytes;
        const uint32_t ca = 4u * (cw & 1) + (gi >> 2);
        const uint32_t inw = (gi & 3) * 4u;
        const uint32_t r0 = 2u * q, r1 = 2u * q + 1u;
        const uint32_t offA0 = box + r0 * 128u + ((ca ^ r0) << 4) + inw;
        const uint32_t offA1 = box + r1 * 128u + ((ca ^ r1) << 4) + inw;
        const uint32_t offB0 = box + r0 * 128u + (((ca + 2u) ^ r0) << 4) + inw;
        const uint32_t offB1 = box + r1 * 128u + (((ca + 2u) ^ r1) << 4) + inw;
        // activations: token row gi (and gi + 8), k pair (2q, 2q+1) of the block and the pair 8 further
        const uint32_t xoff = kGPackedBytes + gi * 128u + 4u * q;

        float y[MT][8][4];
        // running outputs: registers, or [index][consumer thread] in shared memory (conflict-free)
        float *ysm = reinterpret_cast<float *>(smem_aligned + nstages * kGStageBytes + 1024) + (threadIdx.x - 32);
        auto Y = [&](int mt, int j, int c) -> float & {
            if constexpr (YS)
                return ysm[((mt * 8 + j) * 4 + c) * (SETS * kGColWarps * 32)];
            else
                return y[mt][j][c];
        };
        float acc[MT][8][4];
        float accx[MT][4];
        const uint32_t ones[4] = {GMagic<T>::kOnes, GMagic<T>::kOnes, GMagic<T>::kOnes, GMagic<T>::kOnes};
        // constants of the extraction, kept in registers (the logic instruction takes one immediate only)
        const uint32_t nib_mask = opaque_u32(0x000f000fu);
        const uint32_t nib_flip = opaque_u32(GMagic<T>::kExp | 0x00080008u);
        bool ok = true;

        int64_t seg_begin = u_begin;
        while (seg_begin < u_end) {
            const int unit = static_cast<int>(seg_begin / p.ngroups);
            const int64_t unit_begin = static_cast<int64_t>(unit) * p.ngroups;
            const int64_t unit_end = unit_begin + p.ngroups;
            const int64_t seg_end = unit_end < u_end ? unit_end : u_end;
            // first column of this lane's two runs of eight columns: n0 and n0 + 64
            const int64_t n0 = static_cast<int64_t>(unit) * kGUnitN + cw * 128 + gi * 8;
            const bool okA = n0 < w.N, okB = n0 + 64 < w.N;
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                for (int j = 0; j < 8; ++j)
#pragma unroll
                    for (int c = 0; c < 4; ++c) Y(mt, j, c) = 0.0f;

            // first item of this set in the segment: local indices are counted from u_begin
            int64_t it = seg_begin + ((set - (seg_begin - u_begin)) % SETS + SETS) % SETS;
            for (; it < seg_end; it += SETS) {
                const int g = static_cast<int>(it - unit_begin);
                // scale and offset of the group: requested now, used after the group's MMAs
                uint4 sA = make_uint4(0, 0, 0, 0), sB = sA, oA = sA, oB = sA;
                {
                    const int64_t row = static_cast<int64_t>(g) * w.N;
                    if (okA) sA = __ldg(reinterpret_cast<const uint4 *>(scale + row + n0));
                    if (okB) sB = __ldg(reinterpret_cast<const uint4 *>(scale + row + n0 + 64));
                    if (offset != nullptr) {
                        if (okA) oA = __ldg(reinterpret_cast<const uint4 *>(offset + row + n0));
                        if (okB) oB = __ldg(reinterpret_cast<const uint4 *>(offset + row + n0 + 64));
                    }
                }
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
                    for (int j = 0; j < 8; ++j)
#pragma unroll
                        for (int c = 0; c < 4; ++c) acc[mt][j][c] = 0.0f;
#pragma unroll
                    for (int c = 0; c < 4; ++c) accx[mt][c] = 0.0f;
                }
                const uint32_t step0 = static_cast<uint32_t>(it - u_begin) * static_cast<uint32_t>(spg);
                for (int s = 0; s < spg; ++s) {
                    const uint32_t step = step0 + s;
                    const uint32_t st = step % nstages;
                    const uint32_t ph = (step / nstages) & 1u;
                    if (ok && !mbar_wait(smem_u32(&tail->full[st]), ph, abort_flag, 0x41)) ok = false;
                    const uint8_t *sb = smem_aligned + st * kGStageBytes;
#pragma unroll
                    for (int kb = 0; kb < 4; ++kb) {
                        const uint8_t *kbase = sb + kb * 2048u;
                        uint32_t wd[8];
                        wd[0] = *reinterpret_cast<const uint32_t *>(kbase + offA0);          // column gi,     row 2q
                        wd[1] = *reinterpret_cast<const uint32_t *>(kbase + offA1);          //                row 2q+1
                        wd[2] = *reinterpret_cast<const uint32_t *>(kbase + offA0 + 1024u);  //                row 2q+8
                        wd[3] = *reinterpret_cast<const uint32_t *>(kbase + offA1 + 1024u);  //                row 2q+9
                        wd[4] = *reinterpret_cast<const uint32_t *>(kbase + offB0);          // column gi + 8
                        wd[5] = *reinterpret_cast<const uint32_t *>(kbase + offB1);
                        wd[6] = *reinterpret_cast<const uint32_t *>(kbase + offB0 + 1024u);
                        wd[7] = *reinterpret_cast<const uint32_t *>(kbase + offB1 + 1024u);
                        uint32_t xb[MT][2];
#pragma unroll
                        for (int mt = 0; mt < MT; ++mt) {
                            xb[mt][0] = *reinterpret_cast<const uint32_t *>(sb + xoff + mt * 1024u + (((2u * kb) ^ gi) << 4));
                            xb[mt][1] = *reinterpret_cast<const uint32_t *>(sb + xoff + mt * 1024u + (((2u * kb + 1u) ^ gi) << 4));
                        }
                        // Pair the rows first: the low halves of two words side by side hold nibbles 0..3
                        // of rows k and k+1, the high halves nibbles 4..7.  One shift and one logic
                        // operation then yield an operand register (w[k][n], w[k+1][n]) as two 16-bit floats:
                        // (nibble ^ 8) | exponent bits = BIAS + w.
                        uint32_t pr[2][4];
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            // i: 0 = column gi rows 2q,2q+1; 1 = column gi+8, same rows; 2, 3 = rows 8 further
                            const int a = (i & 1) * 4 + (i >> 1) * 2;
                            pr[0][i] = prmt(wd[a], wd[a + 1], 0x5410u);
                            pr[1][i] = prmt(wd[a], wd[a + 1], 0x7632u);
                        }
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            uint32_t a[4];
#pragma unroll
                            for (int i = 0; i < 4; ++i)
                                a[i] = GMagic<T>::finish(and_xor(pr[j >> 2][i] >> (4 * (j & 3)), nib_mask, nib_flip));
#pragma unroll
                            for (int mt = 0; mt < MT; ++mt) GMagic<T>::mma(acc[mt][j], a, xb[mt][0], xb[mt][1]);
                        }
#pragma unroll
                        for (int mt = 0; mt < MT; ++mt) GMagic<T>::mma(accx[mt], ones, xb[mt][0], xb[mt][1]);
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(smem_u32(&tail->empty[st]));
                }
                // scale and offset of the group, applied to the group's sums
                float sf[2][8], of[2][8];
                unpack8<T>(sA, sf[0]);
                unpack8<T>(sB, sf[1]);
                unpack8<T>(oA, of[0]);
                unpack8<T>(oB, of[1]);
#pragma unroll
                for (int r = 0; r < 2; ++r)
#pragma unroll
                    for (int j = 0; j < 8; ++j) of[r][j] -= GMagic<T>::kBias;
#pragma unroll
                for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                    for (int j = 0; j < 8; ++j)
#pragma unroll
                        for (int c = 0; c < 4; ++c) {
                            const int r = c >> 1;  // which run of columns
                            const float xs = accx[mt][c & 1];
                            Y(mt, j, c) = fmaf(sf[r][j], fmaf(of[r][j], xs, acc[mt][j][c]), Y(mt, j, c));
                        }
            }

            // ---- this (CTA, set)'s share of the unit goes to its slot ----
            const int first_cta = g_cta_of_item(unit_begin, total, G);
            const int last_cta = g_cta_of_item(unit_end - 1, total, G);
            const int nslots = (last_cta - first_cta + 1) * SETS;
            const int slot = (static_cast<int>(blockIdx.x) - first_cta) * SETS + set;
            constexpr int64_t kSlotElems = static_cast<int64_t>(8 * MT) * kGUnitN;
            float *unit_slots = p.slots + static_cast<int64_t>(unit) * p.max_slots * kSlotElems;
            // element (token, column) lives at token * 512 + column; this lane owns, per token tile, the
            // tokens 2q and 2q+1 and the column runs [cw*128 + gi*8, +8) and 64 further
            const int col = cw * 128 + gi * 8;
            float *mine = unit_slots + static_cast<int64_t>(slot) * kSlotElems;
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const int token = mt * 8 + 2 * q + (c & 1);
                    if (token < M) {
                        float *dst = mine + token * kGUnitN + col + (c >> 1) * 64;
                        __stcg(reinterpret_cast<float4 *>(dst),
                               make_float4(Y(mt, 0, c), Y(mt, 1, c), Y(mt, 2, c), Y(mt, 3, c)));
                        __stcg(reinterpret_cast<float4 *>(dst) + 1,
                               make_float4(Y(mt, 4, c), Y(mt, 5, c), Y(mt, 6, c), Y(mt, 7, c)));
                    }
                }
            __threadfence();
            set_bar_sync(set);
            if (cw == 0 && lane == 0) {
                const uint32_t old = atomicAdd(p.counters + unit, 1u);
                const bool last = (old + 1 == static_cast<uint32_t>(nslots));
                if (last) p.counters[unit] = 0;
                tail->is_last[set] = last ? 1u : 0u;
                __threadfence();
            }
            set_bar_sync(set);
            if (*reinterpret_cast<volatile uint32_t *>(&tail->is_last[set]) != 0) {
                // the last arriver adds the slots in slot order and writes the unit's outputs
#pragma unroll
                for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        const int token = mt * 8 + 2 * q + (c & 1);
                        const int64_t n = n0 + (c >> 1) * 64;
                        if (token < M && n < w.N) {
                            float v[8];
#pragma unroll
                            for (int j = 0; j < 8; ++j) v[j] = 0.0f;
                            const float *src = unit_slots + token * kGUnitN + col + (c >> 1) * 64;
                            for (int sl = 0; sl < nslots; ++sl) {
                                const float4 lo = __ldcg(reinterpret_cast<const float4 *>(src + sl * kSlotElems));
                                const float4 hi = __ldcg(reinterpret_cast<const float4 *>(src + sl * kSlotElems) + 1);
                                v[0] += lo.x;
                                v[1] += lo.y;
                                v[2] += lo.z;
                                v[3] += lo.w;
                                v[4] += hi.x;
                                v[5] += hi.y;
                                v[6] += hi.z;
                                v[7] += hi.w;
                            }
                            uint4 o;
                            T *oh = reinterpret_cast<T *>(&o);
#pragma unroll
                            for (int j = 0; j < 8; ++j)
                                oh[j] = from_float<T>(v[j] + (bias != nullptr ? to_float(bias[n + j]) : 0.0f));
                            *reinterpret_cast<uint4 *>(out + static_cast<int64_t>(token) * w.ld_out + n) = o;
                        }
                    }
            }
            set_bar_sync(set);  // is_last is rewritten by the next unit
            seg_begin = seg_end;
        }
    }

    __syncthreads();
    if (threadIdx.x == 0 && tail->abort_flag != 0 && p.status != nullptr) atomicMax(p.status, tail->abort_flag);
}

}  // namespace
}  // namespace qmm
