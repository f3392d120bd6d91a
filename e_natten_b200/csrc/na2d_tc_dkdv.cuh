// Persistent, warp-specialised tcgen05 dK/dV kernel.  Included by na2d_tc.cuh.
//
// One CTA per SM walks key tiles (TH x TW keys, row r of every MMA = key r = tensor-memory lane
// r).  The queries that can see a tile form a box (the union of the keys' inverse
// neighbourhoods, clipped to the local query band), walked in chunks of RC rows x HW columns
// (at most 128 queries):
//     S^T = K Q_c^T,  dP^T = V dO_c^T                      (tensor memory, fp32)
//     P^T = exp(S^T - lse),  dS^T = P^T (dP^T - delta)     (softmax warps, registers)
//     dV += P^T dO_c,  dK += dS^T Q_c                      (P^T, dS^T read from tensor memory)
// P^T and dS^T are written back over S^T / dP^T as packed 16-bit pairs; on the bf16 path dS^T
// is written as head + residual (two MMAs), because one bf16 keeps too few bits for dK.
// Twelve warps: 0-7 softmax (warps w and w+4 share 32 keys and split the 16-column blocks),
// 8 TMA producer (K, V tile; ring of Q / dO chunks), 9 MMA issue, 10-11 idle (register donors).
// dK and dV accumulate in tensor memory over all chunks of a tile; no atomics.
#pragma once

namespace na2d_tc {

// The query box of a key tile is walked in chunks of at most 128 queries.  Where a half-width
// strip of the box holds all of its rows (kernel sizes 3 and 5) the box is cut into a left and a
// right strip: every warp's keys are then seen from the same number of queries in each chunk,
// whereas row-wise chunks leave the warps of one half of the tile idle in each chunk (the two
// warps that share a tensor-memory lane quarter also share an SM sub-partition).
constexpr int dkv_w_split(int ks) { return 128 / ((TW + ks - 1) / 2) >= TH + ks - 1 ? 2 : 1; }

template <int D, int KS, bool SPLIT>
struct DkvCfg : Cfg<D, KS, 128, 0, dkv_w_split(KS)> {
    using B = Cfg<D, KS, 128, 0, dkv_w_split(KS)>;
    // names of the base read as "queries per chunk" here: NK = queries in a chunk, NKP padded
    static constexpr int TMEM_ST = 0, TMEM_DPT = 128, TMEM_DV = 256, TMEM_DK = 384;
    static constexpr int TMEM_PT = 0, TMEM_RES = 64, TMEM_DST = 128;      // 16-bit operands over S^T / dP^T
    static constexpr int STAGE = 2 * B::KV_BYTES;                          // Q chunk then dO chunk
    static constexpr int OUT_BYTES = 8 * OutStage<D / 2>::BYTES;          // output staging of the 8 softmax warps
    static constexpr int FIXED = 2 * B::Q_BYTES /*K, V tile*/ + OUT_BYTES + 2 * 2 * 128 * 4 /*lse, delta x 2*/ + 256 + 1024;
    static constexpr int NSTQ = (FIXED + 3 * STAGE <= kSmemLimit) ? 3 : ((FIXED + 2 * STAGE <= kSmemLimit) ? 2 : 1);
    static constexpr int SMEM = FIXED + NSTQ * STAGE;
    static constexpr int NB16 = B::NKP / 16;
    static_assert(SMEM <= kSmemLimit, "dK/dV kernel shared memory");
    static_assert(B::NKP <= 128 && D <= 128, "tensor memory layout");
};

template <typename DT, int D, int KS>
__global__ void __launch_bounds__(384, 1)
dkdv_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
            const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_do,
            const __grid_constant__ CUtensorMap tm_dk, const __grid_constant__ CUtensorMap tm_dv,
            const float* __restrict__ lse, const float* __restrict__ delta,
            DT* __restrict__ d_k, DT* __restrict__ d_v, const Na2dGeom g, const int tiles_r, const int tiles_c,
            const int total_tiles) {
    constexpr bool SPLIT = IsBf16<DT>::value;
    using C = DkvCfg<D, KS, SPLIT>;
    constexpr int NSTQ = C::NSTQ;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sK = smem;                               // key tile   [128 x D]
    uint8_t* sV = sK + C::Q_BYTES;                    // value tile [128 x D]
    uint8_t* sQD = sV + C::Q_BYTES;                   // NSTQ x (query chunk, dO chunk), each [NKP x D]
    uint8_t* sOut = sQD + NSTQ * C::STAGE;            // 8 x output staging (1024-byte aligned)
    float* s_lse = reinterpret_cast<float*>(sOut + C::OUT_BYTES);     // [chunk parity][128]  lse * log2(e)
    float* s_delta = s_lse + 2 * 128;                                   // [chunk parity][128]
    uint64_t* bars = reinterpret_cast<uint64_t*>(s_delta + 2 * 128);
    uint64_t* kv_full = bars + 0;            //       TMA -> MMA
    uint64_t* kv_empty = bars + 1;           //       MMA (commit) -> TMA
    uint64_t* s_full = bars + 2;             //       MMA (commit) -> softmax
    uint64_t* p_full = bars + 3;             //       softmax -> MMA
    uint64_t* acc_full = bars + 4;           //       MMA (commit) -> softmax (epilogue)
    uint64_t* acc_free = bars + 5;           //       softmax -> MMA
    uint64_t* qd_full = bars + 6;            // [3]   TMA -> MMA
    uint64_t* qd_empty = bars + 9;           // [3]   MMA (commit) -> TMA
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 12);
    volatile uint32_t* abort_flag = tmem_slot + 1;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n_my = total_tiles > (int)blockIdx.x ? (total_tiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;

    if (tid == 0) {
        *abort_flag = 0;
        mbar_init(kv_full, 1);
        mbar_init(kv_empty, 1);
        mbar_init(s_full, 1);
        mbar_init(p_full, 8);
        mbar_init(acc_full, 1);
        mbar_init(acc_free, 8);
        for (int i = 0; i < 3; ++i) {
            mbar_init(qd_full + i, 1);
            mbar_init(qd_empty + i, 1);
        }
        mbar_fence_init();
        tma_prefetch_desc(&tm_k);
        tma_prefetch_desc(&tm_v);
        tma_prefetch_desc(&tm_q);
        tma_prefetch_desc(&tm_do);
        tma_prefetch_desc(&tm_dk);
        tma_prefetch_desc(&tm_dv);
    }
    if (warp == 0) {
        __syncwarp();
        tmem_alloc(tmem_slot, 512);
        tmem_relinquish();
    }
    // Rows [NK, NKP) of every query / dO chunk buffer are contraction rows of the output MMAs that
    // TMA never writes: zero them once.
    if constexpr (C::NKP > C::NK) {
        constexpr int pad16 = (C::NKP - C::NK) * C::ROWB / 16;
        for (int i = tid; i < NSTQ * 2 * C::NS * pad16; i += 384) {
            const int which = i / pad16, off = i - which * pad16;          // which = (stage * 2 + q/dO) * NS + slab
            const int slab = which % C::NS, buf = which / C::NS;
            uint8_t* base = sQD + (buf >> 1) * C::STAGE + (buf & 1) * C::KV_BYTES + slab * C::KV_SLAB;
            st_shared_v4(smem_u32(base + C::NK * C::ROWB + off * 16), 0u, 0u, 0u, 0u);
        }
        fence_proxy_async();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    // Geometry of my i-th tile: key tile origin and the query box it is seen from.
    struct TileGeo { int bn, kr0, kc0, qb_r0, q_local_r0, n_rows, qb_c0, n_cc, n_ch; };
    auto tile_geo = [&](int i) {
        TileGeo t;
        int x = (int)blockIdx.x + i * (int)gridDim.x;
        const int tc = x % tiles_c;
        x /= tiles_c;
        t.kr0 = (x % tiles_r) * TH;
        t.kc0 = tc * TW;
        t.bn = x / tiles_r;
        const int kg_first = g.kv_row0 + t.kr0;
        const int kg_last = g.kv_row0 + min(t.kr0 + TH, g.Hkv) - 1;
        t.qb_r0 = max(na2d_bws(kg_first, KS), g.q_row0);                           // global row
        const int qb_r1 = min(na2d_bwe(kg_last, g.Hg, KS), g.q_row0 + g.Hq);
        t.n_rows = max(qb_r1 - t.qb_r0, 0);
        t.q_local_r0 = t.qb_r0 - g.q_row0;
        t.qb_c0 = na2d_bws(t.kc0, KS);
        const int n_cols = na2d_bwe(min(t.kc0 + TW, g.W) - 1, g.W, KS) - t.qb_c0;
        t.n_cc = (n_cols + C::HW - 1) / C::HW;           // 1 inside the image, 2 where both borders stretch the box
        t.n_ch = ((t.n_rows + C::RC - 1) / C::RC) * t.n_cc;
        return t;
    };

    if (warp == 8) {
        // ------------------------------------------------------------------ producer
        reg_dec<kRegsDonor>();
        if (lane == 0) {
            uint32_t n = 0, it = 0;                     // chunk counter, non-empty tile counter
            for (int i = 0; i < n_my; ++i) {
                const TileGeo t = tile_geo(i);
                if (t.n_ch == 0) continue;
                mbar_wait(kv_empty, (it & 1) ^ 1, abort_flag, kErrLoadWait);
                mbar_expect_tx(kv_full, 2u * C::Q_BYTES);
#pragma unroll
                for (int s = 0; s < C::NS; ++s) {
                    tma_load_4d(sK + s * C::Q_SLAB, &tm_k, kv_full, s * 64, t.kc0, t.kr0, t.bn);
                    tma_load_4d(sV + s * C::Q_SLAB, &tm_v, kv_full, s * 64, t.kc0, t.kr0, t.bn);
                }
                ++it;
                for (int ch = 0; ch < t.n_ch; ++ch, ++n) {
                    const int rc = ch / t.n_cc, cc = ch - rc * t.n_cc;
                    const uint32_t st = n % NSTQ;
                    mbar_wait(qd_empty + st, ((n / NSTQ) & 1) ^ 1, abort_flag, kErrLoadWait);
                    mbar_expect_tx(qd_full + st, 2u * C::NS * C::NK * C::ROWB);
                    uint8_t* dst = sQD + st * C::STAGE;
#pragma unroll
                    for (int s = 0; s < C::NS; ++s) {
                        tma_load_4d(dst + s * C::KV_SLAB, &tm_q, qd_full + st, s * 64, t.qb_c0 + cc * C::HW,
                                    t.q_local_r0 + rc * C::RC, t.bn);
                        tma_load_4d(dst + C::KV_BYTES + s * C::KV_SLAB, &tm_do, qd_full + st, s * 64,
                                    t.qb_c0 + cc * C::HW, t.q_local_r0 + rc * C::RC, t.bn);
                    }
                }
            }
        }
    } else if (warp == 9) {
        // ------------------------------------------------------------------ MMA issue
        reg_dec<kRegsDonor>();
        const bool leader = lane == 0;
        constexpr uint32_t idesc_s = umma_idesc(TM, C::NKP, IsBf16<DT>::value, IsBf16<DT>::value, false, false);
        constexpr uint32_t idesc_o = umma_idesc(TM, D, IsBf16<DT>::value, IsBf16<DT>::value, false, true);
        constexpr uint32_t hi = smem_desc_hi(C::ATOM, C::SWZ);
        const uint32_t k_lo = smem_desc_lo(smem_u32(sK), 16), v_lo = smem_desc_lo(smem_u32(sV), 16);
        uint32_t n = 0, it = 0;
        for (int i = 0; i < n_my; ++i) {
            const TileGeo t = tile_geo(i);
            if (t.n_ch == 0) continue;
            mbar_wait(kv_full, it & 1, abort_flag, kErrLoadWait);
            for (int ch = 0; ch < t.n_ch; ++ch, ++n) {
                const uint32_t st = n % NSTQ;
                if (leader) NA2D_TR(2, 0, n);
                mbar_wait(qd_full + st, (n / NSTQ) & 1, abort_flag, kErrLoadWait);
                tc_fence_after();
                if (leader) NA2D_TR(2, 1, n);
                const uint32_t q_addr = smem_u32(sQD + st * C::STAGE), g_addr = q_addr + C::KV_BYTES;
                if (leader) {
                    const uint32_t q_lo = smem_desc_lo(q_addr, 16), g_lo = smem_desc_lo(g_addr, 16);
#pragma unroll
                    for (int kk = 0; kk < D / 16; ++kk) {
                        constexpr int kPerSlab = C::SLAB_C / 16;
                        const int slab = kk / kPerSlab, in_slab = kk % kPerSlab;
                        umma_ss(tmem_base + C::TMEM_ST, desc64(hi, k_lo + ((slab * C::Q_SLAB) >> 4) + 2 * in_slab),
                                desc64(hi, q_lo + ((slab * C::KV_SLAB) >> 4) + 2 * in_slab), idesc_s, kk > 0);
                    }
#pragma unroll
                    for (int kk = 0; kk < D / 16; ++kk) {
                        constexpr int kPerSlab = C::SLAB_C / 16;
                        const int slab = kk / kPerSlab, in_slab = kk % kPerSlab;
                        umma_ss(tmem_base + C::TMEM_DPT, desc64(hi, v_lo + ((slab * C::Q_SLAB) >> 4) + 2 * in_slab),
                                desc64(hi, g_lo + ((slab * C::KV_SLAB) >> 4) + 2 * in_slab), idesc_s, kk > 0);
                    }
                    umma_commit(s_full);
                    if (ch == t.n_ch - 1) umma_commit(kv_empty);       // K and V are only read by the score MMAs
                    NA2D_TR(2, 2, n);
                }
                __syncwarp();
                mbar_wait(p_full, n & 1, abort_flag, kErrMmaWait);
                if (ch == 0) mbar_wait(acc_free, (it & 1) ^ 1, abort_flag, kErrMmaWait);
                tc_fence_after();
                if (leader) NA2D_TR(2, 3, n);
                if (leader) {
                    const uint32_t qm_lo = smem_desc_lo(q_addr, C::KV_SLAB), gm_lo = smem_desc_lo(g_addr, C::KV_SLAB);
                    const uint32_t acc = ch > 0;
#pragma unroll
                    for (int kk = 0; kk < C::NKP / 16; ++kk)
                        umma_ts(tmem_base + C::TMEM_DV, tmem_base + C::TMEM_PT + 8 * kk,
                                desc64(hi, gm_lo + ((kk * 16 * C::ROWB) >> 4)), idesc_o, acc | (kk > 0));
#pragma unroll
                    for (int kk = 0; kk < C::NKP / 16; ++kk)
                        umma_ts(tmem_base + C::TMEM_DK, tmem_base + C::TMEM_DST + 8 * kk,
                                desc64(hi, qm_lo + ((kk * 16 * C::ROWB) >> 4)), idesc_o, acc | (kk > 0));
                    if (SPLIT) {
#pragma unroll
                        for (int kk = 0; kk < C::NKP / 16; ++kk)
                            umma_ts(tmem_base + C::TMEM_DK, tmem_base + C::TMEM_RES + 8 * kk,
                                    desc64(hi, qm_lo + ((kk * 16 * C::ROWB) >> 4)), idesc_o, 1u);
                    }
                    umma_commit(qd_empty + st);
                    if (ch == t.n_ch - 1) umma_commit(acc_full);
                    NA2D_TR(2, 4, n);
                }
                __syncwarp();
            }
            ++it;
        }
    } else if (warp >= 10) {
        reg_dec<kRegsDonor>();
    } else {
        // ------------------------------------------------------------------ softmax warps
        reg_inc<kRegsSoftmax>();
        const int quarter = warp & 3, half = warp >> 2;
        const int row = quarter * 32 + lane;                 // key of the tile = tensor-memory lane
        const int ctid = warp * 32 + lane;                   // 0..255 among the softmax warps
        const uint32_t tmem_lane = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
        constexpr int DH = D / 2;                            // output columns stored by this half
        constexpr int NBH = (C::NB16 + 1) / 2;               // own blocks at most
        // a warp's 32 / TW key rows are seen from at most that many + 2 ks - 2 query rows
        constexpr int kRows = (32 / TW - 1 + 2 * KS - 1) < C::RC ? (32 / TW - 1 + 2 * KS - 1) : C::RC;
        constexpr int kBlocks = (kRows * C::HW - 1) / 16 + 2;
        constexpr int NACT = (kBlocks + 1) / 2 < NBH ? (kBlocks + 1) / 2 : NBH;
        constexpr int NR = (16 + C::HW - 2) / C::HW + 1;     // chunk rows a 16-column block can touch

        uint32_t n = 0, it = 0;
        for (int i = 0; i < n_my; ++i) {
            const TileGeo t = tile_geo(i);
            const int kr_raw = t.kr0 + (row / TW), kc_raw = t.kc0 + (row % TW);
            const bool k_valid = kr_raw < g.Hkv && kc_raw < g.W;
            const int kr = min(kr_raw, g.Hkv - 1), kc = min(kc_raw, g.W - 1);
            const size_t ki = (static_cast<size_t>(t.bn) * g.Hkv + kr) * g.W + kc;
            DT* dv_row = d_v + ki * D + half * DH;
            DT* dk_row = d_k + ki * D + half * DH;
            if (t.n_ch == 0) {                               // no local query sees this tile
                if (k_valid) {
#pragma unroll
                    for (int c8 = 0; c8 < DH / 8; ++c8) {
                        *reinterpret_cast<uint4*>(dv_row + 8 * c8) = make_uint4(0u, 0u, 0u, 0u);
                        *reinterpret_cast<uint4*>(dk_row + 8 * c8) = make_uint4(0u, 0u, 0u, 0u);
                    }
                }
                continue;
            }
            // the queries that see this thread's key: box rows [row_lo, row_hi), box columns [col_lo, col_hi)
            const int kg = g.kv_row0 + kr;
            const int row_lo = max(na2d_bws(kg, KS), g.q_row0) - t.qb_r0;
            const int row_hi = min(na2d_bwe(kg, g.Hg, KS), g.q_row0 + g.Hq) - t.qb_r0;
            const int col_lo = na2d_bws(kc, KS) - t.qb_c0;
            const int col_hi = na2d_bwe(kc, g.W, KS) - t.qb_c0;
            const int wrow_lo = __shfl_sync(0xffffffffu, row_lo, 0);
            const int wrow_hi = __shfl_sync(0xffffffffu, row_hi, 31);

            for (int ch = 0; ch < t.n_ch; ++ch, ++n) {
                const int rc = ch / t.n_cc, cc = ch - rc * t.n_cc;
                const int r_off = rc * C::RC, c_off = cc * C::HW;
                const int par = n & 1;
                if (tid == 0) NA2D_TR(3, 0, n);
                // lse * log2(e) and delta of the chunk's queries -> shared memory (zero outside the band)
                if (ctid < C::NK) {
                    const int br = r_off + ctid / C::HW, qc = t.qb_c0 + c_off + ctid % C::HW;
                    float l2 = 0.f, dl = 0.f;
                    if (br < t.n_rows && qc < g.W) {
                        const size_t qi = (static_cast<size_t>(t.bn) * g.Hq + (t.q_local_r0 + br)) * g.W + qc;
                        l2 = lse[qi] * kLog2e;
                        dl = delta[qi];
                    }
                    s_lse[par * 128 + ctid] = l2;
                    s_delta[par * 128 + ctid] = dl;
                }
                // the warp's keys are seen from chunk rows [ra, rb): its active column range
                const int ra = max(wrow_lo - r_off, 0), rb = min(wrow_hi - r_off, C::RC);
                const int j_lo = ra * C::HW;
                const int j_hi = rb > ra ? min(rb * C::HW, C::NK) : 0;
                const int b_hi = (j_hi + 15) >> 4;
                const int bi_lo = j_hi > 0 ? (((j_lo >> 4) - half + 1) >> 1) : 0;
                // this thread's column segment inside a chunk row
                const int cl = max(col_lo - c_off, 0), chi = min(col_hi - c_off, C::HW);
                const int seg_len = chi - cl;
                const uint32_t seg = seg_len > 0 ? ((1u << seg_len) - 1u) : 0u;
                bar_sync(5, 256);                                           // lse / delta are in place
                if (tid == 0) NA2D_TR(3, 1, n);

                mbar_wait(s_full, n & 1, abort_flag, kErrMmaWait);
                tc_fence_after();
                if (tid == 0) NA2D_TR(3, 2, n);
                uint32_t s[NACT][16], dp[NACT][16];
                uint32_t vmask[NACT];
#pragma unroll
                for (int a = 0; a < NACT; ++a) {
                    const int blk = half + 2 * (bi_lo + a);
                    if (blk < b_hi) {                                       // warp-uniform
                        tmem_ld_32x16(tmem_lane + C::TMEM_ST + 16 * blk, s[a]);
                        tmem_ld_32x16(tmem_lane + C::TMEM_DPT + 16 * blk, dp[a]);
                    }
                }
#pragma unroll
                for (int a = 0; a < NACT; ++a) {                            // validity masks, loads in flight
                    const int blk = half + 2 * (bi_lo + a);
                    const int r_first = (16 * blk) / C::HW;
                    uint32_t m = 0;
#pragma unroll
                    for (int dr = 0; dr < NR; ++dr) {
                        const int r = r_first + dr;                          // chunk row
                        const int rel = r * C::HW + cl - 16 * blk;           // segment start relative to the block
                        const uint32_t bits = rel >= 0 ? (seg << (rel & 31)) : (seg >> ((-rel) & 31));
                        const bool row_ok = r < C::RC && r_off + r >= row_lo && r_off + r < row_hi;
                        if (row_ok && rel > -32 && rel < 16) m |= bits;
                    }
                    vmask[a] = (blk < b_hi) ? (m & 0xffffu) : 0u;
                }
                tmem_ld_wait();
                if (tid == 0) NA2D_TR(3, 3, n);
                // the partner has read its S^T / dP^T blocks too: the 16-bit operands may now be
                // written over them
                bar_sync(1 + quarter, 64);
                if (tid == 0) NA2D_TR(3, 4, n);

#pragma unroll
                for (int a = 0; a < NACT; ++a) {
                    const int blk = half + 2 * (bi_lo + a);
                    if (blk < b_hi) {
                        float l2[16], dl[16];
#pragma unroll
                        for (int v4 = 0; v4 < 4; ++v4) {
                            const float4 x = *reinterpret_cast<const float4*>(s_lse + par * 128 + 16 * blk + 4 * v4);
                            const float4 y = *reinterpret_cast<const float4*>(s_delta + par * 128 + 16 * blk + 4 * v4);
                            l2[4 * v4] = x.x; l2[4 * v4 + 1] = x.y; l2[4 * v4 + 2] = x.z; l2[4 * v4 + 3] = x.w;
                            dl[4 * v4] = y.x; dl[4 * v4 + 1] = y.y; dl[4 * v4 + 2] = y.z; dl[4 * v4 + 3] = y.w;
                        }
                        uint32_t wp[8], wd[8], wr2[8];
#pragma unroll
                        for (int e2 = 0; e2 < 8; ++e2) {
                            float p[2], ds[2];
#pragma unroll
                            for (int h = 0; h < 2; ++h) {
                                const int e = 2 * e2 + h;
                                const float pe = fast_exp2(fmaf(__uint_as_float(s[a][e]), kLog2e, -l2[e]));
                                const bool ok = (vmask[a] >> e) & 1u;      // select, never multiply by zero
                                p[h] = ok ? pe : 0.f;
                                ds[h] = ok ? pe * (__uint_as_float(dp[a][e]) - dl[e]) : 0.f;
                            }
                            wp[e2] = pack2<DT>(p[0], p[1]);
                            wd[e2] = pack2<DT>(ds[0], ds[1]);
                            wr2[e2] = SPLIT ? pack2_residual_bf16(ds[0], ds[1], wd[e2]) : 0u;
                        }
                        tmem_st_32x8(tmem_lane + C::TMEM_PT + 8 * blk, wp);
                        tmem_st_32x8(tmem_lane + C::TMEM_DST + 8 * blk, wd);
                        if (SPLIT) tmem_st_32x8(tmem_lane + C::TMEM_RES + 8 * blk, wr2);
                    }
                }
                {   // own blocks outside the range hold zeros
                    const uint32_t z[8] = {0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u};
                    for (int bi = 0; bi < NBH; ++bi) {
                        const int blk = half + 2 * bi;
                        const bool in_range = bi >= bi_lo && bi < bi_lo + NACT && blk < b_hi;
                        if (!in_range && blk < C::NB16) {
                            tmem_st_32x8(tmem_lane + C::TMEM_PT + 8 * blk, z);
                            tmem_st_32x8(tmem_lane + C::TMEM_DST + 8 * blk, z);
                            if (SPLIT) tmem_st_32x8(tmem_lane + C::TMEM_RES + 8 * blk, z);
                        }
                    }
                }
                tmem_st_wait();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(p_full);
                if (tid == 0) NA2D_TR(3, 5, n);
            }

            // ---- epilogue: this half's columns of the dV and dK rows of the warp's 32 keys
            mbar_wait(acc_full, it & 1, abort_flag, kErrMmaWait);
            tc_fence_after();
            if (tid == 0) NA2D_TR(3, 6, n - 1);
            {
                uint8_t* stage = sOut + warp * OutStage<DH>::BYTES;
                const int h0 = t.kr0 + quarter * (32 / TW);
                uint32_t acc[DH];
#pragma unroll
                for (int which = 0; which < 2; ++which) {
                    const uint32_t col0 = (which == 0 ? C::TMEM_DV : C::TMEM_DK) + half * DH;
#pragma unroll
                    for (int piece = 0; piece < DH / 16; ++piece)
                        tmem_ld_32x16(tmem_lane + col0 + 16 * piece, *reinterpret_cast<uint32_t(*)[16]>(&acc[16 * piece]));
                    tmem_ld_wait();
                    stage_and_store<DT, DH>(which == 0 ? &tm_dv : &tm_dk, stage, acc, 1.f, half * DH, t.kc0, h0, t.bn, lane);
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_free);
            if (tid == 0) NA2D_TR(3, 7, n - 1);
            ++it;
        }
    }

    if (warp < 8 && lane == 0) bulk_wait<0>();          // the staging buffers have been read, the rows written
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}

template <typename DT, int D, int KS>
int launch_dkdv(const Na2dGeom& g, int dtype, const void* q, const void* k, const void* v, const float* lse,
                const void* d_o, const float* delta, void* d_k, void* d_v, int device, cudaStream_t st, int* launched) {
    using C = DkvCfg<D, KS, IsBf16<DT>::value>;
    CUtensorMap tk, tv, tq, tg, tdk, tdv;
    int rc = make_map(&tk, k, dtype, g.BN, g.Hkv, g.W, D, TW, TH);
    if (rc == NA2D_OK) rc = make_map(&tdk, d_k, dtype, g.BN, g.Hkv, g.W, D, TW, 32 / TW, OutStage<D / 2>::RW);
    if (rc == NA2D_OK) rc = make_map(&tdv, d_v, dtype, g.BN, g.Hkv, g.W, D, TW, 32 / TW, OutStage<D / 2>::RW);
    if (rc == NA2D_OK) rc = make_map(&tv, v, dtype, g.BN, g.Hkv, g.W, D, TW, TH);
    if (rc == NA2D_OK) rc = make_map(&tq, q, dtype, g.BN, g.Hq, g.W, D, C::HW, C::RC);
    if (rc == NA2D_OK) rc = make_map(&tg, d_o, dtype, g.BN, g.Hq, g.W, D, C::HW, C::RC);
    if (rc != NA2D_OK) return rc;
    const int tiles_r = (g.Hkv + TH - 1) / TH, tiles_c = (g.W + TW - 1) / TW;
    const long long tiles = (long long)g.BN * tiles_r * tiles_c;
    if (tiles > 0x7fffffffLL) return NA2D_ERR_TOO_LARGE;
    auto kern = dkdv_kernel<DT, D, KS>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM) != cudaSuccess)
        return NA2D_ERR_CUDA;
    const int grid = (int)(tiles < sm_count(device) ? tiles : sm_count(device));
    kern<<<grid, 384, C::SMEM, st>>>(tk, tv, tq, tg, tdk, tdv, lse, delta, (DT*)d_k, (DT*)d_v, g, tiles_r, tiles_c, (int)tiles);
    *launched += 1;
    return cudaGetLastError() == cudaSuccess ? NA2D_OK : NA2D_ERR_CUDA;
}

inline int backward_dkdv(const Na2dGeom& g, int dtype, const void* q, const void* k, const void* v, const float* lse,
                         const void* d_o, const float* delta, void* d_k, void* d_v, int device, cudaStream_t st,
                         int* launched) {
    if (dtype == NA2D_BF16) {
        NA2D_TC_DISPATCH_D(launch_dkdv, __nv_bfloat16, g, dtype, q, k, v, lse, d_o, delta, d_k, d_v, device, st, launched)
    } else {
        NA2D_TC_DISPATCH_D(launch_dkdv, __half, g, dtype, q, k, v, lse, d_o, delta, d_k, d_v, device, st, launched)
    }
}

}  // namespace na2d_tc
