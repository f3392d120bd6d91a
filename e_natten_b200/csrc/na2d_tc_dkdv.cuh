// Persistent, warp-specialised tcgen05 dK/dV kernel.  Included by na2d_tc.cuh.
//
// One CTA per SM walks key tiles (TH x TW keys, row r of every MMA = key r = tensor-memory lane
// r).  The queries that can see a tile form a box (the union of the keys' inverse
// neighbourhoods, clipped to the local query band), walked in chunks of RC rows x HW columns
// (at most 64 queries):
//     S^T = K Q_c^T,  dP^T = V dO_c^T                      (tensor memory, fp32)
//     P^T = exp(S^T - lse),  dS^T = scale P^T (dP^T - delta)   (softmax warps, registers; the scale is dK's)
//     dV += P^T dO_c,  dK += dS^T Q_c                      (P^T, dS^T read from tensor memory)
// P^T and dS^T are written back over S^T / dP^T as packed 16-bit pairs; on the bf16 path dS^T
// is written as head + residual (two MMAs), because one bf16 keeps too few bits for dK.
//
// Tensor memory holds two chunk stages (S^T, dP^T of 64 columns each) next to the dV and dK
// accumulators, so the score MMAs of one chunk run while the softmax warps work on the previous
// one.  Sixteen warps: 0-7 softmax (warps w and w + 4 own the same 32 keys of a lane quarter and split
// the 8-column blocks of every chunk between them), 8 TMA producer of the Q / dO chunk ring, 11 TMA
// producer of the K, V tile, 9 issues the score MMAs, 10 the output MMAs, 12-15 epilogue (dV, dK rows ->
// staging -> TMA store), which
// overlaps the next tile.  dK and dV accumulate in tensor memory over all chunks of a tile; no
// atomics.
#pragma once

namespace na2d_tc {

// Chunks of an interior tile's query box when the box is cut into `split` column strips.
constexpr int dkv_chunks(int ks, int split) {
    const int bw = TW + ks - 1, hh = TH + ks - 1;
    if (bw % split != 0 || 64 / (bw / split) == 0) return 1 << 20;
    const int rc_max = 64 / (bw / split);
    return (hh + rc_max - 1) / rc_max * split;
}
// Fewest chunks wins; on a tie the narrower strips, which spread the work evenly over the lane
// quarters (a key row group sees the same number of queries in every strip).
constexpr int dkv_w_split(int ks) {
    const int c1 = dkv_chunks(ks, 1), c2 = dkv_chunks(ks, 2), c4 = dkv_chunks(ks, 4);
    return (c4 <= c2 && c4 <= c1) ? 4 : (c2 <= c1 ? 2 : 1);
}

constexpr unsigned long long row_repeat(int hw, int rc) {
    unsigned long long m = 0;
    for (int r = 0; r < rc; ++r) m |= 1ull << (r * hw);
    return m;
}

template <int D, int KS, bool SPLIT>
struct DkvCfg : Cfg<D, KS, 64, 0, dkv_w_split(KS)> {
    using B = Cfg<D, KS, 64, 0, dkv_w_split(KS)>;
    // names of the base read as "queries per chunk" here: NK = queries in a chunk, NKP padded
    static constexpr int TMEM_STAGE = 128;                                 // columns per chunk stage
    static constexpr int TMEM_ST = 0, TMEM_DPT = 64, TMEM_DV = 256, TMEM_DK = 384;
    static constexpr int TMEM_PT = 0, TMEM_DST = 32, TMEM_RES = 64;       // 16-bit operands over S^T / dP^T
    static constexpr int STAGE = 2 * B::KV_BYTES;                          // Q chunk then dO chunk
    static constexpr int OUT_BYTES = 4 * 2 * OutStage<32>::BYTES;          // two staging buffers for each of the 4 epilogue warps
    static constexpr int XCHG_BYTES = 2 * 2 * 2 * 64 * 4;                  // [group][parity]{lse, delta}[64]
    static constexpr int FIXED = 2 * B::Q_BYTES /*K, V tile*/ + OUT_BYTES + XCHG_BYTES + 256 + 1024;
    static constexpr int NSTQ = (FIXED + 4 * STAGE <= kSmemLimit) ? 4 : 3;
    static constexpr int SMEM = FIXED + NSTQ * STAGE;
    static constexpr int NB8 = B::NKP / 8;
    static constexpr unsigned long long ROW_REP = row_repeat(B::HW, B::RC);
    static_assert(SMEM <= kSmemLimit, "dK/dV kernel shared memory");
    static_assert(B::NKP <= 64 && D <= 128 && D % 32 == 0, "tensor memory layout");
};

template <typename DT, int D, int KS>
__global__ void __launch_bounds__(512, 1)
dkdv_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
            const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_do,
            const __grid_constant__ CUtensorMap tm_dk, const __grid_constant__ CUtensorMap tm_dv,
            const float* __restrict__ lse, const float* __restrict__ delta, const int f32_out,
            unsigned int* __restrict__ err_word, const Na2dGeom g, const int tiles_r, const int tiles_c,
            const int total_tiles) {
    constexpr bool SPLIT = IsBf16<DT>::value;
    using C = DkvCfg<D, KS, SPLIT>;
    constexpr int NSTQ = C::NSTQ;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sK = smem;                               // key tile   [128 x D]
    uint8_t* sV = sK + C::Q_BYTES;                    // value tile [128 x D]
    uint8_t* sQD = sV + C::Q_BYTES;                   // NSTQ x (query chunk, dO chunk), each [NKP x D]
    uint8_t* sOut = sQD + NSTQ * C::STAGE;            // 4 x output staging (1024-byte aligned)
    float* s_x = reinterpret_cast<float*>(sOut + C::OUT_BYTES);   // [group][parity]{lse * log2(e), delta}[64]
    uint64_t* bars = reinterpret_cast<uint64_t*>(s_x + C::XCHG_BYTES / 4);
    uint64_t* kv_full = bars + 0;            //       TMA -> MMA
    uint64_t* kv_empty = bars + 1;           //       MMA (commit) -> TMA
    uint64_t* acc_full = bars + 2;           //       MMA (commit) -> epilogue
    uint64_t* acc_free = bars + 3;           //       epilogue -> MMA: dV and dK have been read
    uint64_t* s_full = bars + 4;             // [2]   MMA (commit) -> softmax group
    uint64_t* p_full = bars + 6;             // [2]   softmax group -> MMA
    uint64_t* qd_full = bars + 8;            // [4]   TMA -> MMA
    uint64_t* qd_empty = bars + 12;          // [4]   MMA (commit) -> TMA
    uint64_t* st_free = bars + 16;           // [2]   output MMAs (commit) -> score MMAs: the stage is free
    uint64_t* accv_free = bars + 18;         //       epilogue -> MMA: dV has been read (dK follows)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 19);
    const WaitCtx wctx{reinterpret_cast<WaitState*>(bars + 20)};

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n_my = total_tiles > (int)blockIdx.x ? (total_tiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;

    if (tid == 0) {
        wait_state_init(wctx.st, err_word, kWaitLimitNs);
        mbar_init(kv_full, 1);
        mbar_init(kv_empty, 1);
        mbar_init(acc_full, 1);
        mbar_init(acc_free, 4);
        mbar_init(accv_free, 4);
        for (int i = 0; i < 2; ++i) {
            mbar_init(s_full + i, 1);
            mbar_init(p_full + i, 8);
            mbar_init(st_free + i, 1);
        }
        for (int i = 0; i < 4; ++i) {
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
        for (int i = tid; i < NSTQ * 2 * C::NS * pad16; i += 512) {
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
    struct TileGeo { int bn, hn, hb, kr0, kc0, qb_r0, q_local_r0, n_rows, qb_c0, n_cc, n_ch; };
    auto tile_geo = [&](int i) {
        TileGeo t;
        int x = (int)blockIdx.x + i * (int)gridDim.x;
        const int tc = x % tiles_c;
        x /= tiles_c;
        t.kr0 = (x % tiles_r) * TH;
        t.kc0 = tc * TW;
        t.bn = x / tiles_r;
        split_unit(t.bn, g, t.hn, t.hb);
        const int kg_first = g.kv_row0 + t.kr0;
        const int kg_last = g.kv_row0 + min(t.kr0 + TH, g.Hkv) - 1;
        t.qb_r0 = max(na2d_bws(kg_first, KS), g.q_row0);                           // global row
        const int qb_r1 = min(na2d_bwe(kg_last, g.Hg, KS), g.q_row0 + g.Hq);
        t.n_rows = max(qb_r1 - t.qb_r0, 0);
        t.q_local_r0 = t.qb_r0 - g.q_row0;
        t.qb_c0 = na2d_bws(t.kc0, KS);
        const int n_cols = na2d_bwe(min(t.kc0 + TW, g.W) - 1, g.W, KS) - t.qb_c0;
        t.n_cc = (n_cols + C::HW - 1) / C::HW;           // strips; more where both borders stretch the box
        t.n_ch = ((t.n_rows + C::RC - 1) / C::RC) * t.n_cc;
        return t;
    };

    if (warp == 8) {
        // ------------------------------------------------------------------ producer of the Q / dO chunk ring
        // (the K, V tile has a producer of its own, warp 11: a chunk of the next tile can be
        // fetched as soon as a ring slot is free, long before the K, V buffers are)
        reg_dec<kDkvRegsCtl>();
        if (lane == 0) {
            uint32_t n = 0;
            LoadTracker lt(bars);
            for (int i = 0; i < n_my && lt.ok; ++i) {
                const TileGeo t = tile_geo(i);
                for (int ch = 0; ch < t.n_ch; ++ch, ++n) {
                    const int rc = ch / t.n_cc, cc = ch - rc * t.n_cc;
                    const uint32_t st = n % NSTQ;
                    if (!lt.acquire(qd_empty + st, ((n / NSTQ) & 1) ^ 1, wctx)) break;
                    NA2D_TR(2, 7, n);
                    lt.arm(qd_full + st, (n / NSTQ) & 1, 2u * C::NS * C::NK * C::ROWB);
                    uint8_t* dst = sQD + st * C::STAGE;
#pragma unroll
                    for (int s = 0; s < C::NS; ++s) {
                        tma_load_5d(dst + s * C::KV_SLAB, &tm_q, qd_full + st, s * 64, t.qb_c0 + cc * C::HW,
                                    t.q_local_r0 + rc * C::RC, t.hn, t.hb);
                        tma_load_5d(dst + C::KV_BYTES + s * C::KV_SLAB, &tm_do, qd_full + st, s * 64,
                                    t.qb_c0 + cc * C::HW, t.q_local_r0 + rc * C::RC, t.hn, t.hb);
                    }
                }
            }
            lt.drain(wctx);
        }
    } else if (warp == 9) {
        // ------------------------------------------------------------------ MMA issue: scores
        // Two warps issue MMAs, so that the bookkeeping of one runs under the MMAs of the other:
        // this one the score MMAs of chunk n into stage n & 1, as soon as the chunk's Q / dO have
        // landed and the output MMAs of chunk n - 2 (warp 10) have left the stage.  The whole warp
        // walks the loop with uniform control flow; one elected lane issues.
        reg_dec<kDkvRegsCtl>();
        constexpr uint32_t idesc_s = umma_idesc(TM, C::NKP, IsBf16<DT>::value, IsBf16<DT>::value, false, false);
        constexpr uint32_t hi = smem_desc_hi(C::ATOM, C::SWZ);
        const uint32_t k_lo = smem_desc_lo(smem_u32(sK), 16), v_lo = smem_desc_lo(smem_u32(sV), 16);
        const uint32_t qd_base = smem_u32(sQD);
        uint32_t n = 0, it = 0;
        for (int i = 0; i < n_my; ++i) {
            const TileGeo t = tile_geo(i);
            if (t.n_ch == 0) continue;
            for (int ch = 0; ch < t.n_ch; ++ch, ++n) {
                const uint32_t q_addr = qd_base + (n % NSTQ) * C::STAGE, g_addr = q_addr + C::KV_BYTES;
                const uint32_t q_lo = smem_desc_lo(q_addr, 16), g_lo = smem_desc_lo(g_addr, 16);
                const uint32_t tm = tmem_base + (n & 1) * C::TMEM_STAGE;
                if (lane == 0) NA2D_TR(2, 0, n);
                if (ch == 0) mbar_wait(kv_full, it & 1, wctx, kErrLoadWait);
                if (lane == 0) NA2D_TR(2, 1, n);
                mbar_wait(qd_full + n % NSTQ, (n / NSTQ) & 1, wctx, kErrLoadWait);
                if (lane == 0) NA2D_TR(2, 3, n);
                mbar_wait(st_free + (n & 1), ((n >> 1) & 1) ^ 1, wctx, kErrMmaWait);
                if (lane == 0) NA2D_TR(2, 5, n);
                tc_fence_after();
                if (elect_one()) {
                    // the S^T and dP^T chains alternate
#pragma unroll
                    for (int kk = 0; kk < D / 16; ++kk) {
                        constexpr int kPerSlab = C::SLAB_C / 16;
                        const int slab = kk / kPerSlab, in_slab = kk % kPerSlab;
                        umma_ss(tm + C::TMEM_ST, desc64(hi, k_lo + ((slab * C::Q_SLAB) >> 4) + 2 * in_slab),
                                desc64(hi, q_lo + ((slab * C::KV_SLAB) >> 4) + 2 * in_slab), idesc_s, kk > 0);
                        umma_ss(tm + C::TMEM_DPT, desc64(hi, v_lo + ((slab * C::Q_SLAB) >> 4) + 2 * in_slab),
                                desc64(hi, g_lo + ((slab * C::KV_SLAB) >> 4) + 2 * in_slab), idesc_s, kk > 0);
                    }
                    umma_commit(s_full + (n & 1));
                    if (ch == t.n_ch - 1) umma_commit(kv_empty);       // K and V are only read by the score MMAs
                    NA2D_TR(2, 2, n);
                }
                __syncwarp();
            }
            ++it;
        }
    } else if (warp == 10) {
        // ------------------------------------------------------------------ MMA issue: outputs
        // dV += P^T dO, dK += dS^T Q of chunk n out of stage n & 1, when the chunk's softmax group
        // has written the operands (and, for a tile's first chunk, the epilogue has read the
        // previous tile's accumulators).
        reg_dec<kDkvRegsCtl>();
        constexpr uint32_t idesc_o = umma_idesc(TM, D, IsBf16<DT>::value, IsBf16<DT>::value, false, true);
        constexpr uint32_t hi = smem_desc_hi(C::ATOM, C::SWZ);
        const uint32_t qd_base = smem_u32(sQD);
        uint32_t n = 0, it = 0;
        for (int i = 0; i < n_my; ++i) {
            const TileGeo t = tile_geo(i);
            if (t.n_ch == 0) continue;
            for (int ch = 0; ch < t.n_ch; ++ch, ++n) {
                const uint32_t q_addr = qd_base + (n % NSTQ) * C::STAGE, g_addr = q_addr + C::KV_BYTES;
                const uint32_t qm_lo = smem_desc_lo(q_addr, C::KV_SLAB), gm_lo = smem_desc_lo(g_addr, C::KV_SLAB);
                const uint32_t tm = tmem_base + (n & 1) * C::TMEM_STAGE;
                const uint32_t acc = ch == 0 ? 0u : 1u;
                mbar_wait(p_full + (n & 1), (n >> 1) & 1, wctx, kErrMmaWait);
                if (ch == 0) {
                    // A tile's first chunk overwrites the accumulators the epilogue warps are still
                    // reading out for the previous tile.  They read dV first and say so, so its dV
                    // MMAs go ahead of its dK MMAs and only the latter wait for the whole read-out.
                    mbar_wait(accv_free, (it & 1) ^ 1, wctx, kErrMmaWait);
                    tc_fence_after();
                    if (elect_one()) {
#pragma unroll
                        for (int kk = 0; kk < C::NKP / 16; ++kk)
                            umma_ts(tmem_base + C::TMEM_DV, tm + C::TMEM_PT + 8 * kk,
                                    desc64(hi, gm_lo + ((kk * 16 * C::ROWB) >> 4)), idesc_o, kk > 0);
                    }
                    __syncwarp();
                    mbar_wait(acc_free, (it & 1) ^ 1, wctx, kErrMmaWait);
                }
                tc_fence_after();
                if (elect_one()) {
#pragma unroll
                    for (int kk = 0; kk < C::NKP / 16; ++kk) {               // dK and dV chains alternate
                        umma_ts(tmem_base + C::TMEM_DK, tm + C::TMEM_DST + 8 * kk,
                                desc64(hi, qm_lo + ((kk * 16 * C::ROWB) >> 4)), idesc_o, acc | (kk > 0));
                        if (ch != 0)
                            umma_ts(tmem_base + C::TMEM_DV, tm + C::TMEM_PT + 8 * kk,
                                    desc64(hi, gm_lo + ((kk * 16 * C::ROWB) >> 4)), idesc_o, 1u);
                    }
                    if (SPLIT) {
#pragma unroll
                        for (int kk = 0; kk < C::NKP / 16; ++kk)
                            umma_ts(tmem_base + C::TMEM_DK, tm + C::TMEM_RES + 8 * kk,
                                    desc64(hi, qm_lo + ((kk * 16 * C::ROWB) >> 4)), idesc_o, 1u);
                    }
                    umma_commit(qd_empty + (n % NSTQ));
                    umma_commit(st_free + (n & 1));
                    if (ch == t.n_ch - 1) umma_commit(acc_full);
                    NA2D_TR(2, 4, n);
                }
                __syncwarp();
            }
            ++it;
        }
    } else if (warp == 11) {
        // ------------------------------------------------------------------ producer of the K, V tile
        reg_dec<kDkvRegsCtl>();
        if (lane == 0) {
            uint32_t it = 0;                            // non-empty tile counter
            LoadTracker lt(bars);
            for (int i = 0; i < n_my; ++i) {
                const TileGeo t = tile_geo(i);
                if (t.n_ch == 0) continue;
                if (!lt.acquire(kv_empty, (it & 1) ^ 1, wctx)) break;
                lt.arm(kv_full, it & 1, 2u * C::Q_BYTES);
#pragma unroll
                for (int s = 0; s < C::NS; ++s) {
                    tma_load_5d(sK + s * C::Q_SLAB, &tm_k, kv_full, s * 64, t.kc0, t.kr0, t.hn, t.hb);
                    tma_load_5d(sV + s * C::Q_SLAB, &tm_v, kv_full, s * 64, t.kc0, t.kr0, t.hn, t.hb);
                }
                ++it;
                // The single K, V buffer is only free again after this tile's last score MMAs, and a
                // load from HBM issued then is what the next tile would wait for: bring the next
                // tile's K, V into L2 now.
                if (i + 1 < n_my) {
                    const TileGeo tn = tile_geo(i + 1);
#pragma unroll
                    for (int s = 0; s < C::NS; ++s) {
                        tma_prefetch_5d(&tm_k, s * 64, tn.kc0, tn.kr0, tn.hn, tn.hb);
                        tma_prefetch_5d(&tm_v, s * 64, tn.kc0, tn.kr0, tn.hn, tn.hb);
                    }
                }
            }
            lt.drain(wctx);
        }
    } else if (warp >= 12) {
        // ------------------------------------------------------------------ epilogue warps
        reg_dec<kDkvRegsEpi>();
        const int quarter = warp & 3;
        const uint32_t tmem_lane = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
        uint8_t* stage = sOut + quarter * 2 * OutStage<32>::BYTES;
        constexpr int RPO = D / 32;                          // 32-channel rounds per output
        uint32_t it = 0, seq = 0;
        for (int i = 0; i < n_my; ++i) {
            const TileGeo t = tile_geo(i);
            if (t.n_ch == 0) {                               // no local query sees this tile: zeros
                uint32_t z[32];
#pragma unroll
                for (int e = 0; e < 32; ++e) z[e] = 0u;
#pragma unroll
                for (int j = 0; j < 2 * RPO; ++j) {
                    if (f32_out)
                        stage_and_store_f32<32, 2>(j / RPO == 0 ? &tm_dv : &tm_dk, stage, z, 1.f, 32 * (j % RPO), t.kc0,
                                                   t.kr0 + quarter * (32 / TW), t.hn, t.hb, lane, &seq);
                    else
                        stage_and_store<DT, 32, 2>(j / RPO == 0 ? &tm_dv : &tm_dk, stage, z, 1.f, 32 * (j % RPO), t.kc0,
                                                   t.kr0 + quarter * (32 / TW), t.hn, t.hb, lane, &seq);
                }
                continue;
            }
            if (warp == 12 && lane == 0) NA2D_TR(0, 0, it);
            mbar_wait(acc_full, it & 1, wctx, kErrMmaWait);
            tc_fence_after();
            if (warp == 12 && lane == 0) NA2D_TR(0, 1, it);
            const int h0 = t.kr0 + quarter * (32 / TW);
            // 2 * RPO rounds of 32 columns, the load of the next round in flight while one is stored
            uint32_t v[2][32];
            tmem_ld_32x32(tmem_lane + C::TMEM_DV, v[0]);
#pragma unroll
            for (int j = 0; j < 2 * RPO; ++j) {
                tmem_ld_wait();
                if (j == RPO - 1) {                          // dV is in registers (or stored)
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(accv_free);
                }
                if (j + 1 < 2 * RPO) {
                    const int which = (j + 1) / RPO, r = (j + 1) % RPO;
                    tmem_ld_32x32(tmem_lane + (which == 0 ? C::TMEM_DV : C::TMEM_DK) + 32 * r, v[(j + 1) & 1]);
                } else {                                     // both accumulators are in registers
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(acc_free);
                    if (warp == 12 && lane == 0) NA2D_TR(0, 2, it);
                }
                // (the softmax scale of dK is already in dS^T: the epilogue only converts)
                if (f32_out)
                    stage_and_store_f32<32, 2, false>(j / RPO == 0 ? &tm_dv : &tm_dk, stage, v[j & 1], 1.f, 32 * (j % RPO),
                                                      t.kc0, h0, t.hn, t.hb, lane, &seq);
                else
                    stage_and_store<DT, 32, 2, false>(j / RPO == 0 ? &tm_dv : &tm_dk, stage, v[j & 1], 1.f, 32 * (j % RPO),
                                                      t.kc0, h0, t.hn, t.hb, lane, &seq);
            }
            if (warp == 12 && lane == 0) NA2D_TR(0, 3, it);
            ++it;
        }
        if (lane == 0) bulk_wait<0>();                       // the staging buffer has been read, the rows written
    } else {
        // ------------------------------------------------------------------ softmax groups
        // Both groups work on every chunk: warps w and w + 4 own the same 32 keys (tensor-memory
        // lanes) and take alternate 8-column blocks of the warp's active range, so a chunk's S^T and
        // dP^T spend half as long in registers before the output MMAs may start - that time is part
        // of the chain that bounds the kernel (score MMAs -> this -> output MMAs -> stage free).
        reg_inc<kDkvRegsSoftmax>();
        const int quarter = warp & 3, group = warp >> 2;
        const int row = quarter * 32 + lane;                 // key of the tile = tensor-memory lane
        const int gtid = quarter * 32 + lane;                // 0..127 inside the group
        const uint32_t tmem_lane = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
        // a warp's 32 / TW key rows are seen from at most that many + 2 ks - 2 query rows
        constexpr int kRows = (32 / TW - 1 + 2 * KS - 1) < C::RC ? (32 / TW - 1 + 2 * KS - 1) : C::RC;
        constexpr int kBlocks = (kRows * C::HW - 1) / 8 + 2;
        constexpr int NACT = kBlocks < C::NB8 ? kBlocks : C::NB8;   // 8-column blocks a warp pair can have in range
        constexpr int NOWN = (NACT + 1) / 2;                        // of which one warp takes at most
        constexpr unsigned long long kRowRep = C::ROW_REP;          // bit r * HW set for every chunk row r

        // lse and delta of this thread's query of chunk (rc, cc) of tile t (zero outside the band); the
        // values are fetched one chunk ahead, so that their latency runs under the wait for the
        // chunk's scores instead of before it
        auto fetch = [&](const TileGeo& t, int rc, int cc, float& l2, float& dl) {
            l2 = 0.f;
            dl = 0.f;
            if (gtid < C::NK) {
                const int br = rc * C::RC + gtid / C::HW, qc = t.qb_c0 + cc * C::HW + gtid % C::HW;
                if (br < t.n_rows && qc < g.W) {
                    const size_t qi = (static_cast<size_t>(t.bn) * g.Hq + (t.q_local_r0 + br)) * g.W + qc;
                    l2 = lse[qi];
                    dl = delta[qi];
                }
            }
        };
        // first tile with chunks at or after i
        auto next_tile = [&](int i, TileGeo& t) {
            for (; i < n_my; ++i) {
                t = tile_geo(i);
                if (t.n_ch > 0) break;
            }
            return i;
        };

        uint32_t n = 0;
        TileGeo t;
        int i = next_tile(0, t);
        float pre_l2 = 0.f, pre_dl = 0.f;
        if (i < n_my) fetch(t, 0, 0, pre_l2, pre_dl);
        while (i < n_my) {
            const int kr = min(t.kr0 + (row / TW), g.Hkv - 1), kc = min(t.kc0 + (row % TW), g.W - 1);
            // the queries that see this thread's key: box rows [row_lo, row_hi), box columns [col_lo, col_hi)
            const int kg = g.kv_row0 + kr;
            const int row_lo = max(na2d_bws(kg, KS), g.q_row0) - t.qb_r0;
            const int row_hi = min(na2d_bwe(kg, g.Hg, KS), g.q_row0 + g.Hq) - t.qb_r0;
            const int col_lo = na2d_bws(kc, KS) - t.qb_c0;
            const int col_hi = na2d_bwe(kc, g.W, KS) - t.qb_c0;
            const int wrow_lo = __shfl_sync(0xffffffffu, row_lo, 0);
            const int wrow_hi = __shfl_sync(0xffffffffu, row_hi, 31);
            TileGeo t_next = t;
            int i_next = n_my;

            for (int ch = 0, rc = 0, cc = 0; ch < t.n_ch; ++ch, ++n) {
                const uint32_t stage = n & 1u, k = n >> 1;  // tensor-memory stage and its use counter
                const uint32_t t_stage = tmem_lane + stage * C::TMEM_STAGE;
                const int r_off = rc * C::RC, c_off = cc * C::HW;       // chunk ch = rc * n_cc + cc
                if (quarter == 0 && lane == 0) NA2D_TR(3 - 2 * group, 0, n);
                // each group keeps its own copy of the chunk's lse * log2(e) and delta (two buffers: a
                // warp may be one chunk ahead of the others of its group, the barrier below keeps it
                // from two)
                float* x_lse = s_x + ((group * 2 + stage) * 2) * 64;
                float* x_delta = x_lse + 64;
                if (gtid < C::NK) {
                    x_lse[gtid] = pre_l2 * kLog2e;
                    x_delta[gtid] = pre_dl * g.scale;       // dS^T carries the softmax scale of dK: scale p (dP - delta)
                }
                // the warp's keys are seen from chunk rows [ra, rb): its active column range
                const int ra = max(wrow_lo - r_off, 0), rb = min(wrow_hi - r_off, C::RC);
                const int j_lo = ra * C::HW;
                const int j_hi = rb > ra ? min(rb * C::HW, C::NK) : 0;
                const int b_hi = (j_hi + 7) >> 3;
                const int b_lo = j_hi > 0 ? (j_lo >> 3) : 0;
                // this thread's column segment inside a chunk row
                const int cl = max(col_lo - c_off, 0), chi = min(col_hi - c_off, C::HW);
                const int seg_len = chi - cl;
                const uint32_t seg = seg_len > 0 ? ((1u << seg_len) - 1u) : 0u;
                // validity of the chunk's (at most 64) columns for this thread's key, one bit each:
                // its column segment repeated in every chunk row, cut to its row range
                unsigned long long m64 = 0ull;
                {
                    const int ta = max(row_lo - r_off, 0), tb = min(row_hi - r_off, C::RC);
                    const unsigned long long rows_hi = tb * C::HW >= 64 ? ~0ull : ((1ull << (max(tb, 0) * C::HW)) - 1ull);
                    const unsigned long long rows_lo = (1ull << (ta * C::HW)) - 1ull;       // ta * HW < 64
                    if (tb > ta) m64 = ((kRowRep * seg) << cl) & rows_hi & ~rows_lo;
                }
                bar_sync(5 + group, 128);                                   // lse / delta are in place
                if (++cc == t.n_cc) {
                    cc = 0;
                    ++rc;
                }
                if (ch + 1 < t.n_ch) {
                    fetch(t, rc, cc, pre_l2, pre_dl);
                } else {
                    i_next = next_tile(i + 1, t_next);
                    if (i_next < n_my) fetch(t_next, 0, 0, pre_l2, pre_dl);
                }
                if (quarter == 0 && lane == 0) NA2D_TR(3 - 2 * group, 1, n);

                mbar_wait(s_full + stage, k & 1, wctx, kErrMmaWait);
                tc_fence_after();
                if (quarter == 0 && lane == 0) NA2D_TR(3 - 2 * group, 2, n);
                uint32_t s[NOWN][8], dp[NOWN][8];
#pragma unroll
                for (int a = 0; a < NOWN; ++a) {
                    const int blk = b_lo + 2 * a + group;
                    if (blk < b_hi) {                                       // warp-uniform
                        tmem_ld_32x8(t_stage + C::TMEM_ST + 8 * blk, s[a]);
                        tmem_ld_32x8(t_stage + C::TMEM_DPT + 8 * blk, dp[a]);
                    }
                }
                tmem_ld_wait();
                // The 16-bit operands go over S^T / dP^T, a block's over other blocks' columns: the
                // partner warp must have its blocks in registers too before either of them writes.
                bar_sync(1 + quarter, 64);
                if (quarter == 0 && lane == 0) NA2D_TR(3 - 2 * group, 3, n);
                {   // blocks outside the active range hold zeros (this warp: every other one of them)
                    const uint32_t z[4] = {0u, 0u, 0u, 0u};
#pragma unroll
                    for (int blk = 0; blk < C::NB8; ++blk) {
                        const bool in_range = blk >= b_lo && blk < b_lo + NACT && blk < b_hi;
                        if (!in_range && ((blk & 1) == group)) {
                            tmem_st_32x4(t_stage + C::TMEM_PT + 4 * blk, z);
                            tmem_st_32x4(t_stage + C::TMEM_DST + 4 * blk, z);
                            if (SPLIT) tmem_st_32x4(t_stage + C::TMEM_RES + 4 * blk, z);
                        }
                    }
                }
                if (quarter == 0 && lane == 0) NA2D_TR(3 - 2 * group, 6, n);
#pragma unroll
                for (int a = 0; a < NOWN; ++a) {
                    const int blk = b_lo + 2 * a + group;
                    if (blk < b_hi) {
                        const uint32_t vmask = static_cast<uint32_t>(m64 >> (8 * blk)) & 0xffu;
                        float l2[8], dl[8];
#pragma unroll
                        for (int v4 = 0; v4 < 2; ++v4) {
                            const float4 x = *reinterpret_cast<const float4*>(x_lse + 8 * blk + 4 * v4);
                            const float4 y = *reinterpret_cast<const float4*>(x_delta + 8 * blk + 4 * v4);
                            l2[4 * v4] = x.x; l2[4 * v4 + 1] = x.y; l2[4 * v4 + 2] = x.z; l2[4 * v4 + 3] = x.w;
                            dl[4 * v4] = y.x; dl[4 * v4 + 1] = y.y; dl[4 * v4 + 2] = y.z; dl[4 * v4 + 3] = y.w;
                        }
                        uint32_t wp[4], wd[4], wr2[4];
#pragma unroll
                        for (int e2 = 0; e2 < 4; ++e2) {
                            float p[2], ds[2];
#pragma unroll
                            for (int h = 0; h < 2; ++h) {
                                const int e = 2 * e2 + h;
                                const float pe = fast_exp2(fmaf(__uint_as_float(s[a][e]), g.sl2, -l2[e]));
                                const bool ok = (vmask >> e) & 1u;         // select, never multiply by zero
                                p[h] = ok ? pe : 0.f;
                                ds[h] = ok ? pe * fmaf(__uint_as_float(dp[a][e]), g.scale, -dl[e]) : 0.f;
                            }
                            wp[e2] = pack2<DT>(p[0], p[1]);
                            wd[e2] = pack2<DT>(ds[0], ds[1]);
                            wr2[e2] = SPLIT ? pack2_residual_bf16(ds[0], ds[1], wd[e2]) : 0u;
                        }
                        tmem_st_32x4(t_stage + C::TMEM_PT + 4 * blk, wp);
                        tmem_st_32x4(t_stage + C::TMEM_DST + 4 * blk, wd);
                        if (SPLIT) tmem_st_32x4(t_stage + C::TMEM_RES + 4 * blk, wr2);
                    }
                }
                if (quarter == 0 && lane == 0) NA2D_TR(3 - 2 * group, 4, n);
                tmem_st_wait();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(p_full + stage);
                if (quarter == 0 && lane == 0) NA2D_TR(3 - 2 * group, 5, n);
            }
            i = i_next;
            t = t_next;
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}

template <typename DT, int D, int KS>
int launch_dkdv(const LaunchCtx& lc, const TensorArg& q, const TensorArg& k, const TensorArg& v, const float* lse,
                const TensorArg& d_o, const float* delta, const TensorArg& d_k, const TensorArg& d_v) {
    using C = DkvCfg<D, KS, IsBf16<DT>::value>;
    const Na2dGeom& g = lc.g;
    CUtensorMap tk, tv, tq, tg, tdk, tdv;
    int rc = make_map(&tk, k, lc.dtype, lc.B, g.N, g.Hkv, g.W, D, TW, TH);
    const int out_c = lc.dkdv_f32 ? 16 : 32;
    if (rc == NA2D_OK) rc = make_map(&tdk, d_k, lc.dtype, lc.B, g.N, g.Hkv, g.W, D, TW, 32 / TW, out_c, lc.dkdv_f32);
    if (rc == NA2D_OK) rc = make_map(&tdv, d_v, lc.dtype, lc.B, g.N, g.Hkv, g.W, D, TW, 32 / TW, out_c, lc.dkdv_f32);
    if (rc == NA2D_OK) rc = make_map(&tv, v, lc.dtype, lc.B, g.N, g.Hkv, g.W, D, TW, TH);
    if (rc == NA2D_OK) rc = make_map(&tq, q, lc.dtype, lc.B, g.N, g.Hq, g.W, D, C::HW, C::RC);
    if (rc == NA2D_OK) rc = make_map(&tg, d_o, lc.dtype, lc.B, g.N, g.Hq, g.W, D, C::HW, C::RC);
    if (rc != NA2D_OK) return rc;
    const int tiles_r = (g.Hkv + TH - 1) / TH, tiles_c = (g.W + TW - 1) / TW;
    const long long tiles = (long long)g.BN * tiles_r * tiles_c;
    if (tiles > 0x7fffffffLL) return NA2D_ERR_TOO_LARGE;
    auto kern = dkdv_kernel<DT, D, KS>;
    static std::atomic<unsigned long long> opted{0};
    if (opt_in_smem(kern, C::SMEM, lc.device, opted) != cudaSuccess) return NA2D_ERR_CUDA;
    const int grid = persistent_grid(lc, tiles);
    kern<<<grid, 512, C::SMEM, lc.st>>>(tk, tv, tq, tg, tdk, tdv, lse, delta, lc.dkdv_f32 ? 1 : 0, lc.err_word, g,
                                        tiles_r, tiles_c, (int)tiles);
    *lc.launched += 1;
    return cudaGetLastError() == cudaSuccess ? NA2D_OK : NA2D_ERR_CUDA;
}

}  // namespace na2d_tc
