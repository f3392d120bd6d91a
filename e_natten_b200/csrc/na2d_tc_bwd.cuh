// Persistent, warp-specialised tcgen05 dQ kernel (also produces the row delta).  Included by
// na2d_tc_dq.cu.
//
// One CTA per SM walks query tiles (TH x TW queries, row r of every MMA = query r =
// tensor-memory lane r).  The tile's halo box of keys is taken in chunks of whole box rows.
//     S = Q K_c^T,  dP = dO V_c^T                          (tensor memory, fp32)
//     p = exp(S - lse),  delta = sum_j p dP                (softmax warps, registers)
//     dS = p (dP - delta)  -> tensor memory, 16 bit        (head + residual on the bf16 path)
//     dQ += dS K_c                                         (dS read from tensor memory; the softmax
//                                                           scale is applied to the finished dQ)
// delta needs every chunk of the tile before any dS can be formed exactly.  With one chunk (kernel
// sizes up to 5: at most 256 keys) a tile is a single unit and dQ reuses the S columns.  With
// several chunks there are two ways:
//   * one walk with a correction.  The caller hands in an estimate d~ of delta (dO . o from the
//     stored output, see na2d_delta.cuh; off by the rounding of o, a few 1e-2 at most).  Every
//     unit forms dS~ = p (dP - d~), adds dS~ K_c to dQ and, with one more MMA, p K_c to a
//     second accumulator B, while the exact delta = sum_j p dP builds up in registers.  Since
//     sum_j p (dP - delta) k = sum_j p (dP - d~) k - (delta - d~) sum_j p k, the epilogue stores
//     scale (dQ - (delta - d~) B).  B only meets the small factor (delta - d~), so a single 16-bit
//     p is enough for it.  The exact delta is what the kernel writes out for the dK/dV kernel.
//   * two walks (no estimate given): units 0..NCH-1 only add up delta, units NCH..2NCH-1 repeat
//     the two score MMAs and accumulate dQ.
// Twelve warps: 0-7 softmax (warps w and w+4 share 32 queries and split the 16-column blocks),
// 8 TMA producer, 9 MMA issue, 10-11 idle (register donors).
#pragma once

namespace na2d_tc {

// Keys per chunk at most: the whole box where it fits 256 columns (a single unit); else what
// leaves room in tensor memory for S, dP and the two output accumulators dQ and B.
constexpr int dq_nmax(int d, int ks) {
    return (TH + ks - 1) * (TW + ks - 1) <= 256 ? 256 : (d == 128 ? 128 : 192);
}

template <int D, int KS, bool SPLIT>
struct DqCfg : Cfg<D, KS, dq_nmax(D, KS)> {
    using B = Cfg<D, KS, dq_nmax(D, KS)>;
    static constexpr bool ONE = B::NCH == 1;
    static constexpr int NMAX = dq_nmax(D, KS);
    static constexpr int TMEM_S = 0;
    static constexpr int TMEM_DP = NMAX;
    static constexpr int TMEM_DQ = ONE ? 0 : 2 * NMAX;                 // one chunk: dQ reuses the S columns
    static constexpr int TMEM_BK = ONE ? 0 : 2 * NMAX + D;             // sum_j p k (several chunks only)
    static constexpr int TMEM_DSH = TMEM_DP;                           // dS (head) over dP
    static constexpr int TMEM_RES = ONE ? 384 : 0;                     // dS residual: upper dP half / lower half of S
    static constexpr int TMEM_PH = B::NKP / 2;                         // p (head): upper half of S (several chunks only)
    static constexpr int OUT_BYTES = 8 * OutStage<D / 2>::BYTES;       // output staging of the 8 softmax warps
    static constexpr int FIXED = 2 * B::Q_BYTES + OUT_BYTES + 2 * 2 * 128 * 4 /*delta exchange*/ + 256 + 1024;
    // K and V chunk rings: two stages each where they fit, so that a chunk's loads run under the
    // previous chunk's MMAs (a K chunk is only free again after the dQ MMAs that read it)
    static constexpr int NST = (FIXED + 4 * B::KV_BYTES <= kSmemLimit) ? 2 : 1;
    static constexpr int SMEM = FIXED + 2 * NST * B::KV_BYTES;
    static constexpr int NB16 = (B::NKP + 15) / 16;
    static_assert(SMEM <= kSmemLimit, "dQ kernel shared memory");
    static_assert(B::NKP <= NMAX, "tensor memory layout");
    static_assert(ONE || TMEM_BK + D <= 512, "tensor memory layout");
    static_assert(!SPLIT || !ONE || B::NKP / 2 <= 128, "residual operand does not fit");
    static_assert((B::NKP / 2) % 8 == 0, "operand halves start on a block boundary");
};

template <typename DT, int D, int KS>
__global__ void __launch_bounds__(384, 1)
dq_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_do,
          const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
          const __grid_constant__ CUtensorMap tm_dq, const float* __restrict__ lse, float* __restrict__ delta,
          const float* __restrict__ delta_in, const int want_dq_arg, unsigned int* __restrict__ err_word,
          const Na2dGeom g, const int tiles_r, const int tiles_c, const int total_tiles) {
    constexpr bool SPLIT = IsBf16<DT>::value;
    using C = DqCfg<D, KS, SPLIT>;
    constexpr int NCH = C::NCH;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sQ = smem;
    uint8_t* sDO = sQ + C::Q_BYTES;
    constexpr int NST = C::NST;
    uint8_t* sK = sDO + C::Q_BYTES;                   // NST x key chunk   [NKP x D]
    uint8_t* sV = sK + NST * C::KV_BYTES;             // NST x value chunk [NKP x D]
    uint8_t* sOut = sV + NST * C::KV_BYTES;           // 8 x output staging (1024-byte aligned)
    float* x_sum = reinterpret_cast<float*>(sOut + C::OUT_BYTES);     // [tile parity][half][row]
    uint64_t* bars = reinterpret_cast<uint64_t*>(x_sum + 2 * 2 * 128);
    uint64_t* q_full = bars + 0;             // TMA -> MMA (Q and dO tile)
    uint64_t* q_empty = bars + 1;            // MMA (commit) -> TMA
    uint64_t* k_full = bars + 2;             // [2]
    uint64_t* k_empty = bars + 4;            // [2]
    uint64_t* v_full = bars + 6;             // [2]
    uint64_t* v_empty = bars + 8;            // [2]
    uint64_t* s_full = bars + 10;            // MMA (commit) -> softmax: S and dP are complete
    uint64_t* s_free = bars + 11;            // softmax -> MMA: S and dP have been read (delta-only units)
    uint64_t* p_full = bars + 12;            // softmax -> MMA: dS is in tensor memory
    uint64_t* dq_full = bars + 13;           // MMA (commit) -> softmax (epilogue)
    uint64_t* dq_free = bars + 14;           // softmax -> MMA
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 15);
    const WaitCtx wctx{reinterpret_cast<WaitState*>(bars + 16)};

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n_my = total_tiles > (int)blockIdx.x ? (total_tiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;
    const bool want_dq = want_dq_arg != 0;

    if (tid == 0) {
        wait_state_init(wctx.st, err_word, kWaitLimitNs);
        mbar_init(q_full, 1);
        mbar_init(q_empty, 1);
        for (int i = 0; i < 2; ++i) {
            mbar_init(k_full + i, 1);
            mbar_init(k_empty + i, 1);
            mbar_init(v_full + i, 1);
            mbar_init(v_empty + i, 1);
        }
        mbar_init(s_full, 1);
        mbar_init(s_free, 8);
        mbar_init(p_full, 8);
        mbar_init(dq_full, 1);
        mbar_init(dq_free, 8);
        mbar_fence_init();
        tma_prefetch_desc(&tm_q);
        tma_prefetch_desc(&tm_do);
        tma_prefetch_desc(&tm_k);
        tma_prefetch_desc(&tm_v);
        tma_prefetch_desc(&tm_dq);
    }
    if (warp == 0) {
        __syncwarp();
        tmem_alloc(tmem_slot, 512);
        tmem_relinquish();
    }
    // K rows [NK, NKP) of every stage are contraction rows of dQ = dS K that TMA never writes: zero them once.
    if constexpr (C::NKP > C::NK) {
        constexpr int pad16 = (C::NKP - C::NK) * C::ROWB / 16;
        for (int i = tid; i < NST * C::NS * pad16; i += 384) {
            const int which = i / pad16, off = i - which * pad16;             // which = stage * NS + slab
            st_shared_v4(smem_u32(sK + (which / C::NS) * C::KV_BYTES + (which % C::NS) * C::KV_SLAB + C::NK * C::ROWB +
                                  off * 16), 0u, 0u, 0u, 0u);
        }
        fence_proxy_async();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    // my i-th tile: unit bn (head bn % N of batch bn / N, split where a TMA coordinate needs it),
    // first row r0, first column c0
    auto decode = [&](int i, int& bn, int& r0, int& c0) {
        int t = (int)blockIdx.x + i * (int)gridDim.x;
        const int tc = t % tiles_c;
        t /= tiles_c;
        r0 = (t % tiles_r) * TH;
        c0 = tc * TW;
        bn = t / tiles_r;
    };
    // A unit u of a tile works on chunk u % NCH.  Units from first_ds on form dS and add to dQ; the
    // units before it (a first walk, only when no estimate of delta is given) add up delta.
    // Without a dQ output only the delta units run.
    const bool given = !C::ONE && want_dq && delta_in != nullptr;      // one walk with the correction
    const int first_ds = (C::ONE || given) ? 0 : NCH;
    const int units_run = want_dq ? first_ds + NCH : NCH;

    if (warp == 8) {
        // ------------------------------------------------------------------ producer
        reg_dec<kRegsDonor>();
        if (lane == 0) {
            uint32_t n = 0;
            LoadTracker lt(bars);
            for (int i = 0; i < n_my && lt.ok; ++i) {
                int bn, r0, c0, hn, hb;
                decode(i, bn, r0, c0);
                split_unit(bn, g, hn, hb);
                const int box_r0 = na2d_ws(g.q_row0 + r0, g.Hg, KS) - g.kv_row0;
                const int box_c0 = na2d_ws(c0, g.W, KS);
                if (!lt.acquire(q_empty, (i & 1) ^ 1, wctx)) break;
                lt.arm(q_full, i & 1, 2u * C::Q_BYTES);
#pragma unroll
                for (int s = 0; s < C::NS; ++s) {
                    tma_load_5d(sQ + s * C::Q_SLAB, &tm_q, q_full, s * 64, c0, r0, hn, hb);
                    tma_load_5d(sDO + s * C::Q_SLAB, &tm_do, q_full, s * 64, c0, r0, hn, hb);
                }
                for (int u = 0; u < units_run; ++u, ++n) {
                    const int c = u % NCH;
                    const uint32_t st = n % NST, par = (n / NST) & 1;
                    if (!lt.acquire(v_empty + st, par ^ 1, wctx)) break;
                    lt.arm(v_full + st, par, (uint32_t)C::NS * C::NK * C::ROWB);
#pragma unroll
                    for (int s = 0; s < C::NS; ++s)
                        tma_load_5d(sV + st * C::KV_BYTES + s * C::KV_SLAB, &tm_v, v_full + st, s * 64, box_c0,
                                    box_r0 + c * C::RC, hn, hb);
                    if (!lt.acquire(k_empty + st, par ^ 1, wctx)) break;
                    lt.arm(k_full + st, par, (uint32_t)C::NS * C::NK * C::ROWB);
#pragma unroll
                    for (int s = 0; s < C::NS; ++s)
                        tma_load_5d(sK + st * C::KV_BYTES + s * C::KV_SLAB, &tm_k, k_full + st, s * 64, box_c0,
                                    box_r0 + c * C::RC, hn, hb);
                }
            }
            lt.drain(wctx);
        }
    } else if (warp == 9) {
        // ------------------------------------------------------------------ MMA issue
        reg_dec<kRegsDonor>();
        const bool leader = lane == 0;
        constexpr uint32_t idesc_s = umma_idesc(TM, C::NKP, IsBf16<DT>::value, IsBf16<DT>::value, false, false);
        constexpr uint32_t idesc_o = umma_idesc(TM, D, IsBf16<DT>::value, IsBf16<DT>::value, false, true);
        constexpr uint32_t hi = smem_desc_hi(C::ATOM, C::SWZ);
        const uint32_t q_lo = smem_desc_lo(smem_u32(sQ), 16), g_lo = smem_desc_lo(smem_u32(sDO), 16);
        uint32_t n = 0, n_free = 0, n_p = 0;          // units, delta-only units, dS units so far
        for (int i = 0; i < n_my; ++i) {
            mbar_wait(q_full, i & 1, wctx, kErrLoadWait);
            for (int u = 0; u < units_run; ++u, ++n) {
                const bool forms_ds = want_dq && u >= first_ds;
                const uint32_t st = n % NST, par = (n / NST) & 1;
                const uint32_t k_lo = smem_desc_lo(smem_u32(sK + st * C::KV_BYTES), 16);
                const uint32_t v_lo = smem_desc_lo(smem_u32(sV + st * C::KV_BYTES), 16);
                const uint32_t km_lo = smem_desc_lo(smem_u32(sK + st * C::KV_BYTES), C::KV_SLAB);
                if (leader) NA2D_TR(2, 0, n);
                mbar_wait(k_full + st, par, wctx, kErrLoadWait);
                mbar_wait(v_full + st, par, wctx, kErrLoadWait);
                // the accumulators the score MMAs overwrite must have been read
                if (u > 0 && !(want_dq && u - 1 >= first_ds)) {  // previous unit was delta-only
                    mbar_wait(s_free, (n_free & 1) ^ 1, wctx, kErrMmaWait);
                }
                if (u == 0 && i > 0) {
                    if (C::ONE || !want_dq) {
                        // previous tile: its last unit either left dQ over S (epilogue must have read
                        // it) or was delta-only (S must have been read)
                        if (want_dq) mbar_wait(dq_free, (i & 1) ^ 1, wctx, kErrMmaWait);
                        else mbar_wait(s_free, (n_free & 1) ^ 1, wctx, kErrMmaWait);
                    }
                }
                tc_fence_after();
                if (elect_one()) {
                    NA2D_TR(2, 1, n);
#pragma unroll
                    for (int kk = 0; kk < D / 16; ++kk) {
                        constexpr int kPerSlab = C::SLAB_C / 16;
                        const int slab = kk / kPerSlab, in_slab = kk % kPerSlab;
                        umma_ss(tmem_base + C::TMEM_S, desc64(hi, q_lo + ((slab * C::Q_SLAB) >> 4) + 2 * in_slab),
                                desc64(hi, k_lo + ((slab * C::KV_SLAB) >> 4) + 2 * in_slab), idesc_s, kk > 0);
                    }
#pragma unroll
                    for (int kk = 0; kk < D / 16; ++kk) {
                        constexpr int kPerSlab = C::SLAB_C / 16;
                        const int slab = kk / kPerSlab, in_slab = kk % kPerSlab;
                        umma_ss(tmem_base + C::TMEM_DP, desc64(hi, g_lo + ((slab * C::Q_SLAB) >> 4) + 2 * in_slab),
                                desc64(hi, v_lo + ((slab * C::KV_SLAB) >> 4) + 2 * in_slab), idesc_s, kk > 0);
                    }
                    umma_commit(s_full);
                    umma_commit(v_empty + st);
                    if (!forms_ds) umma_commit(k_empty + st);
                    if (u == units_run - 1) umma_commit(q_empty);     // last score MMAs of the tile
                    NA2D_TR(2, 2, n);
                }
                __syncwarp();
                if (!forms_ds) { ++n_free; continue; }
                mbar_wait(p_full, n_p & 1, wctx, kErrMmaWait);
                ++n_p;
                if (!C::ONE && u == first_ds && i > 0) mbar_wait(dq_free, (i & 1) ^ 1, wctx, kErrMmaWait);
                tc_fence_after();
                if (elect_one()) {
                    NA2D_TR(2, 3, n);
                    const uint32_t acc = (!C::ONE && u > first_ds) ? 1u : 0u;
#pragma unroll
                    for (int kk = 0; kk < C::NKP / 16; ++kk)
                        umma_ts(tmem_base + C::TMEM_DQ, tmem_base + C::TMEM_DSH + 8 * kk,
                                desc64(hi, km_lo + ((kk * 16 * C::ROWB) >> 4)), idesc_o, acc | (kk > 0));
                    if (SPLIT) {
#pragma unroll
                        for (int kk = 0; kk < C::NKP / 16; ++kk)
                            umma_ts(tmem_base + C::TMEM_DQ, tmem_base + C::TMEM_RES + 8 * kk,
                                    desc64(hi, km_lo + ((kk * 16 * C::ROWB) >> 4)), idesc_o, 1u);
                    }
                    if (given) {                                 // B (+)= p K_c
#pragma unroll
                        for (int kk = 0; kk < C::NKP / 16; ++kk)
                            umma_ts(tmem_base + C::TMEM_BK, tmem_base + C::TMEM_PH + 8 * kk,
                                    desc64(hi, km_lo + ((kk * 16 * C::ROWB) >> 4)), idesc_o, acc | (kk > 0));
                    }
                    umma_commit(k_empty + st);
                    if (u == units_run - 1) umma_commit(dq_full);
                    NA2D_TR(2, 4, n);
                }
                __syncwarp();
            }
        }
    } else if (warp >= 10) {
        reg_dec<kRegsDonor>();
    } else {
        // ------------------------------------------------------------------ softmax warps
        reg_inc<kRegsSoftmax>();
        const int quarter = warp & 3, half = warp >> 2;
        const int row = quarter * 32 + lane;                 // query of the tile = tensor-memory lane
        const uint32_t tmem_lane = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
        constexpr int DH = D / 2;                            // output columns stored by this half
        constexpr int NBH = (C::NB16 + 1) / 2;               // own blocks at most
        constexpr int kRows = (32 / TW - 1 + KS) < C::RC ? (32 / TW - 1 + KS) : C::RC;
        constexpr int kBlocks = (kRows * C::HW - 1) / 16 + 2;
        constexpr int NACT = (kBlocks + 1) / 2 < NBH ? (kBlocks + 1) / 2 : NBH;

        uint32_t n = 0, n_x = 0;                             // units, delta exchanges so far
        for (int i = 0; i < n_my; ++i) {
            int bn, r0, c0;
            decode(i, bn, r0, c0);
            const int box_r0 = na2d_ws(g.q_row0 + r0, g.Hg, KS) - g.kv_row0;
            const int box_c0 = na2d_ws(c0, g.W, KS);
            const int qr_raw = r0 + (row / TW), qc_raw = c0 + (row % TW);
            const bool q_valid = qr_raw < g.Hq && qc_raw < g.W;
            const int qr = min(qr_raw, g.Hq - 1), qc = min(qc_raw, g.W - 1);
            const size_t qi = (static_cast<size_t>(bn) * g.Hq + qr) * g.W + qc;
            const int wr = na2d_ws(g.q_row0 + qr, g.Hg, KS) - g.kv_row0 - box_r0;   // in [0, TH)
            const int wc = na2d_ws(qc, g.W, KS) - box_c0;                            // in [0, TW)
            const int wr_lo = __shfl_sync(0xffffffffu, wr, 0);
            const int wr_hi = __shfl_sync(0xffffffffu, wr, 31);
            const float lse2 = lse[qi] * kLog2e;
            float dl_part = 0.f;                             // this half's part of delta
            float dl = 0.f;                                  // delta, once every chunk has been seen
            // The estimate is read before this tile's first partner barrier and the exact value
            // written (by the partner warp of half 0, to the same address when delta_in == delta)
            // after its last one, so the read never sees the new value.
            const float d_est = given ? delta_in[qi] : 0.f;

            for (int u = 0; u < units_run; ++u, ++n) {
                const int ch = u % NCH;
                const bool forms_ds = want_dq && u >= first_ds;
                const bool adds_delta = C::ONE || given || u < NCH;
                const int row_off = ch * C::RC;
                const int j_lo = max(wr_lo - row_off, 0) * C::HW;
                const int j_hi = min(min(wr_hi + KS - row_off, C::RC) * C::HW, C::NK);       // exclusive
                const int b_hi = (max(j_hi, 0) + 15) >> 4;
                const int bi_lo = ((j_lo >> 4) - half + 1) >> 1;

                if (tid == 0) NA2D_TR(3, 0, n);
                mbar_wait(s_full, n & 1, wctx, kErrMmaWait);
                tc_fence_after();
                if (tid == 0) NA2D_TR(3, 1, n);
                uint32_t s[NACT][16], dp[NACT][16];
                uint32_t vmask[NACT];
#pragma unroll
                for (int a = 0; a < NACT; ++a) {
                    const int blk = half + 2 * (bi_lo + a);
                    if (blk < b_hi) {                                        // warp-uniform
                        tmem_ld_32x16(tmem_lane + C::TMEM_S + 16 * blk, s[a]);
                        tmem_ld_32x16(tmem_lane + C::TMEM_DP + 16 * blk, dp[a]);
                    }
                }
#pragma unroll
                for (int a = 0; a < NACT; ++a) {                             // validity masks, loads in flight
                    const int blk = half + 2 * (bi_lo + a);
                    vmask[a] = (blk < b_hi) ? block_mask16<C::HW, KS, C::RC>(blk, wr - row_off, wc) : 0u;
                }
                tmem_ld_wait();
                if (tid == 0) NA2D_TR(3, 2, n);

                // p = exp(s - lse) in place of s; this half's part of delta
                float d0 = 0.f, d1 = 0.f;
#pragma unroll
                for (int a = 0; a < NACT; ++a) {
                    if (half + 2 * (bi_lo + a) < b_hi) {
#pragma unroll
                        for (int e = 0; e < 16; e += 2) {
                            const float p0 = ((vmask[a] >> e) & 1u)
                                                 ? fast_exp2(fmaf(__uint_as_float(s[a][e]), g.sl2, -lse2)) : 0.f;
                            const float p1 = ((vmask[a] >> (e + 1)) & 1u)
                                                 ? fast_exp2(fmaf(__uint_as_float(s[a][e + 1]), g.sl2, -lse2)) : 0.f;
                            s[a][e] = __float_as_uint(p0);
                            s[a][e + 1] = __float_as_uint(p1);
                            // masked columns may hold anything (padding keys): keep them out by
                            // selection, never by multiplying with zero
                            if (!((vmask[a] >> e) & 1u)) dp[a][e] = 0u;
                            if (!((vmask[a] >> (e + 1)) & 1u)) dp[a][e + 1] = 0u;
                            d0 = fmaf(p0, __uint_as_float(dp[a][e]), d0);
                            d1 = fmaf(p1, __uint_as_float(dp[a][e + 1]), d1);
                        }
                    }
                }
                if (adds_delta) dl_part += d0 + d1;

                if (adds_delta && (C::ONE || u == NCH - 1)) {
                    // all chunks seen: add the partner's part; both now hold delta
                    x_sum[((n_x & 1) * 2 + half) * 128 + row] = dl_part;
                    bar_sync(1 + quarter, 64);
                    dl = dl_part + x_sum[((n_x & 1) * 2 + (half ^ 1)) * 128 + row];
                    ++n_x;
                    if (q_valid && half == 0) delta[qi] = dl;
                } else {
                    // the partner must have read its blocks before 16-bit operands go over them
                    bar_sync(1 + quarter, 64);
                }

                if (tid == 0) NA2D_TR(3, 3, n);
                if (!forms_ds) {
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(s_free);
                    continue;
                }

                // dS = p (dP - delta) as packed 16-bit pairs (head, and residual on the bf16 path);
                // with the one-walk scheme delta is the estimate, and p goes along as a third operand
                const float dlu = given ? d_est : dl;
#pragma unroll
                for (int a = 0; a < NACT; ++a) {
                    const int blk = half + 2 * (bi_lo + a);
                    if (blk < b_hi) {
                        uint32_t wd[8], wr2[8];
#pragma unroll
                        for (int e2 = 0; e2 < 8; ++e2) {
                            const float ds0 = ((vmask[a] >> (2 * e2)) & 1u)
                                ? __uint_as_float(s[a][2 * e2]) * (__uint_as_float(dp[a][2 * e2]) - dlu) : 0.f;
                            const float ds1 = ((vmask[a] >> (2 * e2 + 1)) & 1u)
                                ? __uint_as_float(s[a][2 * e2 + 1]) * (__uint_as_float(dp[a][2 * e2 + 1]) - dlu) : 0.f;
                            wd[e2] = pack2<DT>(ds0, ds1);
                            wr2[e2] = SPLIT ? pack2_residual_bf16(ds0, ds1, wd[e2]) : 0u;
                        }
                        tmem_st_32x8(tmem_lane + C::TMEM_DSH + 8 * blk, wd);
                        if (SPLIT) tmem_st_32x8(tmem_lane + C::TMEM_RES + 8 * blk, wr2);
                        if (given) {                             // p of masked columns is an exact zero
#pragma unroll
                            for (int e2 = 0; e2 < 8; ++e2)
                                wd[e2] = pack2<DT>(__uint_as_float(s[a][2 * e2]), __uint_as_float(s[a][2 * e2 + 1]));
                            tmem_st_32x8(tmem_lane + C::TMEM_PH + 8 * blk, wd);
                        }
                    }
                }
                {   // own blocks outside the range hold zeros
                    const uint32_t z[8] = {0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u};
                    for (int bi = 0; bi < NBH; ++bi) {
                        const int blk = half + 2 * bi;
                        const bool in_range = bi >= bi_lo && bi < bi_lo + NACT && blk < b_hi;
                        if (!in_range && 16 * blk < C::NKP) {
                            tmem_st_32x8(tmem_lane + C::TMEM_DSH + 8 * blk, z);
                            if (SPLIT) tmem_st_32x8(tmem_lane + C::TMEM_RES + 8 * blk, z);
                            if (given) tmem_st_32x8(tmem_lane + C::TMEM_PH + 8 * blk, z);
                        }
                    }
                }
                tmem_st_wait();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(p_full);
                if (tid == 0) NA2D_TR(3, 4, n);
            }

            if (want_dq) {
                // ---- epilogue: this half's columns of the thread's dQ row
                mbar_wait(dq_full, i & 1, wctx, kErrMmaWait);
                tc_fence_after();
                if (tid == 0) NA2D_TR(3, 5, n - 1);
                uint32_t acc[DH];
#pragma unroll
                for (int piece = 0; piece < DH / 16; ++piece)
                    tmem_ld_32x16(tmem_lane + C::TMEM_DQ + half * DH + 16 * piece,
                                  *reinterpret_cast<uint32_t(*)[16]>(&acc[16 * piece]));
                if (given) {
                    // dQ - (delta - estimate) B, piece by piece
                    const float corr = dl - d_est;
#pragma unroll
                    for (int piece = 0; piece < DH / 16; ++piece) {
                        uint32_t bk[16];
                        tmem_ld_32x16(tmem_lane + C::TMEM_BK + half * DH + 16 * piece, bk);
                        tmem_ld_wait();
#pragma unroll
                        for (int e = 0; e < 16; ++e)
                            acc[16 * piece + e] = __float_as_uint(fmaf(-corr, __uint_as_float(bk[e]), __uint_as_float(acc[16 * piece + e])));
                    }
                }
                tmem_ld_wait();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(dq_free);
                if (tid == 0) NA2D_TR(3, 6, n - 1);
                int hn, hb;
                split_unit(bn, g, hn, hb);
                stage_and_store<DT, DH>(&tm_dq, sOut + warp * OutStage<DH>::BYTES, acc, g.scale, half * DH, c0,
                                        r0 + quarter * (32 / TW), hn, hb, lane);
                if (tid == 0) NA2D_TR(3, 7, n - 1);
            }
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

// delta_in: row deltas formed beforehand (or null: the kernel forms them itself and writes `delta`).
template <typename DT, int D, int KS>
int launch_dq(const LaunchCtx& lc, const TensorArg& q, const TensorArg& k, const TensorArg& v, const float* lse,
              const TensorArg& d_o, const TensorArg& d_q, float* delta, const float* delta_in) {
    // kernel sizes 3 and 5 with a dQ output go to the strip kernel; this one keeps the larger
    // windows and the delta-only call
    if constexpr (KS <= 5) {
        if (d_q.ptr != nullptr) return launch_dq1<DT, D, KS>(lc, q, k, v, lse, d_o, d_q, delta);
    }
    using C = DqCfg<D, KS, IsBf16<DT>::value>;
    const Na2dGeom& g = lc.g;
    CUtensorMap tq, tg, tk, tv, tdq;
    int rc = make_map(&tq, q, lc.dtype, lc.B, g.N, g.Hq, g.W, D, TW, TH);
    // without a dQ buffer the kernel only writes delta; the map then points at q and is never used
    if (rc == NA2D_OK) rc = make_map(&tdq, d_q.ptr ? d_q : q, lc.dtype, lc.B, g.N, g.Hq, g.W, D, TW, 32 / TW, OutStage<D / 2>::RW);
    if (rc == NA2D_OK) rc = make_map(&tg, d_o, lc.dtype, lc.B, g.N, g.Hq, g.W, D, TW, TH);
    if (rc == NA2D_OK) rc = make_map(&tk, k, lc.dtype, lc.B, g.N, g.Hkv, g.W, D, C::HW, C::RC);
    if (rc == NA2D_OK) rc = make_map(&tv, v, lc.dtype, lc.B, g.N, g.Hkv, g.W, D, C::HW, C::RC);
    if (rc != NA2D_OK) return rc;
    const int tiles_r = (g.Hq + TH - 1) / TH, tiles_c = (g.W + TW - 1) / TW;
    const long long tiles = (long long)g.BN * tiles_r * tiles_c;
    if (tiles > 0x7fffffffLL) return NA2D_ERR_TOO_LARGE;
    auto kern = dq_kernel<DT, D, KS>;
    static std::atomic<unsigned long long> opted{0};
    if (opt_in_smem(kern, C::SMEM, lc.device, opted) != cudaSuccess) return NA2D_ERR_CUDA;
    const int grid = persistent_grid(lc, tiles);
    kern<<<grid, 384, C::SMEM, lc.st>>>(tq, tg, tk, tv, tdq, lse, delta, delta_in, d_q.ptr != nullptr, lc.err_word, g,
                                        tiles_r, tiles_c, (int)tiles);
    *lc.launched += 1;
    return cudaGetLastError() == cudaSuccess ? NA2D_OK : NA2D_ERR_CUDA;
}

}  // namespace na2d_tc
