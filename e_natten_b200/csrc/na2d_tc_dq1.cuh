// Persistent, warp-specialised tcgen05 dQ kernel for kernel sizes whose key box splits into two
// column strips of at most 128 keys (3 and 5).  Included by na2d_tc.cuh.
//
// One CTA per SM walks query tiles (TH x TW queries = tensor-memory lanes).  The key box of a tile
// is cut into a left strip A and a right strip B (box rows x half the box columns each):
//     S_x = Q K_x^T,  dP_x = dO V_x^T          (x = A, B; four accumulators fill tensor memory)
//     p = exp(S - lse),  delta = sum_j p_j dP_j over both strips     (softmax warps, registers)
//     dS_x = scale p_x (dP_x - delta)  ->  tensor memory, over dP_x   (head + residual on bf16)
//     dQ = dS_A K_A + dS_B K_B                  (accumulated over S_B, which is in registers by then)
// Splitting the box lets the tensor pipe work under the softmax warps: the score MMAs of strip B
// run while strip A is read, dS_A K_A runs while dS_B is formed, and the score MMAs of the next
// tile run under this tile's epilogue.  The four strip buffers in shared memory
// change roles from tile to tile (K_A, V_A, K_B, V_B of tile i+1 go where V_A, V_B, K_A, K_B of
// tile i were), so the next tile's K_A and V_A can be fetched as soon as the score MMAs are done.
// Twelve warps: 0-7 softmax (warps w and w+4 share 32 queries and split the 16-column blocks),
// 8 TMA producer, 9 MMA issue, 10-11 idle (register donors).
#pragma once

namespace na2d_tc {

template <int D, int KS, bool SPLIT>
struct Dq1Cfg : Cfg<D, KS, 128, 0, 2> {
    using B = Cfg<D, KS, 128, 0, 2>;
    static_assert(B::NCH == 1, "a strip must hold all box rows");
    static constexpr int TMEM_SA = 0, TMEM_DPA = 128, TMEM_SB = 256, TMEM_DPB = 384;
    static constexpr int TMEM_DQ = TMEM_SB;                               // dQ accumulates over S_B
    // Two output staging buffers for each of the 8 softmax warps where they fit.  They only fit
    // (head dim 128) because the kernel asks for its dynamic shared memory on a 1024-byte boundary
    // instead of keeping 1024 bytes of slack to round the base up itself.
    static constexpr int NOUT = (2 * B::Q_BYTES + 4 * B::KV_BYTES + 16 * OutStage<D / 2>::BYTES + 2 * 2 * 128 * 4 + 256 <= kSmemLimit) ? 2 : 1;
    static constexpr int OUT_BYTES = 8 * NOUT * OutStage<D / 2>::BYTES;
    static constexpr int SMEM = 2 * B::Q_BYTES + 4 * B::KV_BYTES + OUT_BYTES + 2 * 2 * 128 * 4 + 256;
    static constexpr int NB16 = B::NKP / 16;
    static constexpr unsigned long long REP_LO = row_repeat_lo(B::HW, KS), REP_HI = row_repeat_hi(B::HW, KS);
    static_assert(SMEM <= kSmemLimit, "dQ strip kernel shared memory");
    static_assert(B::NKP <= 128 && D <= 128, "tensor memory layout");
};

template <typename DT, int D, int KS>
__global__ void __launch_bounds__(384, 1)
dq1_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_do,
           const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
           const __grid_constant__ CUtensorMap tm_dq, const float* __restrict__ lse, float* __restrict__ delta,
           unsigned int* __restrict__ err_word, const Na2dGeom g, const int tiles_r, const int tiles_c,
           const int total_tiles) {
    constexpr bool SPLIT = IsBf16<DT>::value;
    using C = Dq1Cfg<D, KS, SPLIT>;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = smem_raw;
    if (smem_u32(smem_raw) & 1023u) {                 // the swizzled operand layouts need it; never seen
        if (threadIdx.x == 0) atomicOr(err_word, kErrSmemBase);
        return;
    }
    uint8_t* sQ = smem;
    uint8_t* sDO = sQ + C::Q_BYTES;
    uint8_t* sStrip = sDO + C::Q_BYTES;               // 4 strip buffers [NKP x D]
    uint8_t* sOut = sStrip + 4 * C::KV_BYTES;         // 8 x output staging (1024-byte aligned)
    float* x_sum = reinterpret_cast<float*>(sOut + C::OUT_BYTES);     // [tile parity][half][row]
    uint64_t* bars = reinterpret_cast<uint64_t*>(x_sum + 2 * 2 * 128);
    uint64_t* q_full = bars + 0;             // TMA -> MMA (Q and dO tile)
    uint64_t* q_empty = bars + 1;            // MMA (commit) -> TMA
    uint64_t* s_full = bars + 2;             // [2]  MMA (commit) -> softmax: S_x and dP_x are complete
    uint64_t* p_full = bars + 4;             // [2]  softmax -> MMA: dS_x is in tensor memory
    uint64_t* dq_full = bars + 6;            //      MMA (commit) -> softmax (epilogue)
    uint64_t* dq_free = bars + 7;            //      softmax -> MMA
    uint64_t* st_full = bars + 8;            // [4]  TMA -> MMA, per strip buffer
    uint64_t* st_empty = bars + 12;          // [4]  MMA (commit) -> TMA
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);
    const WaitCtx wctx{reinterpret_cast<WaitState*>(bars + 17)};

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n_my = total_tiles > (int)blockIdx.x ? (total_tiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;

    if (tid == 0) {
        wait_state_init(wctx.st, err_word, kWaitLimitNs);
        mbar_init(q_full, 1);
        mbar_init(q_empty, 1);
        mbar_init(dq_full, 1);
        mbar_init(dq_free, 8);
        for (int i = 0; i < 2; ++i) {
            mbar_init(s_full + i, 1);
            mbar_init(p_full + i, 8);
        }
        for (int i = 0; i < 4; ++i) {
            mbar_init(st_full + i, 1);
            mbar_init(st_empty + i, 1);
        }
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
    // Rows [NK, NKP) of a strip buffer are contraction rows of dQ = dS K that TMA never writes:
    // zero them once in all four buffers (each holds a K strip sooner or later).
    if constexpr (C::NKP > C::NK) {
        constexpr int pad16 = (C::NKP - C::NK) * C::ROWB / 16;
        for (int i = tid; i < 4 * C::NS * pad16; i += 384) {
            const int which = i / pad16, off = i - which * pad16;           // which = buffer * NS + slab
            st_shared_v4(smem_u32(sStrip + (which / C::NS) * C::KV_BYTES + (which % C::NS) * C::KV_SLAB +
                                  C::NK * C::ROWB + off * 16), 0u, 0u, 0u, 0u);
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
    // Strip buffers of tile i: every tile the roles rotate (K_A, V_A, K_B, V_B) <- (V_A, V_B, K_A, K_B),
    // a cycle of length four.  Each buffer is filled and released exactly once per tile, so the
    // phase of its barriers is the tile's parity.
    struct Slots { int ka, va, kb, vb; };
    auto slots_of = [](int i) {
        // tile 0: ka 0, va 1, kb 2, vb 3; then ka' = va, va' = vb, kb' = ka, vb' = kb
        Slots s{0, 1, 2, 3};
        for (int t = 0; t < (i & 3); ++t) s = Slots{s.va, s.vb, s.ka, s.kb};
        return s;
    };

    if (warp == 8) {
        // ------------------------------------------------------------------ producer
        reg_dec<kRegsDonor>();
        if (lane == 0) {
            LoadTracker lt(bars);
            for (int i = 0; i < n_my && lt.ok; ++i) {
                int bn, r0, c0, hn, hb;
                decode(i, bn, r0, c0);
                split_unit(bn, g, hn, hb);
                const int box_r0 = na2d_ws(g.q_row0 + r0, g.Hg, KS) - g.kv_row0;
                const int box_c0 = na2d_ws(c0, g.W, KS);
                const Slots s = slots_of(i);
                const uint32_t par_free = (i & 1) ^ 1;
                if (!lt.acquire(q_empty, par_free, wctx)) break;
                lt.arm(q_full, i & 1, 2u * C::Q_BYTES);
#pragma unroll
                for (int sl = 0; sl < C::NS; ++sl) {
                    tma_load_5d(sQ + sl * C::Q_SLAB, &tm_q, q_full, sl * 64, c0, r0, hn, hb);
                    tma_load_5d(sDO + sl * C::Q_SLAB, &tm_do, q_full, sl * 64, c0, r0, hn, hb);
                }
                // K_A, V_A first: their buffers were released by the previous tile's score MMAs
                const int slot[4] = {s.ka, s.va, s.kb, s.vb};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    if (!lt.acquire(st_empty + slot[j], par_free, wctx)) break;
                    lt.arm(st_full + slot[j], i & 1, (uint32_t)C::NS * C::NK * C::ROWB);
                    uint8_t* dst = sStrip + slot[j] * C::KV_BYTES;
                    // (the tensor map is named in each call: a map chosen through a run-time pointer
                    // may be copied to local memory, where TMA cannot read it)
#pragma unroll
                    for (int sl = 0; sl < C::NS; ++sl) {
                        if (j & 1) tma_load_5d(dst + sl * C::KV_SLAB, &tm_v, st_full + slot[j], sl * 64, box_c0 + (j >> 1) * C::HW, box_r0, hn, hb);
                        else tma_load_5d(dst + sl * C::KV_SLAB, &tm_k, st_full + slot[j], sl * 64, box_c0 + (j >> 1) * C::HW, box_r0, hn, hb);
                    }
                }
            }
            lt.drain(wctx);
        }
    } else if (warp == 9) {
        // ------------------------------------------------------------------ MMA issue
        // Order on the tensor pipe: A1(0) B1(0) | A2(i) B2(i) A1(i+1) B1(i+1) | ...  where x1 are the
        // score MMAs of strip x and x2 its dQ MMAs.  The whole warp walks the loop; one elected lane
        // issues.
        reg_dec<kRegsDonor>();
        constexpr uint32_t idesc_s = umma_idesc(TM, C::NKP, IsBf16<DT>::value, IsBf16<DT>::value, false, false);
        constexpr uint32_t idesc_o = umma_idesc(TM, D, IsBf16<DT>::value, IsBf16<DT>::value, false, true);
        constexpr uint32_t hi = smem_desc_hi(C::ATOM, C::SWZ);
        const uint32_t q_lo = smem_desc_lo(smem_u32(sQ), 16), g_lo = smem_desc_lo(smem_u32(sDO), 16);
        const uint32_t strip_base = smem_u32(sStrip);

        // score MMAs of strip x (0 = A, 1 = B) of tile i
        auto scores = [&](int i, int x) {
            const Slots s = slots_of(i);
            const int sk = x ? s.kb : s.ka, sv = x ? s.vb : s.va;
            const uint32_t par = i & 1;
            if (x == 0 && lane == 0) NA2D_TR(0, 0, i);
            if (x == 0) mbar_wait(q_full, par, wctx, kErrLoadWait);
            if (x == 0 && lane == 0) NA2D_TR(0, 1, i);
            mbar_wait(st_full + sk, par, wctx, kErrLoadWait);
            if (x == 0 && lane == 0) NA2D_TR(0, 2, i);
            mbar_wait(st_full + sv, par, wctx, kErrLoadWait);
            if (x == 0 && lane == 0) NA2D_TR(0, 3, i);
            if (x == 1 && lane == 0) NA2D_TR(0, 4, i);
            if (x == 1) mbar_wait(dq_free, par ^ 1, wctx, kErrMmaWait);     // dQ of tile i - 1 sits over S_B
            if (x == 1 && lane == 0) NA2D_TR(0, 5, i);
            tc_fence_after();
            const uint32_t k_lo = smem_desc_lo(strip_base + sk * C::KV_BYTES, 16);
            const uint32_t v_lo = smem_desc_lo(strip_base + sv * C::KV_BYTES, 16);
            const uint32_t t_s = tmem_base + (x ? C::TMEM_SB : C::TMEM_SA), t_dp = tmem_base + (x ? C::TMEM_DPB : C::TMEM_DPA);
            if (elect_one()) {
                NA2D_TR(2, x ? 2 : 0, i);
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk) {
                    constexpr int kPerSlab = C::SLAB_C / 16;
                    const int slab = kk / kPerSlab, in_slab = kk % kPerSlab;
                    umma_ss(t_s, desc64(hi, q_lo + ((slab * C::Q_SLAB) >> 4) + 2 * in_slab),
                            desc64(hi, k_lo + ((slab * C::KV_SLAB) >> 4) + 2 * in_slab), idesc_s, kk > 0);
                    umma_ss(t_dp, desc64(hi, g_lo + ((slab * C::Q_SLAB) >> 4) + 2 * in_slab),
                            desc64(hi, v_lo + ((slab * C::KV_SLAB) >> 4) + 2 * in_slab), idesc_s, kk > 0);
                }
                umma_commit(s_full + x);
                umma_commit(st_empty + sv);                          // V_x is only read here
                if (x == 1) umma_commit(q_empty);                    // last reader of the Q and dO tiles
                NA2D_TR(2, x ? 3 : 1, i);
            }
            __syncwarp();
        };
        // dQ (+)= dS_x K_x of tile i
        auto outputs = [&](int i, int x) {
            const Slots s = slots_of(i);
            const int sk = x ? s.kb : s.ka;
            mbar_wait(p_full + x, i & 1, wctx, kErrMmaWait);
            tc_fence_after();
            const uint32_t km_lo = smem_desc_lo(strip_base + sk * C::KV_BYTES, C::KV_SLAB);
            const uint32_t t_ds = tmem_base + (x ? C::TMEM_DPB : C::TMEM_DPA);
            if (elect_one()) {
                NA2D_TR(2, x ? 6 : 4, i);
#pragma unroll
                for (int kk = 0; kk < C::NKP / 16; ++kk)
                    umma_ts(tmem_base + C::TMEM_DQ, t_ds + 8 * kk, desc64(hi, km_lo + ((kk * 16 * C::ROWB) >> 4)), idesc_o,
                            (x > 0) || (kk > 0));
                if (SPLIT) {
#pragma unroll
                    for (int kk = 0; kk < C::NKP / 16; ++kk)
                        umma_ts(tmem_base + C::TMEM_DQ, t_ds + 64 + 8 * kk, desc64(hi, km_lo + ((kk * 16 * C::ROWB) >> 4)),
                                idesc_o, 1u);
                }
                umma_commit(st_empty + sk);
                if (x == 1) umma_commit(dq_full);
                NA2D_TR(2, x ? 7 : 5, i);
            }
            __syncwarp();
        };
        if (n_my > 0) {
            scores(0, 0);
            scores(0, 1);
        }
        for (int i = 0; i < n_my; ++i) {
            outputs(i, 0);
            outputs(i, 1);                              // dQ complete: the softmax warps wait for it
            if (i + 1 < n_my) {
                scores(i + 1, 0);                       // under the epilogue of tile i
                scores(i + 1, 1);
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
        constexpr int NBH = (C::NB16 + 1) / 2;               // own blocks of a strip at most
        constexpr int kRows = (32 / TW - 1 + KS) < C::RC ? (32 / TW - 1 + KS) : C::RC;
        constexpr int kBlocks = (kRows * C::HW - 1) / 16 + 2;
        constexpr int NACT = (kBlocks + 1) / 2 < NBH ? (kBlocks + 1) / 2 : NBH;
        constexpr unsigned long long kRepLo = C::REP_LO, kRepHi = C::REP_HI;   // bit r * HW for the ks window rows

        // What the softmax warps need to know of a tile before its scores arrive: where it lies,
        // which of its 16-column blocks this warp takes, the validity masks of this thread's query
        // in both strips, and the query's lse.  It is worked out for tile i + 1 while the dQ MMAs of
        // tile i run (the warps would only wait there), so that none of it - about 1.8 k cycles of
        // divisions, 64-bit shifts and a global load - stands between two tiles.
        struct TileState {
            int bn, r0, c0;
            bool q_valid;
            size_t qi;
            float lse2;
            int b_hi, bi_lo;
            unsigned long long m_lo[2], m_hi[2];
        };
        auto prepare = [&](int i) {
            TileState t;
            decode(i, t.bn, t.r0, t.c0);
            const int box_r0 = na2d_ws(g.q_row0 + t.r0, g.Hg, KS) - g.kv_row0;
            const int box_c0 = na2d_ws(t.c0, g.W, KS);
            const int qr_raw = t.r0 + (row / TW), qc_raw = t.c0 + (row % TW);
            t.q_valid = qr_raw < g.Hq && qc_raw < g.W;
            const int qr = min(qr_raw, g.Hq - 1), qc = min(qc_raw, g.W - 1);
            t.qi = (static_cast<size_t>(t.bn) * g.Hq + qr) * g.W + qc;
            const int wr = na2d_ws(g.q_row0 + qr, g.Hg, KS) - g.kv_row0 - box_r0;   // in [0, TH)
            const int wc = na2d_ws(qc, g.W, KS) - box_c0;                            // in [0, TW)
            const int wr_lo = __shfl_sync(0xffffffffu, wr, 0);
            const int wr_hi = __shfl_sync(0xffffffffu, wr, 31);
            t.lse2 = lse[t.qi] * kLog2e;
            // the warp's queries see strip rows [wr_lo, wr_hi + ks): of the 16-column blocks in that
            // range this warp takes every other one, at most NACT per strip
            const int j_lo = wr_lo * C::HW;
            const int j_hi = min((wr_hi + KS) * C::HW, C::NK);
            t.b_hi = (j_hi + 15) >> 4;
            t.bi_lo = ((j_lo >> 4) - half + 1) >> 1;
#pragma unroll
            for (int x = 0; x < 2; ++x) {
                // this query's window columns inside strip x: [cl, chi) of [0, HW); the mask has that
                // segment in each of its ks window rows
                const int cl = max(wc - x * C::HW, 0), chi = min(wc + KS - x * C::HW, C::HW);
                unsigned long long m_lo = 0, m_hi = 0;
                if (chi > cl) {
                    const unsigned long long seg = (1ull << (chi - cl)) - 1ull;
                    m_lo = kRepLo * seg;
                    m_hi = kRepHi * seg + __umul64hi(kRepLo, seg);
                    shl128(m_lo, m_hi, cl);
                    // move the ks-row pattern down to window row wr: shift by wr * HW (< 128)
                    const int sh = wr * C::HW;
                    if (sh >= 64) {
                        m_hi = m_lo;
                        m_lo = 0;
                        shl128(m_lo, m_hi, sh - 64);
                    } else {
                        shl128(m_lo, m_hi, sh);
                    }
                }
                t.m_lo[x] = m_lo;
                t.m_hi[x] = m_hi;
            }
            return t;
        };

        TileState cur;
        uint32_t out_seq = 0;
        if (n_my > 0) cur = prepare(0);
        for (int i = 0; i < n_my; ++i) {
            const uint32_t par = i & 1;
            const int bn = cur.bn, r0 = cur.r0, c0 = cur.c0;
            const bool q_valid = cur.q_valid;
            const size_t qi = cur.qi;
            const float lse2 = cur.lse2;
            const int b_hi = cur.b_hi, bi_lo = cur.bi_lo;
            if (tid == 0) NA2D_TR(1, 1, i);

            uint32_t s[2][NACT][16], dp[2][NACT][16];
            uint32_t vmask[2][NACT];
            float d0 = 0.f, d1 = 0.f;
#pragma unroll
            for (int x = 0; x < 2; ++x) {
                const uint32_t t_s = tmem_lane + (x ? C::TMEM_SB : C::TMEM_SA), t_dp = tmem_lane + (x ? C::TMEM_DPB : C::TMEM_DPA);
                const unsigned long long m_lo = cur.m_lo[x], m_hi = cur.m_hi[x];
                if (tid == 0) NA2D_TR(3, x ? 2 : 0, i);
                mbar_wait(s_full + x, par, wctx, kErrMmaWait);
                tc_fence_after();
                if (tid == 0) NA2D_TR(3, x ? 3 : 1, i);
#pragma unroll
                for (int a = 0; a < NACT; ++a) {
                    const int blk = half + 2 * (bi_lo + a);
                    if (blk < b_hi) {                                        // warp-uniform
                        tmem_ld_32x16(t_s + 16 * blk, s[x][a]);
                        tmem_ld_32x16(t_dp + 16 * blk, dp[x][a]);
                    }
                }
#pragma unroll
                for (int a = 0; a < NACT; ++a) {
                    const int blk = half + 2 * (bi_lo + a);
                    const unsigned long long w = blk < 4 ? (m_lo >> (16 * (blk & 3))) : (m_hi >> (16 * (blk & 3)));
                    vmask[x][a] = (blk < b_hi) ? (static_cast<uint32_t>(w) & 0xffffu) : 0u;
                }
                tmem_ld_wait();
                // p = exp(s - lse) in place of s; this half's part of delta
#pragma unroll
                for (int a = 0; a < NACT; ++a) {
                    if (half + 2 * (bi_lo + a) < b_hi) {
#pragma unroll
                        for (int e = 0; e < 16; e += 2) {
                            const bool ok0 = (vmask[x][a] >> e) & 1u, ok1 = (vmask[x][a] >> (e + 1)) & 1u;
                            const float p0 = ok0 ? fast_exp2(fmaf(__uint_as_float(s[x][a][e]), g.sl2, -lse2)) : 0.f;
                            const float p1 = ok1 ? fast_exp2(fmaf(__uint_as_float(s[x][a][e + 1]), g.sl2, -lse2)) : 0.f;
                            s[x][a][e] = __float_as_uint(p0);
                            s[x][a][e + 1] = __float_as_uint(p1);
                            // masked columns may hold anything: keep them out by selection, never by
                            // multiplying with zero
                            if (!ok0) dp[x][a][e] = 0u;
                            if (!ok1) dp[x][a][e + 1] = 0u;
                            d0 = fmaf(p0, __uint_as_float(dp[x][a][e]), d0);
                            d1 = fmaf(p1, __uint_as_float(dp[x][a][e + 1]), d1);
                        }
                    }
                }
            }
            // both strips seen: add the partner's part; both halves now hold delta.  The barrier also
            // tells that the partner has read its blocks, so 16-bit operands may go over them.
            if (tid == 0) NA2D_TR(3, 4, i);
            x_sum[(par * 2 + half) * 128 + row] = d0 + d1;
            bar_sync(1 + quarter, 64);
            const float dl = (d0 + d1) + x_sum[(par * 2 + (half ^ 1)) * 128 + row];
            if (q_valid && half == 0) delta[qi] = dl;

            // dS = scale p (dP - delta) as packed 16-bit pairs (head, and residual on the bf16 path); the
            // softmax scale of dQ goes in here, inside a multiply-add that replaces the subtraction
            const float dls = dl * g.scale;
#pragma unroll
            for (int x = 0; x < 2; ++x) {
                const uint32_t t_ds = tmem_lane + (x ? C::TMEM_DPB : C::TMEM_DPA);
#pragma unroll
                for (int a = 0; a < NACT; ++a) {
                    const int blk = half + 2 * (bi_lo + a);
                    if (blk < b_hi) {
                        uint32_t wd[8], wr2[8];
#pragma unroll
                        for (int e2 = 0; e2 < 8; ++e2) {
                            // p and dP of masked columns are exact zeros here
                            const float ds0 = __uint_as_float(s[x][a][2 * e2]) * fmaf(__uint_as_float(dp[x][a][2 * e2]), g.scale, -dls);
                            const float ds1 = __uint_as_float(s[x][a][2 * e2 + 1]) * fmaf(__uint_as_float(dp[x][a][2 * e2 + 1]), g.scale, -dls);
                            wd[e2] = pack2<DT>(ds0, ds1);
                            wr2[e2] = SPLIT ? pack2_residual_bf16(ds0, ds1, wd[e2]) : 0u;
                        }
                        tmem_st_32x8(t_ds + 8 * blk, wd);
                        if (SPLIT) tmem_st_32x8(t_ds + 64 + 8 * blk, wr2);
                    }
                }
                {   // own blocks outside the range hold zeros
                    const uint32_t z[8] = {0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u};
                    for (int bi = 0; bi < NBH; ++bi) {
                        const int blk = half + 2 * bi;
                        const bool in_range = bi >= bi_lo && bi < bi_lo + NACT && blk < b_hi;
                        if (!in_range && 16 * blk < C::NKP) {
                            tmem_st_32x8(t_ds + 8 * blk, z);
                            if (SPLIT) tmem_st_32x8(t_ds + 64 + 8 * blk, z);
                        }
                    }
                }
                tmem_st_wait();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(p_full + x);
                if (tid == 0) NA2D_TR(3, x ? 6 : 5, i);
            }

            // the next tile's state, under the dQ MMAs
            TileState nxt = cur;
            if (i + 1 < n_my) nxt = prepare(i + 1);

            // ---- epilogue: this half's columns of the dQ rows of the warp's 32 queries
            mbar_wait(dq_full, par, wctx, kErrMmaWait);
            tc_fence_after();
            uint32_t acc[DH];
#pragma unroll
            for (int piece = 0; piece < DH / 16; ++piece)
                tmem_ld_32x16(tmem_lane + C::TMEM_DQ + half * DH + 16 * piece, *reinterpret_cast<uint32_t(*)[16]>(&acc[16 * piece]));
            tmem_ld_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(dq_free);
            if (tid == 0) NA2D_TR(3, 7, i);
            int hn, hb;
            split_unit(bn, g, hn, hb);
            stage_and_store<DT, DH, C::NOUT, false>(&tm_dq, sOut + warp * C::NOUT * OutStage<DH>::BYTES, acc, 1.f, half * DH, c0,
                                                    r0 + quarter * (32 / TW), hn, hb, lane, &out_seq);
            if (tid == 0) NA2D_TR(1, 0, i);
            cur = nxt;
        }
        if (lane == 0) bulk_wait<0>();          // the staging buffer has been read, the rows written
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}

template <typename DT, int D, int KS>
int launch_dq1(const LaunchCtx& lc, const TensorArg& q, const TensorArg& k, const TensorArg& v, const float* lse,
               const TensorArg& d_o, const TensorArg& d_q, float* delta) {
    using C = Dq1Cfg<D, KS, IsBf16<DT>::value>;
    const Na2dGeom& g = lc.g;
    CUtensorMap tq, tg, tk, tv, tdq;
    int rc = make_map(&tq, q, lc.dtype, lc.B, g.N, g.Hq, g.W, D, TW, TH);
    if (rc == NA2D_OK) rc = make_map(&tdq, d_q, lc.dtype, lc.B, g.N, g.Hq, g.W, D, TW, 32 / TW, OutStage<D / 2>::RW);
    if (rc == NA2D_OK) rc = make_map(&tg, d_o, lc.dtype, lc.B, g.N, g.Hq, g.W, D, TW, TH);
    if (rc == NA2D_OK) rc = make_map(&tk, k, lc.dtype, lc.B, g.N, g.Hkv, g.W, D, C::HW, C::RC);
    if (rc == NA2D_OK) rc = make_map(&tv, v, lc.dtype, lc.B, g.N, g.Hkv, g.W, D, C::HW, C::RC);
    if (rc != NA2D_OK) return rc;
    const int tiles_r = (g.Hq + TH - 1) / TH, tiles_c = (g.W + TW - 1) / TW;
    const long long tiles = (long long)g.BN * tiles_r * tiles_c;
    if (tiles > 0x7fffffffLL) return NA2D_ERR_TOO_LARGE;
    auto kern = dq1_kernel<DT, D, KS>;
    static std::atomic<unsigned long long> opted{0};
    if (opt_in_smem(kern, C::SMEM, lc.device, opted) != cudaSuccess) return NA2D_ERR_CUDA;
    const int grid = persistent_grid(lc, tiles);
    kern<<<grid, 384, C::SMEM, lc.st>>>(tq, tg, tk, tv, tdq, lse, delta, lc.err_word, g, tiles_r, tiles_c, (int)tiles);
    *lc.launched += 1;
    return cudaGetLastError() == cudaSuccess ? NA2D_OK : NA2D_ERR_CUDA;
}

}  // namespace na2d_tc
