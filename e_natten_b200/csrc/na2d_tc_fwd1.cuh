// Persistent, warp-specialised tcgen05 forward kernel for kernel sizes whose key box splits into
// two column strips of at most 128 keys (3 and 5).  Included by na2d_tc.cuh.
//
// One CTA per SM walks query tiles (TH x TW queries = tensor-memory lanes).  The key box of a tile
// is cut into a left strip A and a right strip B:
//     S_x = Q K_x^T                                   (x = A, B; tensor memory, fp32)
//     m = max over both strips, P_x = exp(S_x - m)    (softmax warps; P_x packed over S_x)
//     O = P_A V_A + P_B V_B                           (tensor memory), o = O / sum, lse = m + ln sum
// Tensor memory holds three strip buffers and O.  A tile uses two of the strip buffers, the next
// tile's S_A goes into the third one and its S_B into the buffer P_A V_A has just left, so the
// score MMAs of tile i+1 run while the softmax warps work on tile i, and P V of tile i runs while
// they read tile i+1.  Four epilogue warps normalise and store the output of tile i meanwhile
// (the next tile's P V waits for O to be read, nothing else does).
// Sixteen warps: 0-7 softmax (warps w and w+4 share 32 queries and split the 16-column blocks),
// 8 TMA producer (Q, K strips), 10 TMA producer (V strips), 9 MMA issue, 11 idle (register donor),
// 12-15 epilogue (one per tensor-memory lane quarter).
#pragma once

namespace na2d_tc {

template <int D, int KS>
struct Fwd1Cfg : Cfg<D, KS, 128, 0, 2> {
    using B = Cfg<D, KS, 128, 0, 2>;
    static_assert(B::NCH == 1, "a strip must hold all box rows");
    static constexpr int TMEM_STRIP = 128;                               // three strip buffers at 0, 128, 256
    static constexpr int TMEM_O = 384;
    static constexpr int OUT_BYTES = 4 * OutStage<32>::BYTES;            // output staging of the 4 epilogue warps
    static constexpr int XCHG_BYTES = (4 * 2 + 2) * 128 * 4;             // row max [2][2][128], row sum [2][2][128], final max [2][128]
    static constexpr int SMEM = B::Q_BYTES + 4 * B::KV_BYTES + OUT_BYTES + XCHG_BYTES + 256 + 1024;
    static constexpr int NB16 = B::NKP / 16;
    static constexpr unsigned long long REP_LO = row_repeat_lo(B::HW, KS), REP_HI = row_repeat_hi(B::HW, KS);
    static_assert(SMEM <= kSmemLimit, "forward strip kernel shared memory");
    static_assert(B::NKP <= 128 && D <= 128, "tensor memory layout");
};

template <typename DT, int D, int KS>
__global__ void __launch_bounds__(512, 1)
fwd1_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
            const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_o,
            float* __restrict__ lse, unsigned int* __restrict__ err_word, const Na2dGeom g, const int tiles_r,
            const int tiles_c, const int total_tiles) {
    using C = Fwd1Cfg<D, KS>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sQ = smem;                                   // Q tile
    uint8_t* sKV = sQ + C::Q_BYTES;                       // K_A, K_B, V_A, V_B strips [NKP x D]
    uint8_t* sOut = sKV + 4 * C::KV_BYTES;                // 8 x output staging (1024-byte aligned)
    float* x_max = reinterpret_cast<float*>(sOut + C::OUT_BYTES);     // [tile parity][half][row]
    float* x_sum = x_max + 2 * 2 * 128;                               // [tile parity][half][row]
    float* x_fin = x_sum + 2 * 2 * 128;                               // [tile parity][row]  final max * log2(e)
    uint64_t* bars = reinterpret_cast<uint64_t*>(x_fin + 2 * 128);
    uint64_t* q_full = bars + 0;             //      TMA -> MMA
    uint64_t* q_empty = bars + 1;            //      MMA (commit) -> TMA
    uint64_t* o_full = bars + 2;             //      MMA (commit) -> softmax
    uint64_t* o_free = bars + 3;             //      softmax -> MMA
    uint64_t* s_full = bars + 4;             // [2]  MMA (commit) -> softmax: S_x is complete
    uint64_t* p_full = bars + 6;             // [2]  softmax -> MMA: P_x is in tensor memory
    uint64_t* kv_full = bars + 8;            // [4]  TMA -> MMA: K_A, K_B, V_A, V_B
    uint64_t* kv_empty = bars + 12;          // [4]  MMA (commit) -> TMA
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);
    const WaitCtx wctx{reinterpret_cast<WaitState*>(bars + 17)};

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n_my = total_tiles > (int)blockIdx.x ? (total_tiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;

    if (tid == 0) {
        wait_state_init(wctx.st, err_word, kWaitLimitNs);
        mbar_init(q_full, 1);
        mbar_init(q_empty, 1);
        mbar_init(o_full, 1);
        mbar_init(o_free, 4);
        for (int i = 0; i < 2; ++i) {
            mbar_init(s_full + i, 1);
            mbar_init(p_full + i, 8);
        }
        for (int i = 0; i < 4; ++i) {
            mbar_init(kv_full + i, 1);
            mbar_init(kv_empty + i, 1);
        }
        mbar_fence_init();
        tma_prefetch_desc(&tm_q);
        tma_prefetch_desc(&tm_k);
        tma_prefetch_desc(&tm_v);
        tma_prefetch_desc(&tm_o);
    }
    if (warp == 0) {
        __syncwarp();
        tmem_alloc(tmem_slot, 512);
        tmem_relinquish();
    }
    // Rows [NK, NKP) of the V strips are contraction rows of O = P V that TMA never writes: zero them once.
    if constexpr (C::NKP > C::NK) {
        constexpr int pad16 = (C::NKP - C::NK) * C::ROWB / 16;
        for (int i = tid; i < 2 * C::NS * pad16; i += 512) {
            const int which = i / pad16, off = i - which * pad16;           // which = strip * NS + slab
            st_shared_v4(smem_u32(sKV + (2 + which / C::NS) * C::KV_BYTES + (which % C::NS) * C::KV_SLAB +
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
    // strip buffer of strip x of tile i: tile i uses (2i) % 3 and (2i + 1) % 3
    auto strip_col = [](int i, int x) { return ((2 * i + x) % 3) * C::TMEM_STRIP; };

    if (warp == 8 || warp == 10) {
        // ------------------------------------------------------------------ producers
        // Warp 8 fetches the Q tile and the K strips, whose buffers the score MMAs release early in
        // a tile; warp 10 the V strips, whose buffers are only released by P V.  One producer for
        // both would hold the next tile's Q and K back behind the wait for a V buffer.
        reg_dec<kDkvRegsCtl>();
        if (lane == 0) {
            const int j0 = warp == 8 ? 0 : 2;
            LoadTracker lt(bars);
            for (int i = 0; i < n_my; ++i) {
                int bn, r0, c0, hn, hb;
                decode(i, bn, r0, c0);
                split_unit(bn, g, hn, hb);
                const int box_r0 = na2d_ws(g.q_row0 + r0, g.Hg, KS) - g.kv_row0;
                const int box_c0 = na2d_ws(c0, g.W, KS);
                const uint32_t par_free = (i & 1) ^ 1;
                if (warp == 8) {
                    if (!lt.acquire(q_empty, par_free, wctx)) break;
                    lt.arm(q_full, i & 1, (uint32_t)C::Q_BYTES);
#pragma unroll
                    for (int sl = 0; sl < C::NS; ++sl) tma_load_5d(sQ + sl * C::Q_SLAB, &tm_q, q_full, sl * 64, c0, r0, hn, hb);
                }
                // (the tensor map is named in each call: a map chosen through a run-time pointer
                // may be copied to local memory, where TMA cannot read it)
#pragma unroll
                for (int x = 0; x < 2; ++x) {
                    const int j = j0 + x;                               // K_A, K_B or V_A, V_B
                    if (!lt.acquire(kv_empty + j, par_free, wctx)) break;
                    lt.arm(kv_full + j, i & 1, (uint32_t)C::NS * C::NK * C::ROWB);
                    uint8_t* dst = sKV + j * C::KV_BYTES;
#pragma unroll
                    for (int sl = 0; sl < C::NS; ++sl) {
                        if (warp == 8) tma_load_5d(dst + sl * C::KV_SLAB, &tm_k, kv_full + j, sl * 64, box_c0 + x * C::HW, box_r0, hn, hb);
                        else tma_load_5d(dst + sl * C::KV_SLAB, &tm_v, kv_full + j, sl * 64, box_c0 + x * C::HW, box_r0, hn, hb);
                    }
                }
                if (!lt.ok) break;
            }
            lt.drain(wctx);
        }
    } else if (warp == 9) {
        // ------------------------------------------------------------------ MMA issue
        // Order on the tensor pipe: S_A(0) S_B(0) | S_A(i+1) PV_A(i) S_B(i+1) PV_B(i) | ...
        // The whole warp walks the loop; one elected lane issues.
        reg_dec<kDkvRegsCtl>();
        constexpr uint32_t idesc_s = umma_idesc(TM, C::NKP, IsBf16<DT>::value, IsBf16<DT>::value, false, false);
        constexpr uint32_t idesc_o = umma_idesc(TM, D, IsBf16<DT>::value, IsBf16<DT>::value, false, true);
        constexpr uint32_t hi = smem_desc_hi(C::ATOM, C::SWZ);
        const uint32_t q_lo = smem_desc_lo(smem_u32(sQ), 16);
        const uint32_t kv_base = smem_u32(sKV);

        auto scores = [&](int i, int x) {
            const uint32_t par = i & 1;
            if (x == 0) mbar_wait(q_full, par, wctx, kErrLoadWait);
            mbar_wait(kv_full + x, par, wctx, kErrLoadWait);
            tc_fence_after();
            const uint32_t k_lo = smem_desc_lo(kv_base + x * C::KV_BYTES, 16);
            const uint32_t t_s = tmem_base + strip_col(i, x);
            if (elect_one()) {
                NA2D_TR(2, x ? 2 : 0, i);
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk) {
                    constexpr int kPerSlab = C::SLAB_C / 16;
                    const int slab = kk / kPerSlab, in_slab = kk % kPerSlab;
                    umma_ss(t_s, desc64(hi, q_lo + ((slab * C::Q_SLAB) >> 4) + 2 * in_slab),
                            desc64(hi, k_lo + ((slab * C::KV_SLAB) >> 4) + 2 * in_slab), idesc_s, kk > 0);
                }
                umma_commit(s_full + x);
                umma_commit(kv_empty + x);
                if (x == 1) umma_commit(q_empty);                    // last reader of the Q tile
                NA2D_TR(2, x ? 3 : 1, i);
            }
            __syncwarp();
        };
        auto outputs = [&](int i, int x) {
            const uint32_t par = i & 1;
            mbar_wait(p_full + x, par, wctx, kErrMmaWait);
            mbar_wait(kv_full + 2 + x, par, wctx, kErrLoadWait);
            if (x == 0) mbar_wait(o_free, par ^ 1, wctx, kErrMmaWait);      // O of tile i - 1 has been read
            tc_fence_after();
            const uint32_t v_lo = smem_desc_lo(kv_base + (2 + x) * C::KV_BYTES, C::KV_SLAB);
            const uint32_t t_p = tmem_base + strip_col(i, x);
            if (elect_one()) {
                NA2D_TR(2, x ? 6 : 4, i);
#pragma unroll
                for (int kk = 0; kk < C::NKP / 16; ++kk)
                    umma_ts(tmem_base + C::TMEM_O, t_p + 8 * kk, desc64(hi, v_lo + ((kk * 16 * C::ROWB) >> 4)), idesc_o,
                            (x > 0) || (kk > 0));
                umma_commit(kv_empty + 2 + x);
                if (x == 1) umma_commit(o_full);
                NA2D_TR(2, x ? 7 : 5, i);
            }
            __syncwarp();
        };
        if (n_my > 0) {
            scores(0, 0);
            scores(0, 1);
        }
        for (int i = 0; i < n_my; ++i) {
            if (i + 1 < n_my) scores(i + 1, 0);          // into the third strip buffer
            outputs(i, 0);
            if (i + 1 < n_my) scores(i + 1, 1);          // into the buffer P_A V_A has left
            outputs(i, 1);
        }
    } else if (warp == 11) {
        reg_dec<kDkvRegsCtl>();
    } else if (warp >= 12) {
        // ------------------------------------------------------------------ epilogue warps
        reg_dec<kDkvRegsEpi>();
        const int quarter = warp & 3;
        const int row = quarter * 32 + lane;                 // query of the tile = tensor-memory lane
        const uint32_t tmem_lane = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
        uint8_t* stage = sOut + quarter * OutStage<32>::BYTES;
        constexpr int RPO = D / 32;                          // 32-channel rounds
        for (int i = 0; i < n_my; ++i) {
            int bn, r0, c0, hn, hb;
            decode(i, bn, r0, c0);
            split_unit(bn, g, hn, hb);
            const uint32_t par = i & 1;
            const int qr = r0 + (row / TW), qc = c0 + (row % TW);
            mbar_wait(o_full, par, wctx, kErrMmaWait);            // also: the softmax warps' sums are written
            tc_fence_after();
            const float total = x_sum[(par * 2 + 0) * 128 + row] + x_sum[(par * 2 + 1) * 128 + row];
            const float fin = x_fin[par * 128 + row];
            const float inv = 1.f / total;
            uint32_t v[2][32];
            tmem_ld_32x32(tmem_lane + C::TMEM_O, v[0]);
#pragma unroll
            for (int j = 0; j < RPO; ++j) {
                tmem_ld_wait();
                if (j + 1 < RPO) {
                    tmem_ld_32x32(tmem_lane + C::TMEM_O + 32 * (j + 1), v[(j + 1) & 1]);
                } else {                                     // O is in registers
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(o_free);
                }
                stage_and_store<DT, 32>(&tm_o, stage, v[j & 1], inv, 32 * j, c0, r0 + quarter * (32 / TW), hn, hb, lane);
            }
            if (qr < g.Hq && qc < g.W)
                lse[(static_cast<size_t>(bn) * g.Hq + qr) * g.W + qc] = (fin + log2f(total)) * kLn2;
        }
        if (lane == 0) bulk_wait<0>();                       // the staging buffer has been read, the rows written
    } else {
        // ------------------------------------------------------------------ softmax warps
        reg_inc<kDkvRegsSoftmax>();
        const int quarter = warp & 3, half = warp >> 2;
        const int row = quarter * 32 + lane;                 // query of the tile = tensor-memory lane
        const uint32_t tmem_lane = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
        constexpr int NBH = (C::NB16 + 1) / 2;               // own blocks of a strip at most
        constexpr int kRows = (32 / TW - 1 + KS) < C::RC ? (32 / TW - 1 + KS) : C::RC;
        constexpr int kBlocks = (kRows * C::HW - 1) / 16 + 2;
        constexpr int NACT = (kBlocks + 1) / 2 < NBH ? (kBlocks + 1) / 2 : NBH;
        constexpr unsigned long long kRepLo = C::REP_LO, kRepHi = C::REP_HI;   // bit r * HW for the ks window rows

        for (int i = 0; i < n_my; ++i) {
            int bn, r0, c0;
            decode(i, bn, r0, c0);
            const uint32_t par = i & 1;
            const int box_r0 = na2d_ws(g.q_row0 + r0, g.Hg, KS) - g.kv_row0;
            const int box_c0 = na2d_ws(c0, g.W, KS);
            const int qr_raw = r0 + (row / TW), qc_raw = c0 + (row % TW);
            const int qr = min(qr_raw, g.Hq - 1), qc = min(qc_raw, g.W - 1);
            const int wr = na2d_ws(g.q_row0 + qr, g.Hg, KS) - g.kv_row0 - box_r0;   // in [0, TH)
            const int wc = na2d_ws(qc, g.W, KS) - box_c0;                            // in [0, TW)
            const int wr_lo = __shfl_sync(0xffffffffu, wr, 0);
            const int wr_hi = __shfl_sync(0xffffffffu, wr, 31);
            // the warp's queries see strip rows [wr_lo, wr_hi + ks): of the 16-column blocks in that
            // range this warp takes every other one, at most NACT per strip
            const int j_lo = wr_lo * C::HW;
            const int j_hi = min((wr_hi + KS) * C::HW, C::NK);
            const int b_hi = (j_hi + 15) >> 4;
            const int bi_lo = ((j_lo >> 4) - half + 1) >> 1;

            uint32_t s[2][NACT][16];
            uint32_t vmask[2][NACT];
#pragma unroll
            for (int x = 0; x < 2; ++x) {
                const uint32_t t_s = tmem_lane + strip_col(i, x);
                // this query's window columns inside strip x: [cl, chi) of [0, HW); the mask has that
                // segment in each of its ks window rows
                const int cl = max(wc - x * C::HW, 0), chi = min(wc + KS - x * C::HW, C::HW);
                unsigned long long m_lo = 0, m_hi = 0;
                if (chi > cl) {
                    const unsigned long long seg = (1ull << (chi - cl)) - 1ull;
                    m_lo = kRepLo * seg;
                    m_hi = kRepHi * seg + __umul64hi(kRepLo, seg);
                    shl128(m_lo, m_hi, cl);
                    const int sh = wr * C::HW;                              // down to window row wr (< 128)
                    if (sh >= 64) {
                        m_hi = m_lo;
                        m_lo = 0;
                        shl128(m_lo, m_hi, sh - 64);
                    } else {
                        shl128(m_lo, m_hi, sh);
                    }
                }
                if (tid == 0) NA2D_TR(3, x ? 2 : 0, i);
                mbar_wait(s_full + x, par, wctx, kErrMmaWait);
                tc_fence_after();
                if (tid == 0) NA2D_TR(3, x ? 3 : 1, i);
#pragma unroll
                for (int a = 0; a < NACT; ++a) {
                    const int blk = half + 2 * (bi_lo + a);
                    if (blk < b_hi) tmem_ld_32x16(t_s + 16 * blk, s[x][a]);          // warp-uniform
                }
#pragma unroll
                for (int a = 0; a < NACT; ++a) {
                    const int blk = half + 2 * (bi_lo + a);
                    const unsigned long long w = blk < 4 ? (m_lo >> (16 * (blk & 3))) : (m_hi >> (16 * (blk & 3)));
                    vmask[x][a] = (blk < b_hi) ? (static_cast<uint32_t>(w) & 0xffffu) : 0u;
                }
            }
            tmem_ld_wait();

            // masked maximum over this half's blocks of both strips, then over both halves
            float m0 = -CUDART_INF_F, m1 = -CUDART_INF_F;
#pragma unroll
            for (int x = 0; x < 2; ++x) {
#pragma unroll
                for (int a = 0; a < NACT; ++a) {
                    if (half + 2 * (bi_lo + a) < b_hi) {
#pragma unroll
                        for (int e = 0; e < 16; e += 2) {
                            m0 = fmaxf(m0, ((vmask[x][a] >> e) & 1u) ? __uint_as_float(s[x][a][e]) : -CUDART_INF_F);
                            m1 = fmaxf(m1, ((vmask[x][a] >> (e + 1)) & 1u) ? __uint_as_float(s[x][a][e + 1]) : -CUDART_INF_F);
                        }
                    }
                }
            }
            float cmax = fmaxf(m0, m1);
            if (tid == 0) NA2D_TR(3, 4, i);
            x_max[(par * 2 + half) * 128 + row] = cmax;
            // This barrier also orders the partner's reads of S before this thread's writes of P,
            // which land in the same tensor-memory columns.
            bar_sync(1 + quarter, 64);
            cmax = fmaxf(cmax, x_max[(par * 2 + (half ^ 1)) * 128 + row]) * g.sl2;
            const float safe_max = (cmax == -CUDART_INF_F) ? 0.f : cmax;

            // P = exp2(s * log2e - max) as packed 16-bit pairs -> tensor memory (over S), row sum
            float c0s = 0.f, c1s = 0.f;
#pragma unroll
            for (int x = 0; x < 2; ++x) {
                const uint32_t t_s = tmem_lane + strip_col(i, x);
#pragma unroll
                for (int a = 0; a < NACT; ++a) {
                    const int blk = half + 2 * (bi_lo + a);
                    if (blk < b_hi) {
                        uint32_t w[8];
#pragma unroll
                        for (int e2 = 0; e2 < 8; ++e2) {
                            const float e0 = fast_exp2(fmaf(__uint_as_float(s[x][a][2 * e2]), g.sl2, -safe_max));
                            const float e1 = fast_exp2(fmaf(__uint_as_float(s[x][a][2 * e2 + 1]), g.sl2, -safe_max));
                            const float p0 = ((vmask[x][a] >> (2 * e2)) & 1u) ? e0 : 0.f;
                            const float p1 = ((vmask[x][a] >> (2 * e2 + 1)) & 1u) ? e1 : 0.f;
                            c0s += p0;
                            c1s += p1;
                            w[e2] = pack2<DT>(p0, p1);
                        }
                        tmem_st_32x8(t_s + 8 * blk, w);
                    }
                }
                {   // own blocks outside the range hold zeros
                    const uint32_t z[8] = {0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u};
                    for (int bi = 0; bi < NBH; ++bi) {
                        const int blk = half + 2 * bi;
                        const bool in_range = bi >= bi_lo && bi < bi_lo + NACT && blk < b_hi;
                        if (!in_range && 16 * blk < C::NKP) tmem_st_32x8(t_s + 8 * blk, z);
                    }
                }
                if (x == 1) {
                    // what the epilogue warps need, written before the arrival that lets the last
                    // P V go: this half's row sum, and the row maximum
                    x_sum[(par * 2 + half) * 128 + row] = c0s + c1s;
                    if (half == 0) x_fin[par * 128 + row] = safe_max;
                }
                tmem_st_wait();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(p_full + x);
                if (tid == 0) NA2D_TR(3, x ? 6 : 5, i);
            }
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
int launch_forward1(const LaunchCtx& lc, const TensorArg& q, const TensorArg& k, const TensorArg& v, const TensorArg& o,
                    float* lse) {
    using C = Fwd1Cfg<D, KS>;
    const Na2dGeom& g = lc.g;
    CUtensorMap tq, tk, tv, to;
    int rc = make_map(&tq, q, lc.dtype, lc.B, g.N, g.Hq, g.W, D, TW, TH);
    if (rc == NA2D_OK) rc = make_map(&to, o, lc.dtype, lc.B, g.N, g.Hq, g.W, D, TW, 32 / TW, 32);
    if (rc == NA2D_OK) rc = make_map(&tk, k, lc.dtype, lc.B, g.N, g.Hkv, g.W, D, C::HW, C::RC);
    if (rc == NA2D_OK) rc = make_map(&tv, v, lc.dtype, lc.B, g.N, g.Hkv, g.W, D, C::HW, C::RC);
    if (rc != NA2D_OK) return rc;
    const int tiles_r = (g.Hq + TH - 1) / TH, tiles_c = (g.W + TW - 1) / TW;
    const long long tiles = (long long)g.BN * tiles_r * tiles_c;
    if (tiles > 0x7fffffffLL) return NA2D_ERR_TOO_LARGE;
    auto kern = fwd1_kernel<DT, D, KS>;
    static std::atomic<unsigned long long> opted{0};
    if (opt_in_smem(kern, C::SMEM, lc.device, opted) != cudaSuccess) return NA2D_ERR_CUDA;
    const int grid = persistent_grid(lc, tiles);
    kern<<<grid, 512, C::SMEM, lc.st>>>(tq, tk, tv, to, lse, lc.err_word, g, tiles_r, tiles_c, (int)tiles);
    *lc.launched += 1;
    return cudaGetLastError() == cudaSuccess ? NA2D_OK : NA2D_ERR_CUDA;
}

}  // namespace na2d_tc
