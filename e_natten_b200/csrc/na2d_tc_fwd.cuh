// Persistent, warp-specialised tcgen05 forward kernel for the larger windows (kernel sizes >= 7).
// Included by na2d_tc_fwd.cu.
//
// One CTA per SM walks tiles blockIdx.x, blockIdx.x + gridDim.x, ...  A tile is TH x TW queries;
// its halo box of keys is taken in chunks of whole box rows with at most 192 keys.  Twelve warps
// in three groups of four:
//   warps 0-7  softmax.  Warps w and w+4 own the same 32 queries (tensor-memory lanes
//              32*(w%4)..) and split the 16-column blocks of S between them (even / odd); they
//              read their blocks of S from tensor memory once, exchange the row maximum through
//              shared memory, and write P back into tensor memory over S as packed 16-bit
//              pairs, where it is the A operand of the second MMA.  The output accumulates in
//              tensor memory across the chunks of a tile and is rescaled there only when a row's
//              maximum grows by more than 2^8 (until then the older maximum keeps being used,
//              which leaves the result unchanged).  The tile's epilogue (normalise, store o and
//              lse) is deferred into the next tile, whose MMAs and loads it overlaps.
//   warp 8     producer: TMA loads of Q tiles (two buffers), K chunks and V chunks (separate
//              rings: a K slot is free again as soon as S = Q K^T has been computed);
//   warp 9     MMA issue: S = Q K^T, then O += P V with P read from tensor memory;
//   warps 10-11 idle (they fill the third group, which hands its registers to warps 0-7).
// Tensor memory holds two S / P buffers, so the tensor pipe computes the scores of chunk n+1 (and
// n+2, once P V of chunk n has left its buffer) while the softmax warps work on chunk n: on the
// pipe the order is S(0) S(1) | PV(0) S(2) | PV(1) S(3) | ...  The rest holds the output
// accumulator, twice where the head dim leaves room (the epilogue of tile t then never holds up
// the first P V of tile t+1).
// Shared-memory traffic is what the design economises: every UMMA with both operands in shared
// memory re-reads a 128-row A operand, so S is computed with the widest N that fits and P never
// touches shared memory.  Every hand-over is an mbarrier with a bounded wait.
#pragma once

#include <type_traits>

namespace na2d_tc {


template <int D, int KS>
struct FwdCfg : Cfg<D, KS, 192> {
    using B = Cfg<D, KS, 192>;
    // The K chunk keeps only the rows TMA writes (rounded to the swizzle period): the UMMA reads
    // NKP rows, and the few it reads past the end only feed S columns that are masked anyway.
    // The V chunk keeps all NKP rows, the padding ones zeroed, because they are contraction rows.
    static constexpr int K_ROWS = B::ROWB == 128 ? (B::NK + 7) / 8 * 8 : B::NKP;
    static constexpr int K_SLAB = K_ROWS * B::ROWB;
    static constexpr int K_BYTES = B::NS * K_SLAB;
    static constexpr int V_BYTES = B::KV_BYTES;
    static constexpr int XCHG_BYTES = 4 * 2 * 128 * 4;                  // row max [2][2][128], row sum [2][2][128]
    static constexpr int OUT_BYTES = 8 * 2 * OutStage<D / 2>::BYTES;     // two output staging buffers for each of the 8 softmax warps
    static constexpr int FIXED = XCHG_BYTES + OUT_BYTES + 256 /*barriers*/ + 1024 /*alignment*/;
    // Ring depths, given out in the order that pays most: a second V slot first (a V slot is only
    // free after the chunk's last MMA, so its refill is what the next tile would wait for), then a
    // second K slot, then a second Q tile.
    static constexpr bool fits(int nq, int nk, int nv) {
        return FIXED + nq * B::Q_BYTES + nk * K_BYTES + nv * V_BYTES <= kSmemLimit;
    }
    static constexpr int NSTV = fits(1, 1, 2) ? 2 : 1;
    static constexpr int NSTK = fits(1, 2, NSTV) ? 2 : 1;
    static constexpr int NQ = fits(2, NSTK, NSTV) ? 2 : 1;
    static constexpr int SMEM = FIXED + NQ * B::Q_BYTES + NSTK * K_BYTES + NSTV * V_BYTES;
    static constexpr int NB16 = (B::NKP + 15) / 16;                     // 16-column blocks of S
    static constexpr int TMEM_S = 0, TMEM_SSTRIDE = 192;                // two S / P buffers at 0 and 192
    static constexpr int TMEM_O0 = 384, TMEM_OSTRIDE = D;               // O at 384 (and 384 + D where it fits)
    static constexpr int NOB = (TMEM_O0 + 2 * D <= 512) ? 2 : 1;
    static_assert(SMEM <= kSmemLimit, "forward kernel shared memory");
    static_assert(B::NKP <= 192 && TMEM_O0 + NOB * D <= 512, "tensor memory layout");
};

template <typename DT, int D, int KS>
__global__ void __launch_bounds__(384, 1)
fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
           const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_o,
           float* __restrict__ lse, unsigned int* __restrict__ err_word,
           const Na2dGeom g, const int tiles_r, const int tiles_c, const int total_tiles) {
    using C = FwdCfg<D, KS>;
    constexpr int NSTK = C::NSTK, NSTV = C::NSTV, NQ = C::NQ;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sQ = smem;                                   // NQ x Q tile
    uint8_t* sK = sQ + NQ * C::Q_BYTES;                   // NSTK x K chunk
    uint8_t* sV = sK + NSTK * C::K_BYTES;                 // NSTV x V chunk
    uint8_t* sOut = sV + NSTV * C::V_BYTES;               // 8 x output staging (1024-byte aligned)
    float* x_max = reinterpret_cast<float*>(sOut + C::OUT_BYTES);     // [unit parity][half][row]
    float* x_sum = x_max + 2 * 2 * 128;                               // [tile parity][half][row]
    uint64_t* bars = reinterpret_cast<uint64_t*>(x_sum + 2 * 2 * 128);
    uint64_t* q_full = bars;                 // [2]   TMA -> MMA
    uint64_t* q_empty = bars + 2;            // [2]   MMA (commit) -> TMA
    uint64_t* o_full = bars + 4;             // [2]   MMA (commit) -> softmax
    uint64_t* o_free = bars + 6;             // [2]   softmax -> MMA
    uint64_t* k_full = bars + 8;             // [2]   TMA -> MMA
    uint64_t* k_empty = bars + 10;           // [2]   MMA (commit) -> TMA
    uint64_t* v_full = bars + 12;            // [2]   TMA -> MMA
    uint64_t* v_empty = bars + 14;           // [2]   MMA (commit) -> TMA
    uint64_t* s_full = bars + 16;            // [2]   MMA (commit) -> softmax, per S buffer
    uint64_t* p_full = bars + 18;            // [2]   softmax -> MMA, per S buffer
    uint64_t* pv_done = bars + 20;           //       MMA (commit) -> softmax: O holds this chunk
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 21);
    const WaitCtx wctx{reinterpret_cast<WaitState*>(bars + 22)};

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n_my = total_tiles > (int)blockIdx.x ? (total_tiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;
    const uint32_t total_units = (uint32_t)n_my * C::NCH;

    if (tid == 0) {
        wait_state_init(wctx.st, err_word, kWaitLimitNs);
        for (int i = 0; i < 2; ++i) {
            mbar_init(q_full + i, 1);
            mbar_init(q_empty + i, 1);
            mbar_init(o_full + i, 1);
            mbar_init(o_free + i, 8);
            mbar_init(k_full + i, 1);
            mbar_init(k_empty + i, 1);
            mbar_init(v_full + i, 1);
            mbar_init(v_empty + i, 1);
            mbar_init(s_full + i, 1);
            mbar_init(p_full + i, 8);
        }
        mbar_init(pv_done, 1);
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
    // V rows [NK, NKP) of every stage are contraction rows of P V that TMA never writes.
    if constexpr (C::NKP > C::NK) {
        constexpr int pad16 = (C::NKP - C::NK) * C::ROWB / 16;
        for (int i = tid; i < NSTV * C::NS * pad16; i += 384) {
            const int which = i / pad16, off = i - which * pad16;
            const int st = which / C::NS, slab = which % C::NS;
            uint8_t* base = sV + st * C::V_BYTES + slab * C::KV_SLAB;
            st_shared_v4(smem_u32(base + C::NK * C::ROWB + off * 16), 0u, 0u, 0u, 0u);
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
                const int qb = i % NQ;
                if (!lt.acquire(q_empty + qb, ((i / NQ) & 1) ^ 1, wctx)) break;
                lt.arm(q_full + qb, (i / NQ) & 1, C::Q_BYTES);
#pragma unroll
                for (int s = 0; s < C::NS; ++s)
                    tma_load_5d(sQ + qb * C::Q_BYTES + s * C::Q_SLAB, &tm_q, q_full + qb, s * 64, c0, r0, hn, hb);
                for (int c = 0; c < C::NCH; ++c, ++n) {
                    const uint32_t sk = n % NSTK, sv = n % NSTV;
                    NA2D_TR(1, 0, n);
                    if (!lt.acquire(k_empty + sk, ((n / NSTK) & 1) ^ 1, wctx)) break;
                    NA2D_TR(1, 1, n);
                    lt.arm(k_full + sk, (n / NSTK) & 1, (uint32_t)C::NS * C::NK * C::ROWB);
#pragma unroll
                    for (int s = 0; s < C::NS; ++s)
                        tma_load_5d(sK + sk * C::K_BYTES + s * C::K_SLAB, &tm_k, k_full + sk, s * 64, box_c0,
                                    box_r0 + c * C::RC, hn, hb);
                    if (!lt.acquire(v_empty + sv, ((n / NSTV) & 1) ^ 1, wctx)) break;
                    NA2D_TR(1, 2, n);
                    lt.arm(v_full + sv, (n / NSTV) & 1, (uint32_t)C::NS * C::NK * C::ROWB);
#pragma unroll
                    for (int s = 0; s < C::NS; ++s)
                        tma_load_5d(sV + sv * C::V_BYTES + s * C::KV_SLAB, &tm_v, v_full + sv, s * 64, box_c0,
                                    box_r0 + c * C::RC, hn, hb);
                }
            }
            lt.drain(wctx);
        }
    } else if (warp == 9) {
        // ------------------------------------------------------------------ MMA issue
        // (the whole warp walks the loop so that addresses stay warp-uniform; one lane issues)
        reg_dec<kRegsDonor>();
        constexpr uint32_t idesc_s = umma_idesc(TM, C::NKP, IsBf16<DT>::value, IsBf16<DT>::value, false, false);
        constexpr uint32_t idesc_o = umma_idesc(TM, D, IsBf16<DT>::value, IsBf16<DT>::value, false, true);
        constexpr uint32_t hi = smem_desc_hi(C::ATOM, C::SWZ);
        // O buffer and phase of tile i
        auto o_buf = [](uint32_t i) { return C::NOB == 2 ? (i & 1u) : 0u; };
        auto o_par = [](uint32_t i) { return C::NOB == 2 ? ((i >> 1) & 1u) : (i & 1u); };
        // S(n) = Q K_c^T into S buffer n & 1
        auto scores = [&](uint32_t n) {
            const uint32_t i = n / C::NCH, c = n % C::NCH, sk = n % NSTK, qb = i % NQ;
            if (lane == 0) NA2D_TR(2, 0, n);
            if (c == 0) mbar_wait(q_full + qb, (i / NQ) & 1, wctx, kErrLoadWait);
            mbar_wait(k_full + sk, (n / NSTK) & 1, wctx, kErrLoadWait);
            if (lane == 0) NA2D_TR(2, 1, n);
            tc_fence_after();
            const uint32_t q_lo = smem_desc_lo(smem_u32(sQ + qb * C::Q_BYTES), 16);
            const uint32_t k_lo = smem_desc_lo(smem_u32(sK + sk * C::K_BYTES), 16);
            const uint32_t t_s = tmem_base + C::TMEM_S + (n & 1) * C::TMEM_SSTRIDE;
            if (elect_one()) {
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk) {
                    constexpr int kPerSlab = C::SLAB_C / 16;
                    const int slab = kk / kPerSlab, in_slab = kk % kPerSlab;
                    umma_ss(t_s, desc64(hi, q_lo + ((slab * C::Q_SLAB) >> 4) + 2 * in_slab),
                            desc64(hi, k_lo + ((slab * C::K_SLAB) >> 4) + 2 * in_slab), idesc_s, kk > 0);
                }
                umma_commit(s_full + (n & 1));
                umma_commit(k_empty + sk);
                if (c == C::NCH - 1) umma_commit(q_empty + qb);           // the tile's Q buffer is free
            }
            __syncwarp();
            if (lane == 0) NA2D_TR(2, 2, n);
        };
        // O (+)= P(n) V_c, P read from S buffer n & 1
        auto outputs = [&](uint32_t n) {
            const uint32_t i = n / C::NCH, c = n % C::NCH, sv = n % NSTV, ob = o_buf(i);
            mbar_wait(v_full + sv, (n / NSTV) & 1, wctx, kErrLoadWait);
            mbar_wait(p_full + (n & 1), (n >> 1) & 1, wctx, kErrMmaWait);
            if (lane == 0) NA2D_TR(2, 3, n);
            if (c == 0) mbar_wait(o_free + ob, o_par(i) ^ 1, wctx, kErrMmaWait);   // the tile before has been read out
            tc_fence_after();
            const uint32_t v_lo = smem_desc_lo(smem_u32(sV + sv * C::V_BYTES), C::KV_SLAB);
            const uint32_t t_p = tmem_base + C::TMEM_S + (n & 1) * C::TMEM_SSTRIDE;
            if (elect_one()) {
#pragma unroll
                for (int kk = 0; kk < C::NKP / 16; ++kk) {
                    umma_ts(tmem_base + C::TMEM_O0 + ob * C::TMEM_OSTRIDE, t_p + 8 * kk,
                            desc64(hi, v_lo + ((kk * 16 * C::ROWB) >> 4)), idesc_o, (c > 0) || (kk > 0));
                }
                umma_commit(v_empty + sv);
                umma_commit(pv_done);
                if (c == C::NCH - 1) umma_commit(o_full + ob);
            }
            __syncwarp();
            if (lane == 0) NA2D_TR(2, 4, n);
        };
        // On the pipe: S(0) S(1) | PV(0) S(2) | PV(1) S(3) | ...  S(n + 2) goes into the buffer PV(n)
        // has just read; the pipe runs its MMAs in the order they were issued.
        if (total_units > 0) scores(0);
        if (total_units > 1) scores(1);
        for (uint32_t n = 0; n < total_units; ++n) {
            outputs(n);
            if (n + 2 < total_units) scores(n + 2);
        }
    } else if (warp >= 10) {
        reg_dec<kRegsDonor>();                 // spare warps of the data-movement group
    } else {
        // ------------------------------------------------------------------ softmax warps
        reg_inc<kRegsSoftmax>();
        const int quarter = warp & 3, half = warp >> 2;
        const int row = quarter * 32 + lane;                 // query of the tile = tensor-memory lane
        const uint32_t tmem_lane = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
        constexpr float kRescaleStep = 8.f;      // log2 units: rescale O when the maximum grows by > 2^8
        constexpr int DH = D / 2;                // output columns of this half
        // epilogue of the previous tile, deferred until the next tile's first chunk is under way
        bool pend = false, pend_valid = false;
        uint32_t pend_tile = 0, out_seq = 0;
        float pend_max = 0.f, pend_sum = 1.f;
        size_t pend_qi = 0;
        int pend_bn = 0, pend_r0 = 0, pend_c0 = 0;

        auto epilogue = [&]() {
            const uint32_t ob = C::NOB == 2 ? (pend_tile & 1u) : 0u;
            bar_sync(1 + quarter, 64);                                       // partner's row sum is in x_sum
            const float total = pend_sum + x_sum[((pend_tile & 1) * 2 + (half ^ 1)) * 128 + row];
            mbar_wait(o_full + ob, C::NOB == 2 ? ((pend_tile >> 1) & 1u) : (pend_tile & 1u), wctx, kErrMmaWait);
            tc_fence_after();
            const float inv = 1.f / total;
            uint32_t acc[DH];
#pragma unroll
            for (int piece = 0; piece < DH / 16; ++piece)
                tmem_ld_32x16(tmem_lane + C::TMEM_O0 + ob * C::TMEM_OSTRIDE + half * DH + 16 * piece,
                              *reinterpret_cast<uint32_t(*)[16]>(&acc[16 * piece]));
            tmem_ld_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(o_free + ob);                         // O is in registers
            int hn, hb;
            split_unit(pend_bn, g, hn, hb);
            stage_and_store<DT, DH, 2>(&tm_o, sOut + warp * 2 * OutStage<DH>::BYTES, acc, inv, half * DH, pend_c0,
                                       pend_r0 + quarter * (32 / TW), hn, hb, lane, &out_seq);
            if (pend_valid && half == 0) lse[pend_qi] = (pend_max + log2f(total)) * kLn2;
            pend = false;
        };

        uint32_t n = 0;
        for (int i = 0; i < n_my; ++i) {
            int bn, r0, c0;
            decode(i, bn, r0, c0);
            const int box_r0 = na2d_ws(g.q_row0 + r0, g.Hg, KS) - g.kv_row0;
            const int box_c0 = na2d_ws(c0, g.W, KS);
            const int qr_raw = r0 + (row / TW), qc_raw = c0 + (row % TW);
            const bool q_valid = qr_raw < g.Hq && qc_raw < g.W;
            const int qr = min(qr_raw, g.Hq - 1), qc = min(qc_raw, g.W - 1);
            const int wr = na2d_ws(g.q_row0 + qr, g.Hg, KS) - g.kv_row0 - box_r0;   // in [0, TH)
            const int wc = na2d_ws(qc, g.W, KS) - box_c0;                            // in [0, TW)
            const int wr_lo = __shfl_sync(0xffffffffu, wr, 0);
            const int wr_hi = __shfl_sync(0xffffffffu, wr, 31);
            const uint32_t o_addr = tmem_lane + C::TMEM_O0 + (C::NOB == 2 ? (i & 1) : 0) * C::TMEM_OSTRIDE + half * DH;
            float run_max = -CUDART_INF_F, run_sum = 0.f;        // run_sum: this half's columns only

            // One chunk.  The warp's queries can only see a contiguous range of the chunk's columns
            // (box rows wr_lo .. wr_hi + ks); of the 16-column blocks in that range this warp takes
            // every other one, at most NACT of them, reads each once into registers and keeps a
            // 16-bit validity mask per block (built from the query's ks window rows) beside it.
            auto unit = [&](const int ch) {
                constexpr int NBH = (C::NB16 + 1) / 2;                      // own blocks at most
                constexpr int kRows = (32 / TW - 1 + KS) < C::RC ? (32 / TW - 1 + KS) : C::RC;
                constexpr int kBlocks = (kRows * C::HW - 1) / 16 + 2;
                constexpr int NACT = (kBlocks + 1) / 2 < NBH ? (kBlocks + 1) / 2 : NBH;
                const uint32_t s_addr = tmem_lane + C::TMEM_S + (n & 1) * C::TMEM_SSTRIDE;
                const int row_off = ch * C::RC;
                const int j_lo = max(wr_lo - row_off, 0) * C::HW;
                const int j_hi = min(min(wr_hi + KS - row_off, C::RC) * C::HW, C::NK);       // exclusive
                const int b_hi = (max(j_hi, 0) + 15) >> 4;                                   // blocks [j_lo/16, b_hi)
                const int bi_lo = ((j_lo >> 4) - half + 1) >> 1;                             // first own block in range
                if (tid == 0) NA2D_TR(3, 0, n);
                mbar_wait(s_full + (n & 1), (n >> 1) & 1, wctx, kErrMmaWait);
                if (tid == 0) NA2D_TR(3, 1, n);
                tc_fence_after();

                uint32_t s[NACT][16];
                uint32_t vmask[NACT];
#pragma unroll
                for (int t = 0; t < NACT; ++t) {
                    const int blk = half + 2 * (bi_lo + t);
                    if (blk < b_hi) tmem_ld_32x16(s_addr + 16 * blk, s[t]);                  // warp-uniform
                }
                // validity masks, while the loads are in flight
#pragma unroll
                for (int t = 0; t < NACT; ++t) {
                    const int blk = half + 2 * (bi_lo + t);
                    vmask[t] = (blk < b_hi) ? block_mask16<C::HW, KS, C::RC>(blk, wr - row_off, wc) : 0u;
                }
                tmem_ld_wait();
                if (tid == 0) NA2D_TR(3, 2, n);

                // masked maximum over this half's blocks, then over both halves
                float m0 = -CUDART_INF_F, m1 = -CUDART_INF_F;
#pragma unroll
                for (int t = 0; t < NACT; ++t) {
                    if (half + 2 * (bi_lo + t) < b_hi) {
#pragma unroll
                        for (int e = 0; e < 16; e += 2) {
                            m0 = fmaxf(m0, ((vmask[t] >> e) & 1u) ? __uint_as_float(s[t][e]) : -CUDART_INF_F);
                            m1 = fmaxf(m1, ((vmask[t] >> (e + 1)) & 1u) ? __uint_as_float(s[t][e + 1]) : -CUDART_INF_F);
                        }
                    }
                }
                float cmax = fmaxf(m0, m1);
                if (tid == 0) NA2D_TR(3, 6, n);
                x_max[((n & 1) * 2 + half) * 128 + row] = cmax;
                // This barrier also orders the partner's reads of S before this thread's writes of P,
                // which land in the same tensor-memory columns.
                bar_sync(1 + quarter, 64);
                cmax = fmaxf(cmax, x_max[((n & 1) * 2 + (half ^ 1)) * 128 + row]) * g.sl2;

                // Raise the running maximum only when it would grow by more than the step; a row
                // whose maximum is still -inf has an all-zero O row and takes the new one freely.
                const bool grow = cmax > run_max + kRescaleStep;
                if (C::NCH > 1 && ch > 0) {
                    mbar_wait(pv_done, (n & 1) ^ 1, wctx, kErrMmaWait);     // O holds the previous chunk
                    if (__any_sync(0xffffffffu, grow && run_max != -CUDART_INF_F)) {
                        const float alpha = grow ? fast_exp2(run_max - cmax) : 1.f;
                        tc_fence_after();
#pragma unroll
                        for (int piece = 0; piece < DH / 16; ++piece) {
                            uint32_t v[16];
                            tmem_ld_32x16(o_addr + 16 * piece, v);
                            tmem_ld_wait();
#pragma unroll
                            for (int e = 0; e < 16; ++e) v[e] = __float_as_uint(__uint_as_float(v[e]) * alpha);
                            tmem_st_32x16(o_addr + 16 * piece, v);
                        }
                        run_sum *= alpha;
                        if (grow) run_max = cmax;
                    }
                }
                if (grow && cmax > run_max + kRescaleStep) {      // not taken above: run_max was -inf (or first chunk)
                    run_sum = 0.f;
                    run_max = cmax;
                }
                const float safe_max = (run_max == -CUDART_INF_F) ? 0.f : run_max;
                if (tid == 0) NA2D_TR(3, 3, n);

                // P = exp2(s * log2e - max) as packed 16-bit pairs -> tensor memory (over S), row sum
                float c0s = 0.f, c1s = 0.f;
#pragma unroll
                for (int t = 0; t < NACT; ++t) {
                    const int blk = half + 2 * (bi_lo + t);
                    if (blk < b_hi) {
                        uint32_t w[8];
#pragma unroll
                        for (int e2 = 0; e2 < 8; ++e2) {
                            const float e0 = fast_exp2(fmaf(__uint_as_float(s[t][2 * e2]), g.sl2, -safe_max));
                            const float e1 = fast_exp2(fmaf(__uint_as_float(s[t][2 * e2 + 1]), g.sl2, -safe_max));
                            const float p0 = ((vmask[t] >> (2 * e2)) & 1u) ? e0 : 0.f;
                            const float p1 = ((vmask[t] >> (2 * e2 + 1)) & 1u) ? e1 : 0.f;
                            c0s += p0;
                            c1s += p1;
                            w[e2] = pack2<DT>(p0, p1);
                        }
                        tmem_st_32x8(s_addr + 8 * blk, w);
                    }
                }
                // own blocks outside the range hold zeros
                {
                    const uint32_t z[8] = {0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u};
                    for (int bi = 0; bi < NBH; ++bi) {
                        const int blk = half + 2 * bi;
                        const bool in_range = bi >= bi_lo && bi < bi_lo + NACT && blk < b_hi;
                        if (!in_range && 16 * blk < C::NKP) tmem_st_32x8(s_addr + 8 * blk, z);
                    }
                }
                run_sum += c0s + c1s;
                if (tid == 0) NA2D_TR(3, 7, n);
                tmem_st_wait();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(p_full + (n & 1));
                if (tid == 0) NA2D_TR(3, 4, n);
            };

            for (int ch = 0; ch < C::NCH; ++ch, ++n) {
                unit(ch);
                if (pend) epilogue();           // previous tile's output, while this chunk's P V runs
                if (tid == 0) NA2D_TR(3, 5, n);
            }
            x_sum[((i & 1) * 2 + half) * 128 + row] = run_sum;
            pend = true;
            pend_tile = (uint32_t)i;
            pend_bn = bn;
            pend_r0 = r0;
            pend_c0 = c0;
            pend_valid = q_valid;
            pend_max = run_max;
            pend_sum = run_sum;
            pend_qi = (static_cast<size_t>(bn) * g.Hq + qr) * g.W + qc;
        }
        if (pend) epilogue();
        if (lane == 0) bulk_wait<0>();      // the staging buffer has been read, the rows written
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}

template <typename DT, int D, int KS>
int launch_forward(const LaunchCtx& lc, const TensorArg& q, const TensorArg& k, const TensorArg& v, const TensorArg& o,
                   float* lse) {
    // kernel sizes 3 and 5 go to the strip kernel
    if constexpr (KS <= 5) {
        return launch_forward1<DT, D, KS>(lc, q, k, v, o, lse);
    } else {
    using C = FwdCfg<D, KS>;
    const Na2dGeom& g = lc.g;
    CUtensorMap tq, tk, tv, to;
    int rc = make_map(&tq, q, lc.dtype, lc.B, g.N, g.Hq, g.W, D, TW, TH);
    if (rc == NA2D_OK) rc = make_map(&to, o, lc.dtype, lc.B, g.N, g.Hq, g.W, D, TW, 32 / TW, OutStage<D / 2>::RW);
    if (rc == NA2D_OK) rc = make_map(&tk, k, lc.dtype, lc.B, g.N, g.Hkv, g.W, D, C::HW, C::RC);
    if (rc == NA2D_OK) rc = make_map(&tv, v, lc.dtype, lc.B, g.N, g.Hkv, g.W, D, C::HW, C::RC);
    if (rc != NA2D_OK) return rc;
    const int tiles_r = (g.Hq + TH - 1) / TH, tiles_c = (g.W + TW - 1) / TW;
    const long long tiles = (long long)g.BN * tiles_r * tiles_c;
    if (tiles > 0x7fffffffLL) return NA2D_ERR_TOO_LARGE;
    auto kern = fwd_kernel<DT, D, KS>;
    static std::atomic<unsigned long long> opted{0};
    if (opt_in_smem(kern, C::SMEM, lc.device, opted) != cudaSuccess) return NA2D_ERR_CUDA;
    const int grid = persistent_grid(lc, tiles);
    kern<<<grid, 384, C::SMEM, lc.st>>>(tq, tk, tv, to, lse, lc.err_word, g, tiles_r, tiles_c, (int)tiles);
    *lc.launched += 1;
    return cudaGetLastError() == cudaSuccess ? NA2D_OK : NA2D_ERR_CUDA;
    }
}

}  // namespace na2d_tc
