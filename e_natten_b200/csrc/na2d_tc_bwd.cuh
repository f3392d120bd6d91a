// tcgen05 backward kernels: dQ (+ row delta) and dK/dV.  Included by na2d_tc.cuh.
//
// Both recompute P from the saved row log-sum-exp: p = exp(s - lse).  The row delta is formed as
// delta = sum_j p_j * dp_j (dp_j = dO . v_j), which equals dO . o exactly and does not depend on
// how o was rounded when it was stored; the dQ kernel writes it to scratch for the dK/dV kernel.
//
// dQ kernel (one CTA per TH x TW query tile, rows = queries):
//   phase A, per key chunk:  S = Q K^T, dP = dO V^T  ->  delta += sum_j p dp      (registers)
//   phase B, per key chunk:  dS = p (dP - delta)  ->  shared  ->  dQ += dS K      (tensor memory)
//   With a single chunk (ks <= 5) S and dP stay in tensor memory between the phases and dQ reuses
//   the S columns; with several chunks phase B reloads the chunk and repeats the two MMAs.
//
// dK/dV kernel (one CTA per TH x TW key tile, rows = keys): the queries that can see the tile are
//   the union of the keys' inverse neighbourhoods, a box of query pixels walked in chunks:
//   S^T = K Q^T, dP^T = V dO^T  ->  P^T, dS^T -> shared  ->  dV += P^T dO, dK += dS^T Q.
#pragma once

namespace na2d_tc {

// ------------------------------------------------------------------------------------ dQ
template <int D, int KS, bool SPLIT>
struct DqCfg : Cfg<D, KS, ((TH + KS - 1) * (TW + KS - 1) <= 256 ? 256 : 192)> {
    using B = Cfg<D, KS, ((TH + KS - 1) * (TW + KS - 1) <= 256 ? 256 : 192)>;
    static constexpr int TMEM_DP = B::NCH == 1 ? 256 : 192;
    static constexpr int TMEM_DQ = B::NCH == 1 ? 0 : 384;      // single chunk: dQ reuses the S columns
    // V chunk and dS share one buffer: V is dead once dP is complete, before dS is written.
    static constexpr int VS_BYTES = B::KV_BYTES > B::P_BYTES ? B::KV_BYTES : B::P_BYTES;
    static constexpr int BASE = 2 * B::Q_BYTES + B::KV_BYTES + VS_BYTES;
    // The residual half of dS (bf16 path) gets its own buffer where that fits; otherwise it
    // reuses the Q / dO tiles, which are dead after the score MMAs of a single-chunk tile.
    static constexpr bool RES_ALIAS = SPLIT && (BASE + B::P_BYTES + 64 + 1024 > kSmemLimit);
    static constexpr int RES_BYTES = (SPLIT && !RES_ALIAS) ? B::P_BYTES : 0;
    static constexpr int SMEM = BASE + RES_BYTES + 64 + 1024;
    static_assert(!RES_ALIAS || (B::NCH == 1 && 2 * B::Q_BYTES >= B::P_BYTES), "residual buffer does not fit");
    static_assert(SMEM <= kSmemLimit, "dQ kernel shared memory");
};

template <typename DT, int D, int KS>
__global__ void __launch_bounds__(128, 1)
dq_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_do,
          const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
          const float* __restrict__ lse, DT* __restrict__ d_q, float* __restrict__ delta,
          const Na2dGeom g, const int tiles_r, const int tiles_c) {
    constexpr bool SPLIT = IsBf16<DT>::value;         // bf16: dS goes to the MMA as head + residual
    using C = DqCfg<D, KS, SPLIT>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sQ = smem;
    uint8_t* sDO = sQ + C::Q_BYTES;
    uint8_t* sK = sDO + C::Q_BYTES;
    uint8_t* sVS = sK + C::KV_BYTES;                  // V chunk, then dS
    uint8_t* sRES = C::RES_ALIAS ? sQ : sVS + C::VS_BYTES;      // residual half of dS
    uint64_t* bars = reinterpret_cast<uint64_t*>(sVS + C::VS_BYTES + C::RES_BYTES);
    uint64_t* bar_load = bars + 0;
    uint64_t* bar_s = bars + 1;
    uint64_t* bar_o = bars + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 3);
    volatile uint32_t* abort_flag = tmem_slot + 1;

    const int tid = threadIdx.x, warp = tid >> 5;
    int t = blockIdx.x;
    const int tc = t % tiles_c;
    t /= tiles_c;
    const int tr = t % tiles_r;
    const int bn = t / tiles_r;
    const int r0 = tr * TH, c0 = tc * TW;
    const int box_r0 = na2d_ws(g.q_row0 + r0, g.Hg, KS) - g.kv_row0;
    const int box_c0 = na2d_ws(c0, g.W, KS);

    if (tid == 0) {
        *abort_flag = 0;
        mbar_init(bar_load, 1);
        mbar_init(bar_s, 1);
        mbar_init(bar_o, 1);
        mbar_fence_init();
        tma_prefetch_desc(&tm_q);
        tma_prefetch_desc(&tm_do);
        tma_prefetch_desc(&tm_k);
        tma_prefetch_desc(&tm_v);
    }
    if (warp == 0) {
        __syncwarp();
        tmem_alloc(tmem_slot, C::TMEM_COLS);
        tmem_relinquish();
    }
    // K rows [NK, NKP) are contraction rows of dQ = dS K and are never written by TMA: zero them.
    // (The same rows of the V buffer only feed masked columns of dP and need no care.)
    if constexpr (C::NKP > C::NK) {
        constexpr int pad16 = (C::NKP - C::NK) * C::ROWB / 16;
        for (int i = tid; i < C::NS * pad16; i += 128) {
            const int which = i / pad16, off = i - which * pad16;
            st_shared_v4(smem_u32(sK + which * C::KV_SLAB + C::NK * C::ROWB + off * 16), 0u, 0u, 0u, 0u);
        }
        fence_proxy_async();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_lane = tmem_base + (static_cast<uint32_t>(warp * 32) << 16);

    const int qr_raw = r0 + (tid / TW), qc_raw = c0 + (tid % TW);
    const bool q_valid = qr_raw < g.Hq && qc_raw < g.W;
    const int qr = min(qr_raw, g.Hq - 1), qc = min(qc_raw, g.W - 1);
    const size_t qi = (static_cast<size_t>(bn) * g.Hq + qr) * g.W + qc;
    const int wr = na2d_ws(g.q_row0 + qr, g.Hg, KS) - g.kv_row0 - box_r0;
    const int wc = na2d_ws(qc, g.W, KS) - box_c0;
    const uint32_t row_mask = ((1u << KS) - 1u) << wr;
    const uint32_t col_mask = ((1u << KS) - 1u) << wc;
    const int wr_lo = __shfl_sync(0xffffffffu, wr, 0);
    const int wr_hi = __shfl_sync(0xffffffffu, wr, 31);
    const float lse2 = lse[qi] * kLog2e;

    constexpr uint32_t idesc_s = umma_idesc(TM, C::NKP, IsBf16<DT>::value, IsBf16<DT>::value, false, false);
    constexpr uint32_t idesc_o = umma_idesc(TM, D, IsBf16<DT>::value, IsBf16<DT>::value, false, true);
    uint32_t ph_load = 0, ph_s = 0, ph_o = 0;

    // Loads chunk `ch` of K and V (plus Q and dO when `with_q`) and issues S = Q K^T, dP = dO V^T.
    auto load_and_score = [&](int ch, bool with_q) {
        const uint32_t kv_bytes = 2u * C::NS * C::NK * C::ROWB;
        mbar_expect_tx(bar_load, kv_bytes + (with_q ? 2u * C::Q_BYTES : 0u));
#pragma unroll
        for (int s = 0; s < C::NS; ++s) {
            if (with_q) {
                tma_load_4d(sQ + s * C::Q_SLAB, &tm_q, bar_load, s * 64, c0, r0, bn);
                tma_load_4d(sDO + s * C::Q_SLAB, &tm_do, bar_load, s * 64, c0, r0, bn);
            }
            tma_load_4d(sK + s * C::KV_SLAB, &tm_k, bar_load, s * 64, box_c0, box_r0 + ch * C::RC, bn);
            tma_load_4d(sVS + s * C::KV_SLAB, &tm_v, bar_load, s * 64, box_c0, box_r0 + ch * C::RC, bn);
        }
        mbar_wait(bar_load, ph_load, abort_flag, kErrLoadWait);
        ph_load ^= 1u;
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
            const int slab = (kk * 16) / C::SLAB_C, in_slab = (kk * 16) % C::SLAB_C;
            const uint64_t aq = smem_desc(smem_u32(sQ + slab * C::Q_SLAB) + in_slab * 2, 16, C::ATOM, C::SWZ);
            const uint64_t bk = smem_desc(smem_u32(sK + slab * C::KV_SLAB) + in_slab * 2, 16, C::ATOM, C::SWZ);
            umma_ss(tmem_base + C::TMEM_S, aq, bk, idesc_s, kk > 0);
        }
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
            const int slab = (kk * 16) / C::SLAB_C, in_slab = (kk * 16) % C::SLAB_C;
            const uint64_t ag = smem_desc(smem_u32(sDO + slab * C::Q_SLAB) + in_slab * 2, 16, C::ATOM, C::SWZ);
            const uint64_t bv = smem_desc(smem_u32(sVS + slab * C::KV_SLAB) + in_slab * 2, 16, C::ATOM, C::SWZ);
            umma_ss(tmem_base + C::TMEM_DP, ag, bv, idesc_s, kk > 0);
        }
        umma_commit(bar_s);
    };

    // ---- phase A: delta = sum_j p_j dp_j -------------------------------------------------------------
    float dl = 0.f;
#pragma unroll
    for (int ch = 0; ch < C::NCH; ++ch) {
        if (tid == 0) load_and_score(ch, ch == 0);
        __syncwarp();
        mbar_wait(bar_s, ph_s, abort_flag, kErrMmaWait);
        ph_s ^= 1u;
        tc_fence_after();
#pragma unroll
        for (int b = 0; b < C::NB; ++b) {
            const int row_first = ch * C::RC + (32 * b) / C::HW;
            const int last_col = (32 * b + 31 < C::NK - 1) ? 32 * b + 31 : C::NK - 1;
            const int row_last = ch * C::RC + last_col / C::HW;
            if (32 * b < C::NK && row_last >= wr_lo && row_first < wr_hi + KS) {
                uint32_t s[32], dp[32];
                tmem_ld_32x32(tmem_lane + C::TMEM_S + 32 * b, s);
                tmem_ld_32x32(tmem_lane + C::TMEM_DP + 32 * b, dp);
                tmem_ld_wait();
#pragma unroll
                for (int e = 0; e < 32; ++e) {
                    const int j = 32 * b + e;
                    if (j < C::NK) {
                        const int hr = ch * C::RC + j / C::HW, hc = j % C::HW;
                        const bool ok = ((row_mask >> hr) & 1u) && ((col_mask >> hc) & 1u);
                        const float p = fast_exp2(fmaf(__uint_as_float(s[e]), kLog2e, -lse2));
                        dl += ok ? p * __uint_as_float(dp[e]) : 0.f;
                    }
                }
            }
        }
        if (C::NCH > 1) {
            tc_fence_before();
            __syncthreads();          // the chunk buffers and the S / dP columns are free again
        }
    }
    if (q_valid) delta[qi] = dl;

    // ---- phase B: dS -> shared, dQ += dS K -------------------------------------------------------------
    if (d_q != nullptr) {
#pragma unroll
        for (int ch = 0; ch < C::NCH; ++ch) {
            if (C::NCH > 1) {
                if (tid == 0) load_and_score(ch, false);
                __syncwarp();
                mbar_wait(bar_s, ph_s, abort_flag, kErrMmaWait);
                ph_s ^= 1u;
                tc_fence_after();
            }
#pragma unroll
            for (int b = 0; b < C::NB; ++b) {
                const int row_first = ch * C::RC + (32 * b) / C::HW;
                const int last_col = (32 * b + 31 < C::NK - 1) ? 32 * b + 31 : C::NK - 1;
                const int row_last = ch * C::RC + last_col / C::HW;
                uint32_t w[16], w2[16];
                if (32 * b < C::NK && row_last >= wr_lo && row_first < wr_hi + KS) {
                    uint32_t s[32], dp[32];
                    tmem_ld_32x32(tmem_lane + C::TMEM_S + 32 * b, s);
                    tmem_ld_32x32(tmem_lane + C::TMEM_DP + 32 * b, dp);
                    tmem_ld_wait();
                    float ds[32];
#pragma unroll
                    for (int e = 0; e < 32; ++e) {
                        const int j = 32 * b + e;
                        ds[e] = 0.f;
                        if (j < C::NK) {
                            const int hr = ch * C::RC + j / C::HW, hc = j % C::HW;
                            const bool ok = ((row_mask >> hr) & 1u) && ((col_mask >> hc) & 1u);
                            const float p = fast_exp2(fmaf(__uint_as_float(s[e]), kLog2e, -lse2));
                            ds[e] = ok ? p * (__uint_as_float(dp[e]) - dl) : 0.f;
                        }
                    }
#pragma unroll
                    for (int e = 0; e < 16; ++e) {
                        w[e] = pack2<DT>(ds[2 * e], ds[2 * e + 1]);
                        w2[e] = SPLIT ? pack2_residual_bf16(ds[2 * e], ds[2 * e + 1], w[e]) : 0u;
                    }
                } else {
#pragma unroll
                    for (int e = 0; e < 16; ++e) { w[e] = 0u; w2[e] = 0u; }
                }
                store_operand_block(smem_u32(sVS), C::P_SLAB, tid, b, w);
                if (SPLIT) store_operand_block(smem_u32(sRES), C::P_SLAB, tid, b, w2);
            }
            fence_proxy_async();
            tc_fence_before();
            __syncthreads();
            if (tid == 0) {
                tc_fence_after();
#pragma unroll
                for (int kk = 0; kk < C::NKP / 16; ++kk) {
                    const uint64_t a = smem_desc(smem_u32(sVS + (kk >> 2) * C::P_SLAB) + (kk & 3) * 32, 16, 1024, 2u);
                    const uint64_t bk = smem_desc(smem_u32(sK) + kk * 16 * C::ROWB, C::KV_SLAB, C::ATOM, C::SWZ);
                    umma_ss(tmem_base + C::TMEM_DQ, a, bk, idesc_o, (ch > 0) || (kk > 0));
                }
                if (SPLIT) {
#pragma unroll
                    for (int kk = 0; kk < C::NKP / 16; ++kk) {
                        const uint64_t a = smem_desc(smem_u32(sRES + (kk >> 2) * C::P_SLAB) + (kk & 3) * 32, 16, 1024, 2u);
                        const uint64_t bk = smem_desc(smem_u32(sK) + kk * 16 * C::ROWB, C::KV_SLAB, C::ATOM, C::SWZ);
                        umma_ss(tmem_base + C::TMEM_DQ, a, bk, idesc_o, 1u);
                    }
                }
                umma_commit(bar_o);
            }
            __syncwarp();
            mbar_wait(bar_o, ph_o, abort_flag, kErrMmaWait);
            ph_o ^= 1u;
            tc_fence_after();
        }

        DT* row = d_q + qi * D;
#pragma unroll
        for (int piece = 0; piece < D / 32; ++piece) {
            uint32_t v[32];
            tmem_ld_32x32(tmem_lane + C::TMEM_DQ + 32 * piece, v);
            tmem_ld_wait();
            if (q_valid) {
#pragma unroll
                for (int gI = 0; gI < 4; ++gI) {
                    uint4 pk;
                    pk.x = pack2<DT>(__uint_as_float(v[8 * gI + 0]), __uint_as_float(v[8 * gI + 1]));
                    pk.y = pack2<DT>(__uint_as_float(v[8 * gI + 2]), __uint_as_float(v[8 * gI + 3]));
                    pk.z = pack2<DT>(__uint_as_float(v[8 * gI + 4]), __uint_as_float(v[8 * gI + 5]));
                    pk.w = pack2<DT>(__uint_as_float(v[8 * gI + 6]), __uint_as_float(v[8 * gI + 7]));
                    *reinterpret_cast<uint4*>(row + 32 * piece + 8 * gI) = pk;
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        tmem_dealloc(tmem_base, C::TMEM_COLS);
    }
}

// ------------------------------------------------------------------------------------ launchers
template <typename DT, int D, int KS>
int launch_dq(const Na2dGeom& g, int dtype, const void* q, const void* k, const void* v, const float* lse,
              const void* d_o, void* d_q, float* delta, cudaStream_t st, int* launched) {
    using C = DqCfg<D, KS, IsBf16<DT>::value>;
    CUtensorMap tq, tg, tk, tv;
    int rc = make_map(&tq, q, dtype, g.BN, g.Hq, g.W, D, TW, TH);
    if (rc == NA2D_OK) rc = make_map(&tg, d_o, dtype, g.BN, g.Hq, g.W, D, TW, TH);
    if (rc == NA2D_OK) rc = make_map(&tk, k, dtype, g.BN, g.Hkv, g.W, D, C::HW, C::RC);
    if (rc == NA2D_OK) rc = make_map(&tv, v, dtype, g.BN, g.Hkv, g.W, D, C::HW, C::RC);
    if (rc != NA2D_OK) return rc;
    const int tiles_r = (g.Hq + TH - 1) / TH, tiles_c = (g.W + TW - 1) / TW;
    const long long tiles = (long long)g.BN * tiles_r * tiles_c;
    if (tiles > 0x7fffffffLL) return NA2D_ERR_TOO_LARGE;
    auto kern = dq_kernel<DT, D, KS>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM) != cudaSuccess)
        return NA2D_ERR_CUDA;
    kern<<<(unsigned)tiles, 128, C::SMEM, st>>>(tq, tg, tk, tv, lse, (DT*)d_q, delta, g, tiles_r, tiles_c);
    *launched += 1;
    return cudaGetLastError() == cudaSuccess ? NA2D_OK : NA2D_ERR_CUDA;
}

inline int backward_dq(const Na2dGeom& g, int dtype, const void* q, const void* k, const void* v, const void* /*o*/,
                       const float* lse, const void* d_o, void* d_q, float* delta, int, cudaStream_t st, int* launched) {
    if (dtype == NA2D_BF16) {
        NA2D_TC_DISPATCH_D(launch_dq, __nv_bfloat16, g, dtype, q, k, v, lse, d_o, d_q, delta, st, launched)
    } else {
        NA2D_TC_DISPATCH_D(launch_dq, __half, g, dtype, q, k, v, lse, d_o, d_q, delta, st, launched)
    }
}

}  // namespace na2d_tc
