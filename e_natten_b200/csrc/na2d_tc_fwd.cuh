// Persistent, warp-specialised tcgen05 forward kernel.  Included by na2d_tc.cuh.
//
// One CTA per SM walks tiles blockIdx.x, blockIdx.x + gridDim.x, ...  A tile is 8 x 16 queries;
// its halo box of keys is streamed in chunks of whole box rows with at most 128 keys.  Six warps:
//   warps 0-3  softmax: read S from tensor memory, mask, online softmax, write P to shared
//              memory; the output accumulates in tensor memory across the chunks of a tile and is
//              rescaled there only when a row's maximum grows by more than 2^8 (until then the
//              older maximum keeps being used, which leaves the result unchanged); store o, lse;
//   warp 4     producer: TMA loads of Q tiles (two buffers) and K/V chunks (a ring of stages);
//   warp 5     MMA issue: S = Q K^T into one of two S accumulators, O += P V into the tile's O
//              accumulator (two, alternating by tile), with the S of the next chunk issued before
//              the P V of the current one so that the tensor pipe and the softmax warps overlap.
// Every hand-over is an mbarrier with a bounded wait.
#pragma once

namespace na2d_tc {

template <int D, int KS>
struct FwdCfg : Cfg<D, KS, 128> {
    using B = Cfg<D, KS, 128>;
    static constexpr int STAGE_BYTES = 2 * B::KV_BYTES;                 // K chunk then V chunk
    static constexpr int FIXED = 2 * B::Q_BYTES + B::P_BYTES + 256 /*barriers*/ + 1024 /*alignment*/;
    static constexpr int NST_FIT = (kSmemLimit - FIXED) / STAGE_BYTES;
    static constexpr int NST = NST_FIT > 4 ? 4 : NST_FIT;               // K/V ring depth
    static constexpr int SMEM = FIXED + NST * STAGE_BYTES;
    static constexpr int TMEM_S0 = 0, TMEM_O0 = 256, TMEM_STRIDE = 128; // S[2] at 0/128, O[2] at 256/384
    static_assert(NST >= 2, "forward kernel needs at least two K/V stages");
    static_assert(B::NKP <= 128 && D <= 128, "tensor memory layout");
};

template <typename DT, int D, int KS>
__global__ void __launch_bounds__(192, 1)
fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
           const __grid_constant__ CUtensorMap tm_v, DT* __restrict__ o, float* __restrict__ lse,
           const Na2dGeom g, const int tiles_r, const int tiles_c, const int total_tiles) {
    using C = FwdCfg<D, KS>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sQ = smem;                                   // 2 x Q tile
    uint8_t* sKV = sQ + 2 * C::Q_BYTES;                   // NST x (K chunk, V chunk)
    uint8_t* sP = sKV + C::NST * C::STAGE_BYTES;          // P of the current chunk
    uint64_t* bars = reinterpret_cast<uint64_t*>(sP + C::P_BYTES);
    uint64_t* q_full = bars;                 // [2]   TMA -> MMA
    uint64_t* q_empty = bars + 2;            // [2]   MMA (commit) -> TMA
    uint64_t* s_full = bars + 4;             // [2]   MMA (commit) -> softmax
    uint64_t* s_free = bars + 6;             // [2]   softmax -> MMA
    uint64_t* o_full = bars + 8;             // [2]   MMA (commit) -> softmax
    uint64_t* o_free = bars + 10;            // [2]   softmax -> MMA
    uint64_t* p_full = bars + 12;            //       softmax -> MMA
    uint64_t* p_free = bars + 13;            //       MMA (commit) -> softmax
    uint64_t* kv_full = bars + 14;           // [NST] TMA -> MMA
    uint64_t* kv_empty = bars + 14 + C::NST; // [NST] MMA (commit) -> TMA
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 14 + 2 * C::NST);
    volatile uint32_t* abort_flag = tmem_slot + 1;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n_my = total_tiles > (int)blockIdx.x ? (total_tiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;
    const uint32_t total_units = (uint32_t)n_my * C::NCH;

    if (tid == 0) {
        *abort_flag = 0;
        for (int i = 0; i < 2; ++i) {
            mbar_init(q_full + i, 1);
            mbar_init(q_empty + i, 1);
            mbar_init(s_full + i, 1);
            mbar_init(s_free + i, 4);
            mbar_init(o_full + i, 1);
            mbar_init(o_free + i, 4);
        }
        mbar_init(p_full, 4);
        mbar_init(p_free, 1);
        for (int i = 0; i < C::NST; ++i) {
            mbar_init(kv_full + i, 1);
            mbar_init(kv_empty + i, 1);
        }
        mbar_fence_init();
        tma_prefetch_desc(&tm_q);
        tma_prefetch_desc(&tm_k);
        tma_prefetch_desc(&tm_v);
    }
    if (warp == 0) {
        __syncwarp();
        tmem_alloc(tmem_slot, 512);
        tmem_relinquish();
    }
    // V rows [NK, NKP) of every stage are contraction rows of P V that TMA never writes.
    if constexpr (C::NKP > C::NK) {
        constexpr int pad16 = (C::NKP - C::NK) * C::ROWB / 16;
        for (int i = tid; i < C::NST * C::NS * pad16; i += 192) {
            const int which = i / pad16, off = i - which * pad16;
            const int st = which / C::NS, slab = which % C::NS;
            uint8_t* base = sKV + st * C::STAGE_BYTES + C::KV_BYTES + slab * C::KV_SLAB;
            st_shared_v4(smem_u32(base + C::NK * C::ROWB + off * 16), 0u, 0u, 0u, 0u);
        }
        fence_proxy_async();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    auto decode = [&](int i, int& bn, int& r0, int& c0) {
        int t = (int)blockIdx.x + i * (int)gridDim.x;
        const int tc = t % tiles_c;
        t /= tiles_c;
        r0 = (t % tiles_r) * TH;
        c0 = tc * TW;
        bn = t / tiles_r;
    };

    if (warp == 4) {
        // ------------------------------------------------------------------ producer
        if (lane == 0) {
            uint32_t n = 0;
            for (int i = 0; i < n_my; ++i) {
                int bn, r0, c0;
                decode(i, bn, r0, c0);
                const int box_r0 = na2d_ws(g.q_row0 + r0, g.Hg, KS) - g.kv_row0;
                const int box_c0 = na2d_ws(c0, g.W, KS);
                const int qb = i & 1;
                mbar_wait(q_empty + qb, ((i >> 1) & 1) ^ 1, abort_flag, kErrLoadWait);
                mbar_expect_tx(q_full + qb, C::Q_BYTES);
#pragma unroll
                for (int s = 0; s < C::NS; ++s)
                    tma_load_4d(sQ + qb * C::Q_BYTES + s * C::Q_SLAB, &tm_q, q_full + qb, s * 64, c0, r0, bn);
                for (int c = 0; c < C::NCH; ++c, ++n) {
                    const uint32_t st = n % C::NST;
                    mbar_wait(kv_empty + st, ((n / C::NST) & 1) ^ 1, abort_flag, kErrLoadWait);
                    mbar_expect_tx(kv_full + st, 2u * C::NS * C::NK * C::ROWB);
                    uint8_t* dst = sKV + st * C::STAGE_BYTES;
#pragma unroll
                    for (int s = 0; s < C::NS; ++s) {
                        tma_load_4d(dst + s * C::KV_SLAB, &tm_k, kv_full + st, s * 64, box_c0, box_r0 + c * C::RC, bn);
                        tma_load_4d(dst + C::KV_BYTES + s * C::KV_SLAB, &tm_v, kv_full + st, s * 64, box_c0,
                                    box_r0 + c * C::RC, bn);
                    }
                }
            }
        }
    } else if (warp == 5) {
        // ------------------------------------------------------------------ MMA issue
        if (lane == 0) {
            constexpr uint32_t idesc_s = umma_idesc(TM, C::NKP, IsBf16<DT>::value, IsBf16<DT>::value, false, false);
            constexpr uint32_t idesc_o = umma_idesc(TM, D, IsBf16<DT>::value, IsBf16<DT>::value, false, true);
            auto issue_s = [&](uint32_t n) {
                const uint32_t i = n / C::NCH, c = n % C::NCH, st = n % C::NST, sb = n & 1;
                if (c == 0) mbar_wait(q_full + (i & 1), (i >> 1) & 1, abort_flag, kErrLoadWait);
                mbar_wait(kv_full + st, (n / C::NST) & 1, abort_flag, kErrLoadWait);
                mbar_wait(s_free + sb, ((n >> 1) & 1) ^ 1, abort_flag, kErrMmaWait);
                tc_fence_after();
                const uint32_t q_addr = smem_u32(sQ + (i & 1) * C::Q_BYTES);
                const uint32_t k_addr = smem_u32(sKV + st * C::STAGE_BYTES);
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk) {
                    const int slab = (kk * 16) / C::SLAB_C, in_slab = (kk * 16) % C::SLAB_C;
                    const uint64_t a = smem_desc(q_addr + slab * C::Q_SLAB + in_slab * 2, 16, C::ATOM, C::SWZ);
                    const uint64_t b = smem_desc(k_addr + slab * C::KV_SLAB + in_slab * 2, 16, C::ATOM, C::SWZ);
                    umma_ss(tmem_base + C::TMEM_S0 + sb * C::TMEM_STRIDE, a, b, idesc_s, kk > 0);
                }
                umma_commit(s_full + sb);
                if (c == C::NCH - 1) umma_commit(q_empty + (i & 1));      // the tile's Q buffer is free
            };
            if (total_units > 0) issue_s(0);
            for (uint32_t n = 0; n < total_units; ++n) {
                if (n + 1 < total_units) issue_s(n + 1);
                const uint32_t i = n / C::NCH, c = n % C::NCH, st = n % C::NST, ob = i & 1;
                mbar_wait(p_full, n & 1, abort_flag, kErrMmaWait);
                if (c == 0) mbar_wait(o_free + ob, ((i >> 1) & 1) ^ 1, abort_flag, kErrMmaWait);
                tc_fence_after();
                const uint32_t v_addr = smem_u32(sKV + st * C::STAGE_BYTES + C::KV_BYTES);
#pragma unroll
                for (int kk = 0; kk < C::NKP / 16; ++kk) {
                    const uint64_t a = smem_desc(smem_u32(sP + (kk >> 2) * C::P_SLAB) + (kk & 3) * 32, 16, 1024, 2u);
                    const uint64_t b = smem_desc(v_addr + kk * 16 * C::ROWB, C::KV_SLAB, C::ATOM, C::SWZ);
                    umma_ss(tmem_base + C::TMEM_O0 + ob * C::TMEM_STRIDE, a, b, idesc_o, (c > 0) || (kk > 0));
                }
                umma_commit(kv_empty + st);
                umma_commit(p_free);                       // also: "this chunk's P V has landed in O"
                if (c == C::NCH - 1) umma_commit(o_full + ob);
            }
        }
    } else {
        // ------------------------------------------------------------------ softmax warps
        const uint32_t tmem_lane = tmem_base + (static_cast<uint32_t>(warp * 32) << 16);
        constexpr float kRescaleStep = 8.f;      // log2 units: rescale O when the maximum grows by > 2^8
        // epilogue of the previous tile, deferred until the next tile's first chunk is under way
        bool pend = false, pend_valid = false;
        uint32_t pend_tile = 0;
        float pend_max = 0.f, pend_sum = 1.f;
        size_t pend_qi = 0;

        auto epilogue = [&]() {
            const uint32_t ob = pend_tile & 1;
            mbar_wait(o_full + ob, (pend_tile >> 1) & 1, abort_flag, kErrMmaWait);
            tc_fence_after();
            const float inv = 1.f / pend_sum;
            DT* orow = o + pend_qi * D;
#pragma unroll
            for (int piece = 0; piece < D / 32; ++piece) {
                uint32_t v[32];
                tmem_ld_32x32(tmem_lane + C::TMEM_O0 + ob * C::TMEM_STRIDE + 32 * piece, v);
                tmem_ld_wait();
                if (pend_valid) {
#pragma unroll
                    for (int gI = 0; gI < 4; ++gI) {
                        uint4 pk;
                        pk.x = pack2<DT>(__uint_as_float(v[8 * gI + 0]) * inv, __uint_as_float(v[8 * gI + 1]) * inv);
                        pk.y = pack2<DT>(__uint_as_float(v[8 * gI + 2]) * inv, __uint_as_float(v[8 * gI + 3]) * inv);
                        pk.z = pack2<DT>(__uint_as_float(v[8 * gI + 4]) * inv, __uint_as_float(v[8 * gI + 5]) * inv);
                        pk.w = pack2<DT>(__uint_as_float(v[8 * gI + 6]) * inv, __uint_as_float(v[8 * gI + 7]) * inv);
                        *reinterpret_cast<uint4*>(orow + 32 * piece + 8 * gI) = pk;
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(o_free + ob);
            if (pend_valid) lse[pend_qi] = (pend_max + log2f(pend_sum)) * kLn2;
            pend = false;
        };

        uint32_t n = 0;
        for (int i = 0; i < n_my; ++i) {
            int bn, r0, c0;
            decode(i, bn, r0, c0);
            const int box_r0 = na2d_ws(g.q_row0 + r0, g.Hg, KS) - g.kv_row0;
            const int box_c0 = na2d_ws(c0, g.W, KS);
            const int qr_raw = r0 + (tid / TW), qc_raw = c0 + (tid % TW);
            const bool q_valid = qr_raw < g.Hq && qc_raw < g.W;
            const int qr = min(qr_raw, g.Hq - 1), qc = min(qc_raw, g.W - 1);
            const int wr = na2d_ws(g.q_row0 + qr, g.Hg, KS) - g.kv_row0 - box_r0;   // in [0, TH)
            const int wc = na2d_ws(qc, g.W, KS) - box_c0;                            // in [0, TW)
            const uint32_t row_mask = ((1u << KS) - 1u) << wr;
            const uint32_t col_mask = ((1u << KS) - 1u) << wc;
            const int wr_lo = __shfl_sync(0xffffffffu, wr, 0);
            const int wr_hi = __shfl_sync(0xffffffffu, wr, 31);
            const uint32_t o_addr = tmem_lane + C::TMEM_O0 + (i & 1) * C::TMEM_STRIDE;
            float run_max = -CUDART_INF_F, run_sum = 0.f;

            for (int ch = 0; ch < C::NCH; ++ch, ++n) {
                const uint32_t sb = n & 1;
                const uint32_t s_addr = tmem_lane + C::TMEM_S0 + sb * C::TMEM_STRIDE;
                const uint32_t rm = row_mask >> (ch * C::RC);            // bit r: chunk row r is in the window
                mbar_wait(s_full + sb, (n >> 1) & 1, abort_flag, kErrMmaWait);
                tc_fence_after();

                // pass 1: masked maximum of the chunk
                float cmax = -CUDART_INF_F;
#pragma unroll
                for (int b = 0; b < C::NB; ++b) {
                    const int row_first = ch * C::RC + (32 * b) / C::HW;
                    constexpr int kNkLast = C::NK - 1;
                    const int last_col = (32 * b + 31 < kNkLast) ? 32 * b + 31 : kNkLast;
                    const int row_last = ch * C::RC + last_col / C::HW;
                    if (32 * b < C::NK && row_last >= wr_lo && row_first < wr_hi + KS) {     // warp-uniform
                        uint32_t s[32];
                        tmem_ld_32x32(s_addr + 32 * b, s);
                        tmem_ld_wait();
#pragma unroll
                        for (int e = 0; e < 32; ++e) {
                            const int j = 32 * b + e;
                            if (j < C::NK) {
                                const bool ok = ((rm >> (j / C::HW)) & 1u) && ((col_mask >> (j % C::HW)) & 1u);
                                cmax = fmaxf(cmax, ok ? __uint_as_float(s[e]) : -CUDART_INF_F);
                            }
                        }
                    }
                }
                cmax *= kLog2e;

                // The previous chunk's P V is complete (so P may be overwritten and O is stable).
                mbar_wait(p_free, (n & 1) ^ 1, abort_flag, kErrMmaWait);

                // Raise the running maximum only when it would grow by more than the step; a row
                // whose maximum is still -inf has an all-zero O row and takes the new one freely.
                const bool grow = cmax > run_max + kRescaleStep;
                if (ch > 0 && __any_sync(0xffffffffu, grow && run_max != -CUDART_INF_F)) {
                    const float alpha = grow ? fast_exp2(run_max - cmax) : 1.f;
                    tc_fence_after();
#pragma unroll
                    for (int piece = 0; piece < D / 32; ++piece) {
                        uint32_t v[32];
                        tmem_ld_32x32(o_addr + 32 * piece, v);
                        tmem_ld_wait();
#pragma unroll
                        for (int e = 0; e < 32; ++e) v[e] = __float_as_uint(__uint_as_float(v[e]) * alpha);
                        tmem_st_32x32(o_addr + 32 * piece, v);
                    }
                    tmem_st_wait();
                    run_sum *= alpha;
                    if (grow) run_max = cmax;
                } else if (grow) {
                    run_sum = 0.f;                  // only reachable with run_max == -inf: nothing summed yet
                    run_max = cmax;
                }
                const float safe_max = (run_max == -CUDART_INF_F) ? 0.f : run_max;

                // pass 2: P = exp2(s * log2e - max) -> shared memory, row sum
                float csum = 0.f;
#pragma unroll
                for (int b = 0; b < C::NB; ++b) {
                    const int row_first = ch * C::RC + (32 * b) / C::HW;
                    constexpr int kNkLast = C::NK - 1;
                    const int last_col = (32 * b + 31 < kNkLast) ? 32 * b + 31 : kNkLast;
                    const int row_last = ch * C::RC + last_col / C::HW;
                    uint32_t w[16];
                    if (32 * b < C::NK && row_last >= wr_lo && row_first < wr_hi + KS) {
                        uint32_t s[32];
                        tmem_ld_32x32(s_addr + 32 * b, s);
                        tmem_ld_wait();
#pragma unroll
                        for (int e2 = 0; e2 < 16; ++e2) {
                            float pp[2] = {0.f, 0.f};
#pragma unroll
                            for (int h = 0; h < 2; ++h) {
                                const int j = 32 * b + 2 * e2 + h;
                                if (j < C::NK) {
                                    const bool ok = ((rm >> (j / C::HW)) & 1u) && ((col_mask >> (j % C::HW)) & 1u);
                                    const float ex = fast_exp2(fmaf(__uint_as_float(s[2 * e2 + h]), kLog2e, -safe_max));
                                    pp[h] = ok ? ex : 0.f;
                                    csum += pp[h];
                                }
                            }
                            w[e2] = pack2<DT>(pp[0], pp[1]);
                        }
                    } else {
#pragma unroll
                        for (int e = 0; e < 16; ++e) w[e] = 0u;
                    }
                    store_operand_block(smem_u32(sP), C::P_SLAB, tid, b, w);
                }
                run_sum += csum;
                tc_fence_before();
                fence_proxy_async();
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(s_free + sb);
                    mbar_arrive(p_full);
                }
                if (pend) epilogue();           // previous tile's output, while this chunk's P V runs
            }
            pend = true;
            pend_tile = (uint32_t)i;
            pend_valid = q_valid;
            pend_max = run_max;
            pend_sum = run_sum;
            pend_qi = (static_cast<size_t>(bn) * g.Hq + qr) * g.W + qc;
        }
        if (pend) epilogue();
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}

template <typename DT, int D, int KS>
int launch_forward(const Na2dGeom& g, int dtype, const void* q, const void* k, const void* v, void* o, float* lse,
                   int device, cudaStream_t st, int* launched) {
    using C = FwdCfg<D, KS>;
    CUtensorMap tq, tk, tv;
    int rc = make_map(&tq, q, dtype, g.BN, g.Hq, g.W, D, TW, TH);
    if (rc == NA2D_OK) rc = make_map(&tk, k, dtype, g.BN, g.Hkv, g.W, D, C::HW, C::RC);
    if (rc == NA2D_OK) rc = make_map(&tv, v, dtype, g.BN, g.Hkv, g.W, D, C::HW, C::RC);
    if (rc != NA2D_OK) return rc;
    const int tiles_r = (g.Hq + TH - 1) / TH, tiles_c = (g.W + TW - 1) / TW;
    const long long tiles = (long long)g.BN * tiles_r * tiles_c;
    if (tiles > 0x7fffffffLL) return NA2D_ERR_TOO_LARGE;
    auto kern = fwd_kernel<DT, D, KS>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM) != cudaSuccess)
        return NA2D_ERR_CUDA;
    const int grid = (int)(tiles < sm_count(device) ? tiles : sm_count(device));
    kern<<<grid, 192, C::SMEM, st>>>(tq, tk, tv, (DT*)o, lse, g, tiles_r, tiles_c, (int)tiles);
    *launched += 1;
    return cudaGetLastError() == cudaSuccess ? NA2D_OK : NA2D_ERR_CUDA;
}

inline int forward(const Na2dGeom& g, int dtype, const void* q, const void* k, const void* v, void* o, float* lse,
                   int device, cudaStream_t st, int* launched) {
    if (dtype == NA2D_BF16) {
        NA2D_TC_DISPATCH_D(launch_forward, __nv_bfloat16, g, dtype, q, k, v, o, lse, device, st, launched)
    } else {
        NA2D_TC_DISPATCH_D(launch_forward, __half, g, dtype, q, k, v, o, lse, device, st, launched)
    }
}

}  // namespace na2d_tc
