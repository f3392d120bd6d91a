// tcgen05 tensor-core kernels for 2D neighborhood attention on sm_100a (bf16 / fp16 inputs,
// fp32 accumulation), and their host-side launchers.
//
// Tiling.  A CTA owns a tile of 8 x 16 = 128 query pixels; query r of the tile is row r of every
// MMA and lane r of tensor memory.  The keys a tile can see are the union of its pixels' clamped
// windows: a (8+ks-1) x (16+ks-1) "halo box" whose origin is the window origin of the tile's
// first pixel.  The box is cut into chunks of whole box rows with at most 256 keys each (the
// UMMA N limit); TMA brings each chunk of K and V into shared memory as [key][channel] rows with
// the 128-byte (64-byte for head dim 32) swizzle, which is at once the K-major B operand of
// S = Q K^T and the MN-major B operand of O = P V.  The per-query window mask is applied in
// registers on the S accumulator read back from tensor memory, followed by an online softmax
// across chunks; P goes back to shared memory as the K-major A operand of the second MMA.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <math_constants.h>

#include <mutex>

#include "../../include/na2d.h"
#include "na2d_index.cuh"
#include "na2d_ptx.cuh"

namespace na2d_tc {

using namespace na2d_ptx;

constexpr int TH = 8;      // tile rows
constexpr int TW = 16;     // tile columns
constexpr int TM = 128;    // queries (or keys) per tile = MMA M
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

// Compile-time geometry of one (head dim, kernel size) instantiation.
// NMAX caps the keys (forward, dQ) or queries (dK/dV) of one chunk; it is set by how many
// tensor-memory columns the kernel can spare for the S-shaped accumulators.
template <int D, int KS, int NMAX = 256>
struct Cfg {
    static constexpr int HH = TH + KS - 1;                 // halo box rows
    static constexpr int HW = TW + KS - 1;                 // halo box columns
    static constexpr int RC_MAX = NMAX / HW;
    static constexpr int NCH = (HH + RC_MAX - 1) / RC_MAX; // key chunks per tile
    static constexpr int RC = (HH + NCH - 1) / NCH;        // box rows per chunk
    static constexpr int NK = RC * HW;                     // keys per chunk
    static constexpr int NKP = (NK + 15) / 16 * 16;        // padded to the UMMA granularity
    static constexpr int NS = (D + 63) / 64;               // channel slabs
    static constexpr int SLAB_C = D < 64 ? D : 64;         // channels per slab
    static constexpr int ROWB = SLAB_C * 2;                // bytes of one row of one slab
    static constexpr uint32_t SWZ = ROWB == 128 ? 2u : 4u; // descriptor swizzle code
    static constexpr int ATOM = 8 * ROWB;                  // bytes of an 8-row group
    static constexpr int Q_SLAB = TM * ROWB;
    static constexpr int Q_BYTES = NS * Q_SLAB;
    static constexpr int KV_SLAB = NKP * ROWB;
    static constexpr int KV_BYTES = NS * KV_SLAB;
    static constexpr int NPS = (NKP + 63) / 64;            // P slabs of 64 keys
    static constexpr int P_SLAB = TM * 128;
    static constexpr int P_BYTES = NPS * P_SLAB;
    static constexpr int NB = (NKP + 31) / 32;             // 32-column blocks of S
    static constexpr int TMEM_S = 0;                       // S accumulator columns [0, 256)
    static constexpr int TMEM_O = 256;                     // O accumulator columns [256, 256 + D)
    static constexpr int TMEM_COLS = 512;
    static constexpr int SMEM_FWD = Q_BYTES + 2 * KV_BYTES + P_BYTES + 64 /*barriers*/ + 1024 /*alignment*/;
    static_assert(NB * 32 <= NPS * 64, "P slabs must hold every S block");
    static_assert(NKP <= NMAX && NKP % 16 == 0, "UMMA N range");
    static_assert(KV_SLAB % 1024 == 0 && Q_SLAB % 1024 == 0, "slabs must keep the swizzle alignment");
};

template <typename DT> struct IsBf16 { static constexpr bool value = false; };
template <> struct IsBf16<__nv_bfloat16> { static constexpr bool value = true; };

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

template <typename DT> __device__ __forceinline__ uint32_t pack2(float lo, float hi);
template <> __device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}
template <> __device__ __forceinline__ uint32_t pack2<__half>(float lo, float hi) {
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// Residual of a packed bf16 pair: packs (lo - value of the low half, hi - value of the high half).
// dS is handed to its MMA as the bf16 pair (head, residual) on the bf16 path: a single bf16
// keeps 8 significant bits, which leaves dQ / dK elements several 1e-2 off in the tails of a
// large tensor; head + residual keeps 16.
__device__ __forceinline__ uint32_t pack2_residual_bf16(float lo, float hi, uint32_t head) {
    const float lo_head = __uint_as_float(head << 16);
    const float hi_head = __uint_as_float(head & 0xffff0000u);
    __nv_bfloat162 v = __floats2bfloat162_rn(lo - lo_head, hi - hi_head);
    return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

// Writes 32 consecutive 16-bit values (already packed in pairs) of row `row` of a K-major,
// 128-byte-swizzled [128 x 64]-slab operand, at columns [32*block, 32*block + 32).
__device__ __forceinline__ void store_operand_block(uint32_t base, int slab_bytes, int row, int block,
                                                    const uint32_t (&w)[16]) {
    const uint32_t row_base = base + (block >> 1) * slab_bytes + row * 128;
#pragma unroll
    for (int gI = 0; gI < 4; ++gI) {
        const int chunk = ((block & 1) * 4 + gI) ^ (row & 7);
        st_shared_v4(row_base + chunk * 16, w[4 * gI], w[4 * gI + 1], w[4 * gI + 2], w[4 * gI + 3]);
    }
}

// ------------------------------------------------------------------------------------ forward
template <typename DT, int D, int KS>
__global__ void __launch_bounds__(128, 1)
fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
           const __grid_constant__ CUtensorMap tm_v, DT* __restrict__ o, float* __restrict__ lse,
           const Na2dGeom g, const int tiles_r, const int tiles_c) {
    using C = Cfg<D, KS>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sQ = smem;
    uint8_t* sK = sQ + C::Q_BYTES;
    uint8_t* sV = sK + C::KV_BYTES;
    uint8_t* sP = sV + C::KV_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(sP + C::P_BYTES);
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
    const int box_r0 = na2d_ws(g.q_row0 + r0, g.Hg, KS) - g.kv_row0;    // key-band row of the box origin
    const int box_c0 = na2d_ws(c0, g.W, KS);

    if (tid == 0) {
        *abort_flag = 0;
        mbar_init(bar_load, 1);
        mbar_init(bar_s, 1);
        mbar_init(bar_o, 1);
        mbar_fence_init();
        tma_prefetch_desc(&tm_q);
        tma_prefetch_desc(&tm_k);
        tma_prefetch_desc(&tm_v);
    }
    if (warp == 0) {
        __syncwarp();
        tmem_alloc(tmem_slot, C::TMEM_COLS);
        tmem_relinquish();
    }
    // Rows [NK, NKP) of every K / V slab are never written by TMA; zero them once so that the
    // padded keys contribute exact zeros (0 * stale bits could be NaN).
    if constexpr (C::NKP > C::NK) {
        constexpr int pad16 = (C::NKP - C::NK) * C::ROWB / 16;
        for (int i = tid; i < 2 * C::NS * pad16; i += 128) {
            const int which = i / pad16, off = i - which * pad16;
            uint8_t* base = (which < C::NS ? sK + which * C::KV_SLAB : sV + (which - C::NS) * C::KV_SLAB);
            st_shared_v4(smem_u32(base + C::NK * C::ROWB + off * 16), 0u, 0u, 0u, 0u);
        }
        fence_proxy_async();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_lane = tmem_base + (static_cast<uint32_t>(warp * 32) << 16);

    // this thread's query and its window inside the halo box
    const int qr_raw = r0 + (tid >> 4), qc_raw = c0 + (tid & 15);
    const bool q_valid = qr_raw < g.Hq && qc_raw < g.W;
    const int qr = min(qr_raw, g.Hq - 1), qc = min(qc_raw, g.W - 1);
    const int wr = na2d_ws(g.q_row0 + qr, g.Hg, KS) - g.kv_row0 - box_r0;   // in [0, TH)
    const int wc = na2d_ws(qc, g.W, KS) - box_c0;                            // in [0, TW)
    const uint32_t row_mask = ((1u << KS) - 1u) << wr;     // bit hr set: box row hr is in the window
    const uint32_t col_mask = ((1u << KS) - 1u) << wc;     // bit hc set: box column hc is in the window
    const int wr_lo = __shfl_sync(0xffffffffu, wr, 0);     // the warp's queries span box rows
    const int wr_hi = __shfl_sync(0xffffffffu, wr, 31);    //   [wr_lo, wr_hi + KS)

    constexpr uint32_t idesc_s = umma_idesc(TM, C::NKP, IsBf16<DT>::value, IsBf16<DT>::value, false, false);
    constexpr uint32_t idesc_o = umma_idesc(TM, D, IsBf16<DT>::value, IsBf16<DT>::value, false, true);

    float run_max = -CUDART_INF_F;      // running row maximum of s * log2(e)
    float run_sum = 0.f;                // running row sum of exp2(s * log2(e) - run_max)
    float o_acc[C::NCH > 1 ? D : 1];    // output accumulator across chunks (multi-chunk only)

#pragma unroll
    for (int ch = 0; ch < C::NCH; ++ch) {
        const uint32_t phase = ch & 1;
        // ---- load this chunk of K and V (and Q the first time), then S = Q K^T ----------------
        if (tid == 0) {
            const uint32_t kv_bytes = 2u * C::NS * C::NK * C::ROWB;
            mbar_expect_tx(bar_load, kv_bytes + (ch == 0 ? C::Q_BYTES : 0));
#pragma unroll
            for (int s = 0; s < C::NS; ++s) {
                if (ch == 0) tma_load_4d(sQ + s * C::Q_SLAB, &tm_q, bar_load, s * 64, c0, r0, bn);
                tma_load_4d(sK + s * C::KV_SLAB, &tm_k, bar_load, s * 64, box_c0, box_r0 + ch * C::RC, bn);
                tma_load_4d(sV + s * C::KV_SLAB, &tm_v, bar_load, s * 64, box_c0, box_r0 + ch * C::RC, bn);
            }
            mbar_wait(bar_load, phase, abort_flag, kErrLoadWait);
            tc_fence_after();
#pragma unroll
            for (int kk = 0; kk < D / 16; ++kk) {
                const int slab = (kk * 16) / C::SLAB_C, in_slab = (kk * 16) % C::SLAB_C;
                const uint64_t a = smem_desc(smem_u32(sQ + slab * C::Q_SLAB) + in_slab * 2, 16, C::ATOM, C::SWZ);
                const uint64_t b = smem_desc(smem_u32(sK + slab * C::KV_SLAB) + in_slab * 2, 16, C::ATOM, C::SWZ);
                umma_ss(tmem_base + C::TMEM_S, a, b, idesc_s, kk > 0);
            }
            umma_commit(bar_s);
        }
        __syncwarp();
        mbar_wait(bar_s, phase, abort_flag, kErrMmaWait);
        tc_fence_after();

        // ---- pass 1: masked row maximum of this chunk -----------------------------------------
        float cmax = -CUDART_INF_F;
#pragma unroll
        for (int b = 0; b < C::NB; ++b) {
            const int row_first = ch * C::RC + (32 * b) / C::HW;
            const int last_col = (32 * b + 31 < C::NK - 1) ? 32 * b + 31 : C::NK - 1;
            const int row_last = ch * C::RC + last_col / C::HW;
            if (32 * b < C::NK && row_last >= wr_lo && row_first < wr_hi + KS) {     // warp-uniform
                uint32_t s[32];
                tmem_ld_32x32(tmem_lane + C::TMEM_S + 32 * b, s);
                tmem_ld_wait();
#pragma unroll
                for (int e = 0; e < 32; ++e) {
                    const int j = 32 * b + e;
                    if (j < C::NK) {
                        const int hr = ch * C::RC + j / C::HW, hc = j % C::HW;
                        const bool ok = ((row_mask >> hr) & 1u) && ((col_mask >> hc) & 1u);
                        cmax = fmaxf(cmax, ok ? __uint_as_float(s[e]) : -CUDART_INF_F);
                    }
                }
            }
        }
        const float new_max = fmaxf(run_max, cmax * kLog2e);
        const float safe_max = (new_max == -CUDART_INF_F) ? 0.f : new_max;
        const float alpha = fast_exp2(run_max - safe_max);        // 0 when run_max is -inf
        run_max = new_max;

        // ---- pass 2: P = exp2(s*log2e - max), row sum, P -> shared memory as the A operand -----
        float csum = 0.f;
#pragma unroll
        for (int b = 0; b < C::NB; ++b) {
            const int row_first = ch * C::RC + (32 * b) / C::HW;
            const int last_col = (32 * b + 31 < C::NK - 1) ? 32 * b + 31 : C::NK - 1;
            const int row_last = ch * C::RC + last_col / C::HW;
            uint32_t w[16];
            if (32 * b < C::NK && row_last >= wr_lo && row_first < wr_hi + KS) {
                uint32_t s[32];
                tmem_ld_32x32(tmem_lane + C::TMEM_S + 32 * b, s);
                tmem_ld_wait();
                float p[32];
#pragma unroll
                for (int e = 0; e < 32; ++e) {
                    const int j = 32 * b + e;
                    p[e] = 0.f;
                    if (j < C::NK) {
                        const int hr = ch * C::RC + j / C::HW, hc = j % C::HW;
                        const bool ok = ((row_mask >> hr) & 1u) && ((col_mask >> hc) & 1u);
                        const float ex = fast_exp2(fmaf(__uint_as_float(s[e]), kLog2e, -safe_max));
                        p[e] = ok ? ex : 0.f;
                        csum += p[e];
                    }
                }
#pragma unroll
                for (int e = 0; e < 16; ++e) w[e] = pack2<DT>(p[2 * e], p[2 * e + 1]);
            } else {
#pragma unroll
                for (int e = 0; e < 16; ++e) w[e] = 0u;
            }
            store_operand_block(smem_u32(sP), C::P_SLAB, tid, b, w);
        }
        run_sum = run_sum * alpha + csum;
        fence_proxy_async();
        tc_fence_before();
        __syncthreads();

        // ---- O_chunk = P V ----------------------------------------------------------------------
        if (tid == 0) {
            tc_fence_after();
#pragma unroll
            for (int kk = 0; kk < C::NKP / 16; ++kk) {
                const uint64_t a = smem_desc(smem_u32(sP + (kk >> 2) * C::P_SLAB) + (kk & 3) * 32, 16, 1024, 2u);
                const uint64_t b = smem_desc(smem_u32(sV) + kk * 16 * C::ROWB, C::KV_SLAB, C::ATOM, C::SWZ);
                umma_ss(tmem_base + C::TMEM_O, a, b, idesc_o, kk > 0);
            }
            umma_commit(bar_o);
        }
        __syncwarp();
        mbar_wait(bar_o, phase, abort_flag, kErrMmaWait);
        tc_fence_after();

        if (C::NCH > 1) {
#pragma unroll
            for (int piece = 0; piece < D / 32; ++piece) {
                uint32_t v[32];
                tmem_ld_32x32(tmem_lane + C::TMEM_O + 32 * piece, v);
                tmem_ld_wait();
#pragma unroll
                for (int e = 0; e < 32; ++e) {
                    const float x = __uint_as_float(v[e]);
                    o_acc[(C::NCH > 1 ? 32 * piece + e : 0)] =
                        (ch == 0) ? x : fmaf(o_acc[(C::NCH > 1 ? 32 * piece + e : 0)], alpha, x);
                }
            }
            tc_fence_before();
            __syncthreads();          // K, V, P and both accumulators are free for the next chunk
        }
    }

    // ---- epilogue: normalise, convert, store o and lse ---------------------------------------------
    const float inv = 1.f / run_sum;
    DT* orow = o + ((static_cast<size_t>(bn) * g.Hq + qr) * g.W + qc) * D;
#pragma unroll
    for (int piece = 0; piece < D / 32; ++piece) {
        float x[32];
        if (C::NCH > 1) {
#pragma unroll
            for (int e = 0; e < 32; ++e) x[e] = o_acc[(C::NCH > 1 ? 32 * piece + e : 0)];
        } else {
            uint32_t v[32];
            tmem_ld_32x32(tmem_lane + C::TMEM_O + 32 * piece, v);
            tmem_ld_wait();
#pragma unroll
            for (int e = 0; e < 32; ++e) x[e] = __uint_as_float(v[e]);
        }
        if (q_valid) {
#pragma unroll
            for (int gI = 0; gI < 4; ++gI) {
                uint4 pk;
                pk.x = pack2<DT>(x[8 * gI + 0] * inv, x[8 * gI + 1] * inv);
                pk.y = pack2<DT>(x[8 * gI + 2] * inv, x[8 * gI + 3] * inv);
                pk.z = pack2<DT>(x[8 * gI + 4] * inv, x[8 * gI + 5] * inv);
                pk.w = pack2<DT>(x[8 * gI + 6] * inv, x[8 * gI + 7] * inv);
                *reinterpret_cast<uint4*>(orow + 32 * piece + 8 * gI) = pk;
            }
        }
    }
    if (q_valid) lse[(static_cast<size_t>(bn) * g.Hq + qr) * g.W + qc] = (run_max + log2f(run_sum)) * kLn2;

    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        tmem_dealloc(tmem_base, C::TMEM_COLS);
    }
}

// ------------------------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    });
    return fn;
}

// Tensor map over a dense (BN, rows, W, C) tensor of 16-bit elements; the box is
// (min(C, 64) channels) x box_w x box_h x 1, swizzled so that one box row is one swizzle span.
inline int make_map(CUtensorMap* map, const void* base, int dtype, long long BN, int rows, int W, int C,
                    int box_w, int box_h) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return NA2D_ERR_CUDA;
    const int slab_c = C < 64 ? C : 64;
    cuuint64_t dims[4] = {(cuuint64_t)C, (cuuint64_t)W, (cuuint64_t)rows, (cuuint64_t)BN};
    cuuint64_t strides[3] = {(cuuint64_t)C * 2, (cuuint64_t)W * C * 2, (cuuint64_t)rows * W * C * 2};
    cuuint32_t box[4] = {(cuuint32_t)slab_c, (cuuint32_t)box_w, (cuuint32_t)box_h, 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    const CUtensorMapDataType dt = dtype == NA2D_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    const CUtensorMapSwizzle sw = slab_c * 2 == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B;
    CUresult r = fn(map, dt, 4, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? NA2D_OK : NA2D_ERR_CUDA;
}

inline bool supported(int dtype, int C, int ks) {
    if (dtype != NA2D_BF16 && dtype != NA2D_F16) return false;
    if (C != 32 && C != 64 && C != 128) return false;
    return ks == 3 || ks == 5 || ks == 7 || ks == 9 || ks == 11 || ks == 13;
}

template <typename DT, int D, int KS>
int launch_forward(const Na2dGeom& g, int dtype, const void* q, const void* k, const void* v, void* o, float* lse,
                   cudaStream_t st, int* launched) {
    using C = Cfg<D, KS>;
    CUtensorMap tq, tk, tv;
    int rc = make_map(&tq, q, dtype, g.BN, g.Hq, g.W, D, TW, TH);
    if (rc == NA2D_OK) rc = make_map(&tk, k, dtype, g.BN, g.Hkv, g.W, D, C::HW, C::RC);
    if (rc == NA2D_OK) rc = make_map(&tv, v, dtype, g.BN, g.Hkv, g.W, D, C::HW, C::RC);
    if (rc != NA2D_OK) return rc;
    const int tiles_r = (g.Hq + TH - 1) / TH, tiles_c = (g.W + TW - 1) / TW;
    const long long tiles = (long long)g.BN * tiles_r * tiles_c;
    if (tiles > 0x7fffffffLL) return NA2D_ERR_TOO_LARGE;
    auto kern = fwd_kernel<DT, D, KS>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_FWD) != cudaSuccess)
        return NA2D_ERR_CUDA;
    kern<<<(unsigned)tiles, 128, C::SMEM_FWD, st>>>(tq, tk, tv, (DT*)o, lse, g, tiles_r, tiles_c);
    *launched += 1;
    return cudaGetLastError() == cudaSuccess ? NA2D_OK : NA2D_ERR_CUDA;
}

#define NA2D_TC_DISPATCH_KS(FN, DT, DD, ...)                                  \
    switch (g.ks) {                                                           \
        case 3: return FN<DT, DD, 3>(__VA_ARGS__);                            \
        case 5: return FN<DT, DD, 5>(__VA_ARGS__);                            \
        case 7: return FN<DT, DD, 7>(__VA_ARGS__);                            \
        case 9: return FN<DT, DD, 9>(__VA_ARGS__);                            \
        case 11: return FN<DT, DD, 11>(__VA_ARGS__);                          \
        case 13: return FN<DT, DD, 13>(__VA_ARGS__);                          \
        default: return NA2D_ERR_UNSUPPORTED;                                 \
    }
#define NA2D_TC_DISPATCH_D(FN, DT, ...)                                       \
    switch (g.C) {                                                            \
        case 32: NA2D_TC_DISPATCH_KS(FN, DT, 32, __VA_ARGS__)                 \
        case 64: NA2D_TC_DISPATCH_KS(FN, DT, 64, __VA_ARGS__)                 \
        case 128: NA2D_TC_DISPATCH_KS(FN, DT, 128, __VA_ARGS__)               \
        default: return NA2D_ERR_UNSUPPORTED;                                 \
    }

inline int forward(const Na2dGeom& g, int dtype, const void* q, const void* k, const void* v, void* o, float* lse,
                   int /*device*/, cudaStream_t st, int* launched) {
    if (dtype == NA2D_BF16) {
        NA2D_TC_DISPATCH_D(launch_forward, __nv_bfloat16, g, dtype, q, k, v, o, lse, st, launched)
    } else {
        NA2D_TC_DISPATCH_D(launch_forward, __half, g, dtype, q, k, v, o, lse, st, launched)
    }
}

}  // namespace na2d_tc

#include "na2d_tc_bwd.cuh"

namespace na2d_tc {

inline int read_and_clear_error(unsigned int* word, cudaStream_t st) {
    if (cudaMemcpyFromSymbolAsync(word, g_error_word, sizeof(unsigned int), 0, cudaMemcpyDeviceToHost, st) != cudaSuccess)
        return NA2D_ERR_CUDA;
    if (cudaStreamSynchronize(st) != cudaSuccess) return NA2D_ERR_CUDA;
    if (*word != 0) {
        unsigned int zero = 0;
        if (cudaMemcpyToSymbolAsync(g_error_word, &zero, sizeof(unsigned int), 0, cudaMemcpyHostToDevice, st) != cudaSuccess)
            return NA2D_ERR_CUDA;
        if (cudaStreamSynchronize(st) != cudaSuccess) return NA2D_ERR_CUDA;
    }
    return NA2D_OK;
}

}  // namespace na2d_tc
