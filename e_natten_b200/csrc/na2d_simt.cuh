// SIMT (CUDA-core) kernels for 2D neighborhood attention: forward, dQ, dK/dV.
//
// One warp per query pixel (forward, dQ) or per key pixel (dK/dV); all accumulation in fp32.
// These kernels serve the fp32 path (tensor cores cannot hold 1e-4 relative error), head dims
// and kernel sizes the tensor-core kernels are not built for, and they are the device-side
// second opinion for shapes the CPU oracle cannot finish.  They are bounds-safe for every
// grid size and use no atomics, so results are bit-stable from run to run.
//
// Math (what e_natten/triton.py:278-291 and 383-423 compute, the backward in flash form):
//   s_j = q . k_j,  lse = max_j s_j + log sum_j exp(s_j - max),  p_j = exp(s_j - lse),
//   o = sum_j p_j v_j;   dp_j = dO . v_j,  delta = sum_j p_j dp_j (= dO . o),  ds_j = p_j (dp_j - delta),
//   dQ = sum_j ds_j k_j,  dK_j += ds_j q,  dV_j += p_j dO   (+= over the inverse neighbourhood).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <math_constants.h>

#include "na2d_index.cuh"

namespace na2d_simt {

constexpr int kWarps = 4;          // warps per block
constexpr int kMaxC = 256;         // head dim limit of the SIMT path
constexpr int kMaxKs = 31;         // kernel size limit of the SIMT path
constexpr int kMaxCPerLane = kMaxC / 32;

template <typename T> __device__ __forceinline__ float to_f(T x);
template <> __device__ __forceinline__ float to_f<float>(float x) { return x; }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }
template <> __device__ __forceinline__ float to_f<__half>(__half x) { return __half2float(x); }

template <typename T> __device__ __forceinline__ T from_f(float x);
template <> __device__ __forceinline__ float from_f<float>(float x) { return x; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }
template <> __device__ __forceinline__ __half from_f<__half>(float x) { return __float2half_rn(x); }

__device__ __forceinline__ float warp_max(float x) {
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, d));
    return x;
}
__device__ __forceinline__ float warp_sum(float x) {
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) x += __shfl_xor_sync(0xffffffffu, x, d);
    return x;
}

// Dynamic shared memory per block, in bytes.
inline size_t fwd_smem_bytes(int C, int ks) { return (size_t)kWarps * (C + ks * ks) * sizeof(float); }
inline size_t dq_smem_bytes(int C, int ks) { return (size_t)kWarps * (2 * C + 2 * ks * ks) * sizeof(float); }
inline size_t dkdv_smem_bytes(int C) { return (size_t)kWarps * (2 * C + 64) * sizeof(float); }

// ------------------------------------------------------------------------------------ forward
template <typename T>
__global__ void __launch_bounds__(kWarps * 32)
fwd_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
           T* __restrict__ o, float* __restrict__ lse, Na2dGeom g) {
    extern __shared__ float smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nk = g.ks * g.ks;
    float* qs = smem + warp * (g.C + nk);
    float* ss = qs + g.C;
    const long long n_query = (long long)g.BN * g.Hq * g.W;
    const long long qi = (long long)blockIdx.x * kWarps + warp;
    if (qi >= n_query) return;                       // warp-uniform; no block barrier follows
    const int y = (int)(qi % g.W);
    const int xl = (int)((qi / g.W) % g.Hq);
    const long long bn = qi / ((long long)g.W * g.Hq);
    const int ox = na2d_ws(g.q_row0 + xl, g.Hg, g.ks) - g.kv_row0;
    const int oy = na2d_ws(y, g.W, g.ks);

    const T* qrow = q + qi * g.C;
    for (int c = lane; c < g.C; c += 32) qs[c] = to_f<T>(qrow[c]);
    __syncwarp();

    const T* kb = k + bn * g.Hkv * g.W * g.C;
    const T* vb = v + bn * g.Hkv * g.W * g.C;
    float m = -CUDART_INF_F;
    for (int j = lane; j < nk; j += 32) {
        const int u = j / g.ks, w = j - u * g.ks;
        const T* kr = kb + ((long long)(ox + u) * g.W + (oy + w)) * g.C;
        float s = 0.f;
        for (int c = 0; c < g.C; ++c) s = fmaf(qs[c], to_f<T>(kr[c]), s);
        ss[j] = s;
        m = fmaxf(m, s);
    }
    m = warp_max(m);
    float l = 0.f;
    for (int j = lane; j < nk; j += 32) {
        const float e = expf(ss[j] - m);
        ss[j] = e;
        l += e;
    }
    l = warp_sum(l);
    __syncwarp();
    const float inv = 1.f / l;
    for (int c = lane; c < g.C; c += 32) {
        float acc = 0.f;
        int j = 0;
        for (int u = 0; u < g.ks; ++u) {
            const T* vr = vb + ((long long)(ox + u) * g.W + oy) * g.C + c;
            for (int w = 0; w < g.ks; ++w, ++j) acc = fmaf(ss[j], to_f<T>(vr[(long long)w * g.C]), acc);
        }
        o[qi * g.C + c] = from_f<T>(acc * inv);
    }
    if (lane == 0) lse[qi] = m + logf(l);
}

// ------------------------------------------------------------------------------------ dQ (+ delta)
// delta = sum_j p_j dp_j, which equals dO . o exactly and does not depend on how o was rounded
// when it was stored (the reference's backward does not read o either, e_natten/triton.py:522).
// d_q may be null: then only delta is produced.
template <typename T>
__global__ void __launch_bounds__(kWarps * 32)
dq_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
          const float* __restrict__ lse, const T* __restrict__ d_o,
          T* __restrict__ d_q, float* __restrict__ delta, Na2dGeom g) {
    extern __shared__ float smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nk = g.ks * g.ks;
    float* qs = smem + warp * (2 * g.C + 2 * nk);
    float* gs = qs + g.C;            // dO row
    float* ps = gs + g.C;            // p per window member, then dS
    float* dps = ps + nk;            // dP per window member
    const long long n_query = (long long)g.BN * g.Hq * g.W;
    const long long qi = (long long)blockIdx.x * kWarps + warp;
    if (qi >= n_query) return;
    const int y = (int)(qi % g.W);
    const int xl = (int)((qi / g.W) % g.Hq);
    const long long bn = qi / ((long long)g.W * g.Hq);
    const int ox = na2d_ws(g.q_row0 + xl, g.Hg, g.ks) - g.kv_row0;
    const int oy = na2d_ws(y, g.W, g.ks);

    for (int c = lane; c < g.C; c += 32) {
        qs[c] = to_f<T>(q[qi * g.C + c]);
        gs[c] = to_f<T>(d_o[qi * g.C + c]);
    }
    __syncwarp();

    const float row_lse = lse[qi];
    const T* kb = k + bn * g.Hkv * g.W * g.C;
    const T* vb = v + bn * g.Hkv * g.W * g.C;
    float dl = 0.f;
    for (int j = lane; j < nk; j += 32) {
        const int u = j / g.ks, w = j - u * g.ks;
        const long long off = ((long long)(ox + u) * g.W + (oy + w)) * g.C;
        const T* kr = kb + off;
        const T* vr = vb + off;
        float s = 0.f, dp = 0.f;
        for (int c = 0; c < g.C; ++c) {
            s = fmaf(qs[c], to_f<T>(kr[c]), s);
            dp = fmaf(gs[c], to_f<T>(vr[c]), dp);
        }
        const float p = expf(s - row_lse);
        ps[j] = p;
        dps[j] = dp;
        dl = fmaf(p, dp, dl);
    }
    dl = warp_sum(dl);
    if (lane == 0) delta[qi] = dl;
    if (d_q == nullptr) return;
    for (int j = lane; j < nk; j += 32) ps[j] = ps[j] * (dps[j] - dl);
    __syncwarp();
    for (int c = lane; c < g.C; c += 32) {
        float acc = 0.f;
        int j = 0;
        for (int u = 0; u < g.ks; ++u) {
            const T* kr = kb + ((long long)(ox + u) * g.W + oy) * g.C + c;
            for (int w = 0; w < g.ks; ++w, ++j) acc = fmaf(ps[j], to_f<T>(kr[(long long)w * g.C]), acc);
        }
        d_q[qi * g.C + c] = from_f<T>(acc);
    }
}

// ------------------------------------------------------------------------------------ dK, dV
// One warp per key pixel of the key band; sums over the queries of the local query band whose
// window holds the key (the inverse neighbourhood, a product of two index ranges).
template <typename T>
__global__ void __launch_bounds__(kWarps * 32)
dkdv_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
            const float* __restrict__ lse, const T* __restrict__ d_o, const float* __restrict__ delta,
            T* __restrict__ d_k, T* __restrict__ d_v, Na2dGeom g) {
    extern __shared__ float smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float* ks_ = smem + warp * (2 * g.C + 64);
    float* vs_ = ks_ + g.C;
    float* ps = vs_ + g.C;           // 32 probabilities of the current round
    float* dss = ps + 32;            // 32 dS of the current round
    const long long n_key = (long long)g.BN * g.Hkv * g.W;
    const long long ki = (long long)blockIdx.x * kWarps + warp;
    if (ki >= n_key) return;
    const int y = (int)(ki % g.W);
    const int xl = (int)((ki / g.W) % g.Hkv);
    const long long bn = ki / ((long long)g.W * g.Hkv);
    const int xg = g.kv_row0 + xl;

    for (int c = lane; c < g.C; c += 32) {
        ks_[c] = to_f<T>(k[ki * g.C + c]);
        vs_[c] = to_f<T>(v[ki * g.C + c]);
    }
    __syncwarp();

    // inverse neighbourhood, rows clipped to the local query band
    int r0 = na2d_bws(xg, g.ks), r1 = na2d_bwe(xg, g.Hg, g.ks);
    r0 = max(r0, g.q_row0);
    r1 = min(r1, g.q_row0 + g.Hq);
    const int c0 = na2d_bws(y, g.ks), c1 = na2d_bwe(y, g.W, g.ks);
    const int nr = max(r1 - r0, 0), nc = c1 - c0;
    const int n_in = nr * nc;

    float acc_k[kMaxCPerLane], acc_v[kMaxCPerLane];
#pragma unroll
    for (int i = 0; i < kMaxCPerLane; ++i) { acc_k[i] = 0.f; acc_v[i] = 0.f; }

    const long long qbase = bn * g.Hq * g.W;
    for (int base = 0; base < n_in; base += 32) {
        const int t = base + lane;
        float p = 0.f, dsv = 0.f;
        if (t < n_in) {
            const int rr = t / nc, cc = t - rr * nc;
            const long long qi = qbase + (long long)(r0 + rr - g.q_row0) * g.W + (c0 + cc);
            const T* qr = q + qi * g.C;
            const T* gr = d_o + qi * g.C;
            float s = 0.f, dp = 0.f;
            for (int c = 0; c < g.C; ++c) {
                s = fmaf(to_f<T>(qr[c]), ks_[c], s);
                dp = fmaf(to_f<T>(gr[c]), vs_[c], dp);
            }
            p = expf(s - lse[qi]);
            dsv = p * (dp - delta[qi]);
        }
        ps[lane] = p;
        dss[lane] = dsv;
        __syncwarp();
        const int n_round = min(32, n_in - base);
        for (int i = 0; i < n_round; ++i) {
            const int tt = base + i;
            const int rr = tt / nc, cc = tt - rr * nc;
            const long long qi = qbase + (long long)(r0 + rr - g.q_row0) * g.W + (c0 + cc);
            const float pi = ps[i], dsi = dss[i];
#pragma unroll
            for (int e = 0; e < kMaxCPerLane; ++e) {
                const int c = lane + 32 * e;
                if (c < g.C) {
                    acc_k[e] = fmaf(dsi, to_f<T>(q[qi * g.C + c]), acc_k[e]);
                    acc_v[e] = fmaf(pi, to_f<T>(d_o[qi * g.C + c]), acc_v[e]);
                }
            }
        }
        __syncwarp();
    }
#pragma unroll
    for (int e = 0; e < kMaxCPerLane; ++e) {
        const int c = lane + 32 * e;
        if (c < g.C) {
            d_k[ki * g.C + c] = from_f<T>(acc_k[e]);
            d_v[ki * g.C + c] = from_f<T>(acc_v[e]);
        }
    }
}

// Device evaluation of the index functions, for the bit-exact indexing test.
__global__ void index_dump_kernel(int* ws, int* bws, int* bwe, int seq_len, int ks) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < seq_len) {
        ws[i] = na2d_ws(i, seq_len, ks);
        bws[i] = na2d_bws(i, ks);
        bwe[i] = na2d_bwe(i, seq_len, ks);
    }
}

}  // namespace na2d_simt
