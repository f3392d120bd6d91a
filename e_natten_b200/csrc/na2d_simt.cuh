// SIMT (CUDA-core) kernels for neighborhood attention: fused forward, dQ, dK/dV, and the unfused
// pair (scores / apply) with their backward halves.
//
// One warp per query pixel (forward, dQ, scores, apply) or per key pixel (dK/dV and the key-side
// halves of the unfused backward).  The lanes of a warp split the CHANNELS of a pixel (lane l holds
// channels l, l + 32, ...), so every row of q, k, v, dO that a warp touches is read with coalesced
// loads; the dot products of a pixel's row with 32 neighbour rows are brought together with a
// transposing butterfly (31 shuffles for 32 sums, the m-th sum landing in lane m).  All
// accumulation is fp32.  The window is kh x kw: ks x ks for the 2D operator, 1 x ks for the 1D
// operator on a (B, N, 1, T, C) view, so one set of kernels serves both.
//
// These kernels are the fp32 path (tensor cores cannot hold 1e-4 relative error), the path for
// head dims and kernel sizes the tensor-core kernels are not built for, the 1D operator, and the
// device-side second opinion for shapes the CPU oracle cannot finish.  They are bounds-safe for
// every grid size and use no atomics, so results are bit-stable from run to run.
//
// A block of eight warps works through a compact patch of 64 pixels (8 x 8, or 1 x 64 for a
// one-row image), warp w taking pixels w, w + 8, ...: neighbouring pixels share most of their
// window rows, and a patch keeps those rows in the SM's L1 instead of fetching each of them from
// L2 once per pixel.
//
// Math (what e_natten/triton.py:278-291 and 383-423 compute, the backward in flash form):
//   s_j = scale * q . k_j,  lse = max_j s_j + log sum_j exp(s_j - max),  p_j = exp(s_j - lse),
//   o = sum_j p_j v_j;   dp_j = dO . v_j,  delta = sum_j p_j dp_j (= dO . o),
//   ds_j = scale * p_j (dp_j - delta),  dQ = sum_j ds_j k_j,  dK_j += ds_j q,  dV_j += p_j dO
//   (+= over the inverse neighbourhood).  The reference applies no scale (scale = 1).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <math_constants.h>

#include "na2d_index.cuh"

namespace na2d_simt {

constexpr int kWarps = 8;          // warps per block
constexpr int kPatch = 64;         // pixels per block (8 per warp); kPatchSmall where that leaves most SMs empty
constexpr int kPatchSmall = 8;     // one pixel per warp
constexpr int kMaxC = 256;         // head dim limit of the SIMT path
constexpr int kMaxKs = 31;         // kernel size limit of the SIMT path

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

// Sums each of 32 per-lane values over the warp; the sum of v[m] ends in lane m (returned).
// Step `off` halves the live values: a lane keeps the half its bit `off` selects and adds what
// its partner sends of the same half.
__device__ __forceinline__ float transpose_sum32(float (&v)[32], int lane) {
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) {
        const bool upper = (lane & off) != 0;
#pragma unroll
        for (int i = 0; i < off; ++i) {
            const float keep = upper ? v[i + off] : v[i];
            const float send = upper ? v[i] : v[i + off];
            v[i] = keep + __shfl_xor_sync(0xffffffffu, send, off);
        }
    }
    return v[0];
}

// Patches of a (BN, H, W) pixel grid: 8 x 8 pixels (2 x 4 for the small patch), or one row of
// `patch` pixels for a one-row image.
__host__ __device__ __forceinline__ int patch_h(int H, int patch) { return H == 1 ? 1 : (patch == kPatch ? 8 : 2); }
__host__ __device__ __forceinline__ int patch_w(int H, int patch) { return patch / patch_h(H, patch); }
inline long long patch_count(long long BN, int H, int W, int patch) {
    const int ph = patch_h(H, patch), pw = patch_w(H, patch);
    return BN * ((H + ph - 1) / ph) * ((W + pw - 1) / pw);
}

// A pixel's coordinates and its index in the dense (BN, H, W) arrays (lse, delta, attn).
struct Pixel {
    long long bn, idx;
    int b, n, h, w;
};
// Pixel t of the block's patch; false if it lies outside the grid.
__device__ __forceinline__ bool patch_pixel(Pixel& p, int t, int H, int W, int N, int patch) {
    const int ph = patch_h(H, patch), pw = patch_w(H, patch);
    const int tiles_w = (W + pw - 1) / pw, tiles_h = (H + ph - 1) / ph;
    long long blk = blockIdx.x;
    const int tw = (int)(blk % tiles_w);
    blk /= tiles_w;
    const int th = (int)(blk % tiles_h);
    p.bn = blk / tiles_h;
    p.h = th * ph + t / pw;
    p.w = tw * pw + t % pw;
    p.b = (int)(p.bn / N);
    p.n = (int)(p.bn - (long long)p.b * N);
    p.idx = (p.bn * H + p.h) * W + p.w;
    return p.h < H && p.w < W;
}
__device__ __forceinline__ long long offset_of(const Na2dStride& s, int b, int n, int h, int w) {
    return b * s.b + n * s.n + h * s.h + w * s.w;
}

// Lane l's channels of one pixel row: x[e] = row[l + 32 e] (0 beyond C).
template <typename T, int CPL>
__device__ __forceinline__ void load_row(float (&x)[CPL], const T* row, int C, int lane) {
#pragma unroll
    for (int e = 0; e < CPL; ++e) {
        const int c = lane + 32 * e;
        x[e] = c < C ? to_f<T>(row[c]) : 0.f;
    }
}

// Dot products of x with the rows of up to 32 window members j0 .. j0 + 31 (member j sits at
// window row j / kw, window column j % kw of a window whose first pixel is `origin`); the m-th
// product ends in lane m.  Members >= nk give 0.
template <typename T, int CPL>
__device__ __forceinline__ float dot_members32(const float (&x)[CPL], const T* origin, long long sh, long long sw,
                                               int kw, int j0, int nk, int C, int lane) {
    float part[32];
    int u = j0 / kw, w = j0 - u * kw;
#pragma unroll
    for (int m = 0; m < 32; ++m) {
        float acc = 0.f;
        if (j0 + m < nk) {                                       // warp-uniform
            const T* row = origin + u * sh + w * sw;
#pragma unroll
            for (int e = 0; e < CPL; ++e) {
                const int c = lane + 32 * e;
                if (c < C) acc = fmaf(x[e], to_f<T>(row[c]), acc);
            }
        }
        part[m] = acc;
        if (++w == kw) { w = 0; ++u; }
    }
    return transpose_sum32(part, lane);
}

// acc[e] += sum_j weight[j] * row_j[lane + 32 e] over all nk members of the window at `origin`;
// the weights are read from shared memory (a broadcast).
template <typename T, int CPL>
__device__ __forceinline__ void add_weighted_rows(float (&acc)[CPL], const float* weight, const T* origin, long long sh,
                                                  long long sw, int kh, int kw, int C, int lane) {
    int j = 0;
    for (int u = 0; u < kh; ++u) {
        const T* row = origin + u * sh;
        for (int w = 0; w < kw; ++w, ++j, row += sw) {
            const float wt = weight[j];
#pragma unroll
            for (int e = 0; e < CPL; ++e) {
                const int c = lane + 32 * e;
                if (c < C) acc[e] = fmaf(wt, to_f<T>(row[c]), acc[e]);
            }
        }
    }
}

template <typename T, int CPL>
__device__ __forceinline__ void store_row(T* row, const float (&x)[CPL], float scale, int C, int lane) {
#pragma unroll
    for (int e = 0; e < CPL; ++e) {
        const int c = lane + 32 * e;
        if (c < C) row[c] = from_f<T>(x[e] * scale);
    }
}

// Dynamic shared memory per block, in bytes: per warp the window's weights (and a second set
// for the dQ kernel).
inline size_t window_smem_bytes(int kh, int kw, int sets) { return (size_t)kWarps * sets * kh * kw * sizeof(float); }

// ------------------------------------------------------------------------------------ forward
template <typename T, int CPL>
__global__ void __launch_bounds__(kWarps * 32)
fwd_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v, T* __restrict__ o,
           float* __restrict__ lse, const Na2dStride sq, const Na2dStride sk, const Na2dStride sv, const Na2dStride so,
           const Na2dGeom g) {
    extern __shared__ float smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int kh = g.kh, kw = g.ks, nk = kh * kw;
    float* ss = smem + warp * nk;
    for (int t = warp; t < g.patch; t += kWarps) {
    Pixel px;
    if (!patch_pixel(px, t, g.Hq, g.W, g.N, g.patch)) continue;          // warp-uniform; no block barrier anywhere
    const long long qi = px.idx;
    const int oh = na2d_ws(g.q_row0 + px.h, g.Hg, kh) - g.kv_row0;
    const int ow = na2d_ws(px.w, g.W, kw);

    float x[CPL];
    load_row<T, CPL>(x, q + offset_of(sq, px.b, px.n, px.h, px.w), g.C, lane);
    const T* k0 = k + offset_of(sk, px.b, px.n, oh, ow);
    float m = -CUDART_INF_F;
    for (int j0 = 0; j0 < nk; j0 += 32) {
        const float s = dot_members32<T, CPL>(x, k0, sk.h, sk.w, kw, j0, nk, g.C, lane) * g.scale;
        if (j0 + lane < nk) {
            ss[j0 + lane] = s;
            m = fmaxf(m, s);
        }
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
    float acc[CPL];
#pragma unroll
    for (int e = 0; e < CPL; ++e) acc[e] = 0.f;
    add_weighted_rows<T, CPL>(acc, ss, v + offset_of(sv, px.b, px.n, oh, ow), sv.h, sv.w, kh, kw, g.C, lane);
    store_row<T, CPL>(o + offset_of(so, px.b, px.n, px.h, px.w), acc, 1.f / l, g.C, lane);
    if (lane == 0) lse[qi] = m + logf(l);
    __syncwarp();                                               // ss is reused by the warp's next pixel
    }
}

// ------------------------------------------------------------------------------------ dQ (+ delta)
// delta = sum_j p_j dp_j, which equals dO . o exactly and does not depend on how o was rounded
// when it was stored (the reference's backward does not read o either, e_natten/triton.py:522).
// d_q may be null: then only delta is produced.
template <typename T, int CPL>
__global__ void __launch_bounds__(kWarps * 32, 2)
dq_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v, const float* __restrict__ lse,
          const T* __restrict__ d_o, T* __restrict__ d_q, float* __restrict__ delta, const Na2dStride sq,
          const Na2dStride sk, const Na2dStride sv, const Na2dStride sg, const Na2dStride sdq, const Na2dGeom g) {
    extern __shared__ float smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int kh = g.kh, kw = g.ks, nk = kh * kw;
    float* ps = smem + warp * 2 * nk;          // p per window member, then dS
    float* dps = ps + nk;                      // dP per window member
    for (int t = warp; t < g.patch; t += kWarps) {
    Pixel px;
    if (!patch_pixel(px, t, g.Hq, g.W, g.N, g.patch)) continue;
    const long long qi = px.idx;
    const int oh = na2d_ws(g.q_row0 + px.h, g.Hg, kh) - g.kv_row0;
    const int ow = na2d_ws(px.w, g.W, kw);

    float x[CPL], gx[CPL];
    load_row<T, CPL>(x, q + offset_of(sq, px.b, px.n, px.h, px.w), g.C, lane);
    load_row<T, CPL>(gx, d_o + offset_of(sg, px.b, px.n, px.h, px.w), g.C, lane);
    const T* k0 = k + offset_of(sk, px.b, px.n, oh, ow);
    const T* v0 = v + offset_of(sv, px.b, px.n, oh, ow);
    const float row_lse = lse[qi];
    float dl = 0.f;
    for (int j0 = 0; j0 < nk; j0 += 32) {
        const float s = dot_members32<T, CPL>(x, k0, sk.h, sk.w, kw, j0, nk, g.C, lane) * g.scale;
        const float dp = dot_members32<T, CPL>(gx, v0, sv.h, sv.w, kw, j0, nk, g.C, lane);
        if (j0 + lane < nk) {
            const float p = expf(s - row_lse);
            ps[j0 + lane] = p;
            dps[j0 + lane] = dp;
            dl = fmaf(p, dp, dl);
        }
    }
    dl = warp_sum(dl);
    if (lane == 0) delta[qi] = dl;
    if (d_q != nullptr) {
        for (int j = lane; j < nk; j += 32) ps[j] = g.scale * ps[j] * (dps[j] - dl);
        __syncwarp();
        float acc[CPL];
#pragma unroll
        for (int e = 0; e < CPL; ++e) acc[e] = 0.f;
        add_weighted_rows<T, CPL>(acc, ps, k0, sk.h, sk.w, kh, kw, g.C, lane);
        store_row<T, CPL>(d_q + offset_of(sdq, px.b, px.n, px.h, px.w), acc, 1.f, g.C, lane);
    }
    __syncwarp();                                               // ps / dps are reused by the warp's next pixel
    }
}

// The queries whose window holds key (kh_, kw_): rows [r0, r0 + nr) of the local query band,
// columns [c0, c0 + nc).
struct Inverse {
    int r0, nr, c0, nc;
};
__device__ __forceinline__ Inverse inverse_neighbourhood(int key_row_global, int key_col, const Na2dGeom& g) {
    Inverse iv;
    int r0 = na2d_bws(key_row_global, g.kh), r1 = na2d_bwe(key_row_global, g.Hg, g.kh);
    r0 = max(r0, g.q_row0);
    r1 = min(r1, g.q_row0 + g.Hq);
    iv.r0 = r0;
    iv.nr = max(r1 - r0, 0);
    iv.c0 = na2d_bws(key_col, g.ks);
    iv.nc = na2d_bwe(key_col, g.W, g.ks) - iv.c0;
    return iv;
}

// ------------------------------------------------------------------------------------ dK, dV
// One warp per key pixel of the key band; sums over the queries of the local query band whose
// window holds the key (the inverse neighbourhood, a product of two index ranges), 32 at a time.
template <typename T, int CPL>
__global__ void __launch_bounds__(kWarps * 32, 2)
dkdv_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v, const float* __restrict__ lse,
            const T* __restrict__ d_o, const float* __restrict__ delta, void* __restrict__ d_k, void* __restrict__ d_v,
            const int f32_out, const Na2dStride sq, const Na2dStride sk, const Na2dStride sv, const Na2dStride sg,
            const Na2dStride sdk, const Na2dStride sdv, const Na2dGeom g) {
    __shared__ float s_p[kWarps][32], s_ds[kWarps][32];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int t = warp; t < g.patch; t += kWarps) {
    Pixel px;
    if (!patch_pixel(px, t, g.Hkv, g.W, g.N, g.patch)) continue;
    const Inverse iv = inverse_neighbourhood(g.kv_row0 + px.h, px.w, g);
    const int n_in = iv.nr * iv.nc;

    float kx[CPL], vx[CPL], acc_k[CPL], acc_v[CPL];
    load_row<T, CPL>(kx, k + offset_of(sk, px.b, px.n, px.h, px.w), g.C, lane);
    load_row<T, CPL>(vx, v + offset_of(sv, px.b, px.n, px.h, px.w), g.C, lane);
#pragma unroll
    for (int e = 0; e < CPL; ++e) { acc_k[e] = 0.f; acc_v[e] = 0.f; }

    const int qh0 = iv.r0 - g.q_row0;                            // local row of the first query row
    const T* q0 = q + offset_of(sq, px.b, px.n, qh0, iv.c0);
    const T* g0 = d_o + offset_of(sg, px.b, px.n, qh0, iv.c0);
    const long long stat0 = (px.bn * g.Hq + qh0) * g.W + iv.c0;  // index of that query in lse / delta
    for (int j0 = 0; j0 < n_in; j0 += 32) {
        const float s = dot_members32<T, CPL>(kx, q0, sq.h, sq.w, iv.nc, j0, n_in, g.C, lane) * g.scale;
        const float dp = dot_members32<T, CPL>(vx, g0, sg.h, sg.w, iv.nc, j0, n_in, g.C, lane);
        float p = 0.f, ds = 0.f;
        if (j0 + lane < n_in) {
            const int rr = (j0 + lane) / iv.nc, cc = (j0 + lane) - rr * iv.nc;
            const long long si = stat0 + (long long)rr * g.W + cc;
            p = expf(s - lse[si]);
            ds = g.scale * p * (dp - delta[si]);
        }
        s_p[warp][lane] = p;
        s_ds[warp][lane] = ds;
        __syncwarp();
        const int n_round = min(32, n_in - j0);
        int rr = j0 / iv.nc, cc = j0 - rr * iv.nc;
        for (int i = 0; i < n_round; ++i) {
            const T* qr = q0 + rr * sq.h + cc * sq.w;
            const T* gr = g0 + rr * sg.h + cc * sg.w;
            const float pi = s_p[warp][i], dsi = s_ds[warp][i];
#pragma unroll
            for (int e = 0; e < CPL; ++e) {
                const int c = lane + 32 * e;
                if (c < g.C) {
                    acc_k[e] = fmaf(dsi, to_f<T>(qr[c]), acc_k[e]);
                    acc_v[e] = fmaf(pi, to_f<T>(gr[c]), acc_v[e]);
                }
            }
            if (++cc == iv.nc) { cc = 0; ++rr; }
        }
        __syncwarp();
    }
    if (f32_out) {          // partial sums of a row band, kept in fp32 for their owner to add up
        store_row<float, CPL>(static_cast<float*>(d_k) + offset_of(sdk, px.b, px.n, px.h, px.w), acc_k, 1.f, g.C, lane);
        store_row<float, CPL>(static_cast<float*>(d_v) + offset_of(sdv, px.b, px.n, px.h, px.w), acc_v, 1.f, g.C, lane);
    } else {
        store_row<T, CPL>(static_cast<T*>(d_k) + offset_of(sdk, px.b, px.n, px.h, px.w), acc_k, 1.f, g.C, lane);
        store_row<T, CPL>(static_cast<T*>(d_v) + offset_of(sdv, px.b, px.n, px.h, px.w), acc_v, 1.f, g.C, lane);
    }
    }
}

// ------------------------------------------------------------------------------------ unfused pair
// The two-step form the reference compares itself with (test.py:17-21, bench.py:23, 52-54):
//   scores   attn[b,n,h,w,j] = q[b,n,h,w,:] . k[b,n,window member j,:]      (B, N, H, W, kh*kw)
//   apply    out[b,n,h,w,:]  = sum_j attn[b,n,h,w,j] * v[b,n,window member j,:]
// with the same clamped windows, member j at window row j / kw, column j % kw.  The softmax between
// them is the caller's.  All tensors are dense here.

// rows(x) . rows(y over the window) -> attn: serves scores (x = q, y = k) and the attn-gradient
// of apply (x = dO, y = v).
template <typename T, int CPL>
__global__ void __launch_bounds__(kWarps * 32)
window_dot_kernel(const T* __restrict__ x, const T* __restrict__ y, T* __restrict__ attn, const Na2dStride sx,
                  const Na2dStride sy, const Na2dGeom g) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int kh = g.kh, kw = g.ks, nk = kh * kw;
    for (int t = warp; t < g.patch; t += kWarps) {
    Pixel px;
    if (!patch_pixel(px, t, g.Hq, g.W, g.N, g.patch)) continue;
    const long long qi = px.idx;
    const int oh = na2d_ws(g.q_row0 + px.h, g.Hg, kh) - g.kv_row0;
    const int ow = na2d_ws(px.w, g.W, kw);
    float xr[CPL];
    load_row<T, CPL>(xr, x + offset_of(sx, px.b, px.n, px.h, px.w), g.C, lane);
    const T* y0 = y + offset_of(sy, px.b, px.n, oh, ow);
    for (int j0 = 0; j0 < nk; j0 += 32) {
        const float s = dot_members32<T, CPL>(xr, y0, sy.h, sy.w, kw, j0, nk, g.C, lane);
        if (j0 + lane < nk) attn[qi * nk + j0 + lane] = from_f<T>(s);
    }
    }
}

// out = sum_j attn[., j] * rows(y over the window): serves apply (y = v) and the q-gradient of
// scores (attn = d_attn, y = k).
template <typename T, int CPL>
__global__ void __launch_bounds__(kWarps * 32)
window_apply_kernel(const T* __restrict__ attn, const T* __restrict__ y, T* __restrict__ out, const Na2dStride sy,
                    const Na2dStride so, const Na2dGeom g) {
    extern __shared__ float smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int kh = g.kh, kw = g.ks, nk = kh * kw;
    float* ws = smem + warp * nk;
    for (int t = warp; t < g.patch; t += kWarps) {
    Pixel px;
    if (!patch_pixel(px, t, g.Hq, g.W, g.N, g.patch)) continue;
    const long long qi = px.idx;
    const int oh = na2d_ws(g.q_row0 + px.h, g.Hg, kh) - g.kv_row0;
    const int ow = na2d_ws(px.w, g.W, kw);
    for (int j = lane; j < nk; j += 32) ws[j] = to_f<T>(attn[qi * nk + j]);
    __syncwarp();
    float acc[CPL];
#pragma unroll
    for (int e = 0; e < CPL; ++e) acc[e] = 0.f;
    add_weighted_rows<T, CPL>(acc, ws, y + offset_of(sy, px.b, px.n, oh, ow), sy.h, sy.w, kh, kw, g.C, lane);
    store_row<T, CPL>(out + offset_of(so, px.b, px.n, px.h, px.w), acc, 1.f, g.C, lane);
    __syncwarp();                                               // ws is reused by the warp's next pixel
    }
}

// Key-side gradient of either step: out[key] = sum over the queries i whose window holds the key
// of attn[i, position of the key in i's window] * x[i]: dK of scores (attn = d_attn, x = q) and
// dV of apply (attn = attn, x = dO).
template <typename T, int CPL>
__global__ void __launch_bounds__(kWarps * 32)
window_inverse_kernel(const T* __restrict__ attn, const T* __restrict__ x, T* __restrict__ out, const Na2dStride sx,
                      const Na2dStride so, const Na2dGeom g) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int kh = g.kh, kw = g.ks, nk = kh * kw;
    for (int t = warp; t < g.patch; t += kWarps) {
    Pixel px;
    if (!patch_pixel(px, t, g.Hkv, g.W, g.N, g.patch)) continue;
    const int key_row = g.kv_row0 + px.h;
    const Inverse iv = inverse_neighbourhood(key_row, px.w, g);
    float acc[CPL];
#pragma unroll
    for (int e = 0; e < CPL; ++e) acc[e] = 0.f;
    for (int rr = 0; rr < iv.nr; ++rr) {
        const int qh = iv.r0 + rr;                                         // global query row
        const int u = key_row - na2d_ws(qh, g.Hg, kh);                     // key's row inside that query's window
        for (int cc = 0; cc < iv.nc; ++cc) {
            const int qw = iv.c0 + cc;
            const int w = px.w - na2d_ws(qw, g.W, kw);
            const long long qi = (px.bn * g.Hq + (qh - g.q_row0)) * g.W + qw;
            const float a = to_f<T>(attn[qi * nk + u * kw + w]);
            const T* row = x + offset_of(sx, px.b, px.n, qh - g.q_row0, qw);
#pragma unroll
            for (int e = 0; e < CPL; ++e) {
                const int c = lane + 32 * e;
                if (c < g.C) acc[e] = fmaf(a, to_f<T>(row[c]), acc[e]);
            }
        }
    }
    store_row<T, CPL>(out + offset_of(so, px.b, px.n, px.h, px.w), acc, 1.f, g.C, lane);
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
