// An estimate of the backward's row delta, formed ahead of the dQ kernel: dO . o per query, where
// o is the forward's output as it was stored (16 bit).  The exact delta is sum_j p_j dP_j; dO . o
// differs from it by what o lost to rounding (P went into the forward's second MMA in 16 bits,
// and o was rounded when stored), a few 1e-2 at most.  That is too coarse to form dS from directly
// - the error would enter every dS of the row - but it is all the dQ kernel of the larger windows
// needs to walk its key box once instead of twice: it forms dS from the estimate and corrects
// the result exactly at the end (see na2d_tc_bwd.cuh).
//
// One warp per query pixel, lanes over channels; plain coalesced loads, an HBM-bound pass over
// two tensors.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "na2d_index.cuh"

namespace na2d_delta {

constexpr int kWarps = 8;

template <typename T> __device__ __forceinline__ float2 to_f2(uint32_t w);
template <> __device__ __forceinline__ float2 to_f2<__nv_bfloat16>(uint32_t w) {
    return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
}
template <> __device__ __forceinline__ float2 to_f2<__half>(uint32_t w) {
    return __half22float2(*reinterpret_cast<const __half2*>(&w));
}

// C is a multiple of 2; every row starts on a 4-byte boundary.
template <typename T>
__global__ void __launch_bounds__(kWarps * 32)
delta_kernel(const T* __restrict__ d_o, const T* __restrict__ o, float* __restrict__ delta, const Na2dStride s_do,
             const Na2dStride s_o, const Na2dGeom g) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long n_query = (long long)g.BN * g.Hq * g.W;
    const long long qi = (long long)blockIdx.x * kWarps + warp;
    if (qi >= n_query) return;
    const int w = (int)(qi % g.W);
    const int h = (int)((qi / g.W) % g.Hq);
    const long long bn = qi / ((long long)g.W * g.Hq);
    const long long b = bn / g.N, n = bn - b * g.N;
    const uint32_t* pg = reinterpret_cast<const uint32_t*>(d_o + b * s_do.b + n * s_do.n + h * s_do.h + w * s_do.w);
    const uint32_t* po = reinterpret_cast<const uint32_t*>(o + b * s_o.b + n * s_o.n + h * s_o.h + w * s_o.w);
    float acc = 0.f;
    for (int c2 = lane; c2 < g.C / 2; c2 += 32) {
        const float2 a = to_f2<T>(pg[c2]), x = to_f2<T>(po[c2]);
        acc = fmaf(a.x, x.x, acc);
        acc = fmaf(a.y, x.y, acc);
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, d);
    if (lane == 0) delta[qi] = acc;
}

}  // namespace na2d_delta
