// An estimate of the backward's row delta, formed ahead of the dQ kernel: dO . o per query, where
// o is the forward's output as it was stored (16 bit).  The exact delta is sum_j p_j dP_j; dO . o
// differs from it by what o lost to rounding (P went into the forward's second MMA in 16 bits,
// and o was rounded when stored), a few 1e-2 at most.  That is too coarse to form dS from directly
// - the error would enter every dS of the row - but it is all the dQ kernel of the larger windows
// needs to walk its key box once instead of twice: it forms dS from the estimate and corrects
// the result exactly at the end (see na2d_tc_bwd.cuh).
//
// C / 8 lanes per query pixel, each lane one 16-byte piece of the two rows; a block covers
// 256 / (C / 8) consecutive pixels of one (batch, head) image, so a warp's loads are whole rows
// lying one after another.  An HBM-bound pass over two tensors: no division beyond one 32-bit
// one per thread.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "na2d_index.cuh"

namespace na2d_delta {

constexpr int kThreads = 256;

template <typename T> __device__ __forceinline__ float2 to_f2(uint32_t w);
template <> __device__ __forceinline__ float2 to_f2<__nv_bfloat16>(uint32_t w) {
    return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
}
template <> __device__ __forceinline__ float2 to_f2<__half>(uint32_t w) {
    return __half22float2(*reinterpret_cast<const __half2*>(&w));
}

template <typename T>
__device__ __forceinline__ float dot8(const uint4 a, const uint4 x, float acc) {
    const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, xw[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 fa = to_f2<T>(aw[i]), fx = to_f2<T>(xw[i]);
        acc = fmaf(fa.x, fx.x, acc);
        acc = fmaf(fa.y, fx.y, acc);
    }
    return acc;
}

// Pixels of one image a block covers.
template <int LPP> NA2D_HD constexpr int pixels_per_block() { return kThreads / LPP; }

// LPP = C / 8 lanes per pixel (4, 8 or 16).  Every row starts on a 16-byte boundary.  The grid is
// batch * heads * blocks_per_image blocks, an image's blocks next to one another.
template <typename T, int LPP>
__global__ void __launch_bounds__(kThreads)
delta_kernel(const T* __restrict__ d_o, const T* __restrict__ o, float* __restrict__ delta, const Na2dStride s_do,
             const Na2dStride s_o, const Na2dGeom g, const unsigned blocks_per_image) {
    const unsigned hw = (unsigned)g.Hq * (unsigned)g.W;
    const unsigned bn = blockIdx.x / blocks_per_image;
    const unsigned pix = (blockIdx.x - bn * blocks_per_image) * pixels_per_block<LPP>() + threadIdx.x / LPP;
    const unsigned part = threadIdx.x % LPP;
    float acc = 0.f;
    if (pix < hw) {
        const unsigned h = pix / (unsigned)g.W, w = pix - h * (unsigned)g.W;
        const unsigned b = bn / (unsigned)g.N, n = bn - b * (unsigned)g.N;
        const T* pg = d_o + b * s_do.b + n * s_do.n + h * s_do.h + w * s_do.w;
        const T* po = o + b * s_o.b + n * s_o.n + h * s_o.h + w * s_o.w;
        const uint4 a = __ldg(reinterpret_cast<const uint4*>(pg) + part);
        const uint4 x = __ldg(reinterpret_cast<const uint4*>(po) + part);
        acc = dot8<T>(a, x, 0.f);
    }
#pragma unroll
    for (int d = LPP / 2; d > 0; d >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, d);
    if (part == 0 && pix < hw) delta[(long long)bn * hw + pix] = acc;
}

}  // namespace na2d_delta
