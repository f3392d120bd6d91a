// tcgen05 tensor-core kernels for 2D neighborhood attention on sm_100a (bf16 / fp16 inputs,
// fp32 accumulation), and their host-side launchers.
//
// Tiling.  A tile is TH x TW = 16 x 8 = 128 query pixels; query r of the tile is row r of every MMA and lane
// r of tensor memory.  The keys a tile can see are the union of its pixels' clamped
// windows: a (TH+ks-1) x (TW+ks-1) "halo box" whose origin is the window origin of the tile's
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

constexpr int TH = 16;     // tile rows
constexpr int TW = 8;      // tile columns (a warp covers 32 / TW tile rows)
constexpr int TM = 128;    // queries (or keys) per tile = MMA M
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

// Compile-time geometry of one (head dim, kernel size) instantiation.
// NMAX caps the keys (forward, dQ) or queries (dK/dV) of one chunk; it is set by how many
// tensor-memory columns the kernel can spare for the S-shaped accumulators.
// EXTRA_W widens the box (dK/dV: the inverse neighbourhood of a key tile whose first column is
// below ks starts at column 0 and is up to ks/2 columns wider than TW + ks - 1).
// W_SPLIT cuts the box into that many column strips, each walked as a chunk of its own (dK/dV).
template <int D, int KS, int NMAX = 256, int EXTRA_W = 0, int W_SPLIT = 1>
struct Cfg {
    static constexpr int HH = TH + KS - 1;                 // halo box rows
    static constexpr int HW = (TW + KS - 1 + EXTRA_W) / W_SPLIT;   // halo box (or strip) columns
    static_assert((TW + KS - 1 + EXTRA_W) % W_SPLIT == 0, "strips must tile the box");
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
    static_assert(NKP <= (NMAX + 15) / 16 * 16 && NKP % 16 == 0, "UMMA N range");
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

// Output rows leave through TMA: a thread that wrote its own 16-byte pieces straight to global
// memory would touch 32 different 128-byte lines per warp instruction.  Each softmax warp owns a
// staging buffer of 32 pixels (32 / TW tile rows x TW columns) x OUT_RW channels, laid out as the
// tensor map's swizzle wants it, and hands it to one tiled store per OUT_RW channels.
template <int DH> struct OutStage {
    static constexpr int RW = DH < 32 ? DH : 32;        // channels per store
    static constexpr int ROWB = RW * 2;                 // 32 or 64 bytes per pixel
    static constexpr int BYTES = 32 * ROWB;             // per warp
    static constexpr int ROUNDS = DH / RW;
    static_assert(RW == 16 || RW == 32, "staging row is 32 or 64 bytes");
};

// Stores columns [0, DH) held as fp32 bit patterns in `v` (scaled by `scale`) as 16-bit channels
// [ch0, ch0 + DH) of the warp's 32 pixels, whose first tile row is image row h0 and first column w0.
template <typename DT, int DH>
__device__ __forceinline__ void stage_and_store(const CUtensorMap* map, uint8_t* stage, const uint32_t (&v)[DH],
                                                float scale, int ch0, int w0, int h0, int bn, int lane) {
    using S = OutStage<DH>;
    const uint32_t row = smem_u32(stage) + lane * S::ROWB;
    const int sw = S::ROWB == 64 ? ((lane >> 1) & 3) : ((lane >> 2) & 1);
#pragma unroll
    for (int r = 0; r < S::ROUNDS; ++r) {
        uint32_t w[S::RW / 2];
#pragma unroll
        for (int e = 0; e < S::RW / 2; ++e)
            w[e] = pack2<DT>(__uint_as_float(v[r * S::RW + 2 * e]) * scale, __uint_as_float(v[r * S::RW + 2 * e + 1]) * scale);
        if (lane == 0) bulk_wait_read<0>();             // the previous store has read the buffer
        __syncwarp();
#pragma unroll
        for (int c = 0; c < S::ROWB / 16; ++c)
            st_shared_v4(row + ((c ^ sw) << 4), w[4 * c], w[4 * c + 1], w[4 * c + 2], w[4 * c + 3]);
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) {
            tma_store_4d(map, smem_u32(stage), ch0 + r * S::RW, w0, h0, bn);
            bulk_commit();
        }
    }
}

// Writes 16 consecutive 16-bit values (packed in pairs) of row `row` of the same operand layout,
// at columns [16*block16, 16*block16 + 16).
__device__ __forceinline__ void store_operand_block16(uint32_t base, int slab_bytes, int row, int block16,
                                                      const uint32_t (&w)[8]) {
    const uint32_t row_base = base + (block16 >> 2) * slab_bytes + row * 128;
#pragma unroll
    for (int gI = 0; gI < 2; ++gI) {
        const int chunk = ((block16 & 3) * 2 + gI) ^ (row & 7);
        st_shared_v4(row_base + chunk * 16, w[4 * gI], w[4 * gI + 1], w[4 * gI + 2], w[4 * gI + 3]);
    }
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

// ------------------------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// CUresult of the last failed tensor-map encode on this thread (0 if none), for error messages.
inline int& last_driver_result() {
    thread_local int r = 0;
    return r;
}

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
// box_c = 0 takes min(C, 64) channels; the output maps of the epilogue pass 16 or 32.
inline int make_map(CUtensorMap* map, const void* base, int dtype, long long BN, int rows, int W, int C,
                    int box_w, int box_h, int box_c = 0) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return NA2D_ERR_CUDA;
    const int slab_c = box_c > 0 ? box_c : (C < 64 ? C : 64);
    cuuint64_t dims[4] = {(cuuint64_t)C, (cuuint64_t)W, (cuuint64_t)rows, (cuuint64_t)BN};
    cuuint64_t strides[3] = {(cuuint64_t)C * 2, (cuuint64_t)W * C * 2, (cuuint64_t)rows * W * C * 2};
    cuuint32_t box[4] = {(cuuint32_t)slab_c, (cuuint32_t)box_w, (cuuint32_t)box_h, 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    const CUtensorMapDataType dt = dtype == NA2D_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    const CUtensorMapSwizzle sw = slab_c * 2 == 128 ? CU_TENSOR_MAP_SWIZZLE_128B
                                  : (slab_c * 2 == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B);
    CUresult r = fn(map, dt, 4, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) last_driver_result() = (int)r;
    return r == CUDA_SUCCESS ? NA2D_OK : NA2D_ERR_CUDA;
}

// Register re-balancing of the 384-thread kernels (launched with 168 registers per thread): the
// four warps of the data-movement group shrink to kRegsDonor, the eight softmax warps grow to
// kRegsSoftmax.  setmaxnreg.inc blocks until the registers it asks for have been given up, so
// what the eight warps take must not exceed what the four release.
constexpr int kRegsLaunch = 168, kRegsDonor = 64, kRegsSoftmax = 216;
static_assert((kRegsSoftmax - kRegsLaunch) * 8 <= (kRegsLaunch - kRegsDonor) * 4, "setmaxnreg.inc would wait for ever");

// The same for the kernels of sixteen warps (512 threads, launched with 128 registers each): softmax
// warps, control warps (producers, MMA issue) and epilogue warps.
constexpr int kDkvRegsLaunch = 128, kDkvRegsSoftmax = 176, kDkvRegsCtl = 72, kDkvRegsEpi = 88;
static_assert((kDkvRegsSoftmax - kDkvRegsLaunch) * 8 <= (kDkvRegsLaunch - kDkvRegsCtl) * 4 + (kDkvRegsLaunch - kDkvRegsEpi) * 4,
              "setmaxnreg.inc would wait for ever");

constexpr int kSmemLimit = 232448;     // dynamic shared memory a CTA can opt in to on sm_100

// Number of SMs of `device` (persistent kernels launch one CTA per SM), cached.
inline int sm_count(int device) {
    static std::mutex mu;
    static int cache[64];
    if (device < 0 || device >= 64) return 148;
    std::lock_guard<std::mutex> lock(mu);
    if (cache[device] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || n <= 0) n = 148;
        cache[device] = n;
    }
    return cache[device];
}

inline bool supported(int dtype, int C, int ks) {
    if (dtype != NA2D_BF16 && dtype != NA2D_F16) return false;
    if (C != 32 && C != 64 && C != 128) return false;
    return ks == 3 || ks == 5 || ks == 7 || ks == 9 || ks == 11 || ks == 13;
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


#ifdef NA2D_TRACE
// Development aid (not compiled into the shipped library): CTA 0 records the SM clock at the
// hand-overs between the warps so that they can be laid out on a time line.
__device__ unsigned long long g_trace[8192];     // [role 0..3][unit 0..255][event 0..7]
__device__ unsigned int g_trace_n = 8192;
__device__ __forceinline__ void trace(int role, int ev, unsigned n) {
    if (blockIdx.x != 0 || n >= 256) return;
    g_trace[(role * 256 + n) * 8 + ev] = clock64();
}
#define NA2D_TR(role, ev, n) trace(role, ev, n)
#else
#define NA2D_TR(role, ev, n)
#endif

}  // namespace na2d_tc

#include "na2d_tc_dq1.cuh"
#include "na2d_tc_fwd1.cuh"
#include "na2d_tc_fwd.cuh"
#include "na2d_tc_bwd.cuh"
#include "na2d_tc_dkdv.cuh"

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
