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
// across chunks; P goes back into tensor memory as packed 16-bit pairs, where it is the A operand
// of the second MMA (TS form).
//
// This header holds what the kernel files share.  Each kernel family is compiled in a translation
// unit of its own (na2d_tc_fwd.cu, na2d_tc_dq.cu, na2d_tc_dkdv.cu), once per 16-bit type.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <math_constants.h>

#include <atomic>
#include <cstring>
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

// Unit index bn -> head hn of batch hb.
__device__ __forceinline__ void split_unit(int bn, const Na2dGeom& g, int& hn, int& hb) {
    hb = g.n_magic ? (int)__umulhi((unsigned)bn, g.n_magic) : (g.N == 1 ? bn : bn / g.N);
    hn = bn - hb * g.N;
}

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

// Low and high 64 bits of the mask with bit r * hw set for r < rc (rc * hw <= 128).
constexpr unsigned long long row_repeat_lo(int hw, int rc) {
    unsigned long long m = 0;
    for (int r = 0; r < rc; ++r) if (r * hw < 64) m |= 1ull << (r * hw);
    return m;
}
constexpr unsigned long long row_repeat_hi(int hw, int rc) {
    unsigned long long m = 0;
    for (int r = 0; r < rc; ++r) if (r * hw >= 64) m |= 1ull << (r * hw - 64);
    return m;
}

// 128-bit helpers on (lo, hi) pairs.
__device__ __forceinline__ void shl128(unsigned long long& lo, unsigned long long& hi, int s) {   // 0 <= s < 64
    if (s > 0) {
        hi = (hi << s) | (lo >> (64 - s));
        lo <<= s;
    }
}
// Bits [0, k) set, 0 <= k <= 128.
__device__ __forceinline__ void low_bits128(int k, unsigned long long& lo, unsigned long long& hi) {
    lo = k >= 64 ? ~0ull : ((1ull << k) - 1ull);
    hi = k >= 128 ? ~0ull : (k > 64 ? ((1ull << (k - 64)) - 1ull) : 0ull);
}

// Validity of the 16 chunk columns [16 * blk, 16 * blk + 16) for one query: bit e is set when column
// 16 * blk + e is a key of the query's window.  A chunk holds RC box rows of HW keys each (column
// j = r * HW + c); the window covers chunk rows [wr_rel, wr_rel + KS) (wr_rel may be negative or
// beyond the chunk) and box columns [wc, wc + KS).  Sixteen columns touch at most three box rows.
template <int HW, int KS, int RC>
__device__ __forceinline__ uint32_t block_mask16(int blk, int wr_rel, int wc) {
    static_assert(3 * HW <= 64 && HW >= 8, "three box rows must fit 64 bits");
    const unsigned long long cm = static_cast<unsigned long long>(((1u << KS) - 1u) << wc);
    const int j0 = 16 * blk;
    const int r0 = j0 / HW, c0 = j0 - r0 * HW;
    unsigned long long w = 0;
#pragma unroll
    for (int t = 0; t < 3; ++t) {
        const int r = r0 + t;
        if (r >= wr_rel && r < wr_rel + KS && r < RC) w |= cm << (t * HW);
    }
    return static_cast<uint32_t>(w >> c0) & 0xffffu;
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
// [ch0, ch0 + DH) of the warp's 32 pixels, whose first tile row is image row h0 and first column w0,
// of head n of batch b.
// NBUF staging buffers of OutStage<DH>::BYTES lie one after another at `stage`; `seq` counts the
// warp's rounds and picks the buffer.  With one buffer a round waits until the previous round's
// store has read it (several hundred cycles per round); with two it only waits for the round
// before that.
// SCALED = false stores the values as they are (`scale` is ignored).
template <typename DT, int DH, int NBUF = 1, bool SCALED = true>
__device__ __forceinline__ void stage_and_store(const CUtensorMap* map, uint8_t* stage, const uint32_t (&v)[DH],
                                                float scale, int ch0, int w0, int h0, int n, int b, int lane,
                                                uint32_t* seq = nullptr) {
    using S = OutStage<DH>;
    static_assert(NBUF == 1 || NBUF == 2, "one or two staging buffers");
    const int sw = S::ROWB == 64 ? ((lane >> 1) & 3) : ((lane >> 2) & 1);
#pragma unroll
    for (int r = 0; r < S::ROUNDS; ++r) {
        uint32_t w[S::RW / 2];
#pragma unroll
        for (int e = 0; e < S::RW / 2; ++e)
            w[e] = SCALED ? pack2<DT>(__uint_as_float(v[r * S::RW + 2 * e]) * scale, __uint_as_float(v[r * S::RW + 2 * e + 1]) * scale)
                          : pack2<DT>(__uint_as_float(v[r * S::RW + 2 * e]), __uint_as_float(v[r * S::RW + 2 * e + 1]));
        const uint32_t buf = NBUF == 1 ? 0u : ((*seq)++ & 1u);
        const uint32_t base = smem_u32(stage) + buf * S::BYTES;
        const uint32_t row = base + lane * S::ROWB;
        if (lane == 0) bulk_wait_read<NBUF - 1>();      // the store that last used this buffer has read it
        __syncwarp();
#pragma unroll
        for (int c = 0; c < S::ROWB / 16; ++c)
            st_shared_v4(row + ((c ^ sw) << 4), w[4 * c], w[4 * c + 1], w[4 * c + 2], w[4 * c + 3]);
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) {
            tma_store_5d(map, base, ch0 + r * S::RW, w0, h0, n, b);
            bulk_commit();
        }
    }
}

// The same with fp32 output (the partial dK / dV of a row band, which its owner adds to its own):
// rounds of 16 channels, again 64-byte rows in the 64-byte swizzle of an fp32 tensor map whose box
// is 16 channels wide.  Buffers of 2 KB each.
template <int NCOL, int NBUF = 1, bool SCALED = true>
__device__ __forceinline__ void stage_and_store_f32(const CUtensorMap* map, uint8_t* stage, const uint32_t (&v)[NCOL],
                                                    float scale, int ch0, int w0, int h0, int n, int b, int lane,
                                                    uint32_t* seq = nullptr) {
    static_assert(NCOL % 16 == 0, "rounds of 16 channels");
    static_assert(NBUF == 1 || NBUF == 2, "one or two staging buffers");
    const int sw = (lane >> 1) & 3;
#pragma unroll
    for (int r = 0; r < NCOL / 16; ++r) {
        const uint32_t buf = NBUF == 1 ? 0u : ((*seq)++ & 1u);
        const uint32_t base = smem_u32(stage) + buf * 2048u;
        const uint32_t row = base + lane * 64;
        if (lane == 0) bulk_wait_read<NBUF - 1>();      // the store that last used this buffer has read it
        __syncwarp();
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            if (SCALED)
                st_shared_v4(row + ((c ^ sw) << 4), __float_as_uint(__uint_as_float(v[16 * r + 4 * c]) * scale),
                             __float_as_uint(__uint_as_float(v[16 * r + 4 * c + 1]) * scale),
                             __float_as_uint(__uint_as_float(v[16 * r + 4 * c + 2]) * scale),
                             __float_as_uint(__uint_as_float(v[16 * r + 4 * c + 3]) * scale));
            else
                st_shared_v4(row + ((c ^ sw) << 4), v[16 * r + 4 * c], v[16 * r + 4 * c + 1], v[16 * r + 4 * c + 2],
                             v[16 * r + 4 * c + 3]);
        }
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) {
            tma_store_5d(map, base, ch0 + 16 * r, w0, h0, n, b);
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

// One operand of a launch: base pointer and element strides of a (B, N, rows, W, C) tensor.
struct TensorArg {
    const void* ptr;
    Na2dStride st;
};

// Tensor map over a (B, N, rows, W, C) tensor of 16-bit elements (fp32 when `f32`: an output map)
// with the caller's strides (channels contiguous); coordinates are (channel, column, row, head,
// batch).  The box is box_c channels (0: min(C, 64)) x box_w x box_h x 1 x 1, swizzled so that one
// box row is one swizzle span.  Encoded maps are kept in a small per-thread cache: a training loop
// calls with the same buffers step after step, and the driver call is a visible part of a small
// launch.
inline int make_map(CUtensorMap* map, const TensorArg& t, int dtype, int B, int N, int rows, int W, int C,
                    int box_w, int box_h, int box_c = 0, bool f32 = false) {
    struct Key {
        const void* ptr;
        long long sb, sn, sh, sw;
        int dtype, B, N, rows, W, C, box_w, box_h, box_c, f32;
    };
    struct Entry {
        Key key;
        CUtensorMap map;
        bool used;
    };
    constexpr int kEntries = 64;
    thread_local Entry cache[kEntries];
    thread_local int next = 0;
    Key key;
    std::memset(&key, 0, sizeof(key));
    key.ptr = t.ptr; key.sb = t.st.b; key.sn = t.st.n; key.sh = t.st.h; key.sw = t.st.w;
    key.dtype = dtype; key.B = B; key.N = N; key.rows = rows; key.W = W; key.C = C;
    key.box_w = box_w; key.box_h = box_h; key.box_c = box_c; key.f32 = f32 ? 1 : 0;
    for (int i = 0; i < kEntries; ++i) {
        if (cache[i].used && std::memcmp(&cache[i].key, &key, sizeof(Key)) == 0) {
            *map = cache[i].map;
            return NA2D_OK;
        }
    }
    EncodeTiledFn fn = encode_fn();
    if (!fn) return NA2D_ERR_CUDA;
    const int slab_c = box_c > 0 ? box_c : (C < 64 ? C : 64);
    cuuint64_t dims[5] = {(cuuint64_t)C, (cuuint64_t)W, (cuuint64_t)rows, (cuuint64_t)N, (cuuint64_t)B};
    const cuuint64_t eb = f32 ? 4 : 2;
    cuuint64_t strides[4] = {(cuuint64_t)t.st.w * eb, (cuuint64_t)t.st.h * eb, (cuuint64_t)t.st.n * eb,
                             (cuuint64_t)t.st.b * eb};
    cuuint32_t box[5] = {(cuuint32_t)slab_c, (cuuint32_t)box_w, (cuuint32_t)box_h, 1, 1};
    cuuint32_t estr[5] = {1, 1, 1, 1, 1};
    const CUtensorMapDataType dt = f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                       : (dtype == NA2D_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16);
    const int row_bytes = slab_c * (int)eb;
    const CUtensorMapSwizzle sw = row_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B
                                  : (row_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B);
    CUresult r = fn(map, dt, 5, const_cast<void*>(t.ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        last_driver_result() = (int)r;
        return NA2D_ERR_CUDA;
    }
    cache[next].key = key;
    cache[next].map = *map;
    cache[next].used = true;
    next = (next + 1) % kEntries;
    return NA2D_OK;
}

// cudaFuncSetAttribute(MaxDynamicSharedMemorySize) once per kernel and device instead of on every
// launch.  `done` is a per-kernel bit set (one bit per device ordinal).
template <typename K>
inline cudaError_t opt_in_smem(K kern, int bytes, int device, std::atomic<unsigned long long>& done) {
    const unsigned long long bit = 1ull << (device & 63);
    if (done.load(std::memory_order_acquire) & bit) return cudaSuccess;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e == cudaSuccess) done.fetch_or(bit, std::memory_order_release);
    return e;
}

// What every launcher gets besides the tensors: geometry, element type, device, stream, the device
// error word of `device`, and a counter of launched kernels.
struct LaunchCtx {
    Na2dGeom g;
    int dtype;
    int B;
    int device;
    cudaStream_t st;
    unsigned int* err_word;
    int* launched;
    bool dkdv_f32;         // the dK/dV kernel writes fp32 (partial sums of a row band)
    int sm_margin;         // SMs to leave free for a kernel that runs beside this one
};

// CTAs of a persistent launch over `tiles` tiles.
inline int persistent_grid(const LaunchCtx& lc, long long tiles);

// Register re-balancing of the 384-thread kernels (launched with 168 registers per thread): the
// four warps of the data-movement group shrink to kRegsDonor, the eight softmax warps grow to
// kRegsSoftmax.  setmaxnreg.inc blocks until the registers it asks for have been given up, so
// what the eight warps take must not exceed what the four release.
constexpr int kRegsLaunch = 168, kRegsDonor = 72, kRegsSoftmax = 216;
static_assert((kRegsSoftmax - kRegsLaunch) * 8 <= (kRegsLaunch - kRegsDonor) * 4, "setmaxnreg.inc would wait for ever");

// The same for the kernels of sixteen warps (512 threads, launched with 128 registers each): softmax
// warps, control warps (producers, MMA issue) and epilogue warps.
constexpr int kDkvRegsLaunch = 128, kDkvRegsSoftmax = 176, kDkvRegsCtl = 72, kDkvRegsEpi = 88;
static_assert((kDkvRegsSoftmax - kDkvRegsLaunch) * 8 <= (kDkvRegsLaunch - kDkvRegsCtl) * 4 + (kDkvRegsLaunch - kDkvRegsEpi) * 4,
              "setmaxnreg.inc would wait for ever");

constexpr int kSmemLimit = 232448;     // dynamic shared memory a CTA can opt in to on sm_100

// Number of SMs of `device` (persistent kernels launch one CTA per SM), cached.
inline int sm_count(int device);
inline int persistent_grid(const LaunchCtx& lc, long long tiles) {
    int sms = sm_count(lc.device) - lc.sm_margin;
    if (sms < 1) sms = 1;
    return (int)(tiles < sms ? tiles : sms);
}
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
static __device__ unsigned long long g_trace[8192];     // [role 0..3][unit 0..255][event 0..7]
static __device__ unsigned int g_trace_n = 8192;
__device__ __forceinline__ void trace(int role, int ev, unsigned n) {
    if (blockIdx.x != 0 || n >= 256) return;
    g_trace[(role * 256 + n) * 8 + ev] = clock64();
}
#define NA2D_TR(role, ev, n) trace(role, ev, n)
// Copies this translation unit's trace to the host and clears it (each unit has its own array).
inline int copy_trace(unsigned long long* out, int max_entries) {
    unsigned int n = 8192;
    cudaDeviceSynchronize();
    if ((int)n > max_entries) n = max_entries;
    cudaMemcpyFromSymbol(out, g_trace, n * sizeof(unsigned long long));
    void* arr = nullptr;
    if (cudaGetSymbolAddress(&arr, g_trace) == cudaSuccess) cudaMemset(arr, 0, sizeof(g_trace));
    return (int)n;
}
#else
#define NA2D_TR(role, ev, n)
#endif

}  // namespace na2d_tc
