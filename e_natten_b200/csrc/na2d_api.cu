// C ABI of libna2d.so (declared in include/na2d.h): argument checking, device selection and
// dispatch to the SIMT or tcgen05 kernels.  No framework headers; plain pointers and sizes.
#include <cuda_runtime.h>

#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <type_traits>

#include "../../include/na2d.h"
#include "na2d_delta.cuh"
#include "na2d_index.cuh"
#include "na2d_simt.cuh"
#include "na2d_tc_entry.h"

namespace {

std::atomic<long long> g_launches{0};
thread_local char t_cuda_err[256] = "";

int cuda_fail(cudaError_t e, const char* what) {
    snprintf(t_cuda_err, sizeof(t_cuda_err), "%s: %s", what, cudaGetErrorString(e));
    return NA2D_ERR_CUDA;
}

// Failure of a tcgen05 launcher: either a runtime error or a failed tensor-map encode (a driver call).
int tc_fail(const char* what) {
    int& drv = na2d_tc::last_driver_result();
    if (drv != 0) {
        snprintf(t_cuda_err, sizeof(t_cuda_err), "%s: cuTensorMapEncodeTiled failed with CUresult %d", what, drv);
        drv = 0;
        return NA2D_ERR_CUDA;
    }
    return cuda_fail(cudaGetLastError(), what);
}

#define NA2D_CUDA(call)                                        \
    do {                                                       \
        cudaError_t e__ = (call);                              \
        if (e__ != cudaSuccess) return cuda_fail(e__, #call);  \
    } while (0)

// Makes `device` current for the scope and restores the previous device afterwards.
// cudaSetDevice is called even when `device` already is the thread's current device: a thread that
// has made no runtime call yet (an autograd worker thread, for one) reports device 0 as current
// without having its context bound, and the driver call that encodes tensor maps needs a bound
// context.
struct DeviceScope {
    int prev = -1;
    cudaError_t err = cudaSuccess;
    explicit DeviceScope(int device) {
        err = cudaGetDevice(&prev);
        if (err == cudaSuccess) err = cudaSetDevice(device);
    }
    ~DeviceScope() {
        int cur = -1;
        if (prev >= 0 && cudaGetDevice(&cur) == cudaSuccess && cur != prev) cudaSetDevice(prev);
    }
};

constexpr int kMaxDevices = 64;

// Compute-capability check, cached per device.
int check_device(int device) {
    static std::mutex mu;
    static int state[kMaxDevices];   // 0 unknown, 1 ok, 2 not sm_100
    if (device < 0 || device >= kMaxDevices) return NA2D_ERR_BAD_ARG;
    std::lock_guard<std::mutex> lock(mu);
    if (state[device] == 0) {
        int major = 0;
        cudaError_t e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device);
        if (e != cudaSuccess) { cuda_fail(e, "cudaDeviceGetAttribute"); return NA2D_ERR_NO_DEVICE; }
        state[device] = (major == 10) ? 1 : 2;
    }
    return state[device] == 1 ? NA2D_OK : NA2D_ERR_NO_DEVICE;
}

// ---- device error word ---------------------------------------------------------------------------
// Two words per device (a file-scope device variable has one instance per device context).
// [0]: bits say which kind of bounded wait gave up; kernels get its address as an argument.
// [1]: the limit of a bounded wait in microseconds, 0 = the built-in 4 s.  Set once per device from
// the environment variable NA2D_WAIT_LIMIT_US: a profiler pass that instruments every instruction
// can stretch a healthy hand-over past the built-in limit (seen under `ncu --set full`).
__device__ unsigned int g_error_word[2] = {0u, 0u};

// Device address of g_error_word on `device` (which must be current), looked up once per device.
int error_word_address(int device, unsigned int** out) {
    static std::mutex mu;
    static unsigned int* cache[kMaxDevices];
    if (device < 0 || device >= kMaxDevices) return NA2D_ERR_BAD_ARG;
    std::lock_guard<std::mutex> lock(mu);
    if (cache[device] == nullptr) {
        void* p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_error_word);
        if (e != cudaSuccess) return cuda_fail(e, "cudaGetSymbolAddress(g_error_word)");
        if (const char* env = getenv("NA2D_WAIT_LIMIT_US")) {
            const unsigned long long v = strtoull(env, nullptr, 10);
            if (v > 0 && v <= 0xffffffffull) {
                const unsigned int limit = (unsigned int)v;
                e = cudaMemcpy(static_cast<unsigned int*>(p) + 1, &limit, sizeof(limit), cudaMemcpyHostToDevice);
                if (e != cudaSuccess) return cuda_fail(e, "cudaMemcpy(wait limit)");
            }
        }
        cache[device] = static_cast<unsigned int*>(p);
    }
    *out = cache[device];
    return NA2D_OK;
}

// The kernel of na2d_selftest_wait_timeout: one thread waits on a barrier nothing completes.
__global__ void wait_timeout_kernel(unsigned int* err_word, unsigned long long limit_ns) {
    __shared__ uint64_t bar;
    __shared__ na2d_ptx::WaitState state;
    if (threadIdx.x == 0) {
        na2d_ptx::wait_state_init(&state, err_word, limit_ns);
        state.limit_us = static_cast<uint32_t>(limit_ns / 1000ull);        // the self-test's own limit, whatever is configured
        na2d_ptx::mbar_init(&bar, 1);
        na2d_ptx::mbar_fence_init();
        const na2d_ptx::WaitCtx wctx{&state};
        na2d_ptx::mbar_wait(&bar, 0, wctx, na2d_ptx::kErrOther);
    }
}

// ---- problem description --------------------------------------------------------------------------
struct Tensor {
    void* ptr = nullptr;
    Na2dStride st{0, 0, 0, 0};
};

struct Problem {
    Na2dGeom g;
    int B = 0;
    int dtype = 0;
    bool tensor = false;      // run the tcgen05 kernels
    bool dkdv_f32 = false;    // dK / dV are fp32 tensors
    int sm_margin = 0;        // SMs the persistent kernels leave free
    int device = 0;
    cudaStream_t st = nullptr;
    Tensor q, k, v, o, d_o, d_q, d_k, d_v;
    float* lse = nullptr;
    float* delta = nullptr;
};

// Strides of one operand: the caller's, or dense (B, N, rows, W, C) when all four are zero.  The
// stride of a dimension of extent 1 never reaches an address, so whatever the caller passed for
// it is replaced by the dense value (frameworks report arbitrary strides there).
Tensor resolve(const na2d_tensor& t, int B, int N, int rows, int W, int C, bool one_d) {
    Tensor r;
    r.ptr = t.ptr;
    const bool dense = t.stride_b == 0 && t.stride_n == 0 && t.stride_h == 0 && t.stride_w == 0;
    r.st.w = (dense || W == 1) ? C : t.stride_w;
    r.st.h = (dense || rows == 1 || one_d) ? (long long)W * r.st.w : t.stride_h;
    r.st.n = (dense || N == 1) ? (long long)rows * r.st.h : t.stride_n;
    r.st.b = (dense || B == 1) ? (long long)N * r.st.n : t.stride_b;
    return r;
}

// What a TMA tensor map needs of an operand: a 16-byte aligned base, strides that are multiples of
// 16 bytes (8 elements of 16 bits) and below 2^40 bytes.
bool tma_compatible(const Tensor& t) {
    if (t.ptr == nullptr) return true;
    if (reinterpret_cast<uintptr_t>(t.ptr) & 15u) return false;
    const long long s[4] = {t.st.b, t.st.n, t.st.h, t.st.w};
    for (long long x : s)
        if (x <= 0 || (x & 7) != 0 || x >= (1ll << 39)) return false;
    return true;
}

// Pixels per block for the SIMT kernels: 64 (eight per warp, neighbouring windows share L1) unless
// that gives fewer than two blocks per SM, where one pixel per warp fills the GPU better.
int simt_patch(long long BN, int H, int W) {
    return na2d_simt::patch_count(BN, H, W, na2d_simt::kPatch) < 2 * 148 ? na2d_simt::kPatchSmall : na2d_simt::kPatch;
}

// `key_side`: the call is the key half of the backward, whose key band may be any part of the image
// (each key sums over whichever local queries see it); the other calls need a key band that holds
// every window of the query band.
int make_problem(const na2d_args* a, Problem* out, bool key_side = false) {
    if (!a || a->struct_size < sizeof(na2d_args)) return NA2D_ERR_BAD_ARG;
    const int B = a->B, N = a->N, H = a->H, W = a->W, C = a->C, ks = a->kernel_size, dtype = a->dtype, path = a->path;
    if (B <= 0 || N <= 0 || H <= 0 || W <= 0 || C <= 0) return NA2D_ERR_BAD_ARG;
    if (ks <= 0 || (ks & 1) == 0) return NA2D_ERR_BAD_ARG;
    if (dtype != NA2D_F32 && dtype != NA2D_BF16 && dtype != NA2D_F16) return NA2D_ERR_UNSUPPORTED;
    if (path != NA2D_PATH_AUTO && path != NA2D_PATH_SIMT && path != NA2D_PATH_TENSOR) return NA2D_ERR_BAD_ARG;
    if (a->op != NA2D_OP_2D && a->op != NA2D_OP_1D) return NA2D_ERR_BAD_ARG;
    if (!(a->scale > 0.f) || !(a->scale < 3.0e38f)) return NA2D_ERR_BAD_ARG;
    if ((long long)B * N > 0x7fffffffLL) return NA2D_ERR_TOO_LARGE;
    const bool one_d = a->op == NA2D_OP_1D;
    Na2dGeom g;
    g.BN = B * N; g.N = N; g.W = W; g.C = C; g.ks = ks; g.kh = one_d ? 1 : ks;
    g.n_magic = na2d_heads_magic(g.BN, N);
    g.scale = a->scale;
    g.sl2 = a->scale * 1.4426950408889634f;
    if (one_d) {
        if (H != 1 || a->rows) return NA2D_ERR_BAD_ARG;
        g.q_row0 = 0; g.Hq = 1; g.kv_row0 = 0; g.Hkv = 1; g.Hg = 1;
        // the reference reads out of range when the sequence is shorter than the window
        // (e_natten/pytorch.py:7-11 goes negative); here that is an error
        if (W < ks) return NA2D_ERR_WINDOW;
    } else {
        const na2d_rows* rows = a->rows;
        if (rows) {
            g.q_row0 = rows->q_row0; g.Hq = rows->Hq; g.kv_row0 = rows->kv_row0; g.Hkv = rows->Hkv;
            g.Hg = rows->H_global;
            if (g.Hq <= 0 || g.Hkv <= 0 || g.Hg <= 0 || g.q_row0 < 0 || g.kv_row0 < 0) return NA2D_ERR_BAD_ARG;
            if (g.q_row0 + g.Hq > g.Hg || g.kv_row0 + g.Hkv > g.Hg) return NA2D_ERR_BAD_ARG;
        } else {
            g.q_row0 = 0; g.Hq = H; g.kv_row0 = 0; g.Hkv = H; g.Hg = H;
        }
        // The reference silently reads garbage when a grid side is below the kernel size
        // (e_natten/pytorch.py:7-11 goes negative); here that is an error.
        if (g.Hg < ks || W < ks) return NA2D_ERR_WINDOW;
        // the key band must hold every window of the query band
        if (!key_side) {
            if (na2d_ws(g.q_row0, g.Hg, ks) < g.kv_row0) return NA2D_ERR_WINDOW;
            if (na2d_ws(g.q_row0 + g.Hq - 1, g.Hg, ks) + ks > g.kv_row0 + g.Hkv) return NA2D_ERR_WINDOW;
        }
    }
    Problem& p = *out;
    p.q = resolve(a->q, B, N, g.Hq, W, C, one_d);
    p.o = resolve(a->o, B, N, g.Hq, W, C, one_d);
    p.d_o = resolve(a->d_o, B, N, g.Hq, W, C, one_d);
    p.d_q = resolve(a->d_q, B, N, g.Hq, W, C, one_d);
    p.k = resolve(a->k, B, N, g.Hkv, W, C, one_d);
    p.v = resolve(a->v, B, N, g.Hkv, W, C, one_d);
    p.d_k = resolve(a->d_k, B, N, g.Hkv, W, C, one_d);
    p.d_v = resolve(a->d_v, B, N, g.Hkv, W, C, one_d);

    bool tc_ok = !one_d && na2d_tc::supported(dtype, C, ks);
    if (tc_ok) {
        for (const Tensor* t : {&p.q, &p.k, &p.v, &p.o, &p.d_o, &p.d_q, &p.d_k, &p.d_v})
            tc_ok = tc_ok && tma_compatible(*t);
    }
    bool tensor = false;
    if (path == NA2D_PATH_TENSOR) {
        if (!tc_ok) return NA2D_ERR_UNSUPPORTED;
        tensor = true;
    } else if (path == NA2D_PATH_AUTO) {
        tensor = tc_ok;
    }
    if (!tensor && (C > na2d_simt::kMaxC || ks > na2d_simt::kMaxKs)) return NA2D_ERR_UNSUPPORTED;
    g.patch = simt_patch(g.BN, g.Hq, W);
    p.g = g; p.B = B; p.dtype = dtype; p.tensor = tensor;
    p.device = a->device; p.st = (cudaStream_t)a->stream;
    p.lse = a->lse; p.delta = a->delta;
    p.dkdv_f32 = (a->flags & NA2D_FLAG_DKDV_F32) != 0 && dtype != NA2D_F32;
    p.sm_margin = (a->flags >> 8) & 0xff;
    if (a->flags & ~(NA2D_FLAG_DKDV_F32 | NA2D_FLAG_SM_MARGIN(0xff))) return NA2D_ERR_BAD_ARG;
    return NA2D_OK;
}

// ---- dispatch helpers -------------------------------------------------------------------------------
template <int V> using IntTag = std::integral_constant<int, V>;
template <typename T> struct TypeTag { using type = T; };

// Calls f(TypeTag<element type>, IntTag<channels per lane>) for the problem's dtype and head dim.
template <typename F>
int simt_dispatch(int dtype, int C, F&& f) {
    auto by_cpl = [&](auto type_tag) -> int {
        if (C <= 32) return f(type_tag, IntTag<1>{});
        if (C <= 64) return f(type_tag, IntTag<2>{});
        if (C <= 128) return f(type_tag, IntTag<4>{});
        return f(type_tag, IntTag<8>{});
    };
    switch (dtype) {
        case NA2D_F32: return by_cpl(TypeTag<float>{});
        case NA2D_BF16: return by_cpl(TypeTag<__nv_bfloat16>{});
        default: return by_cpl(TypeTag<__half>{});
    }
}

// One block per patch of a (BN, H, W) pixel grid.
int grid_for(long long BN, int H, int W, int patch, unsigned* grid) {
    const long long nb = na2d_simt::patch_count(BN, H, W, patch);
    if (nb > 0x7fffffffLL) return NA2D_ERR_TOO_LARGE;
    *grid = (unsigned)nb;
    return NA2D_OK;
}

constexpr int kSimtThreads = na2d_simt::kWarps * 32;

int after_launch() {
    g_launches.fetch_add(1);
    NA2D_CUDA(cudaGetLastError());
    return NA2D_OK;
}

na2d_tc::TensorArg targ(const Tensor& t) { return na2d_tc::TensorArg{t.ptr, t.st}; }

int launch_ctx(const Problem& p, int* launched, na2d_tc::LaunchCtx* lc) {
    unsigned int* err = nullptr;
    int rc = error_word_address(p.device, &err);
    if (rc != NA2D_OK) return rc;
    *lc = na2d_tc::LaunchCtx{p.g, p.dtype, p.B, p.device, p.st, err, launched, p.dkdv_f32, p.sm_margin};
    return NA2D_OK;
}

// ---- the three compute steps ---------------------------------------------------------------------------
int run_forward(const Problem& p) {
    const Na2dGeom& g = p.g;
    if (p.tensor) {
        int launched = 0;
        na2d_tc::LaunchCtx lc;
        int rc = launch_ctx(p, &launched, &lc);
        if (rc != NA2D_OK) return rc;
        rc = p.dtype == NA2D_BF16 ? na2d_tc::forward_bf16(lc, targ(p.q), targ(p.k), targ(p.v), targ(p.o), p.lse)
                                  : na2d_tc::forward_f16(lc, targ(p.q), targ(p.k), targ(p.v), targ(p.o), p.lse);
        g_launches.fetch_add(launched);
        if (rc == NA2D_ERR_CUDA) return tc_fail("tcgen05 forward launch");
        return rc;
    }
    unsigned grid = 0;
    int rc = grid_for(g.BN, g.Hq, g.W, g.patch, &grid);
    if (rc != NA2D_OK) return rc;
    return simt_dispatch(p.dtype, g.C, [&](auto tt, auto cpl) -> int {
        using T = typename decltype(tt)::type;
        na2d_simt::fwd_kernel<T, decltype(cpl)::value>
            <<<grid, kSimtThreads, na2d_simt::window_smem_bytes(g.kh, g.ks, 1), p.st>>>(
                (const T*)p.q.ptr, (const T*)p.k.ptr, (const T*)p.v.ptr, (T*)p.o.ptr, p.lse, p.q.st, p.k.st, p.v.st,
                p.o.st, g);
        return after_launch();
    });
}

// The dO . o estimate of the row deltas, into p.delta (tensor path: head dim 32, 64 or 128, rows on
// 16-byte boundaries).
template <typename T, int LPP>
int launch_delta_as(const Problem& p) {
    const Na2dGeom& g = p.g;
    const long long hw = (long long)g.Hq * g.W;
    const long long per_image = (hw + na2d_delta::pixels_per_block<LPP>() - 1) / na2d_delta::pixels_per_block<LPP>();
    if (hw > 0x7fffffffLL || per_image * g.BN > 0x7fffffffLL) return NA2D_ERR_TOO_LARGE;
    na2d_delta::delta_kernel<T, LPP><<<(unsigned)(per_image * g.BN), na2d_delta::kThreads, 0, p.st>>>(
        (const T*)p.d_o.ptr, (const T*)p.o.ptr, p.delta, p.d_o.st, p.o.st, g, (unsigned)per_image);
    return after_launch();
}

int launch_delta(const Problem& p) {
    const bool bf = p.dtype == NA2D_BF16;
    switch (p.g.C) {
        case 32: return bf ? launch_delta_as<__nv_bfloat16, 4>(p) : launch_delta_as<__half, 4>(p);
        case 64: return bf ? launch_delta_as<__nv_bfloat16, 8>(p) : launch_delta_as<__half, 8>(p);
        case 128: return bf ? launch_delta_as<__nv_bfloat16, 16>(p) : launch_delta_as<__half, 16>(p);
        default: return NA2D_ERR_UNSUPPORTED;
    }
}

int run_backward_dq(const Problem& p) {
    const Na2dGeom& g = p.g;
    if (p.tensor) {
        int launched = 0;
        na2d_tc::LaunchCtx lc;
        int rc = launch_ctx(p, &launched, &lc);
        if (rc != NA2D_OK) return rc;
        // With the forward's output at hand, the dQ kernel of the larger windows gets an estimate of
        // the row deltas (dO . o) and walks its key box once; it overwrites the estimate with the
        // exact deltas.
        const float* delta_in = nullptr;
        if (g.ks >= 7 && p.o.ptr && p.d_q.ptr) {
            rc = launch_delta(p);
            if (rc != NA2D_OK) return rc;
            delta_in = p.delta;
        }
        rc = p.dtype == NA2D_BF16
                 ? na2d_tc::backward_dq_bf16(lc, targ(p.q), targ(p.k), targ(p.v), p.lse, targ(p.d_o), targ(p.d_q), p.delta, delta_in)
                 : na2d_tc::backward_dq_f16(lc, targ(p.q), targ(p.k), targ(p.v), p.lse, targ(p.d_o), targ(p.d_q), p.delta, delta_in);
        g_launches.fetch_add(launched);
        if (rc == NA2D_ERR_CUDA) return tc_fail("tcgen05 dQ launch");
        return rc;
    }
    unsigned grid = 0;
    int rc = grid_for(g.BN, g.Hq, g.W, g.patch, &grid);
    if (rc != NA2D_OK) return rc;
    return simt_dispatch(p.dtype, g.C, [&](auto tt, auto cpl) -> int {
        using T = typename decltype(tt)::type;
        na2d_simt::dq_kernel<T, decltype(cpl)::value>
            <<<grid, kSimtThreads, na2d_simt::window_smem_bytes(g.kh, g.ks, 2), p.st>>>(
                (const T*)p.q.ptr, (const T*)p.k.ptr, (const T*)p.v.ptr, p.lse, (const T*)p.d_o.ptr, (T*)p.d_q.ptr,
                p.delta, p.q.st, p.k.st, p.v.st, p.d_o.st, p.d_q.st, g);
        return after_launch();
    });
}

int run_backward_dkdv(const Problem& p) {
    const Na2dGeom& g = p.g;
    if (p.tensor) {
        int launched = 0;
        na2d_tc::LaunchCtx lc;
        int rc = launch_ctx(p, &launched, &lc);
        if (rc != NA2D_OK) return rc;
        rc = p.dtype == NA2D_BF16
                 ? na2d_tc::backward_dkdv_bf16(lc, targ(p.q), targ(p.k), targ(p.v), p.lse, targ(p.d_o), p.delta, targ(p.d_k), targ(p.d_v))
                 : na2d_tc::backward_dkdv_f16(lc, targ(p.q), targ(p.k), targ(p.v), p.lse, targ(p.d_o), p.delta, targ(p.d_k), targ(p.d_v));
        g_launches.fetch_add(launched);
        if (rc == NA2D_ERR_CUDA) return tc_fail("tcgen05 dK/dV launch");
        return rc;
    }
    unsigned grid = 0;
    int rc = grid_for(g.BN, g.Hkv, g.W, g.patch, &grid);
    if (rc != NA2D_OK) return rc;
    return simt_dispatch(p.dtype, g.C, [&](auto tt, auto cpl) -> int {
        using T = typename decltype(tt)::type;
        na2d_simt::dkdv_kernel<T, decltype(cpl)::value><<<grid, kSimtThreads, 0, p.st>>>(
            (const T*)p.q.ptr, (const T*)p.k.ptr, (const T*)p.v.ptr, p.lse, (const T*)p.d_o.ptr, p.delta,
            p.d_k.ptr, p.d_v.ptr, p.dkdv_f32 ? 1 : 0, p.q.st, p.k.st, p.v.st, p.d_o.st, p.d_k.st, p.d_v.st, g);
        return after_launch();
    });
}

// Validate, select the device, check it; then run `step`.
template <typename F>
int enter(const na2d_args* a, F&& step, bool key_side = false) {
    Problem p;
    int rc = make_problem(a, &p, key_side);
    if (rc != NA2D_OK) return rc;
    DeviceScope scope(p.device);
    if (scope.err != cudaSuccess) return cuda_fail(scope.err, "cudaSetDevice");
    rc = check_device(p.device);
    if (rc != NA2D_OK) return rc;
    return step(p);
}

na2d_tensor dense(const void* ptr) { return na2d_tensor{const_cast<void*>(ptr), 0, 0, 0, 0}; }

na2d_args dense_args(int op, int B, int N, int H, int W, int C, int ks, int dtype, const na2d_rows* rows, int path,
                     int device, void* stream) {
    na2d_args a;
    std::memset(&a, 0, sizeof(a));
    a.struct_size = sizeof(a);
    a.op = op;
    a.B = B; a.N = N; a.H = H; a.W = W; a.C = C; a.kernel_size = ks; a.dtype = dtype; a.path = path; a.device = device;
    a.scale = 1.f;
    a.stream = stream;
    a.rows = rows;
    return a;
}

// ---- scratch for na2d_backward_static_scratch ----------------------------------------------------
// The backward pair passes the row delta from the dQ kernel to the dK/dV kernel through global
// memory.  Normally the caller provides that buffer; the entry point below keeps it in this
// file-scope device array instead, so that a caller who may not allocate can still run the
// backward.  Every GPU on which the library's device code has been loaded carries the array
// (4 MiB) until the process exits.
constexpr long long kStaticDeltaFloats = 1LL << 20;
static __device__ __align__(256) float g_static_delta[kStaticDeltaFloats];

// Device address of g_static_delta on `device`, looked up once per device.  In host code the
// name g_static_delta is only a handle for the runtime, not an address a kernel could use; the
// address comes from cudaGetSymbolAddress, asked while `device` is the current device.
int static_delta_address(int device, float** out) {
    static std::mutex mu;
    static float* cache[kMaxDevices];
    if (device < 0 || device >= kMaxDevices) return NA2D_ERR_BAD_ARG;
    std::lock_guard<std::mutex> lock(mu);
    if (cache[device] == nullptr) {
        void* p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_static_delta);
        if (e != cudaSuccess) return cuda_fail(e, "cudaGetSymbolAddress(g_static_delta)");
        cache[device] = static_cast<float*>(p);
    }
    *out = cache[device];
    return NA2D_OK;
}

// ---- the unfused pair -------------------------------------------------------------------------------------
struct PairProblem {
    Na2dGeom g;
    int dtype;
    Na2dStride st;          // dense strides of a (B, N, H, W, C) tensor
    cudaStream_t stream;
};

int make_pair_problem(int B, int N, int H, int W, int C, int ks, int dtype, void* stream, PairProblem* out) {
    if (B <= 0 || N <= 0 || H <= 0 || W <= 0 || C <= 0) return NA2D_ERR_BAD_ARG;
    if (ks <= 0 || (ks & 1) == 0) return NA2D_ERR_BAD_ARG;
    if (dtype != NA2D_F32 && dtype != NA2D_BF16 && dtype != NA2D_F16) return NA2D_ERR_UNSUPPORTED;
    if ((long long)B * N > 0x7fffffffLL) return NA2D_ERR_TOO_LARGE;
    if (H < ks || W < ks) return NA2D_ERR_WINDOW;
    if (C > na2d_simt::kMaxC || ks > na2d_simt::kMaxKs) return NA2D_ERR_UNSUPPORTED;
    Na2dGeom g;
    g.BN = B * N; g.N = N; g.n_magic = na2d_heads_magic(g.BN, N); g.Hq = H; g.Hkv = H; g.W = W; g.C = C; g.ks = ks; g.kh = ks;
    g.q_row0 = 0; g.kv_row0 = 0; g.Hg = H; g.scale = 1.f; g.sl2 = 1.4426950408889634f;
    g.patch = simt_patch(g.BN, H, W);
    out->g = g;
    out->dtype = dtype;
    out->st = Na2dStride{(long long)N * H * W * C, (long long)H * W * C, (long long)W * C, C};
    out->stream = (cudaStream_t)stream;
    return NA2D_OK;
}

template <typename F>
int enter_pair(int B, int N, int H, int W, int C, int ks, int dtype, int device, void* stream, F&& step) {
    PairProblem p;
    int rc = make_pair_problem(B, N, H, W, C, ks, dtype, stream, &p);
    if (rc != NA2D_OK) return rc;
    DeviceScope scope(device);
    if (scope.err != cudaSuccess) return cuda_fail(scope.err, "cudaSetDevice");
    rc = check_device(device);
    if (rc != NA2D_OK) return rc;
    return step(p);
}

// x . y over the window -> attn
int pair_dot(const PairProblem& p, const void* x, const void* y, void* attn) {
    unsigned grid = 0;
    int rc = grid_for(p.g.BN, p.g.Hq, p.g.W, p.g.patch, &grid);
    if (rc != NA2D_OK) return rc;
    return simt_dispatch(p.dtype, p.g.C, [&](auto tt, auto cpl) -> int {
        using T = typename decltype(tt)::type;
        na2d_simt::window_dot_kernel<T, decltype(cpl)::value><<<grid, kSimtThreads, 0, p.stream>>>(
            (const T*)x, (const T*)y, (T*)attn, p.st, p.st, p.g);
        return after_launch();
    });
}
// sum_j attn_j y_j -> out
int pair_apply(const PairProblem& p, const void* attn, const void* y, void* out) {
    unsigned grid = 0;
    int rc = grid_for(p.g.BN, p.g.Hq, p.g.W, p.g.patch, &grid);
    if (rc != NA2D_OK) return rc;
    return simt_dispatch(p.dtype, p.g.C, [&](auto tt, auto cpl) -> int {
        using T = typename decltype(tt)::type;
        na2d_simt::window_apply_kernel<T, decltype(cpl)::value>
            <<<grid, kSimtThreads, na2d_simt::window_smem_bytes(p.g.kh, p.g.ks, 1), p.stream>>>(
                (const T*)attn, (const T*)y, (T*)out, p.st, p.st, p.g);
        return after_launch();
    });
}
// key-side sum over the inverse neighbourhood of attn x -> out
int pair_inverse(const PairProblem& p, const void* attn, const void* x, void* out) {
    unsigned grid = 0;
    int rc = grid_for(p.g.BN, p.g.Hkv, p.g.W, p.g.patch, &grid);
    if (rc != NA2D_OK) return rc;
    return simt_dispatch(p.dtype, p.g.C, [&](auto tt, auto cpl) -> int {
        using T = typename decltype(tt)::type;
        na2d_simt::window_inverse_kernel<T, decltype(cpl)::value><<<grid, kSimtThreads, 0, p.stream>>>(
            (const T*)attn, (const T*)x, (T*)out, p.st, p.st, p.g);
        return after_launch();
    });
}

// ---- na2d_poll state -----------------------------------------------------------------------------------------
struct PollState {
    unsigned int* host = nullptr;     // pinned
    cudaEvent_t ev = nullptr;
    bool pending = false;
};
std::mutex g_poll_mu;
PollState g_poll[kMaxDevices];

}  // namespace

extern "C" {

int na2d_version(void) { return 200; }

const char* na2d_strerror(int status) {
    switch (status) {
        case NA2D_OK: return "ok";
        case NA2D_ERR_BAD_ARG: return "bad argument (null pointer, non-positive size, even kernel size, bad scale or bad row view)";
        case NA2D_ERR_UNSUPPORTED: return "unsupported dtype, head dim, kernel size or tensor layout for the requested path";
        case NA2D_ERR_WINDOW: return "grid side smaller than the kernel size, or key band does not cover the query band's windows";
        case NA2D_ERR_CUDA: return "CUDA call failed (see na2d_last_cuda_error)";
        case NA2D_ERR_NO_DEVICE: return "device is not an sm_100 (B200) GPU";
        case NA2D_ERR_TOO_LARGE: return "size beyond a documented maximum";
        case NA2D_ERR_KERNEL_WAIT: return "a bounded wait inside a kernel ran out";
        default: return "unknown status";
    }
}

const char* na2d_last_cuda_error(void) { return t_cuda_err; }

int na2d_window_start(int i, int seq_len, int kernel_size) { return na2d_ws(i, seq_len, kernel_size); }

int na2d_backward_window(int j, int seq_len, int kernel_size, int* lo, int* hi) {
    if (!lo || !hi || kernel_size <= 0 || seq_len <= 0) return NA2D_ERR_BAD_ARG;
    *lo = na2d_bws(j, kernel_size);
    *hi = na2d_bwe(j, seq_len, kernel_size);
    return NA2D_OK;
}

int na2d_dump_index(int32_t* ws, int32_t* bws, int32_t* bwe, int seq_len, int kernel_size,
                    int device, void* stream) {
    if (!ws || !bws || !bwe || seq_len <= 0 || kernel_size <= 0) return NA2D_ERR_BAD_ARG;
    DeviceScope scope(device);
    if (scope.err != cudaSuccess) return cuda_fail(scope.err, "cudaSetDevice");
    na2d_simt::index_dump_kernel<<<(seq_len + 127) / 128, 128, 0, (cudaStream_t)stream>>>(
        ws, bws, bwe, seq_len, kernel_size);
    return after_launch();
}

// ---- strided / scaled / 1D entry points ------------------------------------------------------------------
int na2d_forward_ex(const na2d_args* a) {
    if (!a || !a->q.ptr || !a->k.ptr || !a->v.ptr || !a->o.ptr || !a->lse) return NA2D_ERR_BAD_ARG;
    return enter(a, [](const Problem& p) { return run_forward(p); });
}

int na2d_backward_dq_ex(const na2d_args* a) {
    if (!a || !a->q.ptr || !a->k.ptr || !a->v.ptr || !a->lse || !a->d_o.ptr || !a->delta) return NA2D_ERR_BAD_ARG;
    return enter(a, [](const Problem& p) { return run_backward_dq(p); });
}

int na2d_backward_dkdv_ex(const na2d_args* a) {
    if (!a || !a->q.ptr || !a->k.ptr || !a->v.ptr || !a->lse || !a->d_o.ptr || !a->delta || !a->d_k.ptr || !a->d_v.ptr)
        return NA2D_ERR_BAD_ARG;
    return enter(a, [](const Problem& p) { return run_backward_dkdv(p); }, /*key_side=*/true);
}

int na2d_backward_ex(const na2d_args* a) {
    if (!a) return NA2D_ERR_BAD_ARG;
    if ((a->d_k.ptr == nullptr) != (a->d_v.ptr == nullptr)) return NA2D_ERR_BAD_ARG;
    if (!a->d_q.ptr && !a->d_k.ptr) return NA2D_ERR_BAD_ARG;
    // the query half always runs: it produces delta, which the key half needs
    int rc = na2d_backward_dq_ex(a);
    if (rc != NA2D_OK || a->d_k.ptr == nullptr) return rc;
    return na2d_backward_dkdv_ex(a);
}

// ---- dense entry points -------------------------------------------------------------------------------------
int na2d_forward(const void* q, const void* k, const void* v, void* o, float* lse,
                 int B, int N, int H, int W, int C, int kernel_size, int dtype,
                 const na2d_rows* rows, int path, int device, void* stream) {
    na2d_args a = dense_args(NA2D_OP_2D, B, N, H, W, C, kernel_size, dtype, rows, path, device, stream);
    a.q = dense(q); a.k = dense(k); a.v = dense(v); a.o = dense(o); a.lse = lse;
    return na2d_forward_ex(&a);
}

int na2d_backward_dq(const void* q, const void* k, const void* v, const void* o, const float* lse,
                     const void* d_o, void* d_q, float* delta,
                     int B, int N, int H, int W, int C, int kernel_size, int dtype,
                     const na2d_rows* rows, int path, int device, void* stream) {
    na2d_args a = dense_args(NA2D_OP_2D, B, N, H, W, C, kernel_size, dtype, rows, path, device, stream);
    a.q = dense(q); a.k = dense(k); a.v = dense(v); a.o = dense(o); a.lse = const_cast<float*>(lse);
    a.d_o = dense(d_o); a.d_q = dense(d_q); a.delta = delta;
    return na2d_backward_dq_ex(&a);
}

int na2d_backward_dkdv(const void* q, const void* k, const void* v, const float* lse,
                       const void* d_o, const float* delta, void* d_k, void* d_v,
                       int B, int N, int H, int W, int C, int kernel_size, int dtype,
                       const na2d_rows* rows, int path, int device, void* stream) {
    na2d_args a = dense_args(NA2D_OP_2D, B, N, H, W, C, kernel_size, dtype, rows, path, device, stream);
    a.q = dense(q); a.k = dense(k); a.v = dense(v); a.lse = const_cast<float*>(lse);
    a.d_o = dense(d_o); a.delta = const_cast<float*>(delta); a.d_k = dense(d_k); a.d_v = dense(d_v);
    return na2d_backward_dkdv_ex(&a);
}

int na2d_backward(const void* q, const void* k, const void* v, const void* o, const float* lse,
                  const void* d_o, void* d_q, void* d_k, void* d_v, float* delta,
                  int B, int N, int H, int W, int C, int kernel_size, int dtype,
                  const na2d_rows* rows, int path, int device, void* stream) {
    na2d_args a = dense_args(NA2D_OP_2D, B, N, H, W, C, kernel_size, dtype, rows, path, device, stream);
    a.q = dense(q); a.k = dense(k); a.v = dense(v); a.o = dense(o); a.lse = const_cast<float*>(lse);
    a.d_o = dense(d_o); a.d_q = dense(d_q); a.d_k = dense(d_k); a.d_v = dense(d_v); a.delta = delta;
    return na2d_backward_ex(&a);
}

int na1d_forward(const void* q, const void* k, const void* v, void* o, float* lse,
                 int B, int N, int T, int C, int kernel_size, int dtype, int device, void* stream) {
    na2d_args a = dense_args(NA2D_OP_1D, B, N, 1, T, C, kernel_size, dtype, nullptr, NA2D_PATH_AUTO, device, stream);
    a.q = dense(q); a.k = dense(k); a.v = dense(v); a.o = dense(o); a.lse = lse;
    return na2d_forward_ex(&a);
}

int na1d_backward(const void* q, const void* k, const void* v, const void* o, const float* lse,
                  const void* d_o, void* d_q, void* d_k, void* d_v, float* delta,
                  int B, int N, int T, int C, int kernel_size, int dtype, int device, void* stream) {
    na2d_args a = dense_args(NA2D_OP_1D, B, N, 1, T, C, kernel_size, dtype, nullptr, NA2D_PATH_AUTO, device, stream);
    a.q = dense(q); a.k = dense(k); a.v = dense(v); a.o = dense(o); a.lse = const_cast<float*>(lse);
    a.d_o = dense(d_o); a.d_q = dense(d_q); a.d_k = dense(d_k); a.d_v = dense(d_v); a.delta = delta;
    return na2d_backward_ex(&a);
}

// ---- the unfused pair -------------------------------------------------------------------------------------------
int na2d_qk_forward(const void* q, const void* k, void* attn,
                    int B, int N, int H, int W, int C, int kernel_size, int dtype, int device, void* stream) {
    if (!q || !k || !attn) return NA2D_ERR_BAD_ARG;
    return enter_pair(B, N, H, W, C, kernel_size, dtype, device, stream,
                      [&](const PairProblem& p) { return pair_dot(p, q, k, attn); });
}

int na2d_qk_backward(const void* q, const void* k, const void* d_attn, void* d_q, void* d_k,
                     int B, int N, int H, int W, int C, int kernel_size, int dtype, int device, void* stream) {
    if (!q || !k || !d_attn || !d_q || !d_k) return NA2D_ERR_BAD_ARG;
    return enter_pair(B, N, H, W, C, kernel_size, dtype, device, stream, [&](const PairProblem& p) {
        int rc = pair_apply(p, d_attn, k, d_q);
        if (rc != NA2D_OK) return rc;
        return pair_inverse(p, d_attn, q, d_k);
    });
}

int na2d_av_forward(const void* attn, const void* v, void* out,
                    int B, int N, int H, int W, int C, int kernel_size, int dtype, int device, void* stream) {
    if (!attn || !v || !out) return NA2D_ERR_BAD_ARG;
    return enter_pair(B, N, H, W, C, kernel_size, dtype, device, stream,
                      [&](const PairProblem& p) { return pair_apply(p, attn, v, out); });
}

int na2d_av_backward(const void* attn, const void* v, const void* d_out, void* d_attn, void* d_v,
                     int B, int N, int H, int W, int C, int kernel_size, int dtype, int device, void* stream) {
    if (!attn || !v || !d_out || !d_attn || !d_v) return NA2D_ERR_BAD_ARG;
    return enter_pair(B, N, H, W, C, kernel_size, dtype, device, stream, [&](const PairProblem& p) {
        int rc = pair_dot(p, d_out, v, d_attn);
        if (rc != NA2D_OK) return rc;
        return pair_inverse(p, attn, d_out, d_v);
    });
}

int na2d_backward_static_scratch(const void* q, const void* k, const void* v, const void* o, const float* lse,
                                 const void* d_o, void* d_q, void* d_k, void* d_v,
                                 int B, int N, int H, int W, int C, int kernel_size, int dtype,
                                 const na2d_rows* rows, int path, int device, void* stream) {
    if (B <= 0 || N <= 0 || H <= 0 || W <= 0) return NA2D_ERR_BAD_ARG;
    const long long hq = rows ? rows->Hq : H;
    if (hq <= 0) return NA2D_ERR_BAD_ARG;
    if ((long long)B * N * hq * W > kStaticDeltaFloats) {
        snprintf(t_cuda_err, sizeof(t_cuda_err),
                 "na2d_backward_static_scratch: B*N*Hq*W = %lld exceeds the built-in scratch of %lld floats",
                 (long long)B * N * hq * W, kStaticDeltaFloats);
        return NA2D_ERR_TOO_LARGE;
    }
    float* delta = nullptr;
    {
        DeviceScope scope(device);                        // the lookup needs `device` current
        if (scope.err != cudaSuccess) return cuda_fail(scope.err, "cudaSetDevice");
        int rc = static_delta_address(device, &delta);
        if (rc != NA2D_OK) return rc;
    }
    // delta is fully rewritten by the query half for every query of this call before the key
    // half reads it, so nothing has to be cleared between calls.
    return na2d_backward(q, k, v, o, lse, d_o, d_q, d_k, d_v, delta, B, N, H, W, C, kernel_size, dtype,
                         rows, path, device, stream);
}

int na2d_check(int device, void* stream) {
    DeviceScope scope(device);
    if (scope.err != cudaSuccess) return cuda_fail(scope.err, "cudaSetDevice");
    unsigned int* addr = nullptr;
    int rc = error_word_address(device, &addr);
    if (rc != NA2D_OK) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    unsigned int word = 0;
    NA2D_CUDA(cudaMemcpyAsync(&word, addr, sizeof(word), cudaMemcpyDeviceToHost, st));
    NA2D_CUDA(cudaStreamSynchronize(st));
    if (word != 0) {
        NA2D_CUDA(cudaMemsetAsync(addr, 0, sizeof(word), st));
        NA2D_CUDA(cudaStreamSynchronize(st));
        snprintf(t_cuda_err, sizeof(t_cuda_err),
                 "device error word 0x%x (1: load wait, 2: MMA wait, 4: other wait, 8: shared memory base not 1024-byte aligned)", word);
        return NA2D_ERR_KERNEL_WAIT;
    }
    return NA2D_OK;
}

int na2d_poll(int device, void* stream) {
    if (device < 0 || device >= kMaxDevices) return NA2D_ERR_BAD_ARG;
    DeviceScope scope(device);
    if (scope.err != cudaSuccess) return cuda_fail(scope.err, "cudaSetDevice");
    unsigned int* addr = nullptr;
    int rc = error_word_address(device, &addr);
    if (rc != NA2D_OK) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    std::lock_guard<std::mutex> lock(g_poll_mu);
    PollState& ps = g_poll[device];
    if (ps.host == nullptr) {
        void* h = nullptr;
        NA2D_CUDA(cudaHostAlloc(&h, sizeof(unsigned int), cudaHostAllocDefault));
        ps.host = static_cast<unsigned int*>(h);
        *ps.host = 0;
        NA2D_CUDA(cudaEventCreateWithFlags(&ps.ev, cudaEventDisableTiming));
    }
    int result = NA2D_OK;
    if (ps.pending) {
        cudaError_t e = cudaEventQuery(ps.ev);
        if (e == cudaErrorNotReady) return NA2D_OK;           // the previous copy is still on its way
        if (e != cudaSuccess) return cuda_fail(e, "cudaEventQuery");
        ps.pending = false;
        if (*ps.host != 0) {
            result = NA2D_ERR_KERNEL_WAIT;
            NA2D_CUDA(cudaMemsetAsync(addr, 0, sizeof(unsigned int), st));
        }
    }
    NA2D_CUDA(cudaMemcpyAsync(ps.host, addr, sizeof(unsigned int), cudaMemcpyDeviceToHost, st));
    NA2D_CUDA(cudaEventRecord(ps.ev, st));
    ps.pending = true;
    return result;
}

int na2d_selftest_wait_timeout(int device, void* stream, unsigned int limit_us) {
    DeviceScope scope(device);
    if (scope.err != cudaSuccess) return cuda_fail(scope.err, "cudaSetDevice");
    int rc = check_device(device);
    if (rc != NA2D_OK) return rc;
    if (limit_us == 0 || limit_us > 1000000u) return NA2D_ERR_BAD_ARG;       // at most a second
    unsigned int* addr = nullptr;
    rc = error_word_address(device, &addr);
    if (rc != NA2D_OK) return rc;
    wait_timeout_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(addr, (unsigned long long)limit_us * 1000ull);
    return after_launch();
}

long long na2d_launch_count(void) { return g_launches.load(); }

}  // extern "C"
