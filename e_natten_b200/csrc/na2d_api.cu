// C ABI of libna2d.so (declared in include/na2d.h): argument checking, device selection and
// dispatch to the SIMT or tcgen05 kernels.  No framework headers; plain pointers and sizes.
#include <cuda_runtime.h>

#include <atomic>
#include <cstdio>
#include <cstring>
#include <mutex>

#include "../../include/na2d.h"
#include "na2d_index.cuh"
#include "na2d_simt.cuh"
#include "na2d_tc.cuh"

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

// Compute-capability check, cached per device.
int check_device(int device) {
    static std::mutex mu;
    static int state[64];   // 0 unknown, 1 ok, 2 not sm_100
    if (device < 0 || device >= 64) return NA2D_ERR_BAD_ARG;
    std::lock_guard<std::mutex> lock(mu);
    if (state[device] == 0) {
        int major = 0;
        cudaError_t e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device);
        if (e != cudaSuccess) { cuda_fail(e, "cudaDeviceGetAttribute"); return NA2D_ERR_NO_DEVICE; }
        state[device] = (major == 10) ? 1 : 2;
    }
    return state[device] == 1 ? NA2D_OK : NA2D_ERR_NO_DEVICE;
}

struct Problem {
    Na2dGeom g;
    int dtype;
    bool tensor;      // run the tcgen05 kernels
};

int make_problem(int B, int N, int H, int W, int C, int ks, int dtype, const na2d_rows* rows,
                 int path, Problem* out) {
    if (B <= 0 || N <= 0 || H <= 0 || W <= 0 || C <= 0) return NA2D_ERR_BAD_ARG;
    if (ks <= 0 || (ks & 1) == 0) return NA2D_ERR_BAD_ARG;
    if (dtype != NA2D_F32 && dtype != NA2D_BF16 && dtype != NA2D_F16) return NA2D_ERR_UNSUPPORTED;
    if (path != NA2D_PATH_AUTO && path != NA2D_PATH_SIMT && path != NA2D_PATH_TENSOR) return NA2D_ERR_BAD_ARG;
    if ((long long)B * N > 0x7fffffffLL) return NA2D_ERR_TOO_LARGE;
    Na2dGeom g;
    g.BN = B * N; g.W = W; g.C = C; g.ks = ks;
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
    if (na2d_ws(g.q_row0, g.Hg, ks) < g.kv_row0) return NA2D_ERR_WINDOW;
    if (na2d_ws(g.q_row0 + g.Hq - 1, g.Hg, ks) + ks > g.kv_row0 + g.Hkv) return NA2D_ERR_WINDOW;

    const bool tc_ok = na2d_tc::supported(dtype, C, ks);
    bool tensor = false;
    if (path == NA2D_PATH_TENSOR) {
        if (!tc_ok) return NA2D_ERR_UNSUPPORTED;
        tensor = true;
    } else if (path == NA2D_PATH_AUTO) {
        tensor = tc_ok;
    }
    if (!tensor && (C > na2d_simt::kMaxC || ks > na2d_simt::kMaxKs)) return NA2D_ERR_UNSUPPORTED;
    out->g = g; out->dtype = dtype; out->tensor = tensor;
    return NA2D_OK;
}

long long blocks_for(long long items) { return (items + na2d_simt::kWarps - 1) / na2d_simt::kWarps; }

template <typename T>
int simt_forward(const Problem& p, const void* q, const void* k, const void* v, void* o, float* lse,
                 cudaStream_t st) {
    const Na2dGeom& g = p.g;
    const long long nq = (long long)g.BN * g.Hq * g.W;
    const long long nb = blocks_for(nq);
    if (nb > 0x7fffffffLL) return NA2D_ERR_TOO_LARGE;
    const size_t smem = na2d_simt::fwd_smem_bytes(g.C, g.ks);
    na2d_simt::fwd_kernel<T><<<(unsigned)nb, na2d_simt::kWarps * 32, smem, st>>>(
        (const T*)q, (const T*)k, (const T*)v, (T*)o, lse, g);
    g_launches.fetch_add(1);
    NA2D_CUDA(cudaGetLastError());
    return NA2D_OK;
}

template <typename T>
int simt_backward_dq(const Problem& p, const void* q, const void* k, const void* v,
                     const float* lse, const void* d_o, void* d_q, float* delta, cudaStream_t st) {
    const Na2dGeom& g = p.g;
    const long long nq = (long long)g.BN * g.Hq * g.W;
    if (blocks_for(nq) > 0x7fffffffLL) return NA2D_ERR_TOO_LARGE;
    na2d_simt::dq_kernel<T><<<(unsigned)blocks_for(nq), na2d_simt::kWarps * 32,
                              na2d_simt::dq_smem_bytes(g.C, g.ks), st>>>(
        (const T*)q, (const T*)k, (const T*)v, lse, (const T*)d_o, (T*)d_q, delta, g);
    g_launches.fetch_add(1);
    NA2D_CUDA(cudaGetLastError());
    return NA2D_OK;
}

template <typename T>
int simt_backward_dkdv(const Problem& p, const void* q, const void* k, const void* v, const float* lse,
                       const void* d_o, const float* delta, void* d_k, void* d_v, cudaStream_t st) {
    const Na2dGeom& g = p.g;
    const long long nkey = (long long)g.BN * g.Hkv * g.W;
    if (blocks_for(nkey) > 0x7fffffffLL) return NA2D_ERR_TOO_LARGE;
    na2d_simt::dkdv_kernel<T><<<(unsigned)blocks_for(nkey), na2d_simt::kWarps * 32,
                                na2d_simt::dkdv_smem_bytes(g.C), st>>>(
        (const T*)q, (const T*)k, (const T*)v, lse, (const T*)d_o, delta, (T*)d_k, (T*)d_v, g);
    g_launches.fetch_add(1);
    NA2D_CUDA(cudaGetLastError());
    return NA2D_OK;
}

// ---- scratch for na2d_backward_static_scratch ----------------------------------------------------
// The backward pair passes the row delta from the dQ kernel to the dK/dV kernel through global
// memory.  Normally the caller provides that buffer; the entry point below keeps it in this
// file-scope device array instead, so that a caller who may not allocate can still run the
// backward.  Every GPU that loads the library carries the array (4 MiB) until the process exits.
constexpr long long kStaticDeltaFloats = 1LL << 20;
static __device__ __align__(256) float g_static_delta[kStaticDeltaFloats];

// Device address of g_static_delta on `device`, looked up once per device.  In host code the
// name g_static_delta is only a handle for the runtime, not an address a kernel could use; the
// address comes from cudaGetSymbolAddress, asked while `device` is the current device.
int static_delta_address(int device, float** out) {
    static std::mutex mu;
    static float* cache[64];
    if (device < 0 || device >= 64) return NA2D_ERR_BAD_ARG;
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

// Common prologue of the compute entry points: validate, select the device, check it.
#define NA2D_ENTER()                                                                      \
    Problem p;                                                                            \
    int rc = make_problem(B, N, H, W, C, kernel_size, dtype, rows, path, &p);             \
    if (rc != NA2D_OK) return rc;                                                         \
    DeviceScope scope(device);                                                            \
    if (scope.err != cudaSuccess) return cuda_fail(scope.err, "cudaSetDevice");           \
    rc = check_device(device);                                                            \
    if (rc != NA2D_OK) return rc;                                                         \
    cudaStream_t st = (cudaStream_t)stream;

}  // namespace

extern "C" {

int na2d_version(void) { return 100; }

const char* na2d_strerror(int status) {
    switch (status) {
        case NA2D_OK: return "ok";
        case NA2D_ERR_BAD_ARG: return "bad argument (null pointer, non-positive size, even kernel size or bad row view)";
        case NA2D_ERR_UNSUPPORTED: return "unsupported dtype, head dim or kernel size for the requested path";
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
    g_launches.fetch_add(1);
    NA2D_CUDA(cudaGetLastError());
    return NA2D_OK;
}

int na2d_forward(const void* q, const void* k, const void* v, void* o, float* lse,
                 int B, int N, int H, int W, int C, int kernel_size, int dtype,
                 const na2d_rows* rows, int path, int device, void* stream) {
    if (!q || !k || !v || !o || !lse) return NA2D_ERR_BAD_ARG;
    NA2D_ENTER();
    if (p.tensor) {
        int launched = 0;
        rc = na2d_tc::forward(p.g, dtype, q, k, v, o, lse, device, st, &launched);
        g_launches.fetch_add(launched);
        if (rc == NA2D_ERR_CUDA) return tc_fail("tcgen05 forward launch");
        return rc;
    }
    switch (dtype) {
        case NA2D_F32: return simt_forward<float>(p, q, k, v, o, lse, st);
        case NA2D_BF16: return simt_forward<__nv_bfloat16>(p, q, k, v, o, lse, st);
        default: return simt_forward<__half>(p, q, k, v, o, lse, st);
    }
}

int na2d_backward_dq(const void* q, const void* k, const void* v, const void* o, const float* lse,
                     const void* d_o, void* d_q, float* delta,
                     int B, int N, int H, int W, int C, int kernel_size, int dtype,
                     const na2d_rows* rows, int path, int device, void* stream) {
    (void)o;   // not read: delta is formed as sum_j p_j dp_j, see the header
    if (!q || !k || !v || !lse || !d_o || !delta) return NA2D_ERR_BAD_ARG;
    NA2D_ENTER();
    if (p.tensor) {
        int launched = 0;
        rc = na2d_tc::backward_dq(p.g, dtype, q, k, v, o, lse, d_o, d_q, delta, device, st, &launched);
        g_launches.fetch_add(launched);
        if (rc == NA2D_ERR_CUDA) return tc_fail("tcgen05 dQ launch");
        return rc;
    }
    switch (dtype) {
        case NA2D_F32: return simt_backward_dq<float>(p, q, k, v, lse, d_o, d_q, delta, st);
        case NA2D_BF16: return simt_backward_dq<__nv_bfloat16>(p, q, k, v, lse, d_o, d_q, delta, st);
        default: return simt_backward_dq<__half>(p, q, k, v, lse, d_o, d_q, delta, st);
    }
}

int na2d_backward_dkdv(const void* q, const void* k, const void* v, const float* lse,
                       const void* d_o, const float* delta, void* d_k, void* d_v,
                       int B, int N, int H, int W, int C, int kernel_size, int dtype,
                       const na2d_rows* rows, int path, int device, void* stream) {
    if (!q || !k || !v || !lse || !d_o || !delta || !d_k || !d_v) return NA2D_ERR_BAD_ARG;
    NA2D_ENTER();
    if (p.tensor) {
        int launched = 0;
        rc = na2d_tc::backward_dkdv(p.g, dtype, q, k, v, lse, d_o, delta, d_k, d_v, device, st, &launched);
        g_launches.fetch_add(launched);
        if (rc == NA2D_ERR_CUDA) return tc_fail("tcgen05 dK/dV launch");
        return rc;
    }
    switch (dtype) {
        case NA2D_F32: return simt_backward_dkdv<float>(p, q, k, v, lse, d_o, delta, d_k, d_v, st);
        case NA2D_BF16: return simt_backward_dkdv<__nv_bfloat16>(p, q, k, v, lse, d_o, delta, d_k, d_v, st);
        default: return simt_backward_dkdv<__half>(p, q, k, v, lse, d_o, delta, d_k, d_v, st);
    }
}

int na2d_backward(const void* q, const void* k, const void* v, const void* o, const float* lse,
                  const void* d_o, void* d_q, void* d_k, void* d_v, float* delta,
                  int B, int N, int H, int W, int C, int kernel_size, int dtype,
                  const na2d_rows* rows, int path, int device, void* stream) {
    if ((d_k == nullptr) != (d_v == nullptr)) return NA2D_ERR_BAD_ARG;
    if (!d_q && !d_k) return NA2D_ERR_BAD_ARG;
    // the query half always runs: it produces delta, which the key half needs
    int rc = na2d_backward_dq(q, k, v, o, lse, d_o, d_q, delta, B, N, H, W, C, kernel_size, dtype,
                              rows, path, device, stream);
    if (rc != NA2D_OK || d_k == nullptr) return rc;
    return na2d_backward_dkdv(q, k, v, lse, d_o, delta, d_k, d_v, B, N, H, W, C, kernel_size, dtype,
                              rows, path, device, stream);
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
    unsigned int word = 0;
    int rc = na2d_tc::read_and_clear_error(&word, (cudaStream_t)stream);
    if (rc != NA2D_OK) return cuda_fail(cudaGetLastError(), "error word readback");
    return word == 0 ? NA2D_OK : NA2D_ERR_KERNEL_WAIT;
}

long long na2d_launch_count(void) { return g_launches.load(); }

#ifdef NA2D_TRACE
// Development aid: copies the trace of CTA 0 of the last kernels to the host and clears it.
int na2d_debug_trace(unsigned long long* out, int max_entries) {
    unsigned int n = 0;
    cudaDeviceSynchronize();
    cudaMemcpyFromSymbol(&n, na2d_tc::g_trace_n, sizeof(n));
    if ((int)n > max_entries) n = max_entries;
    if (n > 8192) n = 8192;
    cudaMemcpyFromSymbol(out, na2d_tc::g_trace, n * sizeof(unsigned long long));
    void* arr = nullptr;
    if (cudaGetSymbolAddress(&arr, na2d_tc::g_trace) == cudaSuccess) cudaMemset(arr, 0, sizeof(na2d_tc::g_trace));
    return (int)n;
}
#endif

}  // extern "C"
