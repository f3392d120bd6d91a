/*
 * na2d.h -- C ABI of libna2d.so: fused 2D neighborhood attention for NVIDIA B200 (sm_100a).
 *
 * Every entry point takes plain device pointers and sizes; there are no framework types
 * in the signatures.  Tensors are dense, row-major (B, N, H, W, C) = batch, heads, grid rows,
 * grid columns, head dim, C fastest -- the layout e_natten's fused entry point uses
 * (e_natten/triton.py:500).  All functions return 0 on success or a negative na2d_status;
 * nothing aborts, nothing traps on the device.  Kernels are launched on the given stream of
 * the given device and the call returns without synchronising.
 *
 * Row views.  A caller that holds only a band of image rows (a row shard of one huge image)
 * describes it with na2d_rows: the query-side tensors (q, o, lse, dO, dQ, delta) hold global
 * rows [q_row0, q_row0 + Hq) and the key-side tensors (k, v, dK, dV) hold global rows
 * [kv_row0, kv_row0 + Hkv) of an image that is H_global rows tall; window origins are clamped
 * against H_global.  The key band must cover every window of the query band.  The whole
 * image is {0, H, 0, H, H}.
 */
#ifndef NA2D_H_
#define NA2D_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum na2d_dtype {
    NA2D_F32 = 0,
    NA2D_BF16 = 1,
    NA2D_F16 = 2
} na2d_dtype;

typedef enum na2d_status {
    NA2D_OK = 0,
    NA2D_ERR_BAD_ARG = -1,        /* null pointer, non-positive size, even kernel size ...       */
    NA2D_ERR_UNSUPPORTED = -2,    /* dtype / head dim / kernel size outside what is built        */
    NA2D_ERR_WINDOW = -3,         /* grid side smaller than the kernel size, or key band too small */
    NA2D_ERR_CUDA = -4,           /* a CUDA runtime / driver call failed; see na2d_last_cuda_error */
    NA2D_ERR_NO_DEVICE = -5,      /* no sm_100 device                                              */
    NA2D_ERR_TOO_LARGE = -6,      /* size beyond a documented maximum                              */
    NA2D_ERR_KERNEL_WAIT = -7     /* a bounded wait inside a kernel ran out (reported by na2d_check) */
} na2d_status;

/* Which implementation runs.  AUTO picks the tcgen05 tensor-core kernels for bf16/fp16 with a
 * supported head dim and kernel size, else the fp32-accumulating SIMT kernels. */
typedef enum na2d_path {
    NA2D_PATH_AUTO = 0,
    NA2D_PATH_SIMT = 1,
    NA2D_PATH_TENSOR = 2
} na2d_path;

typedef struct na2d_rows {
    int q_row0;    /* global row of the first query-side row              */
    int Hq;        /* query-side rows held                                */
    int kv_row0;   /* global row of the first key-side row                */
    int Hkv;       /* key-side rows held                                  */
    int H_global;  /* rows of the whole image (clamping uses this)        */
} na2d_rows;

/* Library version, MAJOR*10000 + MINOR*100 + PATCH.  No reference counterpart. */
int na2d_version(void);

/* Text for a status code.  Replaces the Python exceptions Triton raises for the reference
 * (e_natten/triton.py:233-234, 316-319). */
const char* na2d_strerror(int status);

/* Text of the last CUDA error seen by this thread inside the library ("" if none). */
const char* na2d_last_cuda_error(void);

/* Clamped window origin of pixel i on an axis of length seq_len.
 * Replaces get_window_start (e_natten/pytorch.py:7-11, e_natten/triton.py:7-18).  Host-side,
 * the same inline function the kernels compile. */
int na2d_window_start(int i, int seq_len, int kernel_size);

/* Half-open range [*lo, *hi) of query indices whose window holds key j.
 * Replaces get_backward_window_start / get_backward_window_end
 * (e_natten/pytorch.py:13-23, e_natten/triton.py:20-30). */
int na2d_backward_window(int j, int seq_len, int kernel_size, int* lo, int* hi);

/* Device-side evaluation of the three index functions for every i in [0, seq_len): writes
 * ws[i], bws[i], bwe[i] (device int32 arrays of seq_len entries) with the code path the
 * kernels use, so the test-suite can compare device indexing bit for bit with the
 * reference's (e_natten/triton.py:7-12). */
int na2d_dump_index(int32_t* ws, int32_t* bws, int32_t* bwe, int seq_len, int kernel_size,
                    int device, void* stream);

/* Forward: o = softmax_j(q . k_j) v_j over the kernel_size x kernel_size window at the
 * clamped origin; lse = max_j s_j + log(sum_j exp(s_j - max)) in fp32, shape (B, N, Hq, W).
 * Replaces Natten2d.forward + _attn_fwd_2d (e_natten/triton.py:489-518, 224-302), which saves
 * no lse.  o and lse are fully overwritten (no pre-zeroing needed).  rows may be NULL for a
 * whole image of H rows. */
int na2d_forward(const void* q, const void* k, const void* v, void* o, float* lse,
                 int B, int N, int H, int W, int C, int kernel_size, int dtype,
                 const na2d_rows* rows, int path, int device, void* stream);

/* Backward, query half: dQ (optional, may be NULL) and the row delta, fp32 of B*N*Hq*W entries,
 * which the key half reads.  delta is formed as sum_j p_j (dO . v_j), which equals dO . o
 * exactly and is independent of the rounding o went through when it was stored; `o` is
 * therefore accepted for interface symmetry but not read (it may be NULL), as in the reference,
 * whose backward ignores the saved o (e_natten/triton.py:522).  Replaces the dQ part of
 * Natten2d.backward + _attn_bwd_2d (e_natten/triton.py:521-548, 383-409).  dQ is fully
 * overwritten. */
int na2d_backward_dq(const void* q, const void* k, const void* v, const void* o, const float* lse,
                     const void* d_o, void* d_q, float* delta,
                     int B, int N, int H, int W, int C, int kernel_size, int dtype,
                     const na2d_rows* rows, int path, int device, void* stream);

/* Backward, key half: dK and dV, each key summing over the queries whose window holds it (the
 * inverse neighbourhood of e_natten/pytorch.py:261-273).  Reads delta written by
 * na2d_backward_dq on the same stream.  Replaces the atomic-add part of _attn_bwd_2d
 * (e_natten/triton.py:412-423): no atomics, every element is written exactly once, so no
 * pre-zeroing is needed.  With a row view, dK / dV cover the key band and hold the partial sums
 * over the local query band only. */
int na2d_backward_dkdv(const void* q, const void* k, const void* v, const float* lse,
                       const void* d_o, const float* delta, void* d_k, void* d_v,
                       int B, int N, int H, int W, int C, int kernel_size, int dtype,
                       const na2d_rows* rows, int path, int device, void* stream);

/* Backward, both halves: dQ, dK, dV from q, k, v, o, lse, dO.  delta is caller-provided scratch
 * of B*N*Hq*W floats.  Replaces Natten2d.backward (e_natten/triton.py:521-548).  dQ, or dK and
 * dV together, may be NULL to skip that half. */
int na2d_backward(const void* q, const void* k, const void* v, const void* o, const float* lse,
                  const void* d_o, void* d_q, void* d_k, void* d_v, float* delta,
                  int B, int N, int H, int W, int C, int kernel_size, int dtype,
                  const na2d_rows* rows, int path, int device, void* stream);

/* Backward for callers that cannot allocate device memory.  No counterpart in the reference.
 *
 * Same computation and arguments as na2d_backward, minus `delta`: the B*N*Hq*W floats of row
 * deltas that the dQ kernel hands to the dK/dV kernel live in an array built into the library
 * (device memory reserved when the library is loaded, 4 MiB per GPU, held until the process
 * exits).  It is meant for code that runs where cudaMalloc is off limits: a plugin inside a
 * runtime whose arena already owns all of the GPU's memory and hands out no workspace, or a
 * step that must not take the device-wide synchronisation that cudaMalloc / cudaFree imply.
 * The call itself performs no cudaMalloc, cudaFree or other allocating call; inputs and outputs
 * are still the caller's.
 *
 * Limits and rules:
 *  - B*N*Hq*W <= NA2D_STATIC_SCRATCH_FLOATS (1,048,576; e.g. B4 N4 256x256).  Larger problems
 *    return NA2D_ERR_TOO_LARGE (na2d_last_cuda_error() has the numbers); use na2d_backward.
 *  - The first call on each device looks up the array's device address (a host-side runtime
 *    query, no allocation).  Make that first call outside any stream capture.
 *  - All calls on a device share the one array.  Nothing in it needs clearing between calls
 *    (every entry a call reads it has written first), but two calls whose kernels can overlap
 *    on the GPU - different streams, no ordering between them - race on it.  Order them. */
#define NA2D_STATIC_SCRATCH_FLOATS (1 << 20)
int na2d_backward_static_scratch(const void* q, const void* k, const void* v, const void* o, const float* lse,
                                 const void* d_o, void* d_q, void* d_k, void* d_v,
                                 int B, int N, int H, int W, int C, int kernel_size, int dtype,
                                 const na2d_rows* rows, int path, int device, void* stream);

/* Reads and clears the device-side error word that a kernel sets when a bounded wait
 * (mbarrier) ran out.  Synchronises the stream.  Returns NA2D_OK or NA2D_ERR_KERNEL_WAIT.
 * No reference counterpart. */
int na2d_check(int device, void* stream);

/* Number of kernels the library has launched in this process so far.  No reference
 * counterpart; the benchmark reports it. */
long long na2d_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* NA2D_H_ */
