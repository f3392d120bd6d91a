/*
 * na2d.h -- C ABI of libna2d.so: fused neighborhood attention for NVIDIA B200 (sm_100a).
 *
 * Every entry point takes plain device pointers and sizes; there are no framework types
 * in the signatures.  Tensors are (B, N, H, W, C) = batch, heads, grid rows, grid columns,
 * head dim, C fastest -- the layout e_natten's fused entry point uses
 * (e_natten/triton.py:500).  The plain entry points take dense, row-major tensors; the *_ex
 * entry points take element strides per tensor (channels contiguous) and a softmax scale.
 * All functions return 0 on success or a negative na2d_status; nothing aborts, nothing traps
 * on the device.  Kernels are launched on the given stream of the given device and the call
 * returns without synchronising.
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
    NA2D_ERR_KERNEL_WAIT = -7     /* a bounded wait inside a kernel ran out (na2d_check, na2d_poll) */
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
 * exactly and is independent of the rounding o went through when it was stored.  `o` may be
 * NULL (the reference's backward ignores the saved o too, e_natten/triton.py:522).  Where it is
 * given, the tensor-core dQ kernel of kernel sizes >= 7 uses dO . o as a first estimate of delta,
 * which lets it walk a query tile's keys once instead of twice; the result, and the delta it
 * writes, are corrected to the exact values either way.  Replaces the dQ part of
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
 * over the local query band only; for this call the key band may be any rows of the image (it
 * need not hold the query band's windows), so a caller can take the key rows in several calls. */
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

/* ---- Strided tensors, softmax scale, the 1D operator: the *_ex entry points ----------------
 *
 * The reference applies no softmax scale (e_natten/triton.py:280: the caller multiplies q by
 * head_dim^-0.5 in a pass of its own) and refuses tensors whose batch / head strides differ from
 * q's (e_natten/triton.py:233-234, 316-319), so a (B, H, W, 3, heads, C) packed-qkv projection
 * has to be copied three times before the call.  Here the scale is an argument, folded into the
 * kernels' exponent, and every tensor carries its own element strides, which the tensor-core
 * kernels put straight into their TMA tensor maps.
 *
 * na2d_tensor: device pointer plus element strides of the batch, head, row and column
 * dimensions; the channel stride is 1.  All four strides zero means dense (B, N, rows, W, C).
 * For the tensor-core kernels the pointer must be 16-byte aligned and every stride a multiple of
 * 8 elements; other layouts run on the SIMT kernels under NA2D_PATH_AUTO and are refused with
 * NA2D_ERR_UNSUPPORTED under NA2D_PATH_TENSOR (a caller who wants the fast path makes a dense
 * copy first).
 *
 * na2d_args: one struct for all four calls; set struct_size = sizeof(na2d_args) and zero what a
 * call does not use.
 *   op        NA2D_OP_2D: the 2D operator.  NA2D_OP_1D: the 1D operator of the reference
 *             (natten1d, e_natten/triton.py:425-485, 65-222) on (B, N, T, C) tensors: pass H = 1,
 *             W = T, the row stride is ignored, the window is 1 x kernel_size, rows must be NULL.
 *   scale     logits are scale * (q . k); must be > 0; 1.0f reproduces the reference.
 *   o         output of the forward; optional input of the backward (see na2d_backward_dq).
 *   flags     NA2D_FLAG_DKDV_F32: the key half writes dK and dV in fp32.  Meant for row views: the
 *             dK / dV of a band are partial sums that their owner adds to its own, and partial
 *             sums can be far larger than the total, so rounding each of them to 16 bits first
 *             costs accuracy.  NA2D_FLAG_SM_MARGIN(n): leave n SMs to a concurrent kernel.
 *   lse       fp32 (B, N, Hq, W), dense: written by the forward, read by the backward.
 *   delta     fp32 (B, N, Hq, W), dense scratch of the backward.
 */
typedef struct na2d_tensor {
    void* ptr;
    int64_t stride_b, stride_n, stride_h, stride_w;
} na2d_tensor;

typedef enum na2d_op {
    NA2D_OP_2D = 0,
    NA2D_OP_1D = 1
} na2d_op;

/* na2d_args.flags */
#define NA2D_FLAG_DKDV_F32 1   /* d_k, d_v are fp32 tensors (strides in fp32 elements) whatever `dtype` is */
/* Bits 8..15: SMs to leave free.  The tensor-core kernels are persistent, one CTA per SM, and a CTA
 * takes nearly all of an SM's shared memory: a communication kernel launched beside them (the halo
 * exchange of the row-sharded mode) finds no SM until they end.  A launch that should overlap with
 * one asks for n fewer CTAs.  0 = use every SM. */
#define NA2D_FLAG_SM_MARGIN(n) (((n) & 0xff) << 8)

typedef struct na2d_args {
    size_t struct_size;
    int op;
    int B, N, H, W, C, kernel_size, dtype, path, device;
    int flags;
    float scale;
    void* stream;
    const na2d_rows* rows;
    na2d_tensor q, k, v, o, d_o, d_q, d_k, d_v;
    float* lse;
    float* delta;
} na2d_args;

/* As na2d_forward; writes a->o and a->lse.
 * Replaces Natten2d.forward (e_natten/triton.py:489-518) and Natten1d.forward (425-452). */
int na2d_forward_ex(const na2d_args* a);
/* As na2d_backward_dq; a->d_q.ptr may be NULL (delta only). */
int na2d_backward_dq_ex(const na2d_args* a);
/* As na2d_backward_dkdv. */
int na2d_backward_dkdv_ex(const na2d_args* a);
/* As na2d_backward: both halves.  Replaces Natten2d.backward (e_natten/triton.py:521-548) and
 * Natten1d.backward (454-483). */
int na2d_backward_ex(const na2d_args* a);

/* ---- 1D operator, dense tensors (B, N, T, C) ------------------------------------------------
 * natten1d of the reference: e_natten/triton.py:425-485 (autograd wrapper), 65-141 and 143-222
 * (kernels), e_natten/pytorch.py:46-156 (loop restatement).  Window = kernel_size consecutive
 * tokens at the clamped origin.  lse and delta are fp32 (B, N, T). */
int na1d_forward(const void* q, const void* k, const void* v, void* o, float* lse,
                 int B, int N, int T, int C, int kernel_size, int dtype, int device, void* stream);
int na1d_backward(const void* q, const void* k, const void* v, const void* o, const float* lse,
                  const void* d_o, void* d_q, void* d_k, void* d_v, float* delta,
                  int B, int N, int T, int C, int kernel_size, int dtype, int device, void* stream);

/* ---- The unfused pair ------------------------------------------------------------------------
 * The two-step neighborhood attention the reference's test and benchmark compare the fused
 * operator with (natten2dqk + softmax + natten2dav, dilation 1: test.py:17-21, bench.py:23,
 * 52-54).  attn is (B, N, H, W, kernel_size^2) in the tensors' dtype, window member j at window
 * row j / kernel_size, column j % kernel_size of the clamped window; the softmax between the two
 * steps is the caller's.  Dense tensors, whole images.
 *   na2d_qk_forward    attn = q . k over the window
 *   na2d_qk_backward   dQ = sum_j d_attn_j k_j;  dK_j = sum over the inverse neighbourhood of d_attn q
 *   na2d_av_forward    out = sum_j attn_j v_j
 *   na2d_av_backward   d_attn_j = dOut . v_j;  dV_j = sum over the inverse neighbourhood of attn dOut */
int na2d_qk_forward(const void* q, const void* k, void* attn,
                    int B, int N, int H, int W, int C, int kernel_size, int dtype, int device, void* stream);
int na2d_qk_backward(const void* q, const void* k, const void* d_attn, void* d_q, void* d_k,
                     int B, int N, int H, int W, int C, int kernel_size, int dtype, int device, void* stream);
int na2d_av_forward(const void* attn, const void* v, void* out,
                    int B, int N, int H, int W, int C, int kernel_size, int dtype, int device, void* stream);
int na2d_av_backward(const void* attn, const void* v, const void* d_out, void* d_attn, void* d_v,
                     int B, int N, int H, int W, int C, int kernel_size, int dtype, int device, void* stream);

/* Backward for callers that cannot allocate device memory.  No counterpart in the reference.
 *
 * Same computation and arguments as na2d_backward, minus `delta`: the B*N*Hq*W floats of row
 * deltas that the dQ kernel hands to the dK/dV kernel live in an array built into the library
 * (4 MiB of device memory per GPU).  It is meant for code that runs where cudaMalloc is off
 * limits: a plugin inside a runtime whose arena already owns all of the GPU's memory and hands
 * out no workspace, or a step that must not take the device-wide synchronisation that
 * cudaMalloc / cudaFree imply.  The call itself performs no cudaMalloc, cudaFree or other
 * allocating call; inputs and outputs are still the caller's.
 *
 * Limits and rules:
 *  - B*N*Hq*W <= NA2D_STATIC_SCRATCH_FLOATS (1,048,576; e.g. B4 N4 256x256).  Larger problems
 *    return NA2D_ERR_TOO_LARGE (na2d_last_cuda_error() has the numbers); use na2d_backward.
 *  - The array comes into being when the CUDA runtime loads the library's device code into the
 *    device's context, which (with lazy loading, the default of CUDA 12) is at the first library
 *    call on that device, not when the .so is opened.  That first call is therefore the one
 *    that can fail for lack of memory, and it also looks up the array's device address (a
 *    host-side runtime query).  Make one warm-up call on each device at start-up - before an
 *    arena takes the rest of the memory, and outside any stream capture; from then on the array
 *    is held until the process exits and later calls allocate nothing.
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

/* The same check without waiting for the GPU: enqueues a copy of the error word to a pinned host
 * word on `stream` and returns what the previous such copy on this device brought back
 * (NA2D_OK if none has completed yet).  A caller that polls at every entry learns of a tripped
 * wait one call late but never stalls; the host word is allocated at the first poll on a device.
 * Once reported, the error is cleared.  No reference counterpart. */
int na2d_poll(int device, void* stream);

/* Self-test of the bounded waits: launches one small kernel whose only thread waits, with a limit
 * of limit_us microseconds, on a barrier that nothing ever completes.  The wait gives up, the
 * kernel records that in the error word and ends normally; the next na2d_check / na2d_poll
 * reports NA2D_ERR_KERNEL_WAIT.  Nothing faults, traps or hangs.  No reference counterpart. */
int na2d_selftest_wait_timeout(int device, void* stream, unsigned int limit_us);

/* Number of kernels the library has launched in this process so far.  No reference
 * counterpart; the benchmark reports it. */
long long na2d_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* NA2D_H_ */
