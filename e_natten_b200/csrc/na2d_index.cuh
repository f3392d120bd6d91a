// Window index math shared by the host entry points and every kernel.
//
// These three functions are the bit-exact contract with e_natten: they restate
// get_window_start (e_natten/pytorch.py:7-11, device twin e_natten/triton.py:7-12),
// get_backward_window_start (e_natten/pytorch.py:13-17) and get_backward_window_end
// (e_natten/pytorch.py:19-23) in integer arithmetic only.
#pragma once

#if defined(__CUDACC__)
#define NA2D_HD __host__ __device__ __forceinline__
#else
#define NA2D_HD inline
#endif

// Origin of the kernel_size-wide window of pixel i on an axis of seq_len pixels: centred on
// i, shifted inwards at the borders so that it never leaves the axis.
NA2D_HD int na2d_ws(int i, int seq_len, int kernel_size) {
    const int half = kernel_size / 2;
    int start = i - half;
    if (start < 0) start = 0;
    if (i + half >= seq_len) start += seq_len - i - half - 1;
    return start;
}

// First query index whose window holds key j.
NA2D_HD int na2d_bws(int j, int kernel_size) {
    return j < kernel_size ? 0 : j - kernel_size / 2;
}

// One past the last query index whose window holds key j.
NA2D_HD int na2d_bwe(int j, int seq_len, int kernel_size) {
    return j >= seq_len - kernel_size ? seq_len : j + kernel_size / 2 + 1;
}

// Geometry of one call, passed by value to every kernel.
struct Na2dGeom {
    int BN;        // batch * heads
    int N;         // heads (a unit index bn is batch bn / N, head bn % N)
    unsigned n_magic;   // floor(2^32 / N) + 1 where bn / N == umulhi(bn, n_magic) for every unit, else 0
    int Hq;        // query-side rows held
    int Hkv;       // key-side rows held
    int W;         // grid columns
    int C;         // head dim
    int ks;        // kernel size (odd); the window is kh x ks
    int kh;        // window rows: ks for the 2D operator, 1 for the 1D operator (a one-row image)
    int q_row0;    // global row of query-side row 0
    int kv_row0;   // global row of key-side row 0
    int Hg;        // rows of the whole image
    int patch;     // SIMT kernels: pixels per block, 64 (8 per warp) or 8 (1 per warp, small grids)
    float scale;   // softmax scale: the logits are scale * (q . k)
    float sl2;     // scale * log2(e)
};

// Magic multiplier for unit_index / heads: with m = floor(2^32 / N) + 1, umulhi(x, m) == x / N for
// every x with x * N < 2^32.  0 where that does not cover the units (or N == 1): divide then.
NA2D_HD unsigned na2d_heads_magic(long long BN, int N) {
    if (N <= 1 || BN * (long long)N >= (1ll << 32)) return 0u;
    return (unsigned)((1ull << 32) / (unsigned long long)N) + 1u;
}

// Element strides of one (batch, heads, rows, columns, channels) tensor; the channel stride is 1.
struct Na2dStride {
    long long b, n, h, w;
};
