"""GPU parity tests: the CUDA kernels, called through the C ABI, against the CPU oracle and the
fixtures produced by the reference itself.  Patterned on the reference's test.py (shapes,
loss = sum(o**2), atol 1e-5) with the comparison target replaced by the pinned oracle."""
import numpy as np
import pytest
import torch

import e_natten_b200 as na
from oracle import na2d_oracle as orc
from helpers import assert_close, make_inputs

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def run_gpu(q, k, v, d_o, ks, path="auto", rows=None, with_o=True, scale=1.0, dkdv_dtype=None):
    """(o, lse, dq, dk, dv) from the library's raw entry points.  `with_o`: hand the forward's
    output to the backward (what the autograd entry point does; the dQ kernel of the larger
    windows then takes its one-walk form); False runs the backward without it (two walks)."""
    qd, kd, vd, gd = (t.to(DEV) for t in (q, k, v, d_o))
    o, lse = na.natten2d_forward(qd, kd, vd, ks, rows=rows, path=path, scale=scale)
    dq, dk, dv = na.natten2d_backward(qd, kd, vd, o if with_o else None, lse, gd, ks, rows=rows, path=path,
                                      scale=scale, dkdv_dtype=dkdv_dtype)
    na.check_kernels(DEV)
    return o, lse, dq, dk, dv


def check_against_oracle(shape, ks, dtype, seed, path="auto", scale=1.0, q_scale=1.0, with_o=True):
    q, k, v, d_o = make_inputs(shape, dtype, seed, scale, q_scale)
    o, lse, dq, dk, dv = run_gpu(q, k, v, d_o, ks, path, with_o=with_o)
    ro, rlse, rdq, rdk, rdv = orc.natten2d_fwd_bwd(q, k, v, d_o, ks)
    tag = f"{tuple(shape)} ks={ks} {dtype} {path}"
    assert_close(o, ro, dtype, f"o {tag}")
    assert_close(lse, rlse, torch.float32 if dtype == torch.float32 else dtype, f"lse {tag}")
    assert_close(dq, rdq, dtype, f"dq {tag}")
    assert_close(dk, rdk, dtype, f"dk {tag}")
    assert_close(dv, rdv, dtype, f"dv {tag}")


# ------------------------------------------------------------------------------ index contract
@pytest.mark.parametrize("ks", list(range(3, 16, 2)))
def test_device_window_indices_bit_exact(golden, ks):
    for L in [ks, ks + 1, 2 * ks - 1, 2 * ks, 14, 16, 28, 32, 56, 64, 80, 192, 256, 1024]:
        if L < ks:
            continue
        ws, bws, bwe = na.device_index_tables(L, ks, DEV)
        assert np.array_equal(ws.cpu().numpy(), golden[f"idx/ws/{ks}/{L}"])
        assert np.array_equal(bws.cpu().numpy(), golden[f"idx/bws/{ks}/{L}"])
        assert np.array_equal(bwe.cpu().numpy(), golden[f"idx/bwe/{ks}/{L}"])


# ------------------------------------------------------------------------------ reference fixtures
def test_config1_against_reference_pytorch_fixture(golden):
    """B1 N2 16x16 C32 ks5 fp32 seed 0: outputs of e_natten.pytorch.natten2d itself."""
    g = {n: torch.from_numpy(golden[f"pt/c1/{n}"]) for n in ("q", "k", "v", "do", "o", "dk", "dv", "dq_tile00")}
    o, lse, dq, dk, dv = run_gpu(g["q"], g["k"], g["v"], g["do"], 5)
    assert_close(o, g["o"], torch.float32, "o vs reference")
    assert_close(dk, g["dk"], torch.float32, "dk vs reference")
    assert_close(dv, g["dv"], torch.float32, "dv vs reference")
    assert_close(dq[:, :, :3, :3], g["dq_tile00"], torch.float32, "dq tile (0,0) vs reference")


@pytest.mark.parametrize("name", ["k3", "k5", "k7", "k9", "k11"])
def test_against_reference_triton_fixture(golden, name):
    """Outputs of the fused e_natten.natten2d (Triton interpreter), loss = sum(o**2), atol 1e-5
    as in the reference's test.py:36-45, through the autograd entry point."""
    g = {n: torch.from_numpy(golden[f"tr/{name}/{n}"]) for n in ("q", "k", "v", "o", "dq", "dk", "dv")}
    ks = int(golden[f"tr/{name}/ks"])
    q, k, v = (g[n].to(DEV).requires_grad_() for n in ("q", "k", "v"))
    o = na.natten2d(q, k, v, ks)
    torch.sum(o ** 2).backward()
    assert torch.allclose(o.detach().cpu(), g["o"], atol=1e-5)
    assert torch.allclose(q.grad.cpu(), g["dq"], atol=2e-5)
    assert torch.allclose(k.grad.cpu(), g["dk"], atol=2e-5)
    assert torch.allclose(v.grad.cpu(), g["dv"], atol=2e-5)


@pytest.mark.parametrize("ks", [3, 5, 7, 9, 11])
def test_reference_test_script_shape(ks):
    """The reference's own 2D test case: shape (2, 6, 16, 16, 2), fp32, seed 0, loss sum(o**2)
    (test.py:5-8, 39-45, 53), compared with atol 1e-5 against the oracle."""
    torch.manual_seed(0)
    q, k, v = torch.randn(3, 2, 6, 16, 16, 2)
    qd, kd, vd = (t.to(DEV).requires_grad_() for t in (q, k, v))
    o = na.natten2d(qd, kd, vd, ks)
    torch.sum(o ** 2).backward()
    ro, _ = orc.natten2d_fwd(q, k, v, ks)
    rdq, rdk, rdv = orc.natten2d_bwd(q, k, v, 2.0 * ro, ks)
    assert torch.allclose(o.detach().cpu().double(), ro, atol=1e-5)
    assert torch.allclose(qd.grad.cpu().double(), rdq, atol=1e-5)
    assert torch.allclose(kd.grad.cpu().double(), rdk, atol=1e-5)
    assert torch.allclose(vd.grad.cpu().double(), rdv, atol=1e-5)


# ------------------------------------------------------------------------------ oracle sweeps
SMALL = [
    # shape, ks
    ((1, 1, 5, 5, 32), 5),          # window == grid
    ((1, 2, 13, 13, 64), 13),       # window == grid, large
    ((2, 1, 7, 19, 32), 7),         # H == ks, W ragged
    ((1, 2, 9, 10, 64), 3),
    ((1, 1, 17, 23, 128), 5),       # not a multiple of any tile
    ((2, 2, 16, 16, 128), 5),
    ((1, 1, 14, 14, 64), 13),       # window nearly covers the grid
    ((1, 2, 28, 28, 64), 13),
    ((1, 1, 24, 40, 32), 7),
    ((1, 1, 20, 33, 128), 9),
    ((1, 1, 33, 20, 64), 11),
]


@pytest.mark.parametrize("shape,ks", SMALL)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_simt_path_against_oracle(shape, ks, dtype):
    check_against_oracle(shape, ks, dtype, seed=100 + ks, path="simt")


@pytest.mark.parametrize("shape,ks", [((1, 2, 9, 11, 2), 5), ((1, 1, 8, 8, 3), 3), ((1, 1, 9, 9, 48), 7),
                                      ((1, 1, 8, 9, 256), 5), ((1, 1, 33, 34, 8), 15)])
def test_simt_path_odd_head_dims_and_large_kernel(shape, ks):
    check_against_oracle(shape, ks, torch.float32, seed=7, path="simt")


@pytest.mark.parametrize("shape,ks", SMALL)
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_default_path_against_oracle(shape, ks, dtype):
    """Whatever AUTO picks for 16-bit inputs (the tensor-core kernels where they are built).
    q carries the usual head_dim**-0.5 scale, as in the benchmark configuration."""
    check_against_oracle(shape, ks, dtype, seed=200 + ks, path="auto", q_scale=shape[-1] ** -0.5)


@pytest.mark.parametrize("shape,ks", SMALL)
def test_default_path_unscaled_logits_fp16(shape, ks):
    """Unscaled N(0,1) q and k (logit std = sqrt(head_dim), near one-hot softmax) on the fp16
    path, whose P / dS operands keep 11 significant bits."""
    check_against_oracle(shape, ks, torch.float16, seed=300 + ks, path="auto")


# ------------------------------------------------------------------------------ every tensor-core instantiation
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("ks", [3, 5, 7, 9, 11, 13])
@pytest.mark.parametrize("D", [32, 64, 128])
def test_every_tensor_core_instantiation(D, ks, dtype):
    """Each (head dim, kernel size, dtype) triple is a kernel family of its own (chunking, shared
    and tensor memory plan, mask constants): forward, dQ and dK/dV of every one of them against
    the oracle on a ragged grid, with and without the forward's output handed to the backward
    (kernel sizes >= 7: the one-walk and the two-walk form of the dQ kernel), and the row deltas
    of the full and of the delta-only call."""
    shape = (1, 2, ks + 10, ks + 13, D)
    seed = 1000 + 100 * ks + D
    check_against_oracle(shape, ks, dtype, seed, path="tensor", q_scale=D ** -0.5)
    if ks >= 7:
        check_against_oracle(shape, ks, dtype, seed, path="tensor", q_scale=D ** -0.5, with_o=False)
        check_against_oracle(shape, ks, dtype, seed + 1, path="tensor")     # unscaled logits, near one-hot rows
    q, k, v, d_o = make_inputs(shape, dtype, seed, q_scale=D ** -0.5)
    qd, kd, vd, gd = (t.to(DEV) for t in (q, k, v, d_o))
    o, lse = na.natten2d_forward(qd, kd, vd, ks, path="tensor")
    ro, _, _, _, _ = orc.natten2d_fwd_bwd(q, k, v, d_o, ks)
    want = (d_o.double() * ro).sum(-1)
    for dq_buf in (None, torch.empty_like(qd)):
        delta = torch.full_like(lse, float("nan"))
        na.functional.backward_dq_into(qd, kd, vd, o, lse, gd, dq_buf, delta, ks, path="tensor")
        na.check_kernels(DEV)
        assert_close(delta, want, dtype, f"delta D={D} ks={ks} dQ={'yes' if dq_buf is not None else 'no'}")


# ------------------------------------------------------------------------------ BASELINE configs
def test_config1_fp32():
    check_against_oracle((1, 2, 16, 16, 32), 5, torch.float32, seed=0)


@pytest.mark.parametrize("side", [32, 64])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_config2_small_sides(side, dtype):
    check_against_oracle((4, 4, side, side, 128), 5, dtype, seed=0, q_scale=128 ** -0.5)


def test_config3_stage1_shape():
    check_against_oracle((32, 2, 56, 56, 32), 7, torch.bfloat16, seed=1, scale=0.5)


def test_config4a_large_window():
    check_against_oracle((16, 8, 28, 28, 64), 13, torch.bfloat16, seed=2)


def test_config4b_window_nearly_covers_grid():
    check_against_oracle((16, 16, 14, 14, 64), 13, torch.bfloat16, seed=2)


def _band_check(q, k, v, d_o, got, ks, bn_list, bands, dtype):
    """Oracle on row bands of selected (batch, head) units of a large problem."""
    o, lse, dq, dk, dv = got
    H = q.shape[2]
    for (b, n) in bn_list:
        for (a, e) in bands:
            kv0 = orc.window_start(a, H, ks)
            kv1 = orc.window_start(e - 1, H, ks) + ks
            sl = lambda t, r0, r1: t[b:b + 1, n:n + 1, r0:r1].cpu()
            ro, rl, rdq, rdk, rdv = orc.natten2d_fwd_bwd(sl(q, a, e), sl(k, kv0, kv1), sl(v, kv0, kv1),
                                                          sl(d_o, a, e), ks, rows=(a, kv0, H))
            tag = f"unit ({b},{n}) rows [{a},{e})"
            assert_close(sl(o, a, e), ro, dtype, "o " + tag)
            assert_close(sl(lse, a, e), rl, dtype, "lse " + tag)
            assert_close(sl(dq, a, e), rdq, dtype, "dq " + tag)
            # dK / dV rows whose whole inverse neighbourhood lies inside the band
            full = [r for r in range(kv0, kv1)
                    if orc.backward_window_start(r, ks) >= a and orc.backward_window_end(r, H, ks) <= e]
            if full:
                r0, r1 = full[0], full[-1] + 1
                assert_close(sl(dk, r0, r1), rdk[:, :, r0 - kv0:r1 - kv0], dtype, "dk " + tag)
                assert_close(sl(dv, r0, r1), rdv[:, :, r0 - kv0:r1 - kv0], dtype, "dv " + tag)


@pytest.mark.parametrize("side,dtype", [(128, torch.bfloat16), (192, torch.bfloat16), (256, torch.bfloat16),
                                        (128, torch.float16), (256, torch.float16)])
def test_config2_large_sides_bands_and_cross_path(side, dtype):
    """Sides the CPU oracle cannot finish whole: oracle on border / interior row bands of two
    units, plus the two GPU paths against each other on the full tensors."""
    ks = 5
    q, k, v, d_o = make_inputs((4, 4, side, side, 128), dtype, 0, q_scale=128 ** -0.5)
    got = run_gpu(q, k, v, d_o, ks, "auto")
    bands = [(0, 12), (side // 2 - 6, side // 2 + 6), (side - 12, side)]
    _band_check(q, k, v, d_o, got, ks, [(0, 0), (3, 3)], bands, dtype)
    ref = run_gpu(q, k, v, d_o, ks, "simt")
    for name, a, b in zip(("o", "lse", "dq", "dk", "dv"), got, ref):
        assert_close(a, b.double(), dtype, f"{name} auto vs simt, side {side}")


def test_config5_huge_image_bands():
    """B1 N8 1024x1024 C128 ks13 bf16 seed 3, whole image on one GPU: oracle on the top border,
    the bottom border and all seven 8-way shard boundaries +-(ks-1) rows (all columns are kept,
    because a narrower problem would change the clamping; the nine bands are spread over the
    heads, one head each), one interior band of another head, and the SIMT kernels against the
    tensor-core kernels on the whole of one head."""
    dtype, ks, S = torch.bfloat16, 13, 1024
    q, k, v, d_o = make_inputs((1, 8, S, S, 128), dtype, 3)
    got = run_gpu(q, k, v, d_o, ks, "auto")
    bands = [(0, 16), (S - 16, S)] + [(r - 12, r + 12) for r in range(128, S, 128)]
    assert len(bands) == 9
    for i, band in enumerate(bands):
        _band_check(q, k, v, d_o, got, ks, [(0, i % 8)], [band], dtype)
    _band_check(q, k, v, d_o, got, ks, [(0, 2)], [(500, 520)], dtype)
    head = 6
    one = [t[:, head:head + 1] for t in (q, k, v, d_o)]
    ref = run_gpu(*one, ks, "simt")
    for name, a, b in zip(("o", "lse", "dq", "dk", "dv"), got, ref):
        assert_close(a[:, head:head + 1], b.double(), dtype, f"{name} auto vs simt, config 5 head {head}")


# ------------------------------------------------------------------------------ row views
@pytest.mark.parametrize("dtype,path,ks", [(torch.float32, "simt", 7), (torch.bfloat16, "auto", 7),
                                           (torch.bfloat16, "auto", 3), (torch.bfloat16, "auto", 5),
                                           (torch.float16, "auto", 5), (torch.bfloat16, "auto", 13)])
def test_row_bands_reassemble_whole_image(dtype, path, ks):
    """Every kernel family under a row view with non-zero first rows: the strip kernels of kernel
    sizes 3 and 5, the chunked kernels of the larger windows, and the SIMT kernels.  The bands'
    dK / dV are partial sums, kept in fp32 as a row-sharded run keeps them: a partial sum can be
    far larger than the total, and rounding each to 16 bits first would be the test's own error."""
    H, W = 45, 24
    q, k, v, d_o = make_inputs((2, 2, H, W, 64), dtype, 9)
    o, lse, dq, dk, dv = run_gpu(q, k, v, d_o, ks, path)
    dk_sum = torch.zeros_like(dk, dtype=torch.float32)
    dv_sum = torch.zeros_like(dv, dtype=torch.float32)
    for a, e in ((0, 11), (11, 23), (23, 34), (34, 45)):
        kv0 = orc.window_start(a, H, ks)
        kv1 = orc.window_start(e - 1, H, ks) + ks
        rows = na.make_rows(a, e - a, kv0, kv1 - kv0, H)
        ob, lb, dqb, dkb, dvb = run_gpu(q[:, :, a:e], k[:, :, kv0:kv1], v[:, :, kv0:kv1], d_o[:, :, a:e],
                                        ks, path, rows=rows, dkdv_dtype=torch.float32)
        assert dkb.dtype == torch.float32 and dvb.dtype == torch.float32
        if path == "simt":      # same arithmetic in the same order: bitwise equal
            assert torch.equal(ob, o[:, :, a:e]) and torch.equal(lb, lse[:, :, a:e])
            assert torch.equal(dqb, dq[:, :, a:e])
        else:
            assert_close(ob, o[:, :, a:e].double(), dtype, "band o")
            assert_close(dqb, dq[:, :, a:e].double(), dtype, "band dq")
        dk_sum[:, :, kv0:kv1] += dkb.float()
        dv_sum[:, :, kv0:kv1] += dvb.float()
    ro, rlse, rdq, rdk, rdv = orc.natten2d_fwd_bwd(q, k, v, d_o, ks)
    assert_close(dk_sum, rdk, dtype, "sum of band dK partials")
    assert_close(dv_sum, rdv, dtype, "sum of band dV partials")


# ------------------------------------------------------------------------------ memory safety
@pytest.mark.parametrize("dtype,shape,ks", [(torch.float32, (1, 2, 9, 11, 32), 5),
                                            (torch.bfloat16, (1, 3, 17, 21, 128), 5),
                                            (torch.bfloat16, (2, 1, 14, 14, 64), 13)])
def test_outputs_stay_inside_their_buffers_and_are_deterministic(dtype, shape, ks):
    """Each output lives in the middle of a larger canary-filled allocation; nothing outside the
    output may change, and two runs must agree bit for bit (there are no atomics)."""
    import ctypes as C
    from e_natten_b200 import _lib
    from e_natten_b200.functional import _DTYPES
    q, k, v, d_o = (t.to(DEV) for t in make_inputs(shape, dtype, 3))
    B, N, H, W, Cd = shape
    n, pad = q.numel(), 4096
    nl = B * N * H * W

    def guarded(count, dt):
        buf = torch.full((count + 2 * pad,), 7.0, dtype=dt, device=DEV)
        return buf, buf[pad:pad + count]

    results = []
    for _ in range(2):
        bufs = {nm: guarded(n, dtype) for nm in ("o", "dq", "dk", "dv")}
        bufs["lse"] = guarded(nl, torch.float32)
        bufs["delta"] = guarded(nl, torch.float32)
        p = lambda t: C.c_void_p(t.data_ptr())
        st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
        _lib.check(_lib.lib.na2d_forward(p(q), p(k), p(v), p(bufs["o"][1]), p(bufs["lse"][1]), B, N, H, W, Cd,
                                         ks, _DTYPES[dtype], None, 0, 0, st))
        _lib.check(_lib.lib.na2d_backward(p(q), p(k), p(v), p(bufs["o"][1]), p(bufs["lse"][1]), p(d_o),
                                          p(bufs["dq"][1]), p(bufs["dk"][1]), p(bufs["dv"][1]),
                                          p(bufs["delta"][1]), B, N, H, W, Cd, ks, _DTYPES[dtype], None, 0, 0, st))
        na.check_kernels(DEV)
        for nm, (whole, view) in bufs.items():
            assert (whole[:pad] == 7.0).all() and (whole[pad + view.numel():] == 7.0).all(), f"{nm}: canary overwritten"
        results.append({nm: view.clone() for nm, (whole, view) in bufs.items()})
    for nm in results[0]:
        assert torch.equal(results[0][nm], results[1][nm]), f"{nm} differs between two runs"


# ------------------------------------------------------------------------------ autograd semantics
def test_autograd_semantics_match_the_reference_entry_point():
    q, k, v, d_o = (t.to(DEV) for t in make_inputs((1, 2, 12, 12, 32), torch.float32, 4))
    # default kernel size is 7 (e_natten/triton.py:489)
    assert torch.equal(na.natten2d(q, k, v), na.natten2d(q, k, v, 7))
    # output has q's shape and dtype; no graph under no_grad
    qg = q.clone().requires_grad_()
    with torch.no_grad():
        assert not na.natten2d(qg, k, v, 5).requires_grad
    # gradients only where asked
    kg = k.clone().requires_grad_()
    na.natten2d(q, kg, v, 5).backward(d_o)
    assert kg.grad is not None and q.grad is None
    # backward returns (dQ, dK, dV, None): all three at once
    q2, k2, v2 = (t.clone().requires_grad_() for t in (q, k, v))
    o = na.natten2d(q2, k2, v2, 5)
    assert o.shape == q.shape and o.dtype == q.dtype
    o.backward(d_o)
    ro, rlse, rdq, rdk, rdv = orc.natten2d_fwd_bwd(q.cpu(), k.cpu(), v.cpu(), d_o.cpu(), 5)
    assert_close(q2.grad, rdq, torch.float32, "dq")
    assert_close(k2.grad, rdk, torch.float32, "dk")
    assert_close(v2.grad, rdv, torch.float32, "dv")
    # lse is exposed separately and is not differentiable
    o3, lse = na.natten2d_with_lse(q2, k2, v2, 5)
    assert not lse.requires_grad and lse.dtype == torch.float32
    assert_close(lse, rlse, torch.float32, "lse")


@pytest.mark.parametrize("ks", [5, 9])
def test_delta_only_call_matches_the_full_call(ks):
    """`na2d_backward_dq` without a dQ buffer only writes the row deltas (sum_j p_j dP_j, equal to
    dO . o); with a buffer it writes both.  The two calls may run different kernels."""
    dtype = torch.bfloat16
    q, k, v, d_o = make_inputs((1, 2, 40, 24, 64), dtype, 17, q_scale=0.125)
    qd, kd, vd, gd = (t.to(DEV) for t in (q, k, v, d_o))
    o, lse = na.natten2d_forward(qd, kd, vd, ks)
    delta_only = torch.full_like(lse, float("nan"))
    na.functional.backward_dq_into(qd, kd, vd, o, lse, gd, None, delta_only, ks)
    dq = torch.empty_like(qd)
    delta_full = torch.full_like(lse, float("nan"))
    na.functional.backward_dq_into(qd, kd, vd, o, lse, gd, dq, delta_full, ks)
    na.check_kernels(DEV)
    ro, _, _, _, _ = orc.natten2d_fwd_bwd(q, k, v, d_o, ks)
    want = (d_o.double() * ro).sum(-1)
    assert_close(delta_only, want, dtype, "delta (delta-only call)")
    assert_close(delta_full, want, dtype, "delta (full call)")


def test_entry_points_work_from_a_thread_that_made_no_cuda_call():
    """An autograd worker thread may reach the library before any runtime call has bound the
    device's context to it; the tensor-core launchers (which encode tensor maps through the
    driver) must still work there."""
    import threading
    q, k, v, d_o = make_inputs((1, 2, 24, 24, 64), torch.bfloat16, 5, q_scale=0.125)
    o, lse, dq, dk, dv = run_gpu(q, k, v, d_o, 7)
    qd, kd, vd, gd = (t.to(DEV) for t in (q, k, v, d_o))
    outs = [torch.empty_like(qd) for _ in range(3)]
    delta = torch.empty_like(lse)
    torch.cuda.synchronize()
    box = {}

    def work():
        try:
            na.functional.backward_dq_into(qd, kd, vd, o, lse, gd, outs[0], delta, 7)
            na.functional.backward_dkdv_into(qd, kd, vd, lse, gd, delta, outs[1], outs[2], 7)
        except Exception as exc:        # noqa: BLE001 -- reported by the assert below
            box["exc"] = exc

    t = threading.Thread(target=work)
    t.start()
    t.join()
    assert "exc" not in box, box.get("exc")
    torch.cuda.synchronize()
    na.check_kernels(DEV)
    assert torch.equal(outs[0], dq) and torch.equal(outs[1], dk) and torch.equal(outs[2], dv)


def test_non_contiguous_inputs_and_grad_output_are_accepted():
    """The reference asserts equal strides (e_natten/triton.py:233-234); accepting strided views
    is a harmless superset."""
    base = torch.randn(1, 10, 9, 3, 2, 32, device=DEV)            # (B, H, W, 3, N, C) packed qkv
    q, k, v = (base[:, :, :, i].permute(0, 3, 1, 2, 4) for i in range(3))
    assert not q.is_contiguous()
    qg = q.detach().requires_grad_()
    o = na.natten2d(qg, k, v, 3)
    g = torch.randn(1, 10, 9, 2, 32, device=DEV).permute(0, 3, 1, 2, 4)
    o.backward(g)
    ro, _ = orc.natten2d_fwd(q.cpu(), k.cpu(), v.cpu(), 3)
    rdq, _, _ = orc.natten2d_bwd(q.cpu(), k.cpu(), v.cpu(), g.cpu(), 3)
    assert_close(o, ro, torch.float32, "o from strided views")
    assert_close(qg.grad, rdq, torch.float32, "dq from strided grad_output")


def test_errors_are_python_exceptions():
    q = torch.zeros(1, 1, 8, 8, 32, device=DEV)
    with pytest.raises(ValueError):
        na.natten2d(q, q, q, 4)                                   # even kernel size
    with pytest.raises(ValueError):
        na.natten2d(q, q, q, 9)                                   # grid smaller than the window
    with pytest.raises(ValueError):
        na.natten2d(q, q[:, :, :4], q, 3)                         # shape mismatch
    with pytest.raises(ValueError):
        na.natten2d(q, q.half(), q, 3)                            # dtype mismatch
    with pytest.raises(ValueError):
        na.natten2d(q.double(), q.double(), q.double(), 3)        # unsupported dtype
    with pytest.raises(ValueError):
        na.natten2d_forward(q, q, q, 3, path="tensor")            # fp32 has no tensor-core path
    empty = torch.zeros(0, 1, 8, 8, 32, device=DEV)
    assert na.natten2d(empty, empty, empty, 3).shape == empty.shape


# ------------------------------------------------------------------------------ scale and strided layouts
@pytest.mark.parametrize("dtype,shape,ks,path", [(torch.float32, (1, 2, 12, 13, 32), 5, "auto"),
                                                 (torch.bfloat16, (2, 2, 20, 24, 64), 5, "tensor"),
                                                 (torch.bfloat16, (1, 2, 22, 24, 128), 7, "tensor"),
                                                 (torch.float16, (1, 2, 20, 28, 32), 13, "tensor"),
                                                 (torch.bfloat16, (1, 2, 20, 24, 64), 9, "simt")])
def test_softmax_scale_argument(dtype, shape, ks, path):
    """The scale argument of the kernels against the oracle (which scales q); unscaled N(0,1)
    inputs, scale = head_dim**-0.5 as a caller of the reference would apply to q."""
    scale = shape[-1] ** -0.5
    q, k, v, d_o = make_inputs(shape, dtype, 77)
    o, lse, dq, dk, dv = run_gpu(q, k, v, d_o, ks, path, scale=scale)
    ro, rlse, rdq, rdk, rdv = orc.natten2d_fwd_bwd(q, k, v, d_o, ks, scale=scale)
    tag = f"{shape} ks={ks} {dtype} {path} scale"
    for name, a, b in (("o", o, ro), ("lse", lse, rlse), ("dq", dq, rdq), ("dk", dk, rdk), ("dv", dv, rdv)):
        assert_close(a, b, dtype, f"{name} {tag}")
    # and through the autograd entry point
    qd, kd, vd = (t.to(DEV).requires_grad_() for t in (q, k, v))
    na.natten2d(qd, kd, vd, ks, scale).backward(d_o.to(DEV))
    if path == "auto" or (path == "tensor" and dtype != torch.float32):
        assert_close(qd.grad, rdq, dtype, "dq through natten2d(scale=...)")


@pytest.mark.parametrize("dtype,Cd,ks", [(torch.bfloat16, 64, 5), (torch.float16, 128, 7), (torch.float32, 32, 5)])
def test_packed_qkv_views_run_without_copies(dtype, Cd, ks):
    """q, k, v as views of one (B, H, W, 3, heads, C) projection output, the layout the reference
    refuses (e_natten/triton.py:233-234): the kernels read them in place (tensor maps / pointer
    arithmetic built from the views' strides) and write dQ, dK, dV straight into views of a packed
    gradient buffer."""
    B, H, W, N = 2, 20, 24, 2
    g = torch.Generator().manual_seed(5)
    packed = (torch.randn((B, H, W, 3, N, Cd), generator=g) * 0.5).to(dtype).to(DEV)
    d_o = torch.randn((B, H, W, N, Cd), generator=g).to(dtype).to(DEV).permute(0, 3, 1, 2, 4)     # strided too
    q, k, v = (packed[:, :, :, i].permute(0, 3, 1, 2, 4) for i in range(3))
    assert not q.is_contiguous() and all(na.as_kernel_input(t) is t for t in (q, k, v, d_o))
    before = na.launch_count()
    o, lse = na.natten2d_forward(q, k, v, ks)
    d_packed = torch.full_like(packed, float("nan"))
    dq, dk, dv = (d_packed[:, :, :, i].permute(0, 3, 1, 2, 4) for i in range(3))
    delta = torch.empty_like(lse)
    na.functional.backward_dq_into(q, k, v, o, lse, d_o, dq, delta, ks)
    na.functional.backward_dkdv_into(q, k, v, lse, d_o, delta, dk, dv, ks)
    na.check_kernels(DEV)
    # forward, dQ, dK/dV and nothing else (the tensor-core dQ of kernel sizes >= 7 is preceded by its delta estimate)
    assert na.launch_count() - before == (4 if (ks >= 7 and dtype != torch.float32) else 3)
    ro, rlse, rdq, rdk, rdv = orc.natten2d_fwd_bwd(q.cpu(), k.cpu(), v.cpu(), d_o.cpu(), ks)
    assert torch.isfinite(d_packed.float()).all()                            # every element of the packed gradient written
    for name, a, b in (("o", o, ro), ("lse", lse, rlse), ("dq", dq, rdq), ("dk", dk, rdk), ("dv", dv, rdv)):
        assert_close(a, b, dtype, f"{name} from packed qkv views, {dtype}")
    # the autograd entry point takes the same views
    pk = packed.clone().requires_grad_()
    q2, k2, v2 = (pk[:, :, :, i].permute(0, 3, 1, 2, 4) for i in range(3))
    na.natten2d(q2, k2, v2, ks).backward(d_o)
    assert_close(pk.grad[:, :, :, 0].permute(0, 3, 1, 2, 4), rdq, dtype, "packed dq through autograd")
    assert_close(pk.grad[:, :, :, 2].permute(0, 3, 1, 2, 4), rdv, dtype, "packed dv through autograd")


def test_layouts_the_tensor_maps_cannot_take_are_copied():
    """Channels not contiguous, or strides that are not multiples of 16 bytes: the wrapper makes a
    dense copy and the result is unchanged."""
    q, k, v, d_o = make_inputs((1, 2, 16, 18, 32), torch.bfloat16, 6, q_scale=32 ** -0.5)
    wide = torch.zeros((1, 2, 16, 18, 36), dtype=torch.bfloat16, device=DEV)
    wide[..., 2:34] = q.to(DEV)
    qv = wide[..., 2:34]                                       # pixel stride 36 elements, base off by 4 bytes
    assert na.as_kernel_input(qv) is not qv
    o1, _ = na.natten2d_forward(qv, k.to(DEV), v.to(DEV), 5)
    o2, _ = na.natten2d_forward(q.to(DEV), k.to(DEV), v.to(DEV), 5)
    assert torch.equal(o1, o2)


# ------------------------------------------------------------------------------ bounded waits
def test_sm_margin_changes_the_grid_not_the_result():
    """NA2D_FLAG_SM_MARGIN: the persistent kernels launch on fewer SMs (to leave room for a halo
    exchange running beside them); the outputs are bit-identical."""
    dtype, ks, shape = torch.bfloat16, 7, (1, 2, 70, 90, 64)
    q, k, v, d_o = (t.to(DEV) for t in make_inputs(shape, dtype, 5, q_scale=0.125))
    outs = []
    for margin in (0, 16, 147, 255):
        o = torch.empty_like(q)
        lse = torch.empty(shape[:4], dtype=torch.float32, device=DEV)
        na.functional.forward_into(q, k, v, o, lse, ks, sm_margin=margin)
        delta = torch.empty_like(lse)
        dq = torch.empty_like(q)
        na.functional.backward_dq_into(q, k, v, o, lse, d_o, dq, delta, ks)
        dk, dv = torch.empty_like(k), torch.empty_like(v)
        na.functional.backward_dkdv_into(q, k, v, lse, d_o, delta, dk, dv, ks, sm_margin=margin)
        na.check_kernels(DEV)
        outs.append((o, lse, dk, dv))
    for other in outs[1:]:
        for a, b in zip(outs[0], other):
            assert torch.equal(a, b)


def test_bounded_wait_gives_up_and_is_reported_once():
    """A wait that nothing ever satisfies ends by itself: the self-test kernel waits 2 ms on a
    barrier nobody completes, records that, and exits normally.  na2d_check reports it once and
    clears it; the next call is clean and the kernels still compute correctly afterwards."""
    import ctypes as C
    from e_natten_b200 import _lib
    na.check_kernels(DEV)                                       # start clean
    st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    _lib.check(_lib.lib.na2d_selftest_wait_timeout(0, st, 2000))
    assert _lib.lib.na2d_check(0, st) == _lib.ERR_KERNEL_WAIT
    assert _lib.lib.na2d_check(0, st) == 0
    with pytest.raises(ValueError):
        _lib.check(_lib.lib.na2d_selftest_wait_timeout(0, st, 0))
    check_against_oracle((1, 2, 17, 19, 64), 5, torch.bfloat16, seed=3, q_scale=0.125)


def test_poll_reports_a_tripped_wait_without_synchronising():
    """na2d_poll answers from the copy the previous poll started: clean, then (after the
    self-test kernel) the error, then clean again.  The autograd backward polls at its entry and
    raises there."""
    import ctypes as C
    from e_natten_b200 import _lib
    na.check_kernels(DEV)
    st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert _lib.lib.na2d_poll(0, st) == 0
    torch.cuda.synchronize()
    assert _lib.lib.na2d_poll(0, st) == 0                       # the first poll's copy saw a clean word
    _lib.check(_lib.lib.na2d_selftest_wait_timeout(0, st, 1000))
    assert _lib.lib.na2d_poll(0, st) == 0                       # asks; the answer comes with the next poll
    torch.cuda.synchronize()
    assert _lib.lib.na2d_poll(0, st) == _lib.ERR_KERNEL_WAIT
    torch.cuda.synchronize()
    _lib.lib.na2d_poll(0, st)                                   # (the copy enqueued before the clear may still see it)
    torch.cuda.synchronize()
    assert _lib.lib.na2d_poll(0, st) == 0
    # through autograd: the error of an earlier kernel surfaces at the next backward's entry
    q, k, v, d_o = (t.to(DEV) for t in make_inputs((1, 1, 12, 12, 32), torch.bfloat16, 2))
    qg = q.clone().requires_grad_()
    o = na.natten2d(qg, k, v, 5)
    _lib.check(_lib.lib.na2d_selftest_wait_timeout(0, st, 1000))
    na.poll_kernels(DEV)                                        # asks
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError, match="bounded wait"):
        o.backward(d_o)
    torch.cuda.synchronize()
    na.check_kernels(DEV) if False else None
    _lib.lib.na2d_check(0, st)                                  # leave the word clean for the tests that follow
    torch.cuda.synchronize()
    _lib.lib.na2d_poll(0, st)
    torch.cuda.synchronize()
    _lib.lib.na2d_poll(0, st)
