"""CPU tests: the oracle restatement against vectors produced by the reference itself."""
import numpy as np
import pytest
import torch

from oracle import na2d_oracle as orc

KS_ALL = list(range(3, 16, 2))


def _lens(ks):
    return list(range(ks, 81)) + [192, 256, 1024]


@pytest.mark.parametrize("ks", KS_ALL)
def test_index_functions_match_reference_tables(golden, ks):
    for L in _lens(ks):
        ws = np.array([orc.window_start(i, L, ks) for i in range(L)], dtype=np.int32)
        bs = np.array([orc.backward_window_start(i, ks) for i in range(L)], dtype=np.int32)
        be = np.array([orc.backward_window_end(i, L, ks) for i in range(L)], dtype=np.int32)
        assert np.array_equal(ws, golden[f"idx/ws/{ks}/{L}"])
        assert np.array_equal(bs, golden[f"idx/bws/{ks}/{L}"])
        assert np.array_equal(be, golden[f"idx/bwe/{ks}/{L}"])


@pytest.mark.parametrize("ks", KS_ALL)
def test_window_start_is_a_clamp_and_inverse_range_is_exact(golden, ks):
    for L in list(range(ks, 81)):
        ws = golden[f"idx/ws/{ks}/{L}"]
        i = np.arange(L)
        assert np.array_equal(ws, np.clip(i - ks // 2, 0, L - ks))
        bs, be = golden[f"idx/bws/{ks}/{L}"], golden[f"idx/bwe/{ks}/{L}"]
        for j in range(L):
            holders = np.nonzero((ws <= j) & (j < ws + ks))[0]
            assert holders[0] == bs[j] and holders[-1] + 1 == be[j]
            assert len(holders) == be[j] - bs[j]          # contiguous: the range is exact


def _pt_case(golden, name):
    g = {k: torch.from_numpy(golden[f"pt/{name}/{k}"]) for k in ("q", "k", "v", "do", "o", "dk", "dv", "dq_tile00")}
    return g, int(golden[f"pt/{name}/ks"])


@pytest.mark.parametrize("name", ["k5", "k7", "k11", "k13"])
def test_forward_bit_identical_to_reference_pytorch_fp64(golden, name):
    g, ks = _pt_case(golden, name)
    o = orc.natten2d_pixel(g["q"], g["k"], g["v"], ks)
    assert torch.equal(o, g["o"])                                  # bit for bit
    o_vec, _ = orc.natten2d_fwd(g["q"], g["k"], g["v"], ks)
    assert (o_vec - g["o"]).abs().max() < 1e-12


@pytest.mark.parametrize("name", ["k5", "k7", "k11", "k13"])
def test_backward_matches_reference_pytorch_fp64(golden, name):
    g, ks = _pt_case(golden, name)
    dq, dk, dv = orc.natten2d_bwd(g["q"], g["k"], g["v"], g["do"], ks)
    assert (dk - g["dk"]).abs().max() < 1e-12
    assert (dv - g["dv"]).abs().max() < 1e-12
    # the reference fills dQ for its first 3x3 tile only (e_natten/pytorch.py:228-231)
    assert (dq[:, :, :3, :3] - g["dq_tile00"]).abs().max() < 1e-12
    # and the autograd of the per-pixel restatement gives the same three gradients everywhere
    q, k, v = (g[n].clone().requires_grad_() for n in ("q", "k", "v"))
    orc.natten2d_pixel(q, k, v, ks).backward(g["do"])
    assert (dq - q.grad).abs().max() < 1e-12
    assert (dk - k.grad).abs().max() < 1e-12
    assert (dv - v.grad).abs().max() < 1e-12


def test_config1_fp32_against_reference_pytorch(golden):
    g, ks = _pt_case(golden, "c1")
    assert g["q"].dtype == torch.float32 and tuple(g["q"].shape) == (1, 2, 16, 16, 32) and ks == 5
    o, _ = orc.natten2d_fwd(g["q"], g["k"], g["v"], ks)
    dq, dk, dv = orc.natten2d_bwd(g["q"], g["k"], g["v"], g["do"], ks)
    assert (o - g["o"].double()).abs().max() < 1e-5
    assert (dk - g["dk"].double()).abs().max() < 2e-5
    assert (dv - g["dv"].double()).abs().max() < 2e-5
    assert (dq[:, :, :3, :3] - g["dq_tile00"].double()).abs().max() < 2e-5
    # the inputs of the fixture are what the seeded generator gives
    q, k, v, d_o = orc.round_inputs((1, 2, 16, 16, 32), torch.float32, 0)
    assert torch.equal(q, g["q"]) and torch.equal(d_o, g["do"])


@pytest.mark.parametrize("name", ["k3", "k5", "k7", "k9", "k11"])
def test_against_reference_triton_kernels_under_interpreter(golden, name):
    g = {k: torch.from_numpy(golden[f"tr/{name}/{k}"]) for k in ("q", "k", "v", "o", "dq", "dk", "dv")}
    ks = int(golden[f"tr/{name}/ks"])
    o, _ = orc.natten2d_fwd(g["q"], g["k"], g["v"], ks)
    assert (o - g["o"].double()).abs().max() < 1e-5               # tolerance of test.py:36
    d_o = 2.0 * o                                                  # loss = sum(o**2), test.py:39-42
    dq, dk, dv = orc.natten2d_bwd(g["q"], g["k"], g["v"], d_o, ks)
    for mine, ref in ((dq, g["dq"]), (dk, g["dk"]), (dv, g["dv"])):
        assert (mine - ref.double()).abs().max() < 2e-5


@pytest.mark.parametrize("ks,shape", [(3, (1, 2, 7, 9, 3)), (9, (1, 1, 11, 13, 2)), (5, (2, 1, 5, 5, 4))])
def test_vectorised_equals_per_pixel(ks, shape):
    q, k, v, d_o = orc.round_inputs(shape, torch.float64, 7)
    o_pix = orc.natten2d_pixel(q, k, v, ks)
    o, lse = orc.natten2d_fwd(q, k, v, ks)
    assert (o - o_pix).abs().max() < 1e-12
    qq, kk, vv = (t.clone().requires_grad_() for t in (q, k, v))
    orc.natten2d_pixel(qq, kk, vv, ks).backward(d_o)
    dq, dk, dv = orc.natten2d_bwd(q, k, v, d_o, ks)
    assert (dq - qq.grad).abs().max() < 1e-12
    assert (dk - kk.grad).abs().max() < 1e-12
    assert (dv - vv.grad).abs().max() < 1e-12


def test_reference_live_if_present():
    """Where the reference checkout is mounted, compare against it directly as well."""
    import os, sys
    ref_root = os.environ.get("E_NATTEN_REFERENCE", "")
    if not ref_root or not os.path.isdir(os.path.join(ref_root, "e_natten")):
        pytest.skip("set E_NATTEN_REFERENCE to an e_natten source checkout to run this comparison")
    sys.path.insert(0, ref_root)
    try:
        import e_natten.pytorch as ref
    finally:
        sys.path.remove(ref_root)
    q, k, v, _ = orc.round_inputs((1, 1, 8, 9, 2), torch.float64, 21)
    assert torch.equal(ref.natten2d(q, k, v, 5), orc.natten2d_pixel(q, k, v, 5))
    for ks in (3, 5, 13):
        for L in (ks, ks + 1, 30):
            for i in range(L):
                assert ref.get_window_start(i, L, ks) == orc.window_start(i, L, ks)


def test_row_view_bands_reassemble_the_whole_image():
    """Oracle's own row-view form: per-band results equal slices of the whole-image result and
    the bands' partial dK / dV add up to the whole-image gradients."""
    ks, H, W = 5, 19, 8
    q, k, v, d_o = orc.round_inputs((1, 2, H, W, 3), torch.float64, 5)
    o, lse, dq, dk, dv = orc.natten2d_fwd_bwd(q, k, v, d_o, ks)
    dk_sum, dv_sum = torch.zeros_like(dk), torch.zeros_like(dv)
    for a, b in ((0, 6), (6, 13), (13, 19)):
        kv0 = orc.window_start(a, H, ks)
        kv1 = orc.window_start(b - 1, H, ks) + ks
        rows = (a, kv0, H)
        ob, lb, dqb, dkb, dvb = orc.natten2d_fwd_bwd(q[:, :, a:b], k[:, :, kv0:kv1], v[:, :, kv0:kv1],
                                                     d_o[:, :, a:b], ks, rows=rows)
        assert (ob - o[:, :, a:b]).abs().max() < 1e-13 and (lb - lse[:, :, a:b]).abs().max() < 1e-13
        assert (dqb - dq[:, :, a:b]).abs().max() < 1e-13
        dk_sum[:, :, kv0:kv1] += dkb
        dv_sum[:, :, kv0:kv1] += dvb
    assert (dk_sum - dk).abs().max() < 1e-13 and (dv_sum - dv).abs().max() < 1e-13


# ------------------------------------------------------------------------------ 1D operator
@pytest.mark.parametrize("ks", [5, 7, 11, 13])
def test_1d_against_reference_pytorch_fixture(golden, ks):
    """e_natten.pytorch.natten1d (fp32): forward and all three gradients."""
    g = {n: torch.from_numpy(golden[f"pt1d/k{ks}/{n}"]) for n in ("q", "k", "v", "do", "o", "dq", "dk", "dv")}
    o, _ = orc.natten1d_fwd(g["q"], g["k"], g["v"], ks)
    dq, dk, dv = orc.natten1d_bwd(g["q"], g["k"], g["v"], g["do"], ks)
    assert (o - g["o"].double()).abs().max() < 1e-5
    for mine, ref in ((dq, g["dq"]), (dk, g["dk"]), (dv, g["dv"])):
        assert (mine - ref.double()).abs().max() < 2e-5


def test_1d_against_reference_triton_fixtures(golden):
    """The fused e_natten.natten1d under the Triton interpreter, loss = sum(o**2) (test.py:39-42),
    for the kernel sizes whose interpreter run ended cleanly when the fixtures were made."""
    kept = [int(x) for x in golden["tr1d/kept"]]
    assert len(kept) >= 3
    for ks in kept:
        g = {n: torch.from_numpy(golden[f"tr1d/k{ks}/{n}"]) for n in ("q", "k", "v", "o", "dq", "dk", "dv")}
        o, _ = orc.natten1d_fwd(g["q"], g["k"], g["v"], ks)
        assert (o - g["o"].double()).abs().max() < 1e-5
        dq, dk, dv = orc.natten1d_bwd(g["q"], g["k"], g["v"], 2.0 * o, ks)
        for mine, ref in ((dq, g["dq"]), (dk, g["dk"]), (dv, g["dv"])):
            assert (mine - ref.double()).abs().max() < 2e-5


@pytest.mark.parametrize("ks,T", [(3, 3), (3, 8), (7, 9), (9, 30)])
def test_1d_vectorised_equals_per_token_and_finite_differences(ks, T):
    """The 1D restatement against the per-token loop with autograd, and its gradients against
    central differences in fp64 (the pattern of the reference's gradcheck.py: eps 1e-6, atol 1e-4)."""
    g = torch.Generator().manual_seed(50 + ks)
    q, k, v, d_o = (torch.randn((2, 3, T, 2), generator=g, dtype=torch.float64) for _ in range(4))
    qq, kk, vv = (t.clone().requires_grad_() for t in (q, k, v))
    o_pix = orc.natten1d_pixel(qq, kk, vv, ks)
    o_pix.backward(d_o)
    o, _ = orc.natten1d_fwd(q, k, v, ks)
    dq, dk, dv = orc.natten1d_bwd(q, k, v, d_o, ks)
    assert (o - o_pix).abs().max() < 1e-12
    for mine, ref in ((dq, qq.grad), (dk, kk.grad), (dv, vv.grad)):
        assert (mine - ref).abs().max() < 1e-12
    eps = 1e-6
    for which, grad in ((0, dq), (1, dk), (2, dv)):
        d = torch.randn(q.shape, generator=g, dtype=torch.float64)
        hi, lo = [q, k, v], [q, k, v]
        hi[which] = hi[which] + eps * d
        lo[which] = lo[which] - eps * d
        f = lambda ts: (orc.natten1d_fwd(*ts, ks)[0] * d_o).sum()
        assert abs((f(hi) - f(lo)) / (2 * eps) - (grad * d).sum()) < 1e-4


def test_scale_is_the_same_as_prescaling_q():
    q, k, v, d_o = orc.round_inputs((1, 2, 9, 11, 4), torch.float64, 8)
    o_a, lse_a, dq_a, dk_a, dv_a = orc.natten2d_fwd_bwd(q * 0.25, k, v, d_o, 5)
    o_b, lse_b, dq_b, dk_b, dv_b = orc.natten2d_fwd_bwd(q, k, v, d_o, 5, scale=0.25)
    assert (o_a - o_b).abs().max() < 1e-13 and (lse_a - lse_b).abs().max() < 1e-13
    assert (dq_a * 0.25 - dq_b).abs().max() < 1e-13         # chain rule through q * scale
    assert (dk_a - dk_b).abs().max() < 1e-13 and (dv_a - dv_b).abs().max() < 1e-13


@pytest.mark.parametrize("ks", [3, 5, 7])
def test_unfused_pair_composes_to_the_fused_operator(ks):
    """scores -> softmax -> apply (the form test.py:17-21 compares with) equals the fused form,
    forward and gradients."""
    q, k, v, d_o = orc.round_inputs((1, 2, 9, 10, 3), torch.float64, 60 + ks)
    qq, kk, vv = (t.clone().requires_grad_() for t in (q, k, v))
    out = orc.natten2d_av(torch.softmax(orc.natten2d_qk(qq, kk, ks), dim=-1), vv, ks)
    out.backward(d_o)
    o, _, dq, dk, dv = orc.natten2d_fwd_bwd(q, k, v, d_o, ks)
    assert (out - o).abs().max() < 1e-12
    for mine, ref in ((dq, qq.grad), (dk, kk.grad), (dv, vv.grad)):
        assert (mine - ref).abs().max() < 1e-12
