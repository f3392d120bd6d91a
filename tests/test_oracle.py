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
    ref_root = os.environ.get("E_NATTEN_REFERENCE", "/root/reference")
    if not os.path.isdir(os.path.join(ref_root, "e_natten")):
        pytest.skip("reference checkout not present")
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
