"""GPU parity tests of the 1D operator (drop-in for e_natten.natten1d, e_natten/triton.py:425-485)
against the CPU oracle and the fixtures produced by the reference itself; patterned on the
reference's test.py (shape (2, 3, 16, 2), kernel sizes 3..11, loss sum(o**2), atol 1e-5) and
gradcheck.py (finite differences)."""
import pytest
import torch

import e_natten_b200 as na
from oracle import na2d_oracle as orc
from helpers import assert_close

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _inputs(shape, dtype, seed, q_scale=1.0):
    g = torch.Generator().manual_seed(seed)
    q, k, v, d_o = (torch.randn(shape, generator=g, dtype=torch.float32) for _ in range(4))
    return tuple(t.to(dtype) for t in (q * q_scale, k, v, d_o))


@pytest.mark.parametrize("ks", [5, 7, 11, 13])
def test_1d_against_reference_pytorch_fixture(golden, ks):
    g = {n: torch.from_numpy(golden[f"pt1d/k{ks}/{n}"]) for n in ("q", "k", "v", "do", "o", "dq", "dk", "dv")}
    q, k, v = (g[n].to(DEV).requires_grad_() for n in ("q", "k", "v"))
    o = na.natten1d(q, k, v, ks)
    o.backward(g["do"].to(DEV))
    assert torch.allclose(o.detach().cpu(), g["o"], atol=1e-5)
    assert torch.allclose(q.grad.cpu(), g["dq"], atol=2e-5)
    assert torch.allclose(k.grad.cpu(), g["dk"], atol=2e-5)
    assert torch.allclose(v.grad.cpu(), g["dv"], atol=2e-5)


def test_1d_against_reference_triton_fixtures(golden):
    for ks in [int(x) for x in golden["tr1d/kept"]]:
        g = {n: torch.from_numpy(golden[f"tr1d/k{ks}/{n}"]) for n in ("q", "k", "v", "o", "dq", "dk", "dv")}
        q, k, v = (g[n].to(DEV).requires_grad_() for n in ("q", "k", "v"))
        o = na.natten1d(q, k, v, ks)
        torch.sum(o ** 2).backward()
        assert torch.allclose(o.detach().cpu(), g["o"], atol=1e-5), ks
        assert torch.allclose(q.grad.cpu(), g["dq"], atol=2e-5), ks
        assert torch.allclose(k.grad.cpu(), g["dk"], atol=2e-5), ks
        assert torch.allclose(v.grad.cpu(), g["dv"], atol=2e-5), ks


@pytest.mark.parametrize("ks", [3, 5, 7, 9, 11])
def test_1d_reference_test_script_shape(ks):
    """The reference's own 1D test case: (2, 3, 16, 2), fp32, seed 0, loss sum(o**2)
    (test.py:5-8, 39-45, 51); default kernel size 7 (e_natten/triton.py:427)."""
    torch.manual_seed(0)
    q, k, v = torch.randn(3, 2, 3, 16, 2)
    qd, kd, vd = (t.to(DEV).requires_grad_() for t in (q, k, v))
    o = na.natten1d(qd, kd, vd, ks)
    torch.sum(o ** 2).backward()
    ro, _ = orc.natten1d_fwd(q, k, v, ks)
    rdq, rdk, rdv = orc.natten1d_bwd(q, k, v, 2.0 * ro, ks)
    assert torch.allclose(o.detach().cpu().double(), ro, atol=1e-5)
    assert torch.allclose(qd.grad.cpu().double(), rdq, atol=1e-5)
    assert torch.allclose(kd.grad.cpu().double(), rdk, atol=1e-5)
    assert torch.allclose(vd.grad.cpu().double(), rdv, atol=1e-5)
    if ks == 7:
        assert torch.equal(na.natten1d(qd, kd, vd), o)


@pytest.mark.parametrize("shape,ks", [((1, 1, 3, 32), 3), ((2, 2, 40, 64), 13), ((1, 3, 257, 128), 7),
                                      ((2, 1, 31, 48), 31), ((1, 2, 100, 256), 9)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_1d_against_oracle(shape, ks, dtype):
    """Window == sequence, ragged lengths, every dtype, head dims up to 256, kernel sizes up to 31."""
    q, k, v, d_o = _inputs(shape, dtype, 400 + ks, q_scale=shape[-1] ** -0.5)
    qd, kd, vd = (t.to(DEV) for t in (q, k, v))
    o, lse = na.natten1d_forward(qd, kd, vd, ks)
    dq, dk, dv = na.natten1d_backward(qd, kd, vd, o, lse, d_o.to(DEV), ks)
    na.check_kernels(DEV)
    ro, rlse = orc.natten1d_fwd(q, k, v, ks)
    rdq, rdk, rdv = orc.natten1d_bwd(q, k, v, d_o, ks)
    tag = f"{shape} ks={ks} {dtype}"
    for name, a, b in (("o", o, ro), ("lse", lse, rlse), ("dq", dq, rdq), ("dk", dk, rdk), ("dv", dv, rdv)):
        assert_close(a, b, dtype, f"1D {name} {tag}")


def test_1d_scale_and_strided_views():
    """(B, T, 3, heads, C) packed projection views and a softmax scale, fp32."""
    B, T, N, Cd, ks = 2, 50, 3, 32, 7
    g = torch.Generator().manual_seed(9)
    packed = torch.randn((B, T, 3, N, Cd), generator=g).to(DEV)
    q, k, v = (packed[:, :, i].permute(0, 2, 1, 3) for i in range(3))
    d_o = torch.randn((B, N, T, Cd), generator=g).to(DEV)
    assert na.as_kernel_input(q) is q
    qg, kg, vg = (t.detach().requires_grad_() for t in (q, k, v))
    na.natten1d(qg, kg, vg, ks, 0.2).backward(d_o)
    ro, _ = orc.natten1d_fwd(q.cpu(), k.cpu(), v.cpu(), ks, scale=0.2)
    rdq, rdk, rdv = orc.natten1d_bwd(q.cpu(), k.cpu(), v.cpu(), d_o.cpu(), ks, scale=0.2)
    assert_close(na.natten1d(q, k, v, ks, 0.2), ro, torch.float32, "1D o, strided + scale")
    assert_close(qg.grad, rdq, torch.float32, "1D dq, strided + scale")
    assert_close(kg.grad, rdk, torch.float32, "1D dk, strided + scale")
    assert_close(vg.grad, rdv, torch.float32, "1D dv, strided + scale")


def test_1d_gradients_against_finite_differences():
    """The pattern of the reference's gradcheck.py (shape (2, 3, 8, 2), kernel size 7) with the
    operator itself as the function: central differences along random directions.  The library
    computes in fp32, so the step and the tolerance are those of fp32 (the reference checks in
    fp64 with eps 1e-6 / atol 1e-4; the oracle is checked that way in the CPU tests)."""
    torch.manual_seed(1)
    q, k, v = (torch.randn(2, 3, 8, 2, device=DEV) for _ in range(3))
    d_o = torch.randn(2, 3, 8, 2, device=DEV)
    qg, kg, vg = (t.clone().requires_grad_() for t in (q, k, v))
    na.natten1d(qg, kg, vg, 7).backward(d_o)
    f = lambda a, b, c: (na.natten1d(a, b, c, 7).double() * d_o.double()).sum().item()
    eps = 1e-2
    for which, grad in ((0, qg.grad), (1, kg.grad), (2, vg.grad)):
        d = torch.randn(2, 3, 8, 2, device=DEV)
        hi, lo = [q, k, v], [q, k, v]
        hi[which] = hi[which] + eps * d
        lo[which] = lo[which] - eps * d
        fd = (f(*hi) - f(*lo)) / (2 * eps)
        an = (grad.double() * d.double()).sum().item()
        assert abs(fd - an) < 2e-3 * max(1.0, abs(an)), (which, fd, an)


def test_1d_errors():
    q = torch.zeros(1, 1, 8, 32, device=DEV)
    with pytest.raises(ValueError):
        na.natten1d(q, q, q, 4)
    with pytest.raises(ValueError):
        na.natten1d(q, q, q, 9)                                   # sequence shorter than the window
    with pytest.raises(ValueError):
        na.natten1d(q, q[:, :, :4], q, 3)
    with pytest.raises(ValueError):
        na.natten1d(torch.zeros(1, 1, 8, 8, 32, device=DEV), q, q, 3)
    empty = torch.zeros(0, 1, 8, 32, device=DEV)
    assert na.natten1d(empty, empty, empty, 3).shape == empty.shape
