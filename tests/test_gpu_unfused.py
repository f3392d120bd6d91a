"""GPU tests of the unfused pair natten2dqk / natten2dav (the two-step form the reference's test.py
and bench.py compare the fused operator with: test.py:17-21, bench.py:23, 52-54), against the CPU
oracle, and of the reference's own comparison: fused == unfused, forward and gradients, at
atol 1e-5 on shape (2, 6, 16, 16, 2)."""
import pytest
import torch

import e_natten_b200 as na
from oracle import na2d_oracle as orc
from helpers import assert_close, make_inputs

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.mark.parametrize("ks", [3, 5, 7, 9, 11])
def test_fused_equals_unfused_as_in_the_reference_test_script(ks):
    """test.py:7-45 with this repository's two providers: natten2dqk + softmax + natten2dav on one
    side, natten2d on the other, loss sum(o**2), allclose(atol=1e-5) on forward and all gradients."""
    torch.manual_seed(0)
    q, k, v = torch.randn(3, 2, 6, 16, 16, 2).to(DEV)
    q1, k1, v1 = (t.clone().requires_grad_() for t in (q, k, v))
    s_1 = na.natten2dqk(q1, k1, ks, 1)
    p_1 = torch.softmax(s_1, dim=-1)
    o_1 = na.natten2dav(p_1, v1, ks, 1)
    q2, k2, v2 = (t.clone().requires_grad_() for t in (q, k, v))
    o_2 = na.natten2d(q2, k2, v2, ks)
    assert torch.allclose(o_1, o_2, atol=1e-5)
    torch.sum(o_1 ** 2).backward()
    torch.sum(o_2 ** 2).backward()
    assert torch.allclose(q1.grad, q2.grad, atol=1e-5)
    assert torch.allclose(k1.grad, k2.grad, atol=1e-5)
    assert torch.allclose(v1.grad, v2.grad, atol=1e-5)


@pytest.mark.parametrize("shape,ks", [((1, 2, 9, 11, 32), 5), ((2, 1, 13, 13, 64), 13), ((1, 1, 17, 23, 128), 7),
                                      ((1, 2, 8, 9, 48), 3)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_scores_and_apply_against_oracle(shape, ks, dtype):
    q, k, v, d_o = make_inputs(shape, dtype, 500 + ks, q_scale=shape[-1] ** -0.5)
    g = torch.Generator().manual_seed(1)
    d_attn = torch.randn(shape[:4] + (ks * ks,), generator=g).to(dtype)
    # scores and their gradients
    qd, kd = (t.to(DEV).requires_grad_() for t in (q, k))
    attn = na.natten2dqk(qd, kd, ks, 1)
    attn.backward(d_attn.to(DEV))
    qr, kr = (t.double().requires_grad_() for t in (q, k))
    r_attn = orc.natten2d_qk(qr, kr, ks)
    r_attn.backward(d_attn.double())
    assert_close(attn, r_attn.detach(), dtype, f"scores {shape} ks={ks} {dtype}")
    assert_close(qd.grad, qr.grad, dtype, "scores dq")
    assert_close(kd.grad, kr.grad, dtype, "scores dk")
    # apply and its gradients, on normalised weights
    w = torch.softmax(r_attn.detach(), dim=-1).to(dtype)
    wd, vd = w.to(DEV).requires_grad_(), v.to(DEV).requires_grad_()
    out = na.natten2dav(wd, vd, ks, 1)
    out.backward(d_o.to(DEV))
    wr, vr = w.double().requires_grad_(), v.double().requires_grad_()
    r_out = orc.natten2d_av(wr, vr, ks)
    r_out.backward(d_o.double())
    assert_close(out, r_out.detach(), dtype, "apply out")
    assert_close(wd.grad, wr.grad, dtype, "apply d_attn")
    assert_close(vd.grad, vr.grad, dtype, "apply dv")


def test_unfused_errors():
    q = torch.zeros(1, 1, 8, 8, 32, device=DEV)
    with pytest.raises(ValueError):
        na.natten2dqk(q, q, 5, 2)                                 # only dilation 1 is built
    with pytest.raises(ValueError):
        na.natten2dqk(q, q, 4, 1)
    with pytest.raises(ValueError):
        na.natten2dav(torch.zeros(1, 1, 8, 8, 9, device=DEV), q, 5, 1)     # attn of another kernel size
