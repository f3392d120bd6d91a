"""Shared helpers of the parity tests."""
import torch

# Tolerances.  fp32 path: within 1e-4 relative, where an element is measured against
# max(|its value|, rms of the tensor) so that elements that cancel to near zero are judged at
# the tensor's scale (fp32 rounding inside exp() of O(10) logits alone gives ~1e-5 relative).
# 16-bit paths: within 2e-2 absolute + 1e-2 relative.
TOL = {
    torch.float32: dict(rtol=1e-4, atol=0.0, rms_rel=1e-4),
    torch.bfloat16: dict(rtol=1e-2, atol=2e-2, rms_rel=0.0),
    torch.float16: dict(rtol=1e-2, atol=2e-2, rms_rel=0.0),
}


def assert_close(got, want, dtype, what=""):
    """fp32 path: |got - want| <= rtol * max(|want|, rms(want)); 16-bit paths:
    |got - want| <= atol + rtol*|want|.  Compared in fp64."""
    tol = TOL[dtype]
    got = got.detach().to("cpu", torch.float64)
    want = want.detach().to("cpu", torch.float64)
    assert got.shape == want.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(want.shape)}"
    assert torch.isfinite(got).all(), f"{what}: non-finite values"
    err = (got - want).abs()
    rms = want.pow(2).mean().sqrt().item() if want.numel() else 0.0
    if tol["rms_rel"] > 0.0:
        bound = tol["atol"] + torch.maximum(tol["rtol"] * want.abs(), torch.full_like(want, tol["rms_rel"] * rms))
    else:
        bound = tol["atol"] + tol["rtol"] * want.abs()
    bad = err > bound
    if bad.any():
        idx = torch.nonzero(bad)[0].tolist()
        raise AssertionError(
            f"{what}: {int(bad.sum())} of {bad.numel()} elements out of tolerance; max err "
            f"{err.max().item():.3e}; first bad index {idx}: got {got[tuple(idx)].item():.6f} "
            f"want {want[tuple(idx)].item():.6f}")


def make_inputs(shape, dtype, seed, scale=1.0, q_scale=1.0):
    from oracle.na2d_oracle import round_inputs
    return round_inputs(shape, dtype, seed, scale, q_scale)
