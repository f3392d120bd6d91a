"""Shared helpers of the parity tests."""
import torch

# Tolerances: fp32 path within 1e-4 relative (plus the 1e-5 absolute floor the reference's own
# test uses, test.py:36); 16-bit paths within 2e-2 absolute / 1e-2 relative.
TOL = {
    torch.float32: dict(rtol=1e-4, atol=1e-5),
    torch.bfloat16: dict(rtol=1e-2, atol=2e-2),
    torch.float16: dict(rtol=1e-2, atol=2e-2),
}


def assert_close(got, want, dtype, what=""):
    """|got - want| <= atol + rtol*|want| elementwise, compared in fp64."""
    tol = TOL[dtype]
    got = got.detach().to("cpu", torch.float64)
    want = want.detach().to("cpu", torch.float64)
    assert got.shape == want.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(want.shape)}"
    assert torch.isfinite(got).all(), f"{what}: non-finite values"
    err = (got - want).abs()
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
