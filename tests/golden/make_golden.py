"""Generate tests/golden/na2d_golden.npz by running the reference itself on the CPU.

Run where the e_natten sources are available:

    python tests/golden/make_golden.py --reference /path/to/e_natten_checkout

Five groups of vectors are written, all small:

* ``idx/...``   window_start / backward_window_start / backward_window_end tables
                from e_natten/pytorch.py:7-23 (and the identical copies in
                e_natten/triton.py:14-30) for odd kernel sizes 3..15 and a sweep of
                sequence lengths.
* ``pt/...``    inputs and outputs of e_natten.pytorch.natten2d (pytorch.py:158-292) on
                the CPU.  Its dQ is only filled for the first 3x3 tile
                (pytorch.py:228-231) and its forward is wrong for kernel sizes with
                ks//2 % 3 == 1, so only ks in {5, 7, 11, 13} are recorded and dQ is
                recorded for that tile only.
* ``tr/...``    inputs and outputs of the fused entry point e_natten.natten2d
                (triton.py:487-550) executed by the Triton interpreter on the CPU,
                forward and all three gradients, loss = sum(o**2) as in test.py:39-42,
                on the shape family test.py:53 uses (scaled down to interpreter speed).
* ``pt1d/...``  inputs and outputs of e_natten.pytorch.natten1d (pytorch.py:46-156), fp32 (its
                output buffer is fp32 whatever the input), forward and all three gradients.
                Like the 2D one its forward (and with it dQ) is wrong for kernel sizes with
                ks//2 % 3 == 1, so only ks in {5, 7, 11, 13} are recorded.
* ``tr1d/...``  the fused 1D entry point e_natten.natten1d (triton.py:425-485) under the Triton
                interpreter, on the shape of test.py:51.  Its backward kernel loads and adds
                without masks (triton.py:176-181, 215-222), which reads and writes beyond the
                tensors for some sizes; each case therefore runs in a child process and is kept
                only if that process ends cleanly with finite values.
"""
import argparse
import os
import subprocess
import sys
import tempfile

import numpy as np


def triton_1d_case(reference: str, ks: int, seed: int, out_path: str):
    """One 1D case of the fused Triton entry point under the interpreter (run in a child)."""
    os.environ["TRITON_INTERPRET"] = "1"
    sys.path.insert(0, reference)
    import torch
    import e_natten.triton as ref_tr
    g = torch.Generator().manual_seed(seed)
    q, k, v = (torch.randn((2, 3, 16, 2), generator=g, dtype=torch.float32) for _ in range(3))
    qr, kr, vr = (t.clone().requires_grad_() for t in (q, k, v))
    o = ref_tr.natten1d(qr, kr, vr, ks)
    torch.sum(o ** 2).backward()
    vals = {"q": q, "k": k, "v": v, "o": o.detach(), "dq": qr.grad, "dk": kr.grad, "dv": vr.grad}
    if not all(bool(torch.isfinite(t).all()) for t in vals.values()):
        raise SystemExit(3)
    np.savez(out_path, **{n: t.numpy() for n, t in vals.items()})


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path of an e_natten source checkout")
    ap.add_argument("--out", default=os.path.join(os.path.dirname(os.path.abspath(__file__)), "na2d_golden.npz"))
    ap.add_argument("--triton-1d-case", nargs=3, metavar=("KS", "SEED", "OUT"), default=None,
                    help="internal: run one 1D Triton case and write it to OUT")
    args = ap.parse_args()
    if args.triton_1d_case:
        triton_1d_case(args.reference, int(args.triton_1d_case[0]), int(args.triton_1d_case[1]), args.triton_1d_case[2])
        return

    os.environ["TRITON_INTERPRET"] = "1"          # must be set before triton is imported
    sys.path.insert(0, args.reference)
    import torch
    import e_natten.pytorch as ref_pt
    import e_natten.triton as ref_tr

    out = {}

    # ---- index tables --------------------------------------------------------------
    lens_extra = [192, 256, 1024]
    for ks in range(3, 16, 2):
        for L in list(range(ks, 81)) + lens_extra:
            ws = [ref_pt.get_window_start(i, L, ks) for i in range(L)]
            ws2 = [ref_tr.get_window_start(i, L, ks) for i in range(L)]
            assert ws == ws2
            bs = [ref_pt.get_backward_window_start(i, ks) for i in range(L)]
            be = [ref_pt.get_backward_window_end(i, L, ks) for i in range(L)]
            out[f"idx/ws/{ks}/{L}"] = np.asarray(ws, dtype=np.int32)
            out[f"idx/bws/{ks}/{L}"] = np.asarray(bs, dtype=np.int32)
            out[f"idx/bwe/{ks}/{L}"] = np.asarray(be, dtype=np.int32)

    # ---- e_natten.pytorch on CPU -----------------------------------------------------
    pt_cases = [
        # name, shape, ks, dtype, seed
        ("c1", (1, 2, 16, 16, 32), 5, torch.float32, 0),     # the CPU-runnable benchmark config
        ("k5", (2, 2, 14, 14, 4), 5, torch.float64, 1),
        ("k7", (1, 2, 17, 19, 4), 7, torch.float64, 2),
        ("k11", (1, 1, 16, 16, 4), 11, torch.float64, 3),
        ("k13", (1, 1, 14, 14, 4), 13, torch.float64, 4),
    ]
    for name, shape, ks, dt, seed in pt_cases:
        g = torch.Generator().manual_seed(seed)
        q, k, v, d_o = (torch.randn(shape, generator=g, dtype=torch.float32).to(dt) for _ in range(4))
        qr, kr, vr = (t.clone().requires_grad_() for t in (q, k, v))
        o = ref_pt.natten2d(qr, kr, vr, ks)
        o.backward(d_o)
        for nm, t in (("q", q), ("k", k), ("v", v), ("do", d_o), ("o", o.detach()),
                      ("dk", kr.grad), ("dv", vr.grad), ("dq_tile00", qr.grad[:, :, :3, :3])):
            out[f"pt/{name}/{nm}"] = t.numpy()
        out[f"pt/{name}/ks"] = np.asarray(ks)
        print("pytorch ref", name, "done", flush=True)

    # ---- e_natten.natten2d (Triton kernels) under the interpreter ---------------------
    tr_cases = [
        ("k3", (1, 2, 6, 6, 2), 3, 10),
        ("k5", (2, 3, 8, 8, 2), 5, 11),
        ("k7", (1, 2, 9, 10, 4), 7, 12),
        ("k9", (1, 1, 10, 9, 2), 9, 13),
        ("k11", (1, 1, 12, 11, 2), 11, 14),
    ]
    for name, shape, ks, seed in tr_cases:
        g = torch.Generator().manual_seed(seed)
        q, k, v = (torch.randn(shape, generator=g, dtype=torch.float32) for _ in range(3))
        qr, kr, vr = (t.clone().requires_grad_() for t in (q, k, v))
        o = ref_tr.natten2d(qr, kr, vr, ks)
        torch.sum(o ** 2).backward()
        for nm, t in (("q", q), ("k", k), ("v", v), ("o", o.detach()),
                      ("dq", qr.grad), ("dk", kr.grad), ("dv", vr.grad)):
            out[f"tr/{name}/{nm}"] = t.numpy()
        out[f"tr/{name}/ks"] = np.asarray(ks)
        print("triton-interpreter ref", name, "done", flush=True)

    # ---- e_natten.pytorch.natten1d on CPU (fp32) ----------------------------------------
    for ks, seed in ((5, 31), (7, 32), (11, 33), (13, 34)):
        g = torch.Generator().manual_seed(seed)
        q, k, v, d_o = (torch.randn((2, 3, 17, 4), generator=g, dtype=torch.float32) for _ in range(4))
        qr, kr, vr = (t.clone().requires_grad_() for t in (q, k, v))
        o = ref_pt.natten1d(qr, kr, vr, ks)
        o.backward(d_o)
        for nm, t in (("q", q), ("k", k), ("v", v), ("do", d_o), ("o", o.detach()),
                      ("dq", qr.grad), ("dk", kr.grad), ("dv", vr.grad)):
            out[f"pt1d/k{ks}/{nm}"] = t.numpy()
        out[f"pt1d/k{ks}/ks"] = np.asarray(ks)
        print("pytorch 1D ref", ks, "done", flush=True)

    # ---- e_natten.natten1d (Triton) under the interpreter, one child process per case ----
    kept = []
    for ks, seed in ((3, 40), (5, 41), (7, 42), (9, 43), (11, 44)):
        with tempfile.TemporaryDirectory() as tmp:
            piece = os.path.join(tmp, "case.npz")
            rc = subprocess.run([sys.executable, os.path.abspath(__file__), "--reference", args.reference,
                                 "--triton-1d-case", str(ks), str(seed), piece]).returncode
            if rc != 0 or not os.path.exists(piece):
                print(f"triton-interpreter 1D ref k{ks}: child ended with {rc}, case dropped", flush=True)
                continue
            data = np.load(piece)
            for nm in data.files:
                out[f"tr1d/k{ks}/{nm}"] = data[nm]
            out[f"tr1d/k{ks}/ks"] = np.asarray(ks)
            kept.append(ks)
            print("triton-interpreter 1D ref", ks, "done", flush=True)
    out["tr1d/kept"] = np.asarray(kept, dtype=np.int32)

    np.savez_compressed(args.out, **out)
    print("wrote", args.out, os.path.getsize(args.out), "bytes")


if __name__ == "__main__":
    main()
