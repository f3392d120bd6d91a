"""Stage the reference's own CPU implementation next to the oracle.  TEST INFRASTRUCTURE ONLY.

    python oracle/build_ref.py [--reference /path/to/e_natten_checkout]

The reference (vikhyat/e_natten) is pure Python: its CPU implementation of this path is the one
file e_natten/pytorch.py (Natten2d / Natten1d written as loops over torch ops).  There is nothing
to compile; "building" it means placing that file, unchanged, where the benchmark's CPU arm can
import it on a machine that has no checkout of the reference: oracle/_ref/, which is kept out of
version control (the file is the reference's, not this repository's) but travels with the built
artefacts.  Without a checkout at hand nothing happens and the CPU arm falls back to the
restatement in oracle/na2d_oracle.py.

The checkout is looked for in --reference, then in $E_NATTEN_REFERENCE, then in a directory named
"reference" beside this repository.
"""
from __future__ import annotations

import argparse
import importlib.util
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(HERE, "_ref")
STAGED = os.path.join(REF_DIR, "e_natten_pytorch.py")


def find_reference(explicit: str | None = None) -> str | None:
    candidates = [explicit, os.environ.get("E_NATTEN_REFERENCE"),
                  os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")]
    for c in candidates:
        if c and os.path.isfile(os.path.join(c, "e_natten", "pytorch.py")):
            return c
    return None


def build(reference: str | None = None) -> str | None:
    """Copy e_natten/pytorch.py of the checkout to oracle/_ref/; returns the staged path or None."""
    root = find_reference(reference)
    if root is None:
        return STAGED if os.path.isfile(STAGED) else None
    os.makedirs(REF_DIR, exist_ok=True)
    shutil.copyfile(os.path.join(root, "e_natten", "pytorch.py"), STAGED)
    return STAGED


def load():
    """The staged reference module (its ``natten2d`` / ``natten1d`` are the reference's own
    torch.autograd.Functions), or None if it has not been staged."""
    if not os.path.isfile(STAGED):
        return None
    spec = importlib.util.spec_from_file_location("e_natten_pytorch_ref", STAGED)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=None)
    path = build(ap.parse_args().reference)
    print(path if path else "no reference checkout found; nothing staged")
    sys.exit(0)
