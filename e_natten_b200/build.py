"""Build libna2d.so in-tree with nvcc for sm_100a.

    python e_natten_b200/build.py [--force] [--verbose]

The library is plain CUDA C++ behind a C ABI (include/na2d.h); it needs no framework headers.
Its kernels are compiled as seven translation units in parallel (the API with the SIMT kernels,
and each of the three tcgen05 kernel families once per 16-bit element type) and linked into one
shared object.
"""
from __future__ import annotations

import concurrent.futures
import os
import shutil
import subprocess
import sys

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG_DIR, "csrc")
OBJ_DIR = os.path.join(PKG_DIR, "build")
LIB_PATH = os.path.join(PKG_DIR, "libna2d.so")
# (source, extra defines, object name)
UNITS = [
    ("na2d_api.cu", [], "na2d_api.o"),
    ("na2d_tc_fwd.cu", ["-DNA2D_TC_DT=1"], "na2d_tc_fwd_bf16.o"),
    ("na2d_tc_fwd.cu", ["-DNA2D_TC_DT=2"], "na2d_tc_fwd_f16.o"),
    ("na2d_tc_dq.cu", ["-DNA2D_TC_DT=1"], "na2d_tc_dq_bf16.o"),
    ("na2d_tc_dq.cu", ["-DNA2D_TC_DT=2"], "na2d_tc_dq_f16.o"),
    ("na2d_tc_dkdv.cu", ["-DNA2D_TC_DT=1"], "na2d_tc_dkdv_bf16.o"),
    ("na2d_tc_dkdv.cu", ["-DNA2D_TC_DT=2"], "na2d_tc_dkdv_f16.o"),
]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC"]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; libna2d.so cannot be built")
    return exe


def _deps():
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)]
    deps.append(os.path.join(os.path.dirname(PKG_DIR), "include", "na2d.h"))
    return [d for d in deps if os.path.isfile(d)]


def _stale() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    built = os.path.getmtime(LIB_PATH)
    return any(os.path.getmtime(d) > built for d in _deps())


def _compile(unit, verbose: bool, extra, obj_dir):
    src, defines, obj = unit
    cmd = [_nvcc(), *NVCC_FLAGS, *extra, *(["-Xptxas", "-v"] if verbose else []), *defines, "-c",
           os.path.join(CSRC, src), "-o", os.path.join(obj_dir, obj)]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    return obj, proc.returncode, proc.stdout + proc.stderr, " ".join(cmd)


def build(force: bool = False, verbose: bool = False, extra_flags=(), lib_path: str = LIB_PATH) -> str:
    """Compile the library if it is missing or older than its sources; return its path."""
    if not force and lib_path == LIB_PATH and not _stale():
        return LIB_PATH
    # a library built elsewhere with other flags (a development build) keeps its objects apart
    obj_dir = OBJ_DIR if lib_path == LIB_PATH else lib_path + ".objs"
    os.makedirs(obj_dir, exist_ok=True)
    workers = max(1, min(len(UNITS), os.cpu_count() or 1))
    with concurrent.futures.ThreadPoolExecutor(workers) as pool:
        results = list(pool.map(lambda u: _compile(u, verbose, list(extra_flags), obj_dir), UNITS))
    for obj, rc, out, cmd in results:
        if verbose or rc != 0:
            sys.stderr.write(f"--- {obj}\n{out}")
        if rc != 0:
            raise RuntimeError("nvcc failed building %s (command: %s)" % (obj, cmd))
    link = [_nvcc(), "-shared", "-Xcompiler", "-fPIC", "-gencode", "arch=compute_100a,code=sm_100a",
            *[os.path.join(obj_dir, u[2]) for u in UNITS], "-o", lib_path]
    proc = subprocess.run(link, capture_output=True, text=True)
    if proc.returncode != 0:
        sys.stderr.write(proc.stdout + proc.stderr)
        raise RuntimeError("nvcc failed linking libna2d.so (command: %s)" % " ".join(link))
    return lib_path


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
