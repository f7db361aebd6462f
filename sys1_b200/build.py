"""Builds the in-tree native library `sys1_b200/libsys1_b200.so` with nvcc for sm_100a only.

Takes the place of the reference's `build.rs:51-83` (which concatenates `src/kernels/*.cu` and emits generic
PTX for whatever compute capability it finds): here there is exactly one target, `sm_100a`, and the output is
a shared library exporting the C ABI declared in `include/sys1_b200.h`.

Run as `python -m sys1_b200.build` (add `-v` for the ptxas resource report).
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
ROOT = PKG.parent
CSRC = PKG / "csrc"
LIB = PKG / "libsys1_b200.so"
STAMP = PKG / "csrc" / ".build_stamp"

SOURCES = ["api.cu", "linear_static.cu", "batching.cu", "delta_rule.cu", "delta_chunked.cu", "delta_io.cu", "attention.cu", "attention_gqa.cu", "norm_rope.cu", "comm.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC", "-shared",
    "--expt-relaxed-constexpr",
    "-Xcudafe", "--diag_suppress=177",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found; the native library cannot be built")


def _fingerprint() -> str:
    h = hashlib.sha256()
    for f in sorted(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) +
                    [ROOT / "include" / "sys1_b200.h", Path(__file__)]):
        h.update(f.name.encode())
        h.update(f.read_bytes())
    return h.hexdigest()


def build(verbose: bool = False, force: bool = False) -> Path:
    """Compile the library if sources changed since the last build; returns the path of the .so."""
    fp = _fingerprint()
    if not force and LIB.exists() and STAMP.exists() and STAMP.read_text().strip() == fp:
        return LIB
    srcs = [str(CSRC / s) for s in SOURCES if (CSRC / s).exists()]
    cmd = [_nvcc(), *NVCC_FLAGS, "-I", str(ROOT / "include"), "-o", str(LIB), *srcs, "-lcudart", "-ldl"]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed building libsys1_b200.so")
    STAMP.write_text(fp)
    return LIB


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv, force=True))
