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
OBJ = PKG / "csrc" / ".obj"

SOURCES = ["api.cu", "linear_static.cu", "batching.cu", "plan.cu", "delta_rule.cu", "delta_chunked.cu", "delta_io.cu", "attention.cu", "attention_gqa.cu", "norm_rope.cu", "comm.cu", "exchange.cu"]
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


def _deps_digest() -> str:
    """Digest of everything every translation unit may include (headers) and of this script."""
    h = hashlib.sha256()
    for f in sorted(list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + [ROOT / "include" / "sys1_b200.h", Path(__file__)]):
        h.update(f.name.encode())
        h.update(f.read_bytes())
    return h.hexdigest()


def _fingerprint() -> str:
    h = hashlib.sha256(_deps_digest().encode())
    for f in sorted(CSRC.glob("*.cu")):
        h.update(f.name.encode())
        h.update(f.read_bytes())
    return h.hexdigest()


def build(verbose: bool = False, force: bool = False) -> Path:
    """Compile the library if sources changed since the last build; returns the path of the .so. Each `.cu` file is
    compiled to an object of its own (in parallel, and only if it or a header changed), then the objects are linked."""
    from concurrent.futures import ThreadPoolExecutor
    fp = _fingerprint()
    if not force and LIB.exists() and STAMP.exists() and STAMP.read_text().strip() == fp:
        return LIB
    nvcc = _nvcc()
    OBJ.mkdir(exist_ok=True)
    deps = _deps_digest()
    flags = [f for f in NVCC_FLAGS if f != "-shared"]

    def compile_one(name: str):
        src, obj, tag = CSRC / name, OBJ / (name + ".o"), OBJ / (name + ".stamp")
        want = hashlib.sha256(deps.encode() + src.read_bytes()).hexdigest()
        if not force and obj.exists() and tag.exists() and tag.read_text() == want:
            return name, 0, ""
        cmd = [nvcc, *flags, *(["-Xptxas", "-v"] if verbose else []), "-I", str(ROOT / "include"), "-c", str(src), "-o", str(obj)]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode == 0:
            tag.write_text(want)
        return name, res.returncode, res.stdout + res.stderr

    names = [s for s in SOURCES if (CSRC / s).exists()]
    with ThreadPoolExecutor(max_workers=min(len(names), os.cpu_count() or 4)) as pool:
        results = list(pool.map(compile_one, names))
    failed = [n for n, rc, _ in results if rc != 0]
    for n, rc, log in results:
        if log and (verbose or rc != 0):
            sys.stderr.write(f"--- {n}\n{log}")
    if failed:
        raise RuntimeError(f"nvcc failed on {failed}")
    link = [nvcc, "-shared", "-Xcompiler", "-fPIC", "-gencode", "arch=compute_100a,code=sm_100a", "-o", str(LIB),
            *(str(OBJ / (n + ".o")) for n in names), "-lcudart", "-ldl"]
    res = subprocess.run(link, capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
        raise RuntimeError("linking libsys1_b200.so failed")
    STAMP.write_text(fp)
    return LIB


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv, force="--force" in sys.argv or "-v" in sys.argv))
