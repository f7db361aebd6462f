"""Shared fixtures. GPU tests are marked `gpu`; everything else runs on a CPU-only box."""
import os
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (sm_100) GPU")


@pytest.fixture(scope="session", autouse=True)
def _built_artifacts():
    """Build the native library and the C part of the oracle if a compiler is around (no-ops when up to date)."""
    try:
        from sys1_b200 import build as s1build
        s1build.build()
    except Exception as exc:  # pragma: no cover - on the GPU box the prebuilt .so travels with the tree
        if not (ROOT / "sys1_b200" / "libsys1_b200.so").exists():
            raise RuntimeError(f"libsys1_b200.so is missing and could not be built: {exc}")
    so = ROOT / "oracle" / "c" / "liboracle_delta.so"
    if not so.exists():
        subprocess.run(["make", "-C", str(ROOT / "oracle" / "c")], check=False, capture_output=True)
    yield


@pytest.fixture(scope="session")
def ctx():
    import torch
    from sys1_b200 import device
    if not torch.cuda.is_available():
        pytest.fail("a GPU test ran without a GPU")
    c = device.load(0)
    yield c
    c.sync()


def max_rel(actual, expected):
    """max |a - e| / max |e|: the 'max-relative' figure the acceptance bound (2e-2 for bf16) is stated in."""
    import torch
    a = actual.detach().float().cpu()
    e = expected.detach().float().cpu()
    return float((a - e).abs().max() / e.abs().max().clamp_min(1e-12))
