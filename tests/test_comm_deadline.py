"""Failure detection on the exchange, tested on the host: `s1_comm_init` creates its NCCL communicator with a
deadline (`comm_timeout_ms`); a rank that never joins makes the call return S1_ETIMEOUT after aborting the half-built
communicator instead of blocking for ever. The deadline logic (sys1_b200/csrc/comm_init.h) is host-only code; here it
is compiled with g++ against a stand-in table of NCCL entry points whose communicator never becomes ready, becomes
ready late, or fails. No GPU and no NCCL library are touched."""
import shutil
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]


def _include_dirs():
    dirs = [ROOT / "sys1_b200" / "csrc", ROOT / "include"]
    for cand in (Path("/usr/local/cuda/include"), Path("/usr/include")):
        if cand.exists():
            dirs.append(cand)
    return dirs


def test_comm_init_deadline_with_a_stand_in_nccl(tmp_path):
    gxx = shutil.which("g++")
    if gxx is None:
        pytest.skip("no host compiler")
    exe = tmp_path / "comm_deadline_test"
    cmd = [gxx, "-std=c++17", "-O1", "-pthread", *(f"-I{d}" for d in _include_dirs()),
           str(ROOT / "tests" / "native" / "comm_deadline_test.cc"), "-o", str(exe)]
    built = subprocess.run(cmd, capture_output=True, text=True)
    assert built.returncode == 0, built.stderr
    run = subprocess.run([str(exe)], capture_output=True, text=True, timeout=60)
    assert run.returncode == 0, run.stdout + run.stderr
    for case in ("never_joins_times_out", "joins_late_succeeds", "connect_failure_is_reported", "no_deadline_is_blocking",
                 "collective_in_progress_is_polled"):
        assert f"{case}: ok" in run.stdout
