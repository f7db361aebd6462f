"""The C-ABI shared library loads and exports every symbol `include/sys1_b200.h` declares; argument checking
that needs no GPU behaves as documented. No compute call is made here."""
import ctypes as C
import re
from pathlib import Path

import pytest

from sys1_b200 import _lib

ROOT = Path(__file__).resolve().parents[1]
HEADER = ROOT / "include" / "sys1_b200.h"


def declared_functions():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(s1_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_something():
    names = declared_functions()
    assert {"s1_ctx_create", "s1_linear", "s1_delta_rule", "s1_pack_batch", "s1_sync"} <= set(names)


def test_every_declared_symbol_is_exported():
    lib = C.CDLL(str(_lib.LIB_PATH))
    missing = [n for n in declared_functions() if not hasattr(lib, n)]
    assert not missing, f"declared in the header but not exported: {missing}"


def test_python_binding_covers_the_header():
    assert sorted(_lib.SIGNATURES) == declared_functions()


def test_null_and_bad_arguments_are_rejected_without_a_gpu():
    lib = _lib.load_library()
    assert lib.s1_ctx_create(0, None, None) == _lib.S1_EINVAL
    assert lib.s1_sync(None) == _lib.S1_EINVAL
    assert lib.s1_ctx_destroy(None) == _lib.S1_EINVAL
    assert lib.s1_linear(None, None, None, 0, None, 0, None, 0, 1) == _lib.S1_EINVAL
    assert lib.s1_delta_rule(None, *([None] * 6), 1, 1, 1, 128, 128, None) == _lib.S1_EINVAL
    assert lib.s1_last_error(None) == b"null context"


def test_context_creation_fails_loudly_without_a_b200():
    import torch
    if torch.cuda.is_available():
        pytest.skip("this check is for CPU-only machines")
    lib = _lib.load_library()
    h = C.c_void_p()
    assert lib.s1_ctx_create(0, None, C.byref(h)) == _lib.S1_EDEVICE
    assert not h.value
    from sys1_b200 import device
    with pytest.raises(Exception):
        device.Context(0, stream=type("S", (), {"cuda_stream": 0})())


def test_operators_refuse_cpu_tensors():
    import torch
    from sys1_b200 import linear, qwen35
    x = torch.zeros(4, 8, dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="CUDA"):
        linear.fused_linear(x, x)
    f = torch.zeros(1, 1, 4, 128)
    with pytest.raises(ValueError, match="CUDA"):
        qwen35.chunked_delta_rule(f, f, f, f[..., 0], f[..., 0])
