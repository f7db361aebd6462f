"""`s1_linear_static`, the projection entry point for callers that must not allocate device memory (a host whose
GPU memory belongs to another allocator, code under stream capture or in a latency-critical loop): called
through the C ABI and compared with the regular entry point `s1_linear` on the same inputs, twice in a row - the
second call reuses the library's static scratch block with whatever the first left in it.

Collected last on purpose: a run that stops at the first failure has then already run everything else.
It passes alone in a fresh process (the first call performs the per-device set-up) and after the other tests.
"""
import ctypes as C

import pytest
import torch

from sys1_b200 import _lib, linear
from sys1_b200._lib import EPI_GEGLU, EPI_NONE, EPI_SWIGLU

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _static(lib, w, x, y, *, w_up=None, residual=None, epilogue=EPI_NONE, wait=1):
    T, K = x.shape
    d = _lib.LinearDesc(w=w.data_ptr(), ldw=w.stride(0), w_up=0 if w_up is None else w_up.data_ptr(),
                        ldw_up=0 if w_up is None else w_up.stride(0), bias=0, N=w.shape[0], K=K,
                        epilogue=epilogue, act=0)
    err = C.create_string_buffer(256)
    stream = torch.cuda.current_stream(0).cuda_stream
    rc = lib.s1_linear_static(0, C.c_void_p(stream), C.byref(d), C.c_void_p(x.data_ptr()), x.stride(0),
                              C.c_void_p(0 if residual is None else residual.data_ptr()),
                              0 if residual is None else residual.stride(0), C.c_void_p(y.data_ptr()), y.stride(0),
                              T, wait, err, len(err))
    return rc, err.value.decode()


def test_static_entry_point_matches_the_regular_one_twice():
    lib = _lib.load_library()
    g = torch.Generator().manual_seed(2024)
    for round_ in range(2):  # two calls in a row per shape: the second finds the scratch as the first left it
        for (T, N, K) in ((300, 768, 768), (20000, 2304, 768)):
            x = torch.randn(T, K, generator=g).to(torch.bfloat16).to(DEV)
            w = (torch.randn(N, K, generator=g) * 0.02).to(torch.bfloat16).to(DEV)
            w2 = (torch.randn(N, K, generator=g) * 0.02).to(torch.bfloat16).to(DEV)
            res = torch.randn(T, N, generator=g).to(torch.bfloat16).to(DEV)

            want = linear.fused_linear(x, w)
            got = torch.empty_like(want)
            rc, msg = _static(lib, w, x, got)
            assert rc == _lib.S1_OK, msg
            assert torch.equal(got, want)

            want = linear.fused_linear(x, w, residual=res)
            got = torch.empty_like(want)
            rc, msg = _static(lib, w, x, got, residual=res)
            assert rc == _lib.S1_OK, msg
            assert torch.equal(got, want)

            stream_buf = res.clone()  # residual stream updated in place
            rc, msg = _static(lib, w, x, stream_buf, residual=stream_buf)
            assert rc == _lib.S1_OK, msg
            assert (stream_buf.float() - want.float()).abs().max() <= 2 ** -7 * want.float().abs().max()

            want = linear.fused_linear(x, w, epilogue=EPI_GEGLU)
            got = torch.empty_like(want)
            rc, msg = _static(lib, w, x, got, epilogue=EPI_GEGLU)
            assert rc == _lib.S1_OK, msg
            assert torch.equal(got, want)

            want = linear.fused_linear(x, w, weight_up=w2, epilogue=EPI_SWIGLU)
            got = torch.empty_like(want)
            rc, msg = _static(lib, w, x, got, w_up=w2, epilogue=EPI_SWIGLU, wait=0)  # asynchronous form
            assert rc == _lib.S1_OK, msg
            torch.cuda.synchronize()
            assert torch.equal(got, want)


def test_static_entry_point_leaves_device_memory_as_it_found_it():
    """The property the entry point is named for: once its one-time set-up has run, a call neither takes nor gives
    back device memory. The driver's count of free bytes and PyTorch's own allocator are read before and after a
    second round of calls (every tensor the calls touch exists before the first reading)."""
    lib = _lib.load_library()
    g = torch.Generator().manual_seed(7)
    T, N, K = 4096, 768, 768
    x = torch.randn(T, K, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(N, K, generator=g) * 0.02).to(torch.bfloat16).to(DEV)
    w2 = (torch.randn(N, K, generator=g) * 0.02).to(torch.bfloat16).to(DEV)
    res = torch.randn(T, N, generator=g).to(torch.bfloat16).to(DEV)
    y, yg = torch.empty(T, N, dtype=torch.bfloat16, device=DEV), torch.empty(T, N // 2, dtype=torch.bfloat16, device=DEV)

    def calls():
        for kw, out in ((dict(), y), (dict(residual=res), y), (dict(epilogue=EPI_GEGLU), yg), (dict(w_up=w2, epilogue=EPI_SWIGLU), y)):
            rc, msg = _static(lib, w, x, out, **kw)
            assert rc == _lib.S1_OK, msg

    calls()  # first round: includes the per-device set-up and the loading of the kernels
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info(0)
    alloc0, reserved0 = torch.cuda.memory_allocated(0), torch.cuda.memory_reserved(0)
    calls()
    calls()
    torch.cuda.synchronize()
    free1, _ = torch.cuda.mem_get_info(0)
    assert free1 == free0
    assert torch.cuda.memory_allocated(0) == alloc0 and torch.cuda.memory_reserved(0) == reserved0


def test_static_entry_point_keeps_the_callers_device():
    """With more than one GPU visible the call makes its device current only for its own duration."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two visible GPUs")
    lib = _lib.load_library()
    x = torch.randn(256, 64).to(torch.bfloat16).to(DEV)
    w = torch.randn(64, 64).to(torch.bfloat16).to(DEV)
    y = torch.empty(256, 64, dtype=torch.bfloat16, device=DEV)
    torch.cuda.set_device(1)
    try:
        rc, msg = _static(lib, w, x, y)
        assert rc == _lib.S1_OK, msg
        assert torch.cuda.current_device() == 1
    finally:
        torch.cuda.set_device(0)


def test_static_entry_point_rejects_what_it_does_not_cover():
    lib = _lib.load_library()
    x = torch.zeros(8, 64, dtype=torch.bfloat16, device=DEV)
    w = torch.zeros(64, 64, dtype=torch.bfloat16, device=DEV)
    y = torch.zeros(8, 64, dtype=torch.bfloat16, device=DEV)
    T_big = _lib.STATIC_MAX_TOKENS + 1
    d = _lib.LinearDesc(w=w.data_ptr(), ldw=64, w_up=0, ldw_up=0, bias=0, N=64, K=64, epilogue=0, act=0)
    err = C.create_string_buffer(256)
    rc = lib.s1_linear_static(0, None, C.byref(d), C.c_void_p(x.data_ptr()), 64, None, 0, C.c_void_p(y.data_ptr()), 64,
                              T_big, 1, err, len(err))
    assert rc == _lib.S1_ELIMIT and b"exceeds the supported maximum" in err.value
    d.act = 1
    rc = lib.s1_linear_static(0, None, C.byref(d), C.c_void_p(x.data_ptr()), 64, None, 0, C.c_void_p(y.data_ptr()), 64,
                              8, 1, err, len(err))
    assert rc == _lib.S1_EINVAL and b"s1_linear" in err.value
