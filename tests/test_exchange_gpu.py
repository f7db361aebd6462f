"""The symmetric-memory exchange kernel's failure path on ONE GPU: a rank whose peer never shows up gives up after
`exchange_wait_ms`, the host reads S1_EKERNEL from `s1_sync`, and the context goes on working. The "peer" here is a flag
array on the same GPU that nothing ever writes, so the kernel leaves at its first meeting point, before it touches the
multicast address (which is therefore never dereferenced: a plain local buffer stands in for it). The data path itself
needs two GPUs and is covered by the tensor-parallel test."""
import ctypes as C
import time

import pytest
import torch

from sys1_b200 import _lib, linear

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def test_a_rank_whose_peer_never_arrives_gives_up_and_the_context_survives(ctx):
    buf = torch.zeros(1 << 16, dtype=torch.bfloat16, device=DEV)
    mine = torch.zeros(_lib.EXCHANGE_FLAG_BYTES // 4, dtype=torch.int32, device=DEV)
    peer = torch.zeros(_lib.EXCHANGE_FLAG_BYTES // 4, dtype=torch.int32, device=DEV)
    torch.cuda.synchronize()
    ctx.set_option("exchange_wait_ms", 50)
    try:
        ctx.exchange_register(0, 2, buf.data_ptr(), buf.data_ptr(), buf.numel() * 2, [mine.data_ptr(), peer.data_ptr()])
        t0 = time.time()
        ctx.all_reduce_(buf[:4096])
        with pytest.raises(_lib.S1Error) as err:
            ctx.sync()
        took = time.time() - t0
        assert err.value.code == _lib.S1_EKERNEL and "bounded wait" in str(err.value)
        assert took < 5.0, f"the wait ran for {took:.2f} s"
        # this rank did announce itself to the peer before it gave up
        assert int(peer[0]) == 1
        assert float(buf.float().abs().max()) == 0.0   # nothing was reduced
    finally:
        ctx.set_option("exchange_wait_ms", 10000)
        # forget the registration: later sums on this context go back to the communicator path
        ctx._lib.s1_exchange_register(ctx.handle, 0, 0, None, None, 0, None, 0)
    # the context still computes
    x = torch.randn(256, 128, device=DEV).to(torch.bfloat16)
    w = torch.randn(64, 128, device=DEV).to(torch.bfloat16)
    y = linear.fused_linear(x, w)
    ctx.sync()
    assert torch.allclose(y.float(), x.float() @ w.float().t(), rtol=2e-2, atol=2e-1)


def test_registration_is_checked(ctx):
    buf = torch.zeros(1024, dtype=torch.bfloat16, device=DEV)
    flags = torch.zeros(_lib.EXCHANGE_FLAG_BYTES // 4, dtype=torch.int32, device=DEV)
    arr = (C.c_void_p * 2)(flags.data_ptr(), flags.data_ptr())
    lib, h = ctx._lib, ctx.handle
    P = C.c_void_p
    assert lib.s1_exchange_register(h, 2, 2, P(buf.data_ptr()), P(buf.data_ptr()), 2048, arr, 4096) == _lib.S1_EINVAL   # rank outside the group
    assert lib.s1_exchange_register(h, 0, 17, P(buf.data_ptr()), P(buf.data_ptr()), 2048, arr, 4096) == _lib.S1_EINVAL  # too many ranks
    assert lib.s1_exchange_register(h, 0, 2, P(buf.data_ptr() + 2), P(buf.data_ptr()), 2048, arr, 4096) == _lib.S1_EINVAL  # misaligned
    assert lib.s1_exchange_register(h, 0, 2, P(buf.data_ptr()), P(buf.data_ptr()), 2048, arr, 64) == _lib.S1_EINVAL    # flag arrays too small
    assert lib.s1_exchange_register(h, 0, 2, P(buf.data_ptr()), None, 2048, arr, 4096) == _lib.S1_EINVAL
