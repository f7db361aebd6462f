"""ctypes binding of `libsys1_b200.so` (the C ABI in `include/sys1_b200.h`).

There is no fallback of any kind: if the library is missing, or a context cannot be opened on an sm_100 GPU,
the call raises. PyTorch is used by the callers only to hold device memory and streams; the pointers handed
to the library are plain addresses.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

PKG = Path(__file__).resolve().parent
LIB_PATH = PKG / "libsys1_b200.so"

S1_OK = 0
S1_EINVAL, S1_ECUDA, S1_EDEVICE, S1_EKERNEL, S1_ENOMEM, S1_ELIMIT, S1_ETIMEOUT = -1, -2, -3, -4, -5, -6, -7
STATIC_MAX_TOKENS, STATIC_MAX_FEATURES = 262144, 32768
COMM_ID_BYTES = 128
EXCHANGE_FLAG_BYTES = 4096  # S1_EXCHANGE_FLAG_BYTES
EPI_NONE, EPI_GEGLU, EPI_SWIGLU = 0, 1, 2
ACT_NONE, ACT_RELU, ACT_GELU = 0, 1, 2

_ERR_NAMES = {-1: "S1_EINVAL", -2: "S1_ECUDA", -3: "S1_EDEVICE", -4: "S1_EKERNEL", -5: "S1_ENOMEM", -6: "S1_ELIMIT", -7: "S1_ETIMEOUT"}


class S1Error(RuntimeError):
    """A C-ABI call returned a negative status."""

    def __init__(self, code: int, message: str):
        super().__init__(f"{_ERR_NAMES.get(code, code)}: {message}")
        self.code = code


class LinearDesc(C.Structure):
    _fields_ = [
        ("w", C.c_void_p), ("ldw", C.c_longlong),
        ("w_up", C.c_void_p), ("ldw_up", C.c_longlong),
        ("bias", C.c_void_p),
        ("N", C.c_int), ("K", C.c_int), ("epilogue", C.c_int), ("act", C.c_int),
    ]


# name -> (restype, argtypes); kept in one table so the symbol-export test can walk it.
SIGNATURES = {
    "s1_device_count": (C.c_int, [C.POINTER(C.c_int)]),
    "s1_ctx_create": (C.c_int, [C.c_int, C.c_void_p, C.POINTER(C.c_void_p)]),
    "s1_ctx_destroy": (C.c_int, [C.c_void_p]),
    "s1_last_error": (C.c_char_p, [C.c_void_p]),
    "s1_sync": (C.c_int, [C.c_void_p]),
    "s1_launch_count": (C.c_longlong, [C.c_void_p]),
    "s1_set_option": (C.c_int, [C.c_void_p, C.c_char_p, C.c_longlong]),
    "s1_pack_batch": (C.c_int, [C.POINTER(C.c_int32), C.c_int, C.c_int, C.c_int, C.POINTER(C.c_int32),
                                C.POINTER(C.c_int32), C.POINTER(C.c_int), C.POINTER(C.c_int), C.POINTER(C.c_int)]),
    "s1_linear_static": (C.c_int, [C.c_int, C.c_void_p, C.POINTER(LinearDesc), C.c_void_p, C.c_longlong, C.c_void_p,
                                   C.c_longlong, C.c_void_p, C.c_longlong, C.c_int, C.c_int, C.c_char_p, C.c_size_t]),
    "s1_delta_rule": (C.c_int, [C.c_void_p] * 7 + [C.c_int] * 5 + [C.c_void_p]),
    "s1_delta_rule_chunked_workspace": (C.c_size_t, [C.c_int, C.c_int, C.c_int]),
    "s1_delta_rule_chunked": (C.c_int, [C.c_void_p] * 6 + [C.POINTER(C.c_int32)] + [C.c_int] * 5 + [C.c_void_p, C.c_void_p, C.c_size_t]),
    "s1_conv_silu": (C.c_int, [C.c_void_p, C.c_void_p, C.c_longlong, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int,
                               C.c_void_p, C.c_longlong]),
    "s1_delta_inputs": (C.c_int, [C.c_void_p, C.c_void_p, C.c_longlong, C.c_void_p, C.c_void_p, C.c_longlong, C.c_void_p,
                                  C.c_void_p, C.c_int, C.c_int, C.c_int] + [C.c_void_p] * 5),
    "s1_delta_finish": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_longlong, C.c_void_p, C.c_float, C.c_int, C.c_int,
                                  C.c_void_p, C.c_longlong]),
    "s1_gated_delta_rule_workspace": (C.c_size_t, [C.c_int, C.c_int, C.c_int]),
    "s1_gated_delta_rule": (C.c_int, [C.c_void_p, C.c_void_p, C.c_longlong, C.c_void_p, C.c_void_p, C.c_longlong, C.c_void_p,
                                      C.c_void_p, C.c_void_p, C.c_longlong, C.c_void_p, C.c_float, C.POINTER(C.c_int32),
                                      C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_longlong, C.c_void_p, C.c_size_t]),
    "s1_gated_delta_rule_conv": (C.c_int, [C.c_void_p, C.c_void_p, C.c_longlong, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                           C.c_longlong, C.c_void_p, C.c_void_p, C.c_void_p, C.c_longlong, C.c_void_p, C.c_float,
                                           C.POINTER(C.c_int32), C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_longlong,
                                           C.c_void_p, C.c_size_t]),
    "s1_batch_plan_bytes": (C.c_size_t, [C.c_int, C.c_int]),
    "s1_batch_plan": (C.c_int, [C.c_void_p, C.POINTER(C.c_int32), C.c_int, C.c_int, C.c_void_p, C.c_size_t]),
    "s1_use_batch_plan": (C.c_int, [C.c_void_p, C.c_void_p]),
    "s1_batch_plan_release": (C.c_int, [C.c_void_p, C.c_void_p]),
    "s1_attention_workspace": (C.c_size_t, [C.c_int, C.c_int]),
    "s1_attention": (C.c_int, [C.c_void_p, C.c_void_p, C.c_longlong, C.c_void_p, C.c_longlong, C.c_void_p, C.c_longlong,
                               C.POINTER(C.c_int32), C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_float, C.c_void_p,
                               C.c_longlong, C.c_void_p, C.c_size_t]),
    "s1_attention_gqa_workspace": (C.c_size_t, [C.c_int, C.c_int]),
    "s1_attention_gqa": (C.c_int, [C.c_void_p, C.c_void_p, C.c_longlong, C.c_longlong, C.c_void_p, C.c_longlong, C.c_longlong,
                                   C.c_void_p, C.c_longlong, C.c_longlong, C.c_void_p, C.c_longlong, C.c_longlong,
                                   C.POINTER(C.c_int32), C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_float, C.c_void_p,
                                   C.c_longlong, C.c_void_p, C.c_size_t]),
    "s1_comm_unique_id": (C.c_int, [C.c_void_p, C.c_char_p, C.c_size_t]),
    "s1_comm_init": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_int]),
    "s1_comm_destroy": (C.c_int, [C.c_void_p]),
    "s1_allreduce_bf16": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t]),
    "s1_allreduce_wait": (C.c_int, [C.c_void_p]),
    "s1_exchange_register": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_size_t, C.POINTER(C.c_void_p), C.c_size_t]),
    "s1_allreduce_ticket": (C.c_longlong, [C.c_void_p]),
    "s1_allreduce_wait_ticket": (C.c_int, [C.c_void_p, C.c_longlong]),
    "s1_norm": (C.c_int, [C.c_void_p, C.c_void_p, C.c_longlong, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_float, C.c_int, C.c_void_p,
                          C.c_longlong, C.c_longlong, C.c_int]),
    "s1_rope": (C.c_int, [C.c_void_p, C.c_void_p, C.c_longlong, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int,
                          C.c_longlong, C.c_int]),
    "s1_add_rows": (C.c_int, [C.c_void_p, C.c_void_p, C.c_longlong, C.c_void_p, C.c_longlong, C.c_void_p, C.c_int, C.c_void_p,
                              C.c_longlong, C.c_longlong, C.c_int]),
    "s1_selftest_bounded_wait": (C.c_int, [C.c_void_p]),
    "s1_head_norm_rope": (C.c_int, [C.c_void_p, C.c_void_p, C.c_longlong, C.c_longlong, C.c_int, C.c_int, C.c_void_p, C.c_float,
                                    C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int]),
    "s1_linear_rope": (C.c_int, [C.c_void_p, C.POINTER(LinearDesc), C.c_void_p, C.c_longlong, C.c_void_p, C.c_longlong, C.c_int,
                                 C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int]),
    "s1_linear": (C.c_int, [C.c_void_p, C.POINTER(LinearDesc), C.c_void_p, C.c_longlong, C.c_void_p, C.c_longlong,
                            C.c_void_p, C.c_longlong, C.c_int]),
}

_lib = None


def load_library() -> C.CDLL:
    """dlopen the in-tree library and attach signatures. Raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m sys1_b200.build` (nvcc, sm_100a). "
            "There is no CPU or library fallback for this path.")
    lib = C.CDLL(str(LIB_PATH))
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib
