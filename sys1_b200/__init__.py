"""sys1_b200: the dense-projection / gated-delta-rule hot path of sys1, written for B200 (sm_100a).

Python here is host plumbing over the C ABI in `include/sys1_b200.h` (library: `libsys1_b200.so`, built by
`python -m sys1_b200.build`). Importing the package does not need a GPU; calling any operator does.
"""
from ._lib import (ACT_GELU, ACT_NONE, ACT_RELU, EPI_GEGLU, EPI_NONE, EPI_SWIGLU, S1Error,  # noqa: F401
                   load_library)

__all__ = ["EPI_NONE", "EPI_GEGLU", "EPI_SWIGLU", "ACT_NONE", "ACT_RELU", "ACT_GELU", "S1Error", "load_library"]
