"""gograd_b200 — B200-native optimizer-step engine behind gograd's optimizer API.

The product is ``liboptengine.so`` (hand-written sm_100a kernels behind a C ABI,
``include/optengine.h``). This package is the thin binding used by the tests and
the benchmark: it loads the library with ctypes and passes device addresses of
torch tensors; torch is only plumbing here (device memory, streams,
``torch.distributed``). There is no CPU fallback: loading fails loudly when the
library has not been built, and every device call fails without a B200.
"""
from . import _lib  # noqa: F401
from .engine import (AdamWHParams, Plan, SGDHParams, TensorDesc, cast_bf16, init, launch_count,  # noqa: F401
                     launch_count_reset)

__all__ = ["AdamWHParams", "SGDHParams", "TensorDesc", "Plan", "cast_bf16", "init", "launch_count",
           "launch_count_reset"]
