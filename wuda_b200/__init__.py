"""wuda_b200 — B200 (sm_100a) implementation of the DeepSeek-V4-style decode hot path.

The product is libwuda_b200.so (hand-written CUDA behind the C ABI of
include/wuda_b200.h).  This package is the thin host-side mirror of the reference's
Python operator interface on top of that ABI; torch is used only for device memory and
streams.  Importing the package requires the built library (python -m wuda_b200.build).
"""
import sys as _sys


def _running_the_build_module():
    """`python -m wuda_b200.build` imports this package first; it must work before the library exists (and while an
    older library lacks newly declared entry points), so the library is not loaded for that one command."""
    argv = list(getattr(_sys, "orig_argv", []) or [])
    return any(a == "-m" and i + 1 < len(argv) and argv[i + 1] == "wuda_b200.build" for i, a in enumerate(argv))


if not _running_the_build_module():
    from ._lib import WudaError, lib, LIB_PATH  # noqa: F401
    from .ops import *  # noqa: F401,F403
    from .shims import *  # noqa: F401,F403
