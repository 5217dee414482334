"""B200 (sm_100a) sparse FlashAttention forward operators.

Drop-in for the six operators of KLab-AI3/Graph-Processing-Attention-IPDPS-2025. Three layers:

* ``lib/libspfa_b200.so`` -- the C-ABI library (include/spfa_b200.h) with the hand-written CUDA kernels;
* ``lib/spfa_<mask>.*.so`` -- six torch-extension modules with the reference's module names and
  ``forward`` signatures (``import spfa_csr`` etc. once :func:`add_bindings_to_path` ran, or via
  :func:`binding`);
* :mod:`capi` -- a ctypes view of the C ABI that takes torch CUDA tensors (row-range sharding lives
  here, it has no counterpart in the reference's single-GPU API);
* :mod:`hostio` -- forward calls on pinned HOST buffers for the banded masks, with the copies and the row-range
  kernels overlapped.

The directory name is not a valid Python identifier; load the package with ``importlib`` (see
``load()`` in the repository's ``__graft_entry__.py``) under the name ``spfa_b200``.

There is no CPU implementation: every operator raises if the CUDA library is missing.
"""
from __future__ import annotations

import importlib
import importlib.util
import os
import sys

_HERE = os.path.dirname(os.path.abspath(__file__))
LIBDIR = os.path.join(_HERE, "lib")

MODULES = ("spfa_csr", "spfa_coo", "spfa_local", "spfa_local_1d_dilated", "spfa_local_2d_dilated",
           "spfa_global_no_local", "spfa_bigbird")


def add_bindings_to_path() -> str:
    """Put lib/ on sys.path so ``import spfa_csr`` (etc.) finds the built torch extensions."""
    if LIBDIR not in sys.path:
        sys.path.insert(0, LIBDIR)
    return LIBDIR


def binding(name: str):
    """Import one of the six torch-extension modules by the reference's module name."""
    if name not in MODULES:
        raise ValueError(f"unknown module {name!r}; expected one of {MODULES}")
    import torch  # noqa: F401  (the extensions link against libtorch)

    add_bindings_to_path()
    try:
        return importlib.import_module(name)
    except ImportError as e:  # fail loudly: there is no fallback path
        raise ImportError(f"{name} is not built; run `python {os.path.join(_HERE, 'build.py')}` ({e})") from e


def __getattr__(attr):
    if attr in ("capi", "sharding", "build", "hostio"):
        return importlib.import_module(f"{__name__}.{attr}")
    raise AttributeError(attr)
