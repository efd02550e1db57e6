"""zentorch_b200: the quantized-linear hot path of zentorch (amd/ZenDNN-pytorch-plugin) on B200.

Importing the package loads ``libzentorch_b200.so`` (CUDA kernels behind a C ABI) and
``libzentorch_b200_torch.so`` (registers the ``torch.ops.zentorch`` schemas of the reference with a
CUDA dispatch key).  Both are built in-tree by ``python -m zentorch_b200._build``; when they are
missing the import fails -- there is no eager/PyTorch fallback.

After import, the reference's operator calls work unchanged on CUDA tensors::

    y = torch.ops.zentorch.zentorch_woq_linear(x, packed.t(), scales, None, bias)
    y = torch.ops.zentorch.zentorch_dynamic_qlinear(x, w_int8, w_scales, bias)
"""
from __future__ import annotations

import ctypes
from pathlib import Path

from . import _capi

__version__ = "0.1.0"

_TORCH_LIB = Path(__file__).resolve().parent.parent / "lib" / "libzentorch_b200_torch.so"
_loaded = False


def load() -> None:
    """Load both native libraries (idempotent)."""
    global _loaded
    if _loaded:
        return
    import torch

    _capi.lib()
    if not _TORCH_LIB.exists():
        raise ImportError(f"{_TORCH_LIB} is missing: build it with `python -m zentorch_b200._build`")
    # RTLD_GLOBAL so that AOTInductor-generated code can resolve the aoti_torch_cuda_zentorch_* shims
    # (the reference does the same for libzentorch.so: src/cpu/python/zentorch/__init__.py:69-78).
    ctypes.CDLL(str(_TORCH_LIB), mode=ctypes.RTLD_GLOBAL)
    torch.ops.load_library(str(_TORCH_LIB))
    _loaded = True


def is_supported_device() -> bool:
    """True when the current CUDA device is a compute-capability 10.x GPU."""
    import torch

    return torch.cuda.is_available() and bool(_capi.lib().zt_device_supported())


def register_backend() -> None:
    """Register ``torch.compile(..., backend="zentorch_b200")``: Inductor with the WOQ replacement and
    fusion passes as its joint-graph post pass.  Kept out of ``import`` because it pulls in Dynamo."""
    from . import _compile

    _compile.register_backend()


# `python -m zentorch_b200._build` imports this package before it has built (or rebuilt) the libraries.
import sys as _sys

if "zentorch_b200._build" not in getattr(_sys, "orig_argv", ()):
    load()
