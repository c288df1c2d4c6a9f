"""B200-native implementation of the torch-supa data-parallel operator path.

Importing the package loads the two in-tree shared libraries and registers the ``supa`` device with
PyTorch (PrivateUse1): ``torch.device("supa")``, ``tensor.to("supa")``, ``torch.supa.*``.  The operators
registered for it (add / mul / gelu / silu / glu, sum / mean / amax, log_softmax, nll_loss, cross_entropy
and their backward kernels) run hand-written sm_100a CUDA kernels through the C ABI of
``include/supa_b200_kernels.h``.  There is no CPU fallback: an operator without a kernel raises.

The bring-up mirrors ``torch_supa/__init__.py:78-85,133`` of the reference: rename the PrivateUse1
backend, register the device module, generate the ``.supa()`` / ``.is_supa`` methods.
"""
from __future__ import annotations

import ctypes
from pathlib import Path

import torch

from . import capi

__version__ = "0.1.0"

_HOST_LIB = Path(__file__).resolve().parent / "lib" / "libtorch_supa_b200.so"
_host = None


def _load():
    global _host
    if _host is not None:
        return _host
    capi.lib()  # the kernel library first (the host layer links against it); raises if it was not built
    if not _HOST_LIB.exists():
        raise RuntimeError(f"{_HOST_LIB} is missing: build it with `python -m torch_supa_b200._build`")
    torch.ops.load_library(str(_HOST_LIB))  # runs the static registrations (guard, allocator, operators)
    _host = ctypes.CDLL(str(_HOST_LIB))
    _host.supa_last_error.restype = ctypes.c_char_p
    return _host


def _check(rc: int) -> None:
    if rc != 0:
        raise RuntimeError(_load().supa_last_error().decode())


_load()

from . import supa  # noqa: E402  (needs the library)

torch.utils.rename_privateuse1_backend("supa")
torch._register_device_module("supa", supa)
torch.utils.generate_methods_for_privateuse1_backend(for_tensor=True, for_module=True, for_storage=True)

from . import distributed  # noqa: E402,F401

distributed.register_c10d_backend()
