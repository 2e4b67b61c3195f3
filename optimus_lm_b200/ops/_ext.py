"""Loader of the in-tree sm_100a kernel extension (``optimus_lm_b200/_C*.so``).

The extension is built by ``python setup.py build_ext --inplace`` (or
``__graft_entry__.build()``).  On a machine with a GPU the kernels are mandatory: if the
extension cannot be imported, every op raises instead of silently running an eager
fallback.  On a CPU-only machine the plain PyTorch implementations are used (they are also
the numerical oracle of the kernel tests).
"""
from __future__ import annotations

import importlib
import os

import torch

_C = None
_IMPORT_ERROR = None


def _try_import():
    global _C, _IMPORT_ERROR
    if _C is not None or _IMPORT_ERROR is not None:
        return
    try:
        _C = importlib.import_module("optimus_lm_b200._C")
    except Exception as exc:  # pragma: no cover - depends on the build
        _IMPORT_ERROR = exc


def extension():
    """The compiled module, or raise with the import error."""
    _try_import()
    if _C is None:
        raise RuntimeError(
            "optimus_lm_b200._C is not built or failed to load; run `python setup.py build_ext --inplace` "
            f"in the repository root. Import error: {_IMPORT_ERROR!r}")
    return _C


def extension_available() -> bool:
    _try_import()
    return _C is not None


def kernels_disabled() -> bool:
    """``OLB_DISABLE_KERNELS=1`` forces the PyTorch oracle path (debugging only)."""
    return os.environ.get("OLB_DISABLE_KERNELS", "0") == "1"


def use_kernels(*tensors: torch.Tensor) -> bool:
    """True when the given tensors should go through the CUDA kernels: they live on a GPU
    and are bf16 where the kernels need it.  Raises if a GPU is present but the extension
    is missing."""
    if not tensors or not all(t.is_cuda for t in tensors if t is not None):
        return False
    if kernels_disabled():
        return False
    extension()
    return True


# ----------------------------------------------------------------------------- launch accounting
# Kernel launches issued per binding call (see csrc/*.cu launchers).
_LAUNCHES_PER_CALL = {
    "moe_build_index": 4, "sumsq": 2, "attn_bwd": 3,
}


class _CountingProxy:
    """Wraps the extension module and counts the kernel launches made through it."""

    def __init__(self, mod):
        object.__setattr__(self, "_mod", mod)
        object.__setattr__(self, "launches", 0)
        object.__setattr__(self, "by_name", {})

    def __getattr__(self, name):
        fn = getattr(self._mod, name)
        if not callable(fn) or name.endswith("_blocks") or name.endswith("_ints"):
            return fn
        n = _LAUNCHES_PER_CALL.get(name, 1)

        def counted(*a, **k):
            object.__setattr__(self, "launches", self.launches + n)
            self.by_name[name] = self.by_name.get(name, 0) + n
            return fn(*a, **k)

        return counted


def enable_launch_counting():
    """Replace the cached extension handle by a counting proxy; returns the proxy
    (``proxy.launches``, ``proxy.by_name``)."""
    global _C
    mod = extension()
    if not isinstance(mod, _CountingProxy):
        _C = _CountingProxy(mod)
    return _C
