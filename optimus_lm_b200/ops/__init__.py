"""Kernel-backed ops (see functional.py)."""
from . import functional  # noqa: F401
from ._ext import extension, extension_available, use_kernels  # noqa: F401
