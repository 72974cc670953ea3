"""Exception types of the DSL surface.

Same names and hierarchy as upstream ``diagnostics.py:1-14`` plus the driver
error of ``cuda_driver.py:46-57`` so ``except`` clauses written against the
upstream package keep working.
"""
from __future__ import annotations


class BaybridgeError(Exception):
    """Root of every error raised by this package."""


class CompilationError(BaybridgeError):
    """The kernel body could not be traced into portable IR."""


class UnsupportedOperationError(BaybridgeError):
    """The DSL entry point exists upstream but is outside this package's path."""


class BackendNotImplementedError(BaybridgeError):
    """The selected backend cannot lower or launch this IR (there is no CPU fallback)."""


class CudaDriverError(BaybridgeError):
    """A native call returned a non-zero status.

    ``op`` is the failing entry point, ``status`` the integer it returned
    (CUresult-compatible when positive, a library validation code when
    negative), ``name``/``message`` the decoded strings.
    """

    def __init__(self, op: str, status: int, name: str = "", message: str = ""):
        self.op = op
        self.status = int(status)
        self.name = name
        self.message = message
        detail = f"{op} failed with status {self.status}"
        if name:
            detail += f" ({name})"
        if message:
            detail += f": {message}"
        super().__init__(detail)
