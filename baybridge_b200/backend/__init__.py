"""The ``b200`` execution backend: matcher, lowering, native library binding and launchers."""
from .b200 import B200Backend, install_into_upstream

__all__ = ["B200Backend", "install_into_upstream"]
