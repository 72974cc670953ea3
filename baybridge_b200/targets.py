"""Compilation targets.

``NvidiaTarget`` serialises exactly like upstream ``target.py:22-58`` (the
``sm`` value keeps architecture suffixes such as ``sm_100a``), because the
target dictionary is part of the compile-cache key.  ``AMDTarget`` exists only
so code that passes one gets a clear rejection from the b200 backend instead
of an AttributeError.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any


@dataclass(frozen=True)
class NvidiaTarget:
    sm: str | int = "sm_100a"
    ptx_version: str = "8.8"
    warp_size: int = 32
    driver_version: str | None = None

    def __post_init__(self) -> None:
        raw = self.sm
        if isinstance(raw, int) and not isinstance(raw, bool):
            if raw <= 0:
                raise ValueError("NvidiaTarget(sm=...) expects a positive SM value")
            text = str(raw)
        else:
            text = str(raw).strip().lower()
            if not text:
                raise ValueError("NvidiaTarget(sm=...) expects a non-empty SM value")
            text = text[3:] if text.startswith("sm_") else text
            if not text.isalnum():
                raise ValueError("NvidiaTarget(sm=...) expects values like 80, '80', or 'sm_80'")
        object.__setattr__(self, "sm", f"sm_{text}")

    @property
    def arch(self) -> str:
        return str(self.sm)

    def to_dict(self) -> dict[str, Any]:
        return {
            "arch": self.arch,
            "sm": self.sm,
            "ptx_version": self.ptx_version,
            "warp_size": self.warp_size,
            "driver_version": self.driver_version,
            "vendor": "nvidia",
        }


@dataclass(frozen=True)
class AMDTarget:
    arch: str = "gfx942"
    wave_size: int = 64
    rocm_version: str | None = None

    def to_dict(self) -> dict[str, Any]:
        return {"arch": self.arch, "wave_size": self.wave_size, "rocm_version": self.rocm_version, "vendor": "amd"}


B200 = NvidiaTarget(sm="sm_100a", ptx_version="8.8")
