#!/usr/bin/env python3
"""Place an unmodified copy of upstream's pure-Python package under ``oracle/_ref/`` — TEST INFRASTRUCTURE.

    python oracle/make_ref.py [/path/to/upstream/checkout]

Upstream (powderluv/baybridge) has no native code and no dependencies, so "building" it is a plain copy
of ``src/baybridge`` into ``oracle/_ref/baybridge``.  The copy is what ``oracle/ref_runtime.py`` imports
to time upstream's own CPU reference runtime next to the GPU numbers, on machines where no upstream
checkout exists.  ``oracle/_ref/`` is ignored by git: upstream's sources never enter this repository's
history, and nothing under ``baybridge_b200/`` imports them.
"""
from __future__ import annotations

import shutil
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
DESTINATION = HERE / "_ref" / "baybridge"


def default_checkout() -> Path:
    return HERE.parents[1] / "reference"  # a checkout next to this repository


def make_ref(checkout: Path | None = None) -> Path | None:
    """Copy ``<checkout>/src/baybridge`` to ``oracle/_ref/baybridge``; returns the destination, or ``None``
    when there is no checkout to copy from (an existing copy is then left as it is)."""
    source = (checkout or default_checkout()) / "src" / "baybridge"
    if not (source / "__init__.py").exists():
        return DESTINATION if (DESTINATION / "__init__.py").exists() else None
    if DESTINATION.exists():
        shutil.rmtree(DESTINATION)
    DESTINATION.parent.mkdir(parents=True, exist_ok=True)
    shutil.copytree(source, DESTINATION, ignore=shutil.ignore_patterns("__pycache__", "*.pyc"))
    return DESTINATION


if __name__ == "__main__":
    made = make_ref(Path(sys.argv[1]) if len(sys.argv) > 1 else None)
    print(made if made else "no upstream checkout found and no earlier copy present")
    sys.exit(0 if made else 1)
