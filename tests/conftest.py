"""Shared fixtures.  ``gpu``-marked tests need a B200 and the built CUDA library; everything else runs on CPU."""
from __future__ import annotations

import json
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
GOLDEN = ROOT / "tests" / "golden"
for entry in (str(ROOT), str(ROOT / "tests")):
    if entry not in sys.path:
        sys.path.insert(0, entry)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200) and the built libbb200.so")


def golden_ir(case: str) -> dict:
    return json.loads((GOLDEN / f"ir_{case}.json").read_text())


def golden_vec(case: str) -> dict[str, np.ndarray]:
    with np.load(GOLDEN / f"vec_{case}.npz") as blob:
        return {name: blob[name] for name in blob.files}


def golden_cases(prefix: str = "") -> list[str]:
    return sorted(path.stem[len("vec_"):] for path in GOLDEN.glob(f"vec_{prefix}*.npz"))


def mma_attrs(ir: dict) -> dict:
    """Attributes of the (single) mma op of a GEMM listing, whole-tensor or written per program."""
    (op,) = [op for op in ir["operations"] if op["op"] == "mma"]
    return op["attrs"]


def gemm_zoo_kernel(case: str, ir: dict, zoo):
    """The zoo kernel a ``gemm_*`` / ``c3_*`` fixture was generated from."""
    attrs = mma_attrs(ir)
    if case.startswith("gemm_tiled_programs"):
        (m, k), (_, n) = ir["arguments"][0]["spec"]["shape"], ir["arguments"][2]["spec"]["shape"]
        tile_m, tile_n, _ = attrs["tile"]
        return zoo.make_tiled_gemm(m, n, k, tile_m, tile_n, transpose_b=attrs["transpose_b"], block=ir["launch"]["block"][0])
    return {(False, False): zoo.gemm_ab, (False, True): zoo.gemm_abt, (True, False): zoo.gemm_atb, (True, True): zoo.gemm_atbt}[
        (attrs["transpose_a"], attrs["transpose_b"])
    ]


@pytest.fixture(scope="session")
def zoo():
    import baybridge_b200 as cute
    from baybridge_b200.samples import build_zoo

    return build_zoo(cute)
