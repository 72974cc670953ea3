"""Shared fixtures.  ``gpu``-marked tests need a B200 and the built CUDA library; everything else runs on CPU."""
from __future__ import annotations

import json
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
GOLDEN = ROOT / "tests" / "golden"
for entry in (str(ROOT), str(ROOT / "tests"), str(GOLDEN)):
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


def zoo_kernel(case: str, zoo):
    """The sample kernel a golden fixture (``ir_<case>.json`` / ``vec_<case>.npz``) was generated from."""
    from sweep import BY_NAME

    parts = case.split("_")
    if case.startswith("sw_"):
        return BY_NAME[case[3:]].kernel(zoo)
    table = {
        "c1": lambda: zoo.make_indexed_add_2d(256, 256),
        "c3": lambda: zoo.gemm_abt,
        "c4": lambda: zoo.make_rmsnorm(1e-6),
        "clamp": lambda: zoo.make_indexed_clamp_scale(512),
        "masked": lambda: zoo.make_indexed_masked_add(1000),
        "padded": lambda: zoo.make_indexed_padded_increment(1024, 512),
        "accumulate": lambda: zoo.make_indexed_accumulate(int(parts[1])),
        "bin": lambda: zoo.make_indexed_binary(parts[1], int(parts[2])),
        "un": lambda: zoo.make_indexed_unary(parts[1], int(parts[2])),
        "rmsnorm": lambda: zoo.make_rmsnorm(None),
        "layernorm": lambda: zoo.layernorm_kernel,
    }
    if case.startswith("reduce_"):
        return {"row": zoo.row_sum_of_squares, "col": zoo.column_max, "total": zoo.total_sum}[parts[1]]
    if case.startswith("c2_fused_indexed"):
        return zoo.make_fused_mul_add_indexed(2**28 if "2p28" in case else int(parts[3]))
    if case.startswith("c2_fused_ssa"):
        return zoo.fused_mul_add_ssa
    if case.startswith("ssa_"):
        return getattr(zoo, "_".join(parts[:-2]))
    if case.startswith(("c5_", "attn_")):
        return zoo.attention_causal if "causal" in case else zoo.attention_full
    families = {
        "bitwise": lambda: zoo.make_indexed_bitwise(parts[1], int(parts[2])), "cmpsel": lambda: zoo.make_indexed_compare_select(int(parts[1])),
        "ext1_indexed": lambda: zoo.make_indexed_extent1_scalar(int(parts[2])), "ext1_ssa": lambda: zoo.ssa_extent1_scalar,
        "bcast_rowcol": lambda: zoo.ssa_broadcast_row_col, "factory_bundle": lambda: zoo.factory_bundle,
        "rbundle_xor": lambda: zoo.reduce_bundle_xor, "rbundle_add": lambda: zoo.reduce_bundle_add, "rarg_max": lambda: zoo.reduce_argument_max,
    }
    for prefix, make in families.items():
        if case.startswith(prefix + "_"):
            return make()
    if case.startswith("api_"):
        return next(getattr(zoo, name) for name in ("api_vector_copy", "api_tile_mma", "api_topology") if case.startswith(name))
    if case.startswith("gemm_"):
        return gemm_zoo_kernel(case, golden_ir(case)["ir"], zoo)
    return table[parts[0]]()


def sample_scalar(cute, case: str, argument: dict):
    """The value a fixture's scalar parameter was generated with (typed where a bare Python int would trace as an index)."""
    if case.startswith("sw_"):
        from sweep import BY_NAME

        entry = next(a for a in BY_NAME[case[3:]].arguments if a.name == argument["name"])
        return cute.Int32(entry.fill) if entry.dtype == "i32" else entry.fill
    return 0.75


@pytest.fixture(scope="session")
def zoo():
    import baybridge_b200 as cute
    from baybridge_b200.samples import build_zoo

    return build_zoo(cute)
