"""GPU parity for the conformance sweep (``tests/golden/sweep.py``): every kernel of the table through
``compile(..., backend="b200")`` against the outputs upstream's CPU reference runtime produced for the same inputs."""
from __future__ import annotations

import numpy as np
import pytest
from conftest import golden_ir, golden_vec, zoo_kernel
from gpu_util import device_zeros, expect_rounded, to_device, to_host
from sweep import CASES

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("case", CASES, ids=[case.name for case in CASES])
def test_sweep_kernel_matches_upstream_vectors(case, zoo, tmp_path):
    import baybridge_b200 as cute

    vec = golden_vec(f"sw_{case.name}")
    operands, outputs = [], {}
    for argument in case.arguments:
        if argument.shape is None:
            operands.append(cute.Int32(argument.fill) if argument.dtype == "i32" else argument.fill)
            continue
        if argument.role == "out":
            tensor = device_zeros(argument.shape, argument.dtype)
        else:
            tensor = to_device(vec[f"in_{argument.name}"], argument.dtype)
        if argument.role != "in":
            outputs[argument.name] = (tensor, argument.dtype)
        operands.append(tensor)
    artifact = cute.compile(case.kernel(zoo), *operands, backend="b200", cache_dir=tmp_path)
    artifact(*operands)
    reduces = case.factory == "make_reduce" and case.factory_args[0] in ("add", "mul") and outputs and next(iter(outputs.values()))[1] != "i32"
    for name, (tensor, dtype) in outputs.items():
        expected = np.asarray(vec[f"out_{name}"], dtype=np.float64)
        actual = to_host(tensor).astype(np.float64)
        if dtype in ("i32", "i1"):
            assert np.array_equal(actual, expected), f"{name}: {int(np.count_nonzero(actual != expected))} elements differ"
        else:
            # arithmetic is exact against the f64 reference rounded once; libm-style functions and floating-point
            # folds (whose order differs from the sequential loop) may differ by one unit in the last place
            expect_rounded(actual, expected, dtype, max_ulp=1 if (case.max_ulp or reduces) else 0)


@pytest.mark.parametrize("case", ["padded_increment_1024v512_f32", "accumulate_1024_f32"])
def test_guarded_load_and_read_modify_write_forms(case, zoo, tmp_path):
    """A guarded load feeding an unguarded store writes f(else_value) past the bound; ``dst[i] = dst[i] + src[i]`` reads
    what it overwrites.  Both against upstream's CPU runtime."""
    import baybridge_b200 as cute

    vec = golden_vec(case)
    ir = golden_ir(case)["ir"]
    operands = []
    for argument in ir["arguments"]:
        name, spec = argument["name"], argument["spec"]
        operands.append(to_device(vec[f"in_{name}"], spec["dtype"]) if f"in_{name}" in vec else device_zeros(spec["shape"], spec["dtype"]))
    artifact = cute.compile(zoo_kernel(case, zoo), *operands, backend="b200", cache_dir=tmp_path)
    artifact(*operands)
    expect_rounded(to_host(operands[-1]), vec["out_dst"], "f32", max_ulp=0)
