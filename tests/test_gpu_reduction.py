"""GPU parity for reductions (map, then fold): rows, columns and full reductions vs the CPU oracle.

Sums are accumulated in f64 for f32 tensors and f32 for 16-bit tensors, in a different order from the
sequential CPU fold, so results are held to 1 unit in the last place of the storage type; max/min and
integer folds are exact."""
from __future__ import annotations

import numpy as np
import pytest
from conftest import golden_ir, golden_vec
from gpu_util import device_zeros, expect_rounded, to_device, to_host

from oracle import cpu_runtime as oracle

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("case,kernel,dtype,exact", [
    ("reduce_row_sumsq_16x96_f32", "row_sum_of_squares", "f32", False),
    ("reduce_col_max_24x64_bf16", "column_max", "bf16", True),
    ("reduce_total_sum_8x96_f32", "total_sum", "f32", False),
])
def test_compiled_reductions_match_upstream_vectors(case, kernel, dtype, exact, zoo, tmp_path):
    import baybridge_b200 as cute

    vec = golden_vec(case)
    src = to_device(vec["in_src"], dtype)
    dst = device_zeros(vec["out_dst"].shape, dtype)
    artifact = cute.compile(getattr(zoo, kernel), src, dst, backend="b200", cache_dir=tmp_path)
    assert artifact.ir.to_dict()["operations"] == golden_ir(case)["ir"]["operations"]
    artifact(src, dst)
    expect_rounded(to_host(dst), vec["out_dst"], dtype, max_ulp=0 if exact else 1)


@pytest.mark.parametrize("case,kernel,dtype", [
    ("rbundle_xor_6x40_i32", "reduce_bundle_xor", "i32"), ("rbundle_add_6x40_f32", "reduce_bundle_add", "f32"),
])
def test_bundled_reductions_match_upstream_vectors(case, kernel, dtype, zoo, tmp_path):
    """Total, row folds and column folds of one loaded tensor in a single kernel body."""
    import baybridge_b200 as cute

    vec = golden_vec(case)
    src = to_device(vec["in_src"], dtype)
    outputs = {name: device_zeros(vec[f"out_{name}"].shape, dtype) for name in ("dst_scalar", "dst_rows", "dst_cols")}
    artifact = cute.compile(getattr(zoo, kernel), src, *outputs.values(), backend="b200", cache_dir=tmp_path)
    assert artifact.ir.to_dict()["operations"] == golden_ir(case)["ir"]["operations"]
    artifact(src, *outputs.values())
    for name, tensor in outputs.items():
        expect_rounded(to_host(tensor), vec[f"out_{name}"], dtype, max_ulp=0 if dtype == "i32" or name == "dst_cols" else 1)


def test_reduction_taken_straight_from_the_argument(zoo, tmp_path):
    import baybridge_b200 as cute

    vec = golden_vec("rarg_max_256_i32")
    src, dst = to_device(vec["in_src"], "i32"), device_zeros((1,), "i32")
    artifact = cute.compile(zoo.reduce_argument_max, src, dst, backend="b200", cache_dir=tmp_path)
    assert artifact.ir.to_dict()["operations"] == golden_ir("rarg_max_256_i32")["ir"]["operations"]
    artifact(src, dst)
    assert int(to_host(dst)[0]) == int(vec["out_dst"][0])


def _run(kernel, src, dst_shape, dtype, tmp_path):
    import baybridge_b200 as cute

    device_src = to_device(src, dtype) if dtype != "i32" else __import__("torch").from_numpy(src.astype(np.int32)).cuda()
    dst = device_zeros(dst_shape, dtype)
    artifact = cute.compile(kernel, device_src, dst, backend="b200", cache_dir=tmp_path)
    artifact(device_src, dst)
    expected = {"src": np.array(src, dtype=np.float64), "dst": np.zeros(dst_shape)}
    oracle.run_kernel_ir(artifact.ir.to_dict(), expected)
    return to_host(dst), expected["dst"]


@pytest.mark.parametrize("dtype,shape", [("bf16", (4096, 8192)), ("f32", (1000, 999)), ("f16", (3, 40)), ("f32", (2, 100000))])
def test_row_reductions(dtype, shape, zoo, tmp_path):
    rng = np.random.default_rng(shape[0] + shape[1])
    src = oracle.round_to_dtype(rng.uniform(-1, 1, shape), dtype)
    got, expected = _run(zoo.row_sum_of_squares, src, (shape[0],), dtype, tmp_path)
    expect_rounded(got, expected, dtype, max_ulp=1)


@pytest.mark.parametrize("dtype,shape", [("bf16", (8192, 256)), ("f32", (64, 100000)), ("f32", (5, 7)), ("bf16", (100000, 8))])
def test_column_reductions(dtype, shape, zoo, tmp_path):
    rng = np.random.default_rng(shape[0] * 3 + shape[1])
    src = oracle.round_to_dtype(rng.uniform(-4, 4, shape), dtype)
    got, expected = _run(zoo.column_max, src, (shape[1],), dtype, tmp_path)
    expect_rounded(got, expected, dtype)  # max is exact


@pytest.mark.parametrize("n", [1, 1000, 2**24 + 3])
def test_full_reductions(n, zoo, tmp_path):
    import baybridge_b200 as cute

    rng = np.random.default_rng(n)
    src = rng.uniform(-1, 1, (n,)).astype(np.float32)
    got, expected = _run(zoo.total_sum, src, (1,), "f32", tmp_path)
    expect_rounded(got, expected, "f32", max_ulp=1)

    @cute.kernel
    def xor_all(src: cute.Tensor, dst: cute.Tensor):
        dst[0] = src.load().reduce(cute.ReductionOp.XOR, 0)

    bits = rng.integers(-2**31, 2**31 - 1, size=n, dtype=np.int64)
    got, _ = _run(xor_all, bits, (1,), "i32", tmp_path)
    assert int(got[0]) == int(np.bitwise_xor.reduce(bits.astype(np.int32)))
