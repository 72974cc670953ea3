"""GPU parity for LayerNorm with fused residual add: compile(..., backend="b200") and the C ABI vs the CPU oracle.

Tolerance: the same bar as RMSNorm — rel-L2 <= 2e-3 against the f64 reference for 16-bit tensors."""
from __future__ import annotations

import numpy as np
import pytest
from conftest import golden_ir, golden_vec
from gpu_util import current_stream, device_zeros, to_device, to_host, ulp_distance, void_p

from oracle import cpu_runtime as oracle

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("case,dtype", [("layernorm_2x4x128_bf16", "bf16"), ("layernorm_5x256_f32", "f32")])
def test_compiled_layernorm_matches_upstream_vectors(case, dtype, zoo, tmp_path):
    import baybridge_b200 as cute

    vec = golden_vec(case)
    x, residual, weight, bias = (to_device(vec[f"in_{name}"], dtype) for name in ("x", "residual", "weight", "bias"))
    out, out_resid = device_zeros(vec["in_x"].shape, dtype), device_zeros(vec["in_x"].shape, dtype)
    artifact = cute.compile(zoo.layernorm_kernel, x, residual, out, out_resid, weight, bias, backend="b200", cache_dir=tmp_path)
    assert artifact.ir.to_dict()["operations"] == golden_ir(case)["ir"]["operations"]
    artifact(x, residual, out, out_resid, weight, bias)
    tolerance = 2e-3 if dtype == "bf16" else 1e-6
    assert oracle.rel_l2(to_host(out), vec["out_out"]) <= tolerance
    # x + residual is a single rounding of an exact f32/f64 sum: bit-exact
    assert int(ulp_distance(to_host(out_resid), oracle.round_to_dtype(vec["out_out_resid"], dtype), dtype).max()) == 0


@pytest.mark.parametrize("dtype,rows,hidden,full", [
    ("bf16", 3, 8, False), ("bf16", 65, 1000, False), ("bf16", 16, 8192, False), ("bf16", 2, 32768, False),
    ("f16", 7, 2048, True), ("f32", 6, 1020, False), ("f32", 3, 16384, True),
])
def test_c_abi_layernorm_shapes(dtype, rows, hidden, full):
    from baybridge_b200.backend import native

    rng = np.random.default_rng(rows * 7 + hidden)
    x = oracle.round_to_dtype(rng.standard_normal((rows, hidden)), dtype)
    r = oracle.round_to_dtype(rng.standard_normal((rows, hidden)), dtype)
    shape = (rows, hidden) if full else (hidden,)
    w = oracle.round_to_dtype(1 + 0.1 * rng.standard_normal(shape), dtype)
    b = oracle.round_to_dtype(0.1 * rng.standard_normal(shape), dtype)
    d = [to_device(t, dtype) for t in (x, r, w, b)]
    out, out_resid = device_zeros((rows, hidden), dtype), device_zeros((rows, hidden), dtype)
    native.call("bb200_layernorm", native.DTYPE_CODES[dtype], void_p(d[0]), void_p(d[1]), void_p(d[2]), void_p(d[3]), void_p(out),
                void_p(out_resid), rows, hidden, int(full), int(full), 1e-5, current_stream())
    ref_out, ref_mixed = oracle.layernorm(x, r, w, b, 1e-5)
    assert oracle.rel_l2(to_host(out), ref_out) <= (2e-3 if dtype != "f32" else 2e-6)
    assert np.array_equal(to_host(out_resid), oracle.round_to_dtype(ref_mixed, dtype))


def test_c_abi_layernorm_rejects_bad_shapes():
    from baybridge_b200 import CudaDriverError
    from baybridge_b200.backend import native

    x = device_zeros((4, 12), "bf16")
    with pytest.raises(CudaDriverError) as info:
        native.call("bb200_layernorm", 1, void_p(x), void_p(x), void_p(x), void_p(x), void_p(x), void_p(x), 4, 12, 0, 0, 1e-5, current_stream())
    assert info.value.status == -2
