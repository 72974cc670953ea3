"""Pin the CPU oracle against fixtures produced by upstream's own CPU reference runtime."""
from __future__ import annotations

import hashlib

import numpy as np
import pytest
from conftest import golden_cases, golden_ir, golden_vec, mma_attrs, sample_scalar
from sweep import BY_NAME

from oracle import cpu_runtime as oracle

TIGHT = 1e-12  # f64 vs f64; only summation order differs


def _kernel_cases() -> list[str]:
    explicit = ("c3_", "c4_", "c5_", "gemm_", "rmsnorm_", "layernorm_", "attn_")
    return [case for case in golden_cases() if not case.startswith(explicit)]


def c1_inputs() -> tuple[np.ndarray, np.ndarray]:
    rng = np.random.default_rng(1001)
    a = rng.uniform(-1, 1, (256, 256)).astype(np.float32)
    b = rng.uniform(-1, 1, (256, 256)).astype(np.float32)
    return a, b


def test_c1_inputs_reproduce_from_seed():
    a, b = c1_inputs()
    vec = golden_vec("c1_indexed_add_256x256_f32")
    assert hashlib.sha256(a.tobytes() + b.tobytes()).hexdigest() == str(vec["input_sha256"])
    # upstream adds in f64; one RNE of that sum to f32 is the IEEE f32 sum (53 >= 2*24+2 bits)
    assert vec["out_g_c"].dtype == np.float32 and np.array_equal(vec["out_g_c"], a + b)


@pytest.mark.parametrize("case", _kernel_cases())
def test_traced_kernel_interpreter_matches_upstream(case: str):
    ir = golden_ir(case)["ir"]
    vec = golden_vec(case)
    arguments = {}
    if case.startswith("c1_"):
        a, b = c1_inputs()
        vec = dict(vec, in_g_a=a, in_g_b=b)
    for argument in ir["arguments"]:
        name = argument["name"]
        if argument["kind"] == "scalar":
            value = sample_scalar(None, case, argument) if not case.startswith("sw_") else None
            if value is None:
                value = next(a for a in BY_NAME[case[3:]].arguments if a.name == name).fill
            arguments[name] = value
        elif f"in_{name}" in vec:
            arguments[name] = np.array(vec[f"in_{name}"], dtype=np.float64)
        else:
            arguments[name] = np.zeros(argument["spec"]["shape"], dtype=np.float64)
    oracle.run_kernel_ir(ir, arguments)
    outputs = [key for key in vec if key.startswith("out_")]
    assert outputs
    for key in outputs:
        if vec[key].dtype == np.float32:  # config 1 stores upstream's f64 result after one RNE to f32
            assert np.array_equal(arguments[key[4:]].astype(np.float32), vec[key])
            continue
        np.testing.assert_allclose(arguments[key[4:]], np.asarray(vec[key], dtype=np.float64), rtol=TIGHT, atol=0)


@pytest.mark.parametrize("case", golden_cases("c3_") + golden_cases("gemm_"))
def test_gemm_matches_upstream(case: str):
    vec = golden_vec(case)
    attrs = mma_attrs(golden_ir(case)["ir"])
    got = oracle.gemm(vec["in_a"], vec["in_b"], transpose_a=attrs["transpose_a"], transpose_b=attrs["transpose_b"])
    np.testing.assert_allclose(got, vec["out_c"], rtol=TIGHT, atol=1e-15)


def test_gemm_known_answer_ramp_times_identity():
    # upstream tests/test_backend_hipkittens_exec.py:47-57, 380-407: C[:, :16] == A exactly, rest zero
    vec = golden_vec("gemm_ab_ramp_identity_32x32x16")
    got = oracle.gemm(vec["in_a"], vec["in_b"])
    assert np.array_equal(got[:, :16], vec["in_a"]) and not got[:, 16:].any()
    assert np.array_equal(got, vec["out_c"])


@pytest.mark.parametrize("case", golden_cases("c4_") + golden_cases("rmsnorm_"))
def test_rmsnorm_matches_upstream(case: str):
    vec = golden_vec(case)
    epsilon = golden_ir(case)["ir"]["operations"][0]["attrs"]["epsilon"]
    got = oracle.rmsnorm(vec["in_x"], vec["in_gamma"], epsilon)
    np.testing.assert_allclose(got, vec["out_out"], rtol=TIGHT, atol=0)


@pytest.mark.parametrize("case", golden_cases("layernorm_"))
def test_layernorm_matches_upstream(case: str):
    vec = golden_vec(case)
    epsilon = golden_ir(case)["ir"]["operations"][0]["attrs"]["epsilon"]
    out, mixed = oracle.layernorm(vec["in_x"], vec["in_residual"], vec["in_weight"], vec["in_bias"], epsilon)
    np.testing.assert_allclose(out, vec["out_out"], rtol=1e-11, atol=1e-13)
    np.testing.assert_allclose(mixed, vec["out_out_resid"], rtol=TIGHT, atol=0)


@pytest.mark.parametrize("case", golden_cases("c5_") + golden_cases("attn_"))
def test_attention_matches_upstream(case: str):
    vec = golden_vec(case)
    causal = golden_ir(case)["ir"]["operations"][0]["attrs"]["causal"]
    out, lse = oracle.attention(vec["in_q"], vec["in_k"], vec["in_v"], causal=causal)
    np.testing.assert_allclose(out, vec["out_out"], rtol=1e-11, atol=1e-14)
    np.testing.assert_allclose(lse, vec["out_lse"], rtol=TIGHT, atol=1e-14)


def test_bf16_rounding_rule():
    # RNE on the upper half of the f32 pattern (upstream hip_runtime.py:246-249)
    x = np.array([1.0, 1.00390625, 1.01171875, -2.5, 3.0e-39, 65504.0], dtype=np.float32)
    got = oracle.bf16_round(x)
    assert got[0] == 1.0 and got[1] == 1.0  # 1 + 2^-8 is a tie → even (1.0)
    assert got[2] == np.float32(1.015625)  # 1 + 3·2^-8 is a tie → even (1 + 2^-6)
    assert np.array_equal(oracle.round_to_dtype(x.astype(np.float64), "bf16"), got.astype(np.float64))
    rng = np.random.default_rng(7)
    y = rng.standard_normal(4096).astype(np.float32)
    assert np.array_equal(oracle.round_to_dtype(y.astype(np.float64), "bf16"), oracle.bf16_round(y).astype(np.float64))
