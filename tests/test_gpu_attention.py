"""GPU parity for attention forward: compile(..., backend="b200") and the C ABI vs the CPU oracle/golden vectors.

Tolerance (the path's contract): out rel-L2 <= 1e-2 against the f64 reference, lse abs error <= 1e-2."""
from __future__ import annotations

import ctypes

import numpy as np
import pytest
from conftest import golden_cases, golden_ir, golden_vec
from gpu_util import current_stream, device_zeros, to_device, to_host, void_p

from oracle import cpu_runtime as oracle

pytestmark = pytest.mark.gpu
REL_L2 = 1e-2
LSE_ABS = 1e-2


def _check(out, lse, ref_out, ref_lse):
    assert oracle.rel_l2(to_host(out), ref_out) <= REL_L2
    assert float(np.abs(to_host(lse).reshape(ref_lse.shape) - ref_lse).max()) <= LSE_ABS


@pytest.mark.parametrize("case", golden_cases("c5_") + golden_cases("attn_"))
def test_compiled_attention_matches_upstream_vectors(case, zoo, tmp_path):
    import baybridge_b200 as cute

    ir = golden_ir(case)["ir"]
    vec = golden_vec(case)
    causal = ir["operations"][0]["attrs"]["causal"]
    q, k, v = (to_device(vec[f"in_{name}"], "bf16") for name in "qkv")
    out = device_zeros(vec["out_out"].shape, "bf16")
    lse = device_zeros(vec["out_lse"].shape, "f32")
    kernel = zoo.attention_causal if causal else zoo.attention_full
    artifact = cute.compile(kernel, q, k, v, out, lse, backend="b200", cache_dir=tmp_path)
    assert artifact.ir.to_dict()["operations"] == ir["operations"]
    artifact(q, k, v, out, lse)
    _check(out, lse, vec["out_out"], vec["out_lse"])


@pytest.mark.parametrize("batch,seq,heads,kv_heads,dim,causal", [
    (1, 128, 1, 1, 128, True), (1, 128, 1, 1, 128, False), (2, 256, 4, 2, 128, True), (1, 384, 2, 2, 128, False),
    (1, 200, 2, 1, 128, True), (1, 72, 3, 3, 128, False), (2, 512, 2, 2, 64, True), (1, 130, 2, 2, 64, False),
    (1, 1024, 8, 2, 128, True), (1, 40, 2, 2, 32, True), (1, 33, 2, 1, 48, False),
])
def test_c_abi_attention_shapes(batch, seq, heads, kv_heads, dim, causal):
    from baybridge_b200.backend import native

    rng = np.random.default_rng(batch * 1009 + seq * 31 + heads * 7 + dim + causal)
    q = oracle.bf16_round(rng.standard_normal((batch, seq, heads, dim), dtype=np.float32))
    k = oracle.bf16_round(rng.standard_normal((batch, seq, kv_heads, dim), dtype=np.float32))
    v = oracle.bf16_round(rng.standard_normal((batch, seq, kv_heads, dim), dtype=np.float32))
    d_q, d_k, d_v = (to_device(t, "bf16") for t in (q, k, v))
    out = device_zeros(q.shape, "bf16")
    lse = device_zeros((batch, heads, seq), "f32")  # rank-3 lse has the same memory layout as [B, H, 1, S]
    native.call("bb200_attention_fwd", void_p(d_q), void_p(d_k), void_p(d_v), void_p(out), void_p(lse), batch, seq, heads,
                kv_heads, dim, int(causal), current_stream())
    status = ctypes.c_int(-1)
    native.call("bb200_take_device_status", current_stream(), ctypes.byref(status))
    assert status.value == 0, f"a bounded device wait gave up (code {status.value})"
    ref_out, ref_lse = oracle.attention(q, k, v, causal=causal)
    _check(out, lse, ref_out, ref_lse.reshape(batch, heads, seq))


def test_c_abi_attention_rejects_bad_arguments():
    from baybridge_b200 import CudaDriverError
    from baybridge_b200.backend import native

    x = device_zeros((1, 128, 4, 128), "bf16")
    lse = device_zeros((1, 4, 128), "f32")
    with pytest.raises(CudaDriverError) as info:  # 4 heads are not divisible by 3 kv heads
        native.call("bb200_attention_fwd", void_p(x), void_p(x), void_p(x), void_p(x), void_p(lse), 1, 128, 4, 3, 128, 1, current_stream())
    assert info.value.status == -1
    with pytest.raises(CudaDriverError):
        native.call("bb200_attention_fwd", void_p(x), void_p(x), void_p(x), void_p(x), None, 1, 128, 4, 4, 128, 1, current_stream())


def test_config5_full_size_causal_attention(zoo, tmp_path):
    """B16 H32 S4096 D128 through compile().  The f64 oracle is evaluated on sampled (batch, head) slices;
    two size-independent properties cover the rest: (1) causality — output rows < t do not change when
    keys/values at positions >= t change; (2) with V == 1 everywhere the output is exactly 1."""
    import torch

    import baybridge_b200 as cute

    batch, seq, heads, dim = 16, 4096, 32, 128
    generator = torch.Generator(device="cuda").manual_seed(1005)
    shape = (batch, seq, heads, dim)
    q, k, v = (torch.randn(shape, device="cuda", dtype=torch.float32, generator=generator).to(torch.bfloat16) for _ in range(3))
    out = torch.zeros_like(q)
    lse = torch.zeros((batch, heads, 1, seq), device="cuda", dtype=torch.float32)
    artifact = cute.compile(zoo.attention_causal, q, k, v, out, lse, backend="b200", cache_dir=tmp_path)
    artifact(q, k, v, out, lse)
    for b, h in [(0, 0), (7, 13), (15, 31)]:
        rows = slice(0, 1024)  # the oracle is O(S^2); the first 1024 queries only need the first 1024 keys when causal
        ref_out, ref_lse = oracle.attention(to_host(q[b:b + 1, rows, h:h + 1]), to_host(k[b:b + 1, rows, h:h + 1]),
                                            to_host(v[b:b + 1, rows, h:h + 1]), causal=True)
        _check(out[b:b + 1, rows, h:h + 1], lse[b:b + 1, h:h + 1, :, rows], ref_out, ref_lse)
    # last rows of one slice against the full-length oracle
    b, h = 3, 5
    ref_out, ref_lse = oracle.attention(to_host(q[b:b + 1, :, h:h + 1]), to_host(k[b:b + 1, :, h:h + 1]),
                                        to_host(v[b:b + 1, :, h:h + 1]), causal=True)
    _check(out[b:b + 1, :, h:h + 1], lse[b:b + 1, h:h + 1], ref_out, ref_lse)
    # (1) causality
    t = 2048
    k2, v2 = k.clone(), v.clone()
    k2[:, t:] = torch.randn_like(k2[:, t:])
    v2[:, t:] = torch.randn_like(v2[:, t:])
    out2, lse2 = torch.zeros_like(out), torch.zeros_like(lse)
    artifact(q, k2, v2, out2, lse2)
    assert torch.equal(out2[:, :t], out[:, :t]) and torch.equal(lse2[..., :t], lse[..., :t])
    # (2) probabilities sum to one: with V == 1 every output element is 1 up to the bf16 rounding of P and out
    ones = torch.ones_like(v)
    artifact(q, k, ones, out2, lse2)
    assert (out2.float() - 1.0).abs().max().item() <= 2.0 ** -7
