"""The elementwise kernel in its fan-out form: a shard's results stored into several gathered buffers at once.

On one GPU the "peers" are two local buffers, which checks the kernel and its launch path (the peer pointers of a
multi-GPU run come from symmetric memory and are exercised by ``bench.py --gpus N``)."""
from __future__ import annotations

import numpy as np
import pytest
from gpu_util import to_device, to_host

from oracle import cpu_runtime as oracle

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n,fanout,shard_index", [(4096, 2, 1), (100_000, 3, 2), (1003, 2, 0)])
def test_fan_out_kernel_writes_every_destination_at_the_shard_offset(n, fanout, shard_index, zoo):
    import torch

    from baybridge_b200.fused_gather import FusedGather

    rng = np.random.default_rng(n + fanout)
    a = oracle.bf16_round(rng.standard_normal(n).astype(np.float32))
    b = oracle.bf16_round(rng.standard_normal(n).astype(np.float32))
    d_a, d_b = to_device(a, "bf16"), to_device(b, "bf16")
    unused = torch.zeros(n, device="cuda", dtype=torch.bfloat16)
    shards = 3
    buffers = [torch.full((shards * n,), -7.0, device="cuda", dtype=torch.bfloat16) for _ in range(fanout)]
    fused = FusedGather(zoo.make_fused_mul_add_indexed(n), [d_a, d_b, unused],
                        destinations={2: [buffer.data_ptr() for buffer in buffers]}, shard_index=shard_index)
    fused.run(d_a, d_b, unused)
    torch.cuda.synchronize()
    expected = oracle.round_to_dtype(a.astype(np.float64) * b + a, "bf16")
    for buffer in buffers:
        host = to_host(buffer)
        assert np.array_equal(host[shard_index * n:(shard_index + 1) * n], expected)
        untouched = np.delete(host, np.s_[shard_index * n:(shard_index + 1) * n])
        assert np.all(untouched == -7.0)
    assert not unused.any()  # the argument itself is not written in this form


def test_fan_out_refuses_in_place_and_non_flat_kernels(zoo):
    import torch

    import baybridge_b200 as cute
    from baybridge_b200.fused_gather import FusedGather

    t = torch.zeros(256, device="cuda")

    @cute.kernel(launch=cute.LaunchConfig(grid=(1, 1, 1), block=(256, 1, 1)))
    def in_place(x: cute.Tensor):
        i = cute.thread_idx("x")
        x[i] = x[i] + 1.0

    with pytest.raises(cute.BackendNotImplementedError, match="in place"):
        FusedGather(in_place, [t], destinations={0: [t.data_ptr()]}, shard_index=0)
    with pytest.raises(cute.BackendNotImplementedError, match="flat elementwise"):
        FusedGather(zoo.gemm_abt, [torch.zeros(128, 64, device="cuda", dtype=torch.bfloat16)] * 2 + [torch.zeros(128, 128, device="cuda")],
                    destinations={2: [t.data_ptr()]}, shard_index=0)


@pytest.mark.parametrize("m,n,k,c_dtype", [(256, 512, 128, "bf16"), (200, 136, 72, "f32"), (2560, 2048, 136, "bf16"),
                                          (128, 256, 2048, "bf16")])  # the last one is split along K and folded into both copies
def test_gemm_epilogue_stores_its_row_block_into_every_destination(m, n, k, c_dtype, zoo):
    """bb200_gemm_bf16_gather with two local destination buffers standing in for two GPUs' copies of C."""
    import torch

    from baybridge_b200.fused_gather import FusedGatherGemm

    rng = np.random.default_rng(m + n + k)
    a = oracle.bf16_round((rng.standard_normal((m, k)) / np.sqrt(k)).astype(np.float32))
    b = oracle.bf16_round((rng.standard_normal((n, k)) / np.sqrt(k)).astype(np.float32))
    d_a, d_b = to_device(a, "bf16"), to_device(b, "bf16")
    dtype = torch.bfloat16 if c_dtype == "bf16" else torch.float32
    blocks, mine = 3, 1
    copies = [torch.full((blocks * m, n), -3.0, device="cuda", dtype=dtype) for _ in range(2)]
    sample_c = torch.zeros((m, n), device="cuda", dtype=dtype)
    fused = FusedGatherGemm(zoo.gemm_abt, [d_a, d_b, sample_c], destinations=[c.data_ptr() for c in copies], shard_index=mine)
    fused.run(d_a, d_b)
    torch.cuda.synchronize()
    reference = oracle.gemm(a, b, transpose_b=True)
    for copy in copies:
        host = to_host(copy)
        assert oracle.rel_l2(host[mine * m:(mine + 1) * m], reference) <= (1e-2 if c_dtype == "bf16" else 1e-5)
        assert np.all(host[:mine * m] == -3.0) and np.all(host[(mine + 1) * m:] == -3.0)
    assert torch.equal(copies[0], copies[1])


@pytest.mark.parametrize("dtype,rows,hidden", [("bf16", 16, 8192), ("f32", 7, 1020), ("f16", 33, 2048)])
def test_rmsnorm_stores_its_rows_into_every_destination(dtype, rows, hidden, zoo):
    import torch

    from baybridge_b200.fused_gather import FusedGatherRmsNorm

    rng = np.random.default_rng(rows + hidden)
    x = oracle.round_to_dtype(rng.standard_normal((rows, hidden)), dtype)
    w = oracle.round_to_dtype(1 + 0.1 * rng.standard_normal(hidden), dtype)
    d_x, d_w = to_device(x, dtype), to_device(w, dtype)
    torch_dtype = {"bf16": torch.bfloat16, "f16": torch.float16, "f32": torch.float32}[dtype]
    blocks, mine = 3, 2
    copies = [torch.full((blocks * rows, hidden), -3.0, device="cuda", dtype=torch_dtype) for _ in range(2)]
    sample_out = torch.zeros((rows, hidden), device="cuda", dtype=torch_dtype)
    fused = FusedGatherRmsNorm(zoo.make_rmsnorm(1e-6), [d_x, sample_out, d_w], destinations=[c.data_ptr() for c in copies], shard_index=mine)
    fused.run(d_x, d_w)
    torch.cuda.synchronize()
    reference = oracle.rmsnorm(x, w, 1e-6)
    for copy in copies:
        host = to_host(copy)
        assert oracle.rel_l2(host[mine * rows:], reference) <= (2e-3 if dtype != "f32" else 2e-6)
        assert np.all(host[:mine * rows] == -3.0)
    assert torch.equal(copies[0], copies[1])


@pytest.mark.parametrize("batch,seq,heads,kv_heads,dim,causal", [
    (2, 256, 4, 2, 128, True), (1, 200, 2, 1, 128, False), (2, 512, 2, 2, 64, True), (1, 130, 2, 2, 64, False),
])
def test_attention_stores_its_sequences_into_every_destination(batch, seq, heads, kv_heads, dim, causal, zoo):
    """bb200_attention_fwd_gather with two local copies of the gathered out/lse standing in for two GPUs."""
    import torch

    from baybridge_b200.fused_gather import FusedGatherAttention

    rng = np.random.default_rng(batch * 1009 + seq * 31 + heads * 7 + dim + causal)
    q = oracle.bf16_round(rng.standard_normal((batch, seq, heads, dim), dtype=np.float32))
    k = oracle.bf16_round(rng.standard_normal((batch, seq, kv_heads, dim), dtype=np.float32))
    v = oracle.bf16_round(rng.standard_normal((batch, seq, kv_heads, dim), dtype=np.float32))
    d_q, d_k, d_v = (to_device(t, "bf16") for t in (q, k, v))
    blocks, mine = 3, 1
    outs = [torch.full((blocks * batch, seq, heads, dim), -3.0, device="cuda", dtype=torch.bfloat16) for _ in range(2)]
    lses = [torch.full((blocks * batch, heads, 1, seq), -3.0, device="cuda", dtype=torch.float32) for _ in range(2)]
    sample_out = torch.zeros((batch, seq, heads, dim), device="cuda", dtype=torch.bfloat16)
    sample_lse = torch.zeros((batch, heads, 1, seq), device="cuda", dtype=torch.float32)
    kernel = zoo.attention_causal if causal else zoo.attention_full
    fused = FusedGatherAttention(kernel, [d_q, d_k, d_v, sample_out, sample_lse], out_destinations=[t.data_ptr() for t in outs],
                                 lse_destinations=[t.data_ptr() for t in lses], shard_index=mine)
    fused.run(d_q, d_k, d_v)
    torch.cuda.synchronize()
    ref_out, ref_lse = oracle.attention(q, k, v, causal=causal)
    mine_rows = slice(mine * batch, (mine + 1) * batch)
    for out, lse in zip(outs, lses):
        host_out, host_lse = to_host(out), to_host(lse)
        assert oracle.rel_l2(host_out[mine_rows], ref_out) <= 1e-2
        assert float(np.abs(host_lse[mine_rows].reshape(ref_lse.shape) - ref_lse).max()) <= 1e-2
        assert np.all(np.delete(host_out, mine_rows, axis=0) == -3.0) and np.all(np.delete(host_lse, mine_rows, axis=0) == -3.0)
    assert torch.equal(outs[0], outs[1]) and torch.equal(lses[0], lses[1])
    # the gathered rows are bit-identical to what the single-destination kernel writes
    import baybridge_b200 as cute
    artifact = cute.compile(kernel, d_q, d_k, d_v, sample_out, sample_lse, backend="b200")
    artifact(d_q, d_k, d_v, sample_out, sample_lse)
    assert torch.equal(outs[0][mine_rows], sample_out) and torch.equal(lses[0][mine_rows], sample_lse)


@pytest.mark.parametrize("dtype,rows,hidden", [("bf16", 16, 8192), ("f32", 6, 1020), ("f16", 33, 2048)])
def test_layernorm_stores_both_outputs_into_every_destination(dtype, rows, hidden, zoo):
    import torch

    from baybridge_b200.fused_gather import FusedGatherLayerNorm

    rng = np.random.default_rng(rows * 7 + hidden)
    x = oracle.round_to_dtype(rng.standard_normal((rows, hidden)), dtype)
    r = oracle.round_to_dtype(rng.standard_normal((rows, hidden)), dtype)
    w = oracle.round_to_dtype(1 + 0.1 * rng.standard_normal(hidden), dtype)
    b = oracle.round_to_dtype(0.1 * rng.standard_normal(hidden), dtype)
    d_x, d_r, d_w, d_b = (to_device(t, dtype) for t in (x, r, w, b))
    torch_dtype = {"bf16": torch.bfloat16, "f16": torch.float16, "f32": torch.float32}[dtype]
    blocks, mine = 3, 1
    outs = [torch.full((blocks * rows, hidden), -3.0, device="cuda", dtype=torch_dtype) for _ in range(2)]
    resids = [torch.full((blocks * rows, hidden), -3.0, device="cuda", dtype=torch_dtype) for _ in range(2)]
    sample = torch.zeros((rows, hidden), device="cuda", dtype=torch_dtype)
    fused = FusedGatherLayerNorm(zoo.layernorm_kernel, [d_x, d_r, sample, sample.clone(), d_w, d_b],
                                 out_destinations=[t.data_ptr() for t in outs], out_resid_destinations=[t.data_ptr() for t in resids],
                                 shard_index=mine)
    fused.run(d_x, d_r, d_w, d_b)
    torch.cuda.synchronize()
    ref_out, ref_mixed = oracle.layernorm(x, r, w, b, 1e-5)
    block = slice(mine * rows, (mine + 1) * rows)
    for out, resid in zip(outs, resids):
        host_out, host_resid = to_host(out), to_host(resid)
        assert oracle.rel_l2(host_out[block], ref_out) <= (2e-3 if dtype != "f32" else 2e-6)
        assert np.array_equal(host_resid[block], oracle.round_to_dtype(ref_mixed, dtype))
        assert np.all(np.delete(host_out, block, axis=0) == -3.0) and np.all(np.delete(host_resid, block, axis=0) == -3.0)
    assert torch.equal(outs[0], outs[1]) and torch.equal(resids[0], resids[1])
