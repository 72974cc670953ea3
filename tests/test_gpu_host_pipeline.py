"""Host-to-host pipeline (chunked copies overlapped with the kernel) against the one-shot artifact call."""
from __future__ import annotations

import numpy as np
import pytest

from oracle import cpu_runtime as oracle

pytestmark = pytest.mark.gpu


def test_pipeline_matches_one_shot_elementwise_and_gemm(zoo, tmp_path):
    import torch

    from baybridge_b200.host_pipeline import HostPipeline

    n = 1_000_000  # 7 chunks are ragged (142858 / 142857 elements): two artifacts; 8 chunks are even
    rng = np.random.default_rng(3)
    a = torch.from_numpy(oracle.bf16_round(rng.standard_normal(n, dtype=np.float32))).to(torch.bfloat16).pin_memory()
    b = torch.from_numpy(oracle.bf16_round(rng.standard_normal(n, dtype=np.float32))).to(torch.bfloat16).pin_memory()
    for chunks in (1, 7, 8):
        c = torch.zeros(n, dtype=torch.bfloat16).pin_memory()
        pipeline = HostPipeline(lambda rows: zoo.make_fused_mul_add_indexed(rows), [a, b, c], chunks=chunks, cache_dir=tmp_path)
        pipeline.run()
        pipeline.run()  # buffers and events are reusable
        reference = a.double().numpy() * b.double().numpy() + a.double().numpy()
        assert oracle.rel_l2(c.double().numpy(), reference) <= 2e-3
        assert pipeline.h2d_bytes == 2 * n * 2 and pipeline.d2h_bytes == n * 2

    # chunks long enough to be ramped: the first and the last of the 8 become 1/8, 1/8, 1/4, 1/2 pieces (14 chunks, 4 lengths)
    n2 = 1 << 21
    a2r = torch.from_numpy(oracle.bf16_round(rng.standard_normal(n2, dtype=np.float32))).to(torch.bfloat16).pin_memory()
    b2r = torch.from_numpy(oracle.bf16_round(rng.standard_normal(n2, dtype=np.float32))).to(torch.bfloat16).pin_memory()
    for ramp in (True, False):
        c2r = torch.zeros(n2, dtype=torch.bfloat16).pin_memory()
        pipeline = HostPipeline(lambda rows: zoo.make_fused_mul_add_indexed(rows), [a2r, b2r, c2r], chunks=8, cache_dir=tmp_path, ramp=ramp)
        assert pipeline.chunks == (14 if ramp else 8) and len(pipeline.artifacts) == (4 if ramp else 1)
        assert pipeline.bounds[0] == (0, (n2 // 8) // (8 if ramp else 1)) and pipeline.bounds[-1][1] == n2
        pipeline.run()
        reference = a2r.double().numpy() * b2r.double().numpy() + a2r.double().numpy()
        assert np.array_equal(c2r.double().numpy(), oracle.bf16_round(reference.astype(np.float32)).astype(np.float64))

    m, nn, k = 1000, 512, 256  # M sharded in ragged chunks, B replicated
    a2 = torch.from_numpy(oracle.bf16_round((rng.standard_normal((m, k)) / 16).astype(np.float32))).to(torch.bfloat16).pin_memory()
    b2 = torch.from_numpy(oracle.bf16_round((rng.standard_normal((nn, k)) / 16).astype(np.float32))).to(torch.bfloat16).pin_memory()
    c2 = torch.zeros((m, nn), dtype=torch.float32).pin_memory()
    HostPipeline(lambda rows: zoo.gemm_abt, [a2, b2, c2], chunks=3, cache_dir=tmp_path).run()
    assert oracle.rel_l2(c2.double().numpy(), oracle.gemm(a2.double().numpy(), b2.double().numpy(), transpose_b=True)) <= 1e-5


def test_pipeline_rmsnorm_and_attention(zoo, tmp_path):
    import torch

    from baybridge_b200.host_pipeline import HostPipeline

    rng = np.random.default_rng(4)
    x = torch.from_numpy(oracle.bf16_round(rng.standard_normal((300, 1024), dtype=np.float32))).to(torch.bfloat16).pin_memory()
    w = torch.from_numpy(oracle.bf16_round((1 + 0.1 * rng.standard_normal(1024)).astype(np.float32))).to(torch.bfloat16).pin_memory()
    out = torch.zeros_like(x).pin_memory()
    HostPipeline(lambda rows: zoo.make_rmsnorm(1e-6), [x, out, w], chunks=4, cache_dir=tmp_path).run()
    assert oracle.rel_l2(out.double().numpy(), oracle.rmsnorm(x.double().numpy(), w.double().numpy(), 1e-6)) <= 2e-3

    shape = (3, 256, 2, 128)
    q, k, v = (torch.from_numpy(oracle.bf16_round(rng.standard_normal(shape, dtype=np.float32))).to(torch.bfloat16).pin_memory() for _ in range(3))
    o = torch.zeros(shape, dtype=torch.bfloat16).pin_memory()
    lse = torch.zeros((3, 2, 1, 256), dtype=torch.float32).pin_memory()
    HostPipeline(lambda rows: zoo.attention_causal, [q, k, v, o, lse], chunks=3, cache_dir=tmp_path).run()
    ref_out, ref_lse = oracle.attention(q.double().numpy(), k.double().numpy(), v.double().numpy(), causal=True)
    assert oracle.rel_l2(o.double().numpy(), ref_out) <= 1e-2
    assert float(np.abs(lse.double().numpy() - ref_lse).max()) <= 1e-2


def test_pipeline_copies_in_what_the_kernel_reads(zoo, tmp_path):
    """A tensor that is read and written (dst += src) must reach the device before the kernel runs, and an output the
    kernel only partly overwrites must come back with its other elements unchanged."""
    import torch

    from baybridge_b200.host_pipeline import HostPipeline

    n = 40_000
    rng = np.random.default_rng(5)
    src = torch.from_numpy(rng.uniform(-1, 1, n).astype(np.float32)).pin_memory()
    start = rng.uniform(-1, 1, n).astype(np.float32)
    for chunks in (1, 3):
        dst = torch.from_numpy(start.copy()).pin_memory()
        pipeline = HostPipeline(lambda rows: zoo.make_indexed_accumulate(rows), [src, dst], chunks=chunks, cache_dir=tmp_path)
        pipeline.run()
        assert np.array_equal(dst.numpy(), (start.astype(np.float64) + src.numpy().astype(np.float64)).astype(np.float32))
        assert pipeline.h2d_bytes == 2 * n * 4 and pipeline.d2h_bytes == n * 4

    # masked add over 1000 of 1024 elements: the last 24 elements of dst are not the kernel's to write
    a, b = (torch.from_numpy(rng.uniform(-1, 1, 1024).astype(np.float32)).pin_memory() for _ in range(2))
    kept = torch.full((1024,), 7.0).pin_memory()
    HostPipeline(lambda rows: zoo.make_indexed_masked_add(1000), [a, b, kept], chunks=1, cache_dir=tmp_path).run()
    assert np.array_equal(kept.numpy()[:1000], (a.numpy().astype(np.float64) + b.numpy()).astype(np.float32)[:1000])
    assert np.array_equal(kept.numpy()[1000:], np.full(24, 7.0, dtype=np.float32))


def test_pipeline_gemm_with_a_stored_k_by_m(zoo, tmp_path):
    """A stored [k, m] is sharded along its second axis: the pipeline runs whole tensors, with k != m."""
    import torch

    from baybridge_b200.host_pipeline import HostPipeline

    m, n, k = 384, 256, 640
    rng = np.random.default_rng(6)
    a = torch.from_numpy(oracle.bf16_round((rng.standard_normal((k, m)) / 16).astype(np.float32))).to(torch.bfloat16).pin_memory()
    b = torch.from_numpy(oracle.bf16_round((rng.standard_normal((k, n)) / 16).astype(np.float32))).to(torch.bfloat16).pin_memory()
    c = torch.zeros((m, n), dtype=torch.float32).pin_memory()
    pipeline = HostPipeline(lambda rows: zoo.gemm_atb, [a, b, c], chunks=4, cache_dir=tmp_path)
    assert pipeline.chunks == 1
    pipeline.run()
    assert oracle.rel_l2(c.double().numpy(), oracle.gemm(a.double().numpy(), b.double().numpy(), transpose_a=True)) <= 1e-5
