"""Launch graphs: compiled-kernel launches recorded once and replayed with one driver call give the same results as
launching them one at a time, and read the buffers' contents at replay time."""
from __future__ import annotations

import numpy as np
import pytest
from gpu_util import to_device, to_host

from oracle import cpu_runtime as oracle

pytestmark = pytest.mark.gpu


def test_recorded_config1_adds_replay_bit_exact(zoo, tmp_path):
    """Config 1 (256x256 f32 indexed add), chained c = a + b; a = c + b, recorded 8 times: replay equals 16 eager adds."""
    import torch

    import baybridge_b200 as cute
    from baybridge_b200.launch_graph import LaunchGraph

    rng = np.random.default_rng(1001)
    a_host = rng.uniform(-1, 1, (256, 256)).astype(np.float32)
    b_host = rng.uniform(-1, 1, (256, 256)).astype(np.float32)
    a, b = to_device(a_host, "f32"), to_device(b_host, "f32")
    c = torch.zeros_like(a)
    artifact = cute.compile(zoo.make_indexed_add_2d(256, 256), a, b, c, backend="b200", cache_dir=tmp_path)  # synchronising launcher
    graph = LaunchGraph()
    with graph.record() as stream:
        for _ in range(8):
            artifact(a, b, c, stream=stream)   # c = a + b
            artifact(c, b, a, stream=stream)   # a = c + b
    torch.cuda.synchronize()
    assert np.array_equal(to_host(a), a_host) and not to_host(c).any()  # recording runs nothing
    graph.replay()
    torch.cuda.synchronize()
    expected = a_host.copy()
    for _ in range(16):
        expected = (expected.astype(np.float64) + b_host).astype(np.float32)
    assert np.array_equal(to_host(a), expected)
    # a second replay continues from the buffers' current contents
    graph.replay(stream=torch.cuda.current_stream())
    torch.cuda.synchronize()
    for _ in range(16):
        expected = (expected.astype(np.float64) + b_host).astype(np.float32)
    assert np.array_equal(to_host(a), expected)
    graph.close()
    with pytest.raises(RuntimeError, match="nothing has been recorded"):
        graph.replay()


def test_recorded_library_kernels_match_eager_launches(zoo, tmp_path):
    """RMSNorm, the tcgen05 GEMM and attention in one recording: same bits as the same launches made eagerly."""
    import torch

    import baybridge_b200 as cute
    from baybridge_b200.launch_graph import LaunchGraph

    rng = np.random.default_rng(7)
    x = to_device(oracle.bf16_round(rng.standard_normal((64, 1024)).astype(np.float32)), "bf16")
    w = to_device(oracle.bf16_round((1 + 0.1 * rng.standard_normal(1024)).astype(np.float32)), "bf16")
    normed = torch.zeros_like(x)
    weight = to_device(oracle.bf16_round((rng.standard_normal((512, 1024)) / 32).astype(np.float32)), "bf16")
    projected = torch.zeros((64, 512), device="cuda", dtype=torch.float32)
    q, k, v = (to_device(oracle.bf16_round(rng.standard_normal((1, 256, 2, 128)).astype(np.float32)), "bf16") for _ in range(3))
    out, lse = torch.zeros_like(q), torch.zeros((1, 2, 1, 256), device="cuda", dtype=torch.float32)
    norm = cute.compile(zoo.make_rmsnorm(1e-6), x, normed, w, backend="b200", cache_dir=tmp_path)
    gemm = cute.compile(zoo.gemm_abt, normed, weight, projected, backend="b200", cache_dir=tmp_path)
    attention = cute.compile(zoo.attention_causal, q, k, v, out, lse, backend="b200", cache_dir=tmp_path)

    def launch_all(stream):
        norm(x, normed, w, stream=stream)
        gemm(normed, weight, projected, stream=stream)
        attention(q, k, v, out, lse, stream=stream)

    launch_all(None)
    eager = [t.clone() for t in (normed, projected, out, lse)]
    for t in (normed, projected, out, lse):
        t.zero_()
    graph = LaunchGraph()
    with graph.record() as stream:
        launch_all(stream)
    graph.replay()
    torch.cuda.synchronize()
    for got, want in zip((normed, projected, out, lse), eager):
        assert torch.equal(got, want)
    graph.close()


def test_recording_refuses_host_tensors_and_recovers(zoo, tmp_path):
    import torch

    import baybridge_b200 as cute
    from baybridge_b200.launch_graph import LaunchGraph

    a = torch.ones(256, device="cuda")
    b = torch.ones(256, device="cuda")
    c = torch.zeros(256, device="cuda")
    artifact = cute.compile(zoo.make_indexed_binary("add", 256), a, b, c, backend="b200", cache_dir=tmp_path)
    host = cute.tensor([1.0] * 256, dtype="f32")
    graph = LaunchGraph()
    with pytest.raises(cute.BackendNotImplementedError, match="while a launch graph records"):
        with graph.record() as stream:
            artifact(host, b, c, stream=stream)
    # the failed recording left nothing behind: a fresh one on the same object works
    with graph.record() as stream:
        artifact(a, b, c, stream=stream)
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(c, a + b)
    graph.close()
