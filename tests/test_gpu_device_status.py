"""A bounded device-side wait that gives up: the kernel returns, the status word records it, the launcher raises.

Nothing here faults, traps or hangs the GPU: the self-test kernel waits — through the same ``mbar_wait`` every
pipeline of the library uses — on a barrier nobody arrives on, with a 1 ms limit instead of the kernels' 1 s.
Upstream's launchers turn a non-zero native status into an exception (``hipcc_exec.py:181-182``); a give-up inside a
kernel is this backend's equivalent of that status.
"""
from __future__ import annotations

import ctypes

import numpy as np
import pytest
from gpu_util import current_stream, to_device, to_host

from oracle import cpu_runtime as oracle

pytestmark = pytest.mark.gpu

SELFTEST_CODE = 99


def test_abandoned_wait_returns_sets_the_status_word_and_leaves_the_context_usable():
    import torch

    from baybridge_b200.backend import native

    stream = current_stream()
    assert native.take_device_status(stream) == 0
    native.call("bb200_selftest_bounded_wait", 1000, stream)  # 1 ms limit; returns only if the kernel returned
    assert native.take_device_status(stream) == SELFTEST_CODE
    assert native.take_device_status(stream) == 0  # reading clears it
    # the context is alive: ordinary work still runs and is correct
    a = torch.arange(1024, device="cuda", dtype=torch.float32)
    assert float((a + 1).sum().item()) == float(np.arange(1024).sum() + 1024)
    with pytest.raises(Exception, match="limit must be"):
        native.call("bb200_selftest_bounded_wait", 0, stream)


def test_synchronising_launcher_raises_on_a_recorded_give_up_and_recovers(zoo, tmp_path):
    import baybridge_b200 as cute
    from baybridge_b200.backend import native

    rng = np.random.default_rng(11)
    m = n = k = 256
    a_host = oracle.bf16_round((rng.standard_normal((m, k)) / 16).astype(np.float32))
    b_host = oracle.bf16_round((rng.standard_normal((n, k)) / 16).astype(np.float32))
    a, b = to_device(a_host, "bf16"), to_device(b_host, "bf16")
    c = to_device(np.zeros((m, n), dtype=np.float32), "bf16")
    artifact = cute.compile(zoo.gemm_abt, a, b, c, backend="b200", cache_dir=tmp_path)
    artifact(a, b, c)  # clean launch: no status
    native.call("bb200_selftest_bounded_wait", 1000, current_stream())  # a wait gives up on this device
    with pytest.raises(RuntimeError, match=r"launch_\w+ returned device status 99"):
        artifact(a, b, c)
    artifact(a, b, c)  # the word was cleared by the failed call; the launcher works again
    assert oracle.rel_l2(to_host(c), oracle.gemm(a_host, b_host, transpose_b=True)) <= 1e-2

    # host tensors staged by the launcher: its device copies are released on that error path and re-made afterwards
    host = [cute.tensor(a_host.astype(np.float64).tolist(), dtype="bf16"), cute.tensor(b_host.astype(np.float64).tolist(), dtype="bf16"),
            cute.zeros((m, n), dtype="bf16")]
    staged = cute.compile(zoo.gemm_abt, *host, backend="b200", cache_dir=tmp_path)
    with pytest.warns(RuntimeWarning):
        staged(*host)
    native.call("bb200_selftest_bounded_wait", 1000, ctypes.c_void_p(0))
    with pytest.raises(RuntimeError, match="device status 99"):
        staged(*host)
    staged(*host)
    assert oracle.rel_l2(np.asarray(host[2].tolist(), dtype=np.float64), oracle.gemm(a_host, b_host, transpose_b=True)) <= 1e-2


def test_debug_bounds_build_reports_out_of_range_accesses(zoo, tmp_path, monkeypatch):
    """``BB200_DEBUG_BOUNDS=1``: a thread-by-thread kernel whose grid overshoots its tensors raises instead of skipping the
    stray accesses silently (upstream's CPU runtime raises IndexError there; its generated kernels skip, as the default
    build here does).  Nothing faults: the checked access is never performed."""
    import baybridge_b200 as cute

    n = 1000  # 8 blocks of 128 threads: 24 threads index past the end of both tensors
    src_host = np.arange(n, dtype=np.float32)
    src, dst = to_device(src_host, "f32"), to_device(np.zeros(n, dtype=np.float32), "f32")
    quiet = cute.compile(zoo.make_indexed_reverse(n), src, dst, backend="b200", cache_dir=tmp_path / "quiet")
    quiet(src, dst)
    assert np.array_equal(to_host(dst), src_host[::-1].astype(np.float64))
    monkeypatch.setenv("BB200_DEBUG_BOUNDS", "1")
    checked = cute.compile(zoo.make_indexed_reverse(n), src, dst, backend="b200", cache_dir=tmp_path / "checked", use_cache=False)
    with pytest.raises(RuntimeError, match=r"device status 30[12]"):
        checked(src, dst)
    assert np.array_equal(to_host(dst), src_host[::-1].astype(np.float64))  # in-range work is unaffected
    exact = cute.compile(zoo.make_indexed_reverse(1024), to_device(np.arange(1024, dtype=np.float32), "f32"),
                         to_device(np.zeros(1024, dtype=np.float32), "f32"), backend="b200", cache_dir=tmp_path / "exact", use_cache=False)
    exact(to_device(np.arange(1024, dtype=np.float32), "f32"), to_device(np.zeros(1024, dtype=np.float32), "f32"))  # no stray access: no error
