"""The allocation-free GEMM entry point against the regular one.

``bb200_gemm_bf16_noalloc`` exists for embedders that may not allocate device memory at run time
(their own pools already own the GPU, or an allocation could stall or fail in a latency-critical
loop).  It stages the transposed copy of A in a buffer built into the library instead of asking the
driver for a workspace.  The check here: through the C ABI, with A stored [k, m] and m not a multiple
of 8 (the one layout the kernel cannot read in place) so the built-in buffer is really used, the
result must be identical to ``bb200_gemm_bf16`` — twice in a row, with
different inputs, because the buffer keeps the previous call's contents.
"""
from __future__ import annotations

import ctypes

import numpy as np
import pytest
from gpu_util import current_stream, device_zeros, to_device, to_host, void_p

from oracle import cpu_runtime as oracle

pytestmark = pytest.mark.gpu


def _pair(seed: int, m: int, n: int, k: int):
    rng = np.random.default_rng(seed)
    a_km = oracle.bf16_round(rng.standard_normal((k, m)).astype(np.float32) / np.sqrt(k))  # A stored [k, m]
    b_nk = oracle.bf16_round(rng.standard_normal((n, k)).astype(np.float32) / np.sqrt(k))
    return a_km, b_nk


@pytest.mark.parametrize("c_dtype", ["bf16", "f32"])
def test_noalloc_gemm_equals_regular_gemm_on_two_calls_in_a_row(c_dtype):
    import torch

    from baybridge_b200.backend import native

    code = native.DTYPE_CODES[c_dtype]
    # m % 8 != 0: the staged-copy path; the second call is smaller, so stale bytes of the first stay behind it
    for call, (m, n, k) in enumerate([(380, 520, 264), (196, 136, 72)]):
        a_km, b_nk = _pair(100 + call, m, n, k)
        a, b = to_device(a_km, "bf16"), to_device(b_nk, "bf16")
        expected, got = device_zeros((m, n), c_dtype), device_zeros((m, n), c_dtype)
        native.call("bb200_gemm_bf16", void_p(a), void_p(b), void_p(expected), m, n, k, 1, 1, code, current_stream())
        native.call("bb200_gemm_bf16_noalloc", void_p(a), void_p(b), void_p(got), m, n, k, 1, 1, code, current_stream())
        torch.cuda.synchronize()
        status = ctypes.c_int(-1)
        native.call("bb200_take_device_status", current_stream(), ctypes.byref(status))
        assert status.value == 0
        assert torch.equal(got, expected), f"call {call}: results differ"
        reference = oracle.gemm(a_km, b_nk, transpose_a=True, transpose_b=True)
        assert oracle.rel_l2(to_host(got), reference) <= (1e-2 if c_dtype == "bf16" else 1e-5)


def test_noalloc_gemm_without_transposed_a_and_size_limit():
    import torch

    from baybridge_b200 import CudaDriverError
    from baybridge_b200.backend import native

    m, n, k = 256, 256, 128
    a_km, b_nk = _pair(7, m, n, k)
    a_mk = to_device(np.ascontiguousarray(a_km.T), "bf16")
    b = to_device(b_nk, "bf16")
    expected, got = device_zeros((m, n), "bf16"), device_zeros((m, n), "bf16")
    native.call("bb200_gemm_bf16", void_p(a_mk), void_p(b), void_p(expected), m, n, k, 0, 1, 1, current_stream())
    native.call("bb200_gemm_bf16_noalloc", void_p(a_mk), void_p(b), void_p(got), m, n, k, 0, 1, 1, current_stream())
    torch.cuda.synchronize()
    assert torch.equal(got, expected)
    # 8188 x 4096 transposed elements = 64 MiB > the 32 MiB built-in buffer: rejected before anything is launched
    with pytest.raises(CudaDriverError) as info:
        native.call("bb200_gemm_bf16_noalloc", void_p(a_mk), void_p(b), void_p(got), 8188, 256, 4096, 1, 1, 1, current_stream())
    assert info.value.status == -7  # BB200_E_TOO_LARGE
    assert "built-in buffer" in info.value.message


@pytest.mark.parametrize("c_dtype", ["bf16", "f32"])
def test_noalloc_gemm_reads_aligned_transposed_a_in_place(c_dtype):
    """A stored [k, m] with m a multiple of 8 needs no staged copy at all: no size limit applies, and both entry
    points agree with the oracle."""
    import torch

    from baybridge_b200.backend import native

    code = native.DTYPE_CODES[c_dtype]
    m, n, k = 384, 520, 264
    a_km, b_nk = _pair(11, m, n, k)
    a, b = to_device(a_km, "bf16"), to_device(b_nk, "bf16")
    expected, got = device_zeros((m, n), c_dtype), device_zeros((m, n), c_dtype)
    native.call("bb200_gemm_bf16", void_p(a), void_p(b), void_p(expected), m, n, k, 1, 1, code, current_stream())
    native.call("bb200_gemm_bf16_noalloc", void_p(a), void_p(b), void_p(got), m, n, k, 1, 1, code, current_stream())
    torch.cuda.synchronize()
    assert torch.equal(got, expected)
    assert oracle.rel_l2(to_host(got), oracle.gemm(a_km, b_nk, transpose_a=True, transpose_b=True)) <= (1e-2 if c_dtype == "bf16" else 1e-5)
    # 8192 x 4096 elements would not fit the built-in buffer, but nothing is staged for this layout
    big_a, big_b, big_c = device_zeros((4096, 8192), "bf16"), device_zeros((256, 4096), "bf16"), device_zeros((8192, 256), c_dtype)
    native.call("bb200_gemm_bf16_noalloc", void_p(big_a), void_p(big_b), void_p(big_c), 8192, 256, 4096, 1, 1, code, current_stream())
    torch.cuda.synchronize()


def test_long_narrow_transposed_a_fits_the_launch_grid():
    """A stored [k, m] with m = 4 and k over two million is 8.8 Mi elements — inside the built-in buffer's 16 Mi — and its
    transposed copy needs 68 750 tile rows, more than a grid's y extent: every size under the documented limit must launch."""
    import torch

    from baybridge_b200.backend import native

    m, n, k = 4, 8, 2_200_000
    a_km, b_nk = _pair(21, m, n, k)
    a, b = to_device(a_km, "bf16"), to_device(b_nk, "bf16")
    expected, got = device_zeros((m, n), "f32"), device_zeros((m, n), "f32")
    native.call("bb200_gemm_bf16", void_p(a), void_p(b), void_p(expected), m, n, k, 1, 1, 0, current_stream())
    native.call("bb200_gemm_bf16_noalloc", void_p(a), void_p(b), void_p(got), m, n, k, 1, 1, 0, current_stream())
    torch.cuda.synchronize()
    reference = oracle.gemm(a_km, b_nk, transpose_a=True, transpose_b=True)
    # 2.2 million products accumulated on the tensor cores (whose fp32 accumulation truncates): measured 2.2e-3; the bar is
    # the BF16 GEMM bar of the hot path, rel-L2 <= 1e-2
    for label, result in (("no-alloc", got), ("regular", expected)):  # the regular entry may split K: same bar, not bit-equal
        error = oracle.rel_l2(to_host(result), reference)
        assert error <= 1e-2, f"{label} entry: rel-L2 {error:.3e}"
