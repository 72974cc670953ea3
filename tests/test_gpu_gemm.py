"""GPU parity for the BF16 GEMM: compile(..., backend="b200") and the C ABI vs the CPU oracle/golden vectors.

Tolerance (the path's contract): rel-L2 <= 1e-2 against the f64 reference for bf16 output; fp32
output is held to 1e-5 (fp32 accumulation of exact bf16 products)."""
from __future__ import annotations

import numpy as np
import pytest
from conftest import gemm_zoo_kernel, golden_cases, golden_ir, golden_vec
from gpu_util import current_stream, device_zeros, to_device, to_host, void_p

from oracle import cpu_runtime as oracle

pytestmark = pytest.mark.gpu
REL_L2_BF16 = 1e-2
REL_L2_F32 = 1e-5


@pytest.mark.parametrize("case", golden_cases("c3_") + golden_cases("gemm_"))
def test_compiled_gemm_matches_upstream_vectors(case, zoo, tmp_path):
    import baybridge_b200 as cute

    ir = golden_ir(case)["ir"]
    vec = golden_vec(case)
    kernel = gemm_zoo_kernel(case, ir, zoo)
    c_dtype = ir["arguments"][2]["spec"]["dtype"]
    a, b = to_device(vec["in_a"], "bf16"), to_device(vec["in_b"], "bf16")
    c = device_zeros(vec["out_c"].shape, c_dtype)
    artifact = cute.compile(kernel, a, b, c, backend="b200", cache_dir=tmp_path)
    assert artifact.ir.to_dict()["operations"] == ir["operations"]
    artifact(a, b, c)
    got = to_host(c)
    if case.startswith("gemm_ab_ramp_"):
        # upstream tests/test_backend_hipkittens_exec.py:380-440: every column of C picks one column of the ramp A,
        # exactly as the device sees it.  The ramps reach 512 and 2048, beyond bf16's 8 significant bits, so the device operand is
        # RNE(A) (the CPU runtime keeps the unrounded Python floats, which is what the fixture holds).
        expected = oracle.gemm(oracle.bf16_round(vec["in_a"]), vec["in_b"])
        assert np.array_equal(got, expected)
        assert oracle.rel_l2(got, vec["out_c"]) <= REL_L2_BF16
        return
    assert oracle.rel_l2(got, vec["out_c"]) <= (REL_L2_BF16 if c_dtype == "bf16" else REL_L2_F32)


@pytest.mark.parametrize("m,n,k", [
    (128, 256, 64), (256, 512, 128), (128, 256, 1024), (384, 768, 320), (200, 136, 72), (100, 50, 24), (1, 8, 8),
    (129, 257, 8), (1024, 1024, 1024), (4096, 512, 256), (130, 4100, 136),
    (128, 35840, 64),    # one row block, 140 full-width tiles: the 256-column single-CTA kernel
    (256, 8192, 512),    # 128 tiles of 128 columns fit one wave: the 128-column kernel
    (512, 8192, 256),    # 64 pair tiles: the CTA-pair kernel at less than one wave
    (384, 4096, 128),    # three row blocks (no pairs), 192 tiles of 64 columns would not fit: 128 columns
    (512, 512, 4096),    # 32 narrow tiles, deep K: four K-splits folded by the second kernel
    (200, 136, 2048),    # K-split with ragged tiles
    (100, 50, 1024),     # K-split whose rows are not 16-byte multiples (element-wise fold)
])
@pytest.mark.parametrize("c_dtype", ["bf16", "f32"])
def test_c_abi_gemm_abt_shapes(m, n, k, c_dtype):
    from baybridge_b200.backend import native

    rng = np.random.default_rng(m * 7919 + n * 131 + k)
    a = oracle.bf16_round((rng.standard_normal((m, k)) / np.sqrt(k)).astype(np.float32))
    b = oracle.bf16_round((rng.standard_normal((n, k)) / np.sqrt(k)).astype(np.float32))
    d_a, d_b = to_device(a, "bf16"), to_device(b, "bf16")
    d_c = device_zeros((m, n), c_dtype)
    native.call("bb200_gemm_bf16", void_p(d_a), void_p(d_b), void_p(d_c), m, n, k, 0, 1, native.DTYPE_CODES[c_dtype], current_stream())
    status = __import__("ctypes").c_int(-1)
    native.call("bb200_take_device_status", current_stream(), __import__("ctypes").byref(status))
    assert status.value == 0, f"a bounded device wait gave up (code {status.value})"
    reference = oracle.gemm(a, b, transpose_b=True)
    assert oracle.rel_l2(to_host(d_c), reference) <= (REL_L2_BF16 if c_dtype == "bf16" else REL_L2_F32)


@pytest.mark.parametrize("m,n,k", [
    (160, 264, 96),      # everything read in place (m and n multiples of 8)
    (156, 264, 96),      # A stored [k, m] with m % 8 != 0: the transposed-copy path
    (640, 1032, 200),    # several tiles, ragged edges in m, n and k
    (2560, 2048, 136),   # enough 256x256 tiles for the CTA-pair kernel
    (128, 34816, 72),    # 136 full-width tiles in one row block: the 256-column single-CTA kernel
    (256, 8192, 72),     # the 128-column single-CTA kernel
    (160, 264, 1096),    # two K-splits, the last k-block ragged
])
def test_c_abi_gemm_transpose_variants_agree(m, n, k):
    from baybridge_b200.backend import native

    rng = np.random.default_rng(11 + m)
    a = oracle.bf16_round(rng.standard_normal((m, k)).astype(np.float32))
    b = oracle.bf16_round(rng.standard_normal((k, n)).astype(np.float32))
    reference = oracle.gemm(a, b)
    for transpose_a in (0, 1):
        for transpose_b in (0, 1):
            stored_a = to_device(np.ascontiguousarray(a.T) if transpose_a else a, "bf16")
            stored_b = to_device(np.ascontiguousarray(b.T) if transpose_b else b, "bf16")
            c = device_zeros((m, n), "f32")
            native.call("bb200_gemm_bf16", void_p(stored_a), void_p(stored_b), void_p(c), m, n, k, transpose_a, transpose_b, 0, current_stream())
            assert oracle.rel_l2(to_host(c), reference) <= REL_L2_F32, (transpose_a, transpose_b)


def test_c_abi_gemm_rejects_bad_arguments():
    from baybridge_b200 import CudaDriverError
    from baybridge_b200.backend import native

    x = device_zeros((64, 64), "bf16")
    with pytest.raises(CudaDriverError) as info:  # k must be a multiple of 8
        native.call("bb200_gemm_bf16", void_p(x), void_p(x), void_p(x), 64, 64, 12, 0, 1, 1, current_stream())
    assert info.value.status == -2
    with pytest.raises(CudaDriverError):
        native.call("bb200_gemm_bf16", void_p(x), void_p(x), void_p(x), 0, 64, 64, 0, 1, 1, current_stream())
    with pytest.raises(CudaDriverError):
        native.call("bb200_gemm_bf16", void_p(x), void_p(x), void_p(x), 64, 64, 64, 0, 1, 3, current_stream())  # i32 C


def test_config3_full_size_gemm(zoo, tmp_path):
    """8192^3 through compile().  The f64 oracle is evaluated on 256 sampled rows (1/32 of C); every row
    is also checked through a checksum of checksums: sum_n C[m, n] == A[m, :] · (sum_n B[n, :])."""
    import torch

    import baybridge_b200 as cute

    size = 8192
    generator = torch.Generator(device="cuda").manual_seed(1003)
    scale = 1.0 / np.sqrt(size)
    a = (torch.randn((size, size), device="cuda", dtype=torch.float32, generator=generator) * scale).to(torch.bfloat16)
    b = (torch.randn((size, size), device="cuda", dtype=torch.float32, generator=generator) * scale).to(torch.bfloat16)
    c = torch.zeros((size, size), device="cuda", dtype=torch.bfloat16)
    artifact = cute.compile(zoo.gemm_abt, a, b, c, backend="b200", cache_dir=tmp_path)
    artifact(a, b, c)
    rows = np.sort(np.random.default_rng(3).choice(size, 256, replace=False))
    index = torch.from_numpy(rows).cuda()
    reference = oracle.gemm(to_host(a[index]), to_host(b), transpose_b=True)
    assert oracle.rel_l2(to_host(c[index]), reference) <= REL_L2_BF16
    # checksum of checksums over the whole output (bf16 output rounding averages out over 8192 columns)
    row_sums = c.double().sum(dim=1).cpu().numpy()
    expected = (a.double() @ b.double().sum(dim=0)).cpu().numpy()
    assert np.abs(row_sums - expected).max() <= 0.05 * np.abs(expected).max() + 0.5
    # linearity in A: gemm(2A, B) == 2 gemm(A, B) exactly (powers of two commute with every rounding)
    doubled = torch.zeros_like(c)
    artifact(a * 2, b, doubled)
    assert torch.equal(doubled, c * 2)
