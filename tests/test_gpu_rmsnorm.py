"""GPU parity for RMSNorm: compile(..., backend="b200") and the C ABI vs the CPU oracle/golden vectors.

Tolerance (stated by the path's contract): rel-L2 <= 2e-3 against the fp32/f64 reference for bf16."""
from __future__ import annotations

import numpy as np
import pytest
from conftest import golden_ir, golden_vec
from gpu_util import current_stream, device_zeros, to_device, to_host, ulp_distance, void_p

from oracle import cpu_runtime as oracle

pytestmark = pytest.mark.gpu
REL_L2 = 2e-3


@pytest.mark.parametrize("case,eps", [("c4_rmsnorm_6x512_bf16_eps1e-6", 1e-6), ("rmsnorm_2x4x128_fullgamma_default_eps", None)])
def test_compiled_rmsnorm_matches_upstream_vectors(case, eps, zoo, tmp_path):
    import baybridge_b200 as cute

    vec = golden_vec(case)
    x, gamma = to_device(vec["in_x"], "bf16"), to_device(vec["in_gamma"], "bf16")
    out = device_zeros(vec["in_x"].shape, "bf16")
    artifact = cute.compile(zoo.make_rmsnorm(eps), x, out, gamma, backend="b200", cache_dir=tmp_path)
    assert artifact.ir.to_dict()["operations"] == golden_ir(case)["ir"]["operations"]
    artifact(x, out, gamma)
    got = to_host(out)
    assert oracle.rel_l2(got, vec["out_out"]) <= REL_L2
    assert int(ulp_distance(got, oracle.round_to_dtype(vec["out_out"], "bf16"), "bf16").max()) <= 1


@pytest.mark.parametrize("dtype,rows,hidden", [
    ("bf16", 3, 8), ("bf16", 5, 264), ("bf16", 257, 1000), ("bf16", 9, 4096), ("bf16", 4, 8192), ("bf16", 2, 16384),
    ("bf16", 2, 40000), ("f16", 7, 2048), ("f32", 6, 1020), ("f32", 3, 8192), ("f32", 2, 20000),
])
def test_c_abi_rmsnorm_shapes(dtype, rows, hidden):
    from baybridge_b200.backend import native

    rng = np.random.default_rng(rows * 100003 + hidden)
    x = oracle.round_to_dtype(rng.standard_normal((rows, hidden)), dtype)
    w = oracle.round_to_dtype(1 + 0.1 * rng.standard_normal(hidden), dtype)
    d_x, d_w, d_out = to_device(x, dtype), to_device(w, dtype), device_zeros((rows, hidden), dtype)
    native.call("bb200_rmsnorm", native.DTYPE_CODES[dtype], void_p(d_x), void_p(d_w), void_p(d_out), rows, hidden, 0,
                1e-6, current_stream())
    reference = oracle.rmsnorm(x, w, 1e-6)
    got = to_host(d_out)
    assert oracle.rel_l2(got, reference) <= (REL_L2 if dtype != "f32" else 1e-6)
    assert int(ulp_distance(got, oracle.round_to_dtype(reference, dtype), dtype).max()) <= (1 if dtype != "f32" else 4)


def test_c_abi_rmsnorm_rejects_bad_shapes():
    from baybridge_b200 import CudaDriverError
    from baybridge_b200.backend import native

    x = device_zeros((4, 12), "bf16")
    with pytest.raises(CudaDriverError) as info:  # 12 is not a multiple of the 8-element vector
        native.call("bb200_rmsnorm", 1, void_p(x), void_p(x), void_p(x), 4, 12, 0, 1e-6, current_stream())
    assert info.value.status == -2
    with pytest.raises(CudaDriverError):
        native.call("bb200_rmsnorm", 1, void_p(x), void_p(x), void_p(x), 0, 16, 0, 1e-6, current_stream())


def test_config4_full_size_rmsnorm(zoo, tmp_path):
    """65536 x 8192 bf16 through compile(); oracle evaluated in row chunks; plus a scale-invariance property:
    rmsnorm(2x) == rmsnorm(x) up to epsilon, which holds for any size."""
    import torch

    import baybridge_b200 as cute

    rows, hidden = 65536, 8192
    torch.manual_seed(1004)
    x = torch.randn((rows, hidden), device="cuda", dtype=torch.float32).to(torch.bfloat16)
    w = (1 + 0.1 * torch.randn((hidden,), device="cuda", dtype=torch.float32)).to(torch.bfloat16)
    out = torch.zeros_like(x)
    artifact = cute.compile(zoo.make_rmsnorm(1e-6), x, out, w, backend="b200", cache_dir=tmp_path)
    artifact(x, out, w)
    w_host = to_host(w)
    err2 = ref2 = 0.0
    for start in range(0, rows, 8192):
        reference = oracle.rmsnorm(to_host(x[start:start + 8192]), w_host, 1e-6)
        got = to_host(out[start:start + 8192])
        err2 += float(np.sum((got - reference) ** 2))
        ref2 += float(np.sum(reference**2))
    assert (err2 / ref2) ** 0.5 <= REL_L2
    doubled = torch.zeros_like(x)
    artifact(x * 2, doubled, w)
    # at most one bf16 unit in the last place apart (8 significant bits)
    assert bool(((doubled.float() - out.float()).abs() <= out.float().abs() * 2.0 ** -7).all())


def test_back_to_back_norm_launches_keep_stream_order():
    """The single-destination RMSNorm and LayerNorm kernels are launched with programmatic stream serialisation (their
    CTAs may be placed while the kernel before drains; ``griddepcontrol.wait`` holds them until its writes are visible).
    A chain in which every launch reads the rows the launch before wrote, without synchronisation, must give bit for bit
    what the same chain gives with a device synchronise after every launch."""
    import torch

    from baybridge_b200.backend import native

    rows, hidden = 16384, 2048  # 64 MB per tensor: many waves of CTAs per launch
    generator = torch.Generator(device="cuda").manual_seed(4242)
    x = torch.randn((rows, hidden), device="cuda", generator=generator).to(torch.bfloat16)
    weight = (1.0 + 0.25 * torch.randn((hidden,), device="cuda", generator=generator)).to(torch.bfloat16)
    bias = (0.1 * torch.randn((hidden,), device="cuda", generator=generator)).to(torch.bfloat16)
    residual = (0.5 * torch.randn((rows, hidden), device="cuda", generator=generator)).to(torch.bfloat16)
    code = native.DTYPE_CODES["bf16"]

    def chain(synchronise: bool):
        ping, pong, summed = x.clone(), torch.empty_like(x), torch.empty_like(x)
        torch.cuda.synchronize()
        stream = current_stream()
        for index in range(12):
            if index % 3 == 2:
                native.call("bb200_layernorm", code, void_p(ping), void_p(residual), void_p(weight), void_p(bias), void_p(pong),
                            void_p(summed), rows, hidden, 0, 0, 1e-5, stream)
            else:
                native.call("bb200_rmsnorm", code, void_p(ping), void_p(weight), void_p(pong), rows, hidden, 0, 1e-6, stream)
            if synchronise:
                torch.cuda.synchronize()
            ping, pong = pong, ping
        torch.cuda.synchronize()
        return ping

    assert torch.equal(chain(False), chain(True))
