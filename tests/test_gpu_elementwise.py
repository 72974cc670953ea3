"""GPU parity for the elementwise path: compile(..., backend="b200") and the C ABI vs the CPU oracle/golden vectors."""
from __future__ import annotations

import numpy as np
import pytest
from conftest import golden_cases, golden_ir, golden_vec
from gpu_util import current_stream, device_zeros, expect_rounded, to_device, to_host, torch_module, void_p

from oracle import cpu_runtime as oracle

pytestmark = pytest.mark.gpu

EXACT_OPS = {"add", "sub", "mul", "div", "max", "min", "neg", "abs", "copy", "sqrt", "floor", "ceil", "trunc"}


def _kernel_for(case: str, zoo):
    parts = case.split("_")
    if case.startswith("bin_"):
        return zoo.make_indexed_binary(parts[1], int(parts[2])), parts[1]
    if case.startswith("un_"):
        return zoo.make_indexed_unary(parts[1], int(parts[2])), parts[1]
    if case.startswith("clamp_scale"):
        return zoo.make_indexed_clamp_scale(512), "mul"
    if case.startswith("masked_add"):
        return zoo.make_indexed_masked_add(1000), "add"
    if case.startswith("ssa_"):
        return getattr(zoo, "_".join(parts[:-2])), "exp" if "exp" in case else "mul"
    if case.startswith("c2_fused_indexed"):
        return zoo.make_fused_mul_add_indexed(int(parts[3])), "fma"
    if case.startswith("c2_fused_ssa"):
        return zoo.fused_mul_add_ssa, "fma"
    families = {
        "bitwise": lambda: zoo.make_indexed_bitwise(parts[1], int(parts[2])), "cmpsel": lambda: zoo.make_indexed_compare_select(int(parts[1])),
        "ext1_indexed": lambda: zoo.make_indexed_extent1_scalar(int(parts[2])), "ext1_ssa": lambda: zoo.ssa_extent1_scalar,
        "bcast_rowcol": lambda: zoo.ssa_broadcast_row_col, "factory_bundle": lambda: zoo.factory_bundle,
    }
    for prefix, make in families.items():
        if case.startswith(prefix + "_"):
            return make(), "mul"  # integer ops, selects and single-rounded f32 arithmetic: exact
    raise KeyError(case)


ELEMENTWISE_CASES = [c for c in golden_cases() if c.startswith(
    ("bin_", "un_", "clamp_", "masked_", "ssa_", "c2_", "bitwise_", "cmpsel_", "ext1_", "bcast_", "factory_"))]


@pytest.mark.parametrize("case", ELEMENTWISE_CASES)
def test_compiled_elementwise_matches_upstream_vectors(case: str, zoo, tmp_path):
    import baybridge_b200 as cute

    ir = golden_ir(case)["ir"]
    vec = golden_vec(case)
    kernel, op = _kernel_for(case, zoo)
    args = []
    outputs = {}
    for argument in ir["arguments"]:
        name, spec = argument["name"], argument["spec"]
        if argument["kind"] == "scalar":
            args.append(0.75)
        elif f"in_{name}" in vec:
            args.append(to_device(vec[f"in_{name}"], spec["dtype"]))
        else:
            outputs[name] = device_zeros(spec["shape"], spec["dtype"])
            args.append(outputs[name])
    artifact = cute.compile(kernel, *args, backend="b200", cache_dir=tmp_path)
    assert json_equal(artifact.ir.to_dict(), ir)
    artifact(*args)
    for name, tensor in outputs.items():
        dtype = next(a["spec"]["dtype"] for a in ir["arguments"] if a["name"] == name)
        # arithmetic is bit-exact against the f64 reference rounded once; libm-style functions may differ
        # from CPython's libm by one unit in the last place of the storage type
        expect_rounded(to_host(tensor), vec[f"out_{name}"], dtype, max_ulp=0 if op in EXACT_OPS or op == "fma" and dtype == "f32" else 1)


def json_equal(mine: dict, theirs: dict) -> bool:
    import json

    return json.loads(json.dumps(mine)) == theirs


def test_config1_indexed_add_256x256_is_bit_exact(zoo, tmp_path):
    import baybridge_b200 as cute

    rng = np.random.default_rng(1001)
    a = rng.uniform(-1, 1, (256, 256)).astype(np.float32)
    b = rng.uniform(-1, 1, (256, 256)).astype(np.float32)
    g_a, g_b, g_c = to_device(a, "f32"), to_device(b, "f32"), device_zeros((256, 256), "f32")
    artifact = cute.compile(zoo.make_indexed_add_2d(256, 256), g_a, g_b, g_c, backend="b200", cache_dir=tmp_path)
    artifact(g_a, g_b, g_c)
    golden = golden_vec("c1_indexed_add_256x256_f32")["out_g_c"]
    assert np.array_equal(g_c.cpu().numpy(), golden)  # upstream CPU runtime output, bit for bit
    # eager launch path: kernel(...).launch(...) outside a trace compiles for b200 and runs on the device
    g_c.zero_()
    zoo.make_indexed_add_2d(256, 256)(g_a, g_b, g_c)
    assert np.array_equal(g_c.cpu().numpy(), golden)


@pytest.mark.parametrize("form", ["indexed", "ssa"])
def test_config2_full_size_fused_mul_add(form: str, zoo, tmp_path):
    """2^28 bf16 elements through compile(); checked chunk by chunk against the f64 oracle.

    Tolerance: RNE(f64 reference) within 1 bf16 ulp (f32 intermediates can double-round) and rel-L2 <= 2e-3."""
    import torch

    import baybridge_b200 as cute

    n = 2**28
    rng = np.random.default_rng(1002)
    a_host = oracle.bf16_round(rng.standard_normal(n, dtype=np.float32))
    b_host = oracle.bf16_round(rng.standard_normal(n, dtype=np.float32))
    a, b = to_device(a_host, "bf16"), to_device(b_host, "bf16")
    c = device_zeros((n,), "bf16")
    kernel = zoo.make_fused_mul_add_indexed(n) if form == "indexed" else zoo.fused_mul_add_ssa
    artifact = cute.compile(kernel, a, b, c, backend="b200", cache_dir=tmp_path)
    artifact(a, b, c)
    got = c.to(torch.float32).cpu().numpy()
    chunk = 2**24
    worst, err2, ref2, exact = 0, 0.0, 0.0, 0
    for start in range(0, n, chunk):
        av = a_host[start:start + chunk].astype(np.float64)
        bv = b_host[start:start + chunk].astype(np.float64)
        reference = av * bv + av
        expected = oracle.round_to_dtype(reference, "bf16")
        piece = got[start:start + chunk].astype(np.float64)
        from gpu_util import ulp_distance

        distance = ulp_distance(piece, expected, "bf16")
        worst = max(worst, int(distance.max()))
        exact += int(np.count_nonzero(distance == 0))
        err2 += float(np.sum((piece - reference) ** 2))
        ref2 += float(np.sum(reference**2))
    assert worst <= 1, f"worst error {worst} bf16 ulp"
    assert exact / n > 0.999
    assert (err2 / ref2) ** 0.5 <= 2e-3


@pytest.mark.parametrize("dtype,n", [("f32", 1_000_003), ("bf16", 999_999), ("f16", 12_345), ("bf16", 7), ("f32", 1)])
def test_c_abi_binary_and_mul_add_ragged_sizes(dtype: str, n: int):
    """Sizes that are not multiples of the vector width or tile, through the C ABI directly."""
    from baybridge_b200.backend import native

    rng = np.random.default_rng(n)
    x = oracle.round_to_dtype(rng.uniform(0.5, 2.0, n), dtype)
    y = oracle.round_to_dtype(rng.uniform(0.5, 2.0, n), dtype)
    a, b, c = to_device(x, dtype), to_device(y, dtype), device_zeros((n,), dtype)
    code = native.DTYPE_CODES[dtype]
    reference = {"add": x + y, "sub": x - y, "mul": x * y, "div": x / y, "max": np.maximum(x, y), "min": np.minimum(x, y)}
    for op, expected in reference.items():
        c.zero_()
        native.call("bb200_elementwise_binary", native.BINARY_OP_CODES[op], code, void_p(a), void_p(b), void_p(c), n, current_stream())
        expect_rounded(to_host(c), expected, dtype)
    c.zero_()
    native.call("bb200_elementwise_mul_add", code, void_p(a), void_p(b), void_p(c), n, current_stream())
    expect_rounded(to_host(c), x * y + x, dtype, max_ulp=0 if dtype == "f32" else 1)


def test_c_abi_unaligned_pointers_take_the_scalar_path():
    from baybridge_b200.backend import native

    n = 4099
    rng = np.random.default_rng(5)
    x = rng.uniform(-1, 1, n + 1).astype(np.float32)
    y = rng.uniform(-1, 1, n + 1).astype(np.float32)
    a, b, c = to_device(x, "f32"), to_device(y, "f32"), device_zeros((n + 1,), "f32")
    # views that start 4 bytes into the allocation: not 16-byte aligned
    native.call("bb200_elementwise_binary", 0, 0, void_p(a[1:]), void_p(b[1:]), void_p(c[1:]), n, current_stream())
    out = c.cpu().numpy()
    assert out[0] == 0.0 and np.array_equal(out[1:], x[1:] + y[1:])


def test_c_abi_rejects_bad_arguments():
    from baybridge_b200 import CudaDriverError
    from baybridge_b200.backend import native

    a = device_zeros((16,), "f32")
    with pytest.raises(CudaDriverError) as info:
        native.call("bb200_elementwise_binary", 99, 0, void_p(a), void_p(a), void_p(a), 16, current_stream())
    assert info.value.status == -1
    with pytest.raises(CudaDriverError):
        native.call("bb200_elementwise_binary", 0, 0, None, void_p(a), void_p(a), 16, current_stream())
    native.call("bb200_elementwise_binary", 0, 0, void_p(a), void_p(a), void_p(a), 0, current_stream())  # empty is a no-op


def test_runtime_tensor_arguments_are_staged_and_copied_back(zoo, tmp_path):
    import baybridge_b200 as cute

    a = cute.tensor([float(i) for i in range(128)], dtype="f32")
    b = cute.tensor([float(i * 2) for i in range(128)], dtype="f32")
    c = cute.zeros((128,), dtype="f32")
    artifact = cute.compile(zoo.make_indexed_binary("add", 128), a, b, c, backend="b200", cache_dir=tmp_path)
    with pytest.warns(RuntimeWarning, match="staging"):
        artifact(a, b, c)
    assert c.tolist() == [x + y for x, y in zip(a.tolist(), b.tolist())]  # upstream tests/test_backend_ptx_exec.py:2660-2677


# ---- bodies whose indexing is not the identity: lowered literally (one device thread per traced thread) ----
def _run_against_oracle(kernel, host_arrays: dict, dtypes: dict, tmp_path, scalars=()):
    """Compile for b200 with device tensors, run, and compare every tensor with the oracle's interpretation of
    the very IR that was compiled (bit-exact after one rounding to the storage dtype)."""
    import baybridge_b200 as cute

    device = {name: to_device(value, dtypes[name]) for name, value in host_arrays.items()}
    args = list(device.values()) + list(scalars)
    artifact = cute.compile(kernel, *args, backend="b200", cache_dir=tmp_path)
    artifact(*args)
    expected = {name: np.array(value, dtype=np.float64) for name, value in host_arrays.items()}
    names = [argument.name for argument in artifact.ir.arguments]
    oracle_args = dict(expected)
    for name, value in zip(names[len(host_arrays):], scalars):
        oracle_args[name] = value
    oracle.run_kernel_ir(artifact.ir.to_dict(), oracle_args)
    for name in host_arrays:
        expect_rounded(to_host(device[name]), expected[name], dtypes[name])
    return artifact


def test_literal_lowering_reversed_and_strided_indices(tmp_path):
    import baybridge_b200 as cute

    n = 1000

    @cute.kernel(launch=cute.LaunchConfig(grid=(8, 1, 1), block=(128, 1, 1)))
    def reverse_scale(src: cute.Tensor, dst: cute.Tensor):
        i = cute.block_idx("x") * cute.block_dim("x") + cute.thread_idx("x")
        inside = i < n
        value = cute.load(src, (n - 1) - i, predicate=inside, else_value=0.0)
        cute.store(value * 3.0 - 1.0, dst, i, predicate=inside)

    rng = np.random.default_rng(21)
    artifact = _run_against_oracle(reverse_scale, {"src": rng.uniform(-1, 1, n).astype(np.float32), "dst": np.zeros(n, np.float32)},
                                   {"src": "f32", "dst": "f32"}, tmp_path)
    assert artifact.runtime_callable is not None
    from baybridge_b200.backend.matcher import match

    assert match(artifact.ir).mode == "literal"

    @cute.kernel(launch=cute.LaunchConfig(grid=(4, 1, 1), block=(64, 1, 1)))
    def gather_even(src: cute.Tensor, dst: cute.Tensor):
        i = cute.block_idx("x") * cute.block_dim("x") + cute.thread_idx("x")
        dst[i] = src[i * 2] + src[i * 2 + 1]

    _run_against_oracle(gather_even, {"src": oracle.bf16_round(rng.standard_normal(512).astype(np.float32)), "dst": np.zeros(256, np.float32)},
                        {"src": "bf16", "dst": "bf16"}, tmp_path)


def test_two_dimensional_launch_with_scalar_argument(tmp_path):
    import baybridge_b200 as cute

    rows, cols = 48, 80

    @cute.kernel(launch=cute.LaunchConfig(grid=(5, 3, 1), block=(16, 16, 1)))
    def saxpy_2d(x: cute.Tensor, y: cute.Tensor, out: cute.Tensor, alpha: float):
        col = cute.block_idx("x") * cute.block_dim("x") + cute.thread_idx("x")
        row = cute.block_idx("y") * cute.block_dim("y") + cute.thread_idx("y")
        out[row, col] = x[row, col] * alpha + y[row, col]

    rng = np.random.default_rng(22)
    _run_against_oracle(
        saxpy_2d,
        {"x": rng.uniform(-1, 1, (rows, cols)).astype(np.float32), "y": rng.uniform(-1, 1, (rows, cols)).astype(np.float32),
         "out": np.zeros((rows, cols), np.float32)},
        {"x": "f32", "y": "f32", "out": "f32"}, tmp_path, scalars=(0.1,),  # 0.1 is not an f32: the f64 path keeps it exact
    )


def test_multi_dimensional_launches_flat_when_one_shared_bijection_else_literal(tmp_path):
    import baybridge_b200 as cute
    from baybridge_b200.backend.matcher import match

    rng = np.random.default_rng(24)
    rows, cols = 48, 80

    # covers [48, 80] exactly with one thread per element and the same (row, col) in every access: vectorised form
    @cute.kernel(launch=cute.LaunchConfig(grid=(5, 3, 1), block=(16, 16, 1)))
    def scale_shift_2d(x: cute.Tensor, out: cute.Tensor):
        col = cute.block_idx("x") * cute.block_dim("x") + cute.thread_idx("x")
        row = cute.block_idx("y") * cute.block_dim("y") + cute.thread_idx("y")
        value = x[row, col]
        out[row, col] = value * value + value

    artifact = _run_against_oracle(scale_shift_2d, {"x": oracle.bf16_round(rng.standard_normal((rows, cols)).astype(np.float32)),
                                                    "out": np.zeros((rows, cols), np.float32)}, {"x": "bf16", "out": "bf16"}, tmp_path)
    assert match(artifact.ir).mode == "flat"

    # three launch axes onto a rank-3 tensor
    @cute.kernel(launch=cute.LaunchConfig(grid=(2, 5, 6), block=(8, 2, 1)))
    def add_3d(a: cute.Tensor, b: cute.Tensor, c: cute.Tensor):
        x = cute.block_idx("x") * cute.block_dim("x") + cute.thread_idx("x")
        y = cute.block_idx("y") * cute.block_dim("y") + cute.thread_idx("y")
        z = cute.block_idx("z")
        c[z, y, x] = a[z, y, x] + b[z, y, x]

    shape = (6, 10, 16)
    artifact = _run_against_oracle(add_3d, {"a": rng.uniform(-1, 1, shape).astype(np.float32), "b": rng.uniform(-1, 1, shape).astype(np.float32),
                                            "c": np.zeros(shape, np.float32)}, {"a": "f32", "b": "f32", "c": "f32"}, tmp_path)
    assert match(artifact.ir).mode == "flat"

    # a 1-D launch walking a row-major tensor column by column: a permutation, still one shared map
    @cute.kernel(launch=cute.LaunchConfig(grid=(15, 1, 1), block=(256, 1, 1)))
    def column_walk(a: cute.Tensor, c: cute.Tensor):
        i = cute.block_idx("x") * cute.block_dim("x") + cute.thread_idx("x")
        c[i % 48, i // 48] = cute.math.exp(a[i % 48, i // 48])

    artifact = _run_against_oracle(column_walk, {"a": rng.uniform(-1, 1, (rows, cols)).astype(np.float32), "c": np.zeros((rows, cols), np.float32)},
                                   {"a": "f32", "c": "f32"}, tmp_path)
    assert match(artifact.ir).mode == "flat"

    # the transposed write uses two different maps: literal lowering
    @cute.kernel(launch=cute.LaunchConfig(grid=(5, 3, 1), block=(16, 16, 1)))
    def transpose_2d(a: cute.Tensor, c: cute.Tensor):
        col = cute.block_idx("x") * cute.block_dim("x") + cute.thread_idx("x")
        row = cute.block_idx("y") * cute.block_dim("y") + cute.thread_idx("y")
        c[col, row] = a[row, col]

    artifact = _run_against_oracle(transpose_2d, {"a": rng.uniform(-1, 1, (rows, cols)).astype(np.float32), "c": np.zeros((cols, rows), np.float32)},
                                   {"a": "f32", "c": "f32"}, tmp_path)
    assert match(artifact.ir).mode == "literal"


@pytest.mark.parametrize("dtype,shape", [("bf16", (512, 1024)), ("f32", (300, 4096)), ("f32", (37, 50)), ("f16", (64, 24))])
def test_broadcast_operands_row_vector_column_vector_and_one_element_tensor(dtype, shape, zoo, tmp_path):
    """(a + row) * col with row [1, C] and col [R, 1], then + alpha[0]: the vector path fetches the row operand with
    16-byte loads and the column operand once per step; odd widths take the element-by-element path."""
    import baybridge_b200 as cute
    from baybridge_b200.backend.matcher import match

    rng = np.random.default_rng(shape[0] * 131 + shape[1])
    rows, cols = shape
    host = {
        "a": oracle.round_to_dtype(rng.uniform(-1, 1, shape), dtype), "row": oracle.round_to_dtype(rng.uniform(-1, 1, (1, cols)), dtype),
        "col": oracle.round_to_dtype(rng.uniform(-1, 1, (rows, 1)), dtype), "c": np.zeros(shape),
    }
    artifact = _run_against_oracle(zoo.ssa_broadcast_row_col, host, {name: dtype for name in host}, tmp_path)
    plan = match(artifact.ir)
    assert plan.mode == "flat" and plan.inputs == (0,) and plan.gathers == (1, 2)

    @cute.kernel
    def scaled_shift(a: cute.Tensor, row: cute.Tensor, alpha: cute.Tensor, c: cute.Tensor):
        c.store(a.load() * alpha[0] - row.load())

    host = {"a": host["a"], "row": host["row"], "alpha": oracle.round_to_dtype(np.array([0.625]), dtype), "c": np.zeros(shape)}
    _run_against_oracle(scaled_shift, host, {name: dtype for name in host}, tmp_path)


def test_flat_lowering_rank3_digits_and_in_place_update(tmp_path):
    import baybridge_b200 as cute

    shape = (6, 10, 16)
    total = 6 * 10 * 16

    @cute.kernel(launch=cute.LaunchConfig(grid=((total + 127) // 128, 1, 1), block=(128, 1, 1)))
    def rank3_inplace(t: cute.Tensor, bias: cute.Tensor):
        i = cute.block_idx("x") * cute.block_dim("x") + cute.thread_idx("x")
        inside = i < total
        a = i // 160
        b = (i // 16) % 10
        c = i % 16
        value = cute.load(t, (a, b, c), predicate=inside, else_value=0.0)
        other = cute.load(bias, (a, b, c), predicate=inside, else_value=0.0)
        cute.store(cute.math.sqrt(value * value + other * other), t, (a, b, c), predicate=inside)

    rng = np.random.default_rng(23)
    artifact = _run_against_oracle(rank3_inplace, {"t": rng.uniform(0.5, 2, shape).astype(np.float32), "bias": rng.uniform(0.5, 2, shape).astype(np.float32)},
                                   {"t": "f32", "bias": "f32"}, tmp_path)
    from baybridge_b200.backend.matcher import match

    plan = match(artifact.ir)
    assert plan.mode == "flat" and plan.extent == total  # (i//160, (i//16)%10, i%16) on [6,10,16] is proved to be offset i


def test_back_to_back_dependent_launches_keep_stream_order(zoo, tmp_path):
    """Flat elementwise kernels are launched with programmatic stream serialisation: a kernel's CTAs may be placed
    while the kernel before it drains, and ``griddepcontrol.wait`` holds them until its writes are visible.  A chain of
    adds in which every launch reads what the launch before wrote (no synchronisation in between, buffers much larger
    than what one wave of CTAs covers), with a library kernel of another framework in the middle of the chain, must
    give exactly the serial result."""
    import baybridge_b200 as cute
    from baybridge_b200 import B200Backend

    torch = torch_module()
    n = 1 << 23
    rng = np.random.default_rng(77)
    start = rng.integers(-64, 64, n).astype(np.float32)
    step = rng.integers(-8, 8, n).astype(np.float32)
    g_step = to_device(step, "f32")
    ping, pong = to_device(start, "f32"), device_zeros((n,), "f32")
    kernel = zoo.make_indexed_binary("add", n)
    artifact = cute.compile(kernel, ping, g_step, pong, backend=B200Backend(synchronize=False), cache_dir=tmp_path)
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    launches = 24
    with torch.cuda.stream(stream):
        handles = {id(t): cute.from_dlpack(t) for t in (ping, pong, g_step)}
        source, destination = ping, pong
        for index in range(launches):
            artifact(handles[id(source)], handles[id(g_step)], handles[id(destination)], stream=stream.cuda_stream)
            source, destination = destination, source
            if index == launches // 2 - 1:
                source.add_(1.0)  # a torch kernel between two of ours, on the same stream
    stream.synchronize()
    expected = start + launches * step + 1.0  # small integers: every partial sum is exact in f32
    assert np.array_equal(source.cpu().numpy(), expected)


def test_dependent_launches_see_a_cached_operand_rewritten_by_the_kernel_before(zoo, tmp_path):
    """The row vector of a broadcast is fetched with ordinary cached loads (it is shared by every row).  Alternate a
    kernel that uses it with a kernel that rewrites it, back to back and unsynchronised: every use must see the value
    the launch before it stored, although its CTAs may have been placed before that launch had finished."""
    import baybridge_b200 as cute
    from baybridge_b200 import B200Backend

    torch = torch_module()
    rows, cols = 2048, 4096
    rng = np.random.default_rng(78)
    a = rng.integers(-16, 16, (rows, cols)).astype(np.float32)
    row = rng.integers(-4, 4, (1, cols)).astype(np.float32)
    col = np.ones((rows, 1), dtype=np.float32)
    one = np.ones((1, cols), dtype=np.float32)
    g_a, g_row, g_col, g_one = (to_device(v, "f32") for v in (a, row, col, one))
    g_next, g_out = device_zeros((1, cols), "f32"), device_zeros((rows, cols), "f32")
    backend = B200Backend(synchronize=False)
    use = cute.compile(zoo.ssa_broadcast_row_col, g_a, g_row, g_col, g_out, backend=backend, cache_dir=tmp_path)

    @cute.kernel
    def bump(src: cute.Tensor, step: cute.Tensor, dst: cute.Tensor):
        dst.store(src.load() + step.load())

    bump_artifact = cute.compile(bump, g_row, g_one, g_next, backend=backend, cache_dir=tmp_path)
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    handle = {id(t): cute.from_dlpack(t) for t in (g_a, g_row, g_col, g_one, g_next, g_out)}
    rounds = 10
    with torch.cuda.stream(stream):
        current, spare = g_row, g_next
        for _ in range(rounds):
            use(handle[id(g_a)], handle[id(current)], handle[id(g_col)], handle[id(g_out)], stream=stream.cuda_stream)
            bump_artifact(handle[id(current)], handle[id(g_one)], handle[id(spare)], stream=stream.cuda_stream)
            current, spare = spare, current
        use(handle[id(g_a)], handle[id(current)], handle[id(g_col)], handle[id(g_out)], stream=stream.cuda_stream)
    stream.synchronize()
    assert np.array_equal(g_out.cpu().numpy(), a + (row + rounds))
    assert np.array_equal(current.cpu().numpy(), row + rounds)
