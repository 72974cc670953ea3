"""Host-side mirror of the DSL: tracing, IR parity with upstream listings, compile cache, registry, interop.

These mirror upstream's CPU-only test tiers (tests/test_api.py, test_elementwise.py, test_cache.py,
test_interop.py, test_backend_ptx_exec.py's fake-DLPack launcher tests) for the b200 path.
"""

import json
import os
import sys
from pathlib import Path

import pytest
from conftest import GOLDEN, golden_ir, sample_scalar, zoo_kernel

import baybridge_b200 as cute
from baybridge_b200.backend.matcher import match
from baybridge_b200.driver import cache_key_for
from baybridge_b200.portable_ir import PortableKernelIR

TARGET = cute.NvidiaTarget("sm_100a", "8.8")


class FakeCudaTensor:
    """DLPack-looking device tensor (upstream tests/test_backend_ptx_exec.py:2557-2576)."""

    def __init__(self, shape, dtype, ptr=4096, device=(2, 0), stride=None):
        self.shape, self.dtype, self._ptr, self._device, self._stride = tuple(shape), dtype, ptr, device, stride
        self.dlpack_streams = []

    def __dlpack__(self, stream=None):
        self.dlpack_streams.append(stream)
        return "capsule"

    def __dlpack_device__(self):
        return self._device

    def data_ptr(self):
        return self._ptr

    def stride(self):
        return self._stride


def _carriers(ir: dict, case: str = ""):
    names = {"f32": "float32", "bf16": "bfloat16", "f16": "float16", "i32": "int32", "i1": "bool"}
    out = []
    for argument in ir["arguments"]:
        if argument["kind"] == "scalar":
            out.append(sample_scalar(cute, case, argument))
        else:
            out.append(FakeCudaTensor(argument["spec"]["shape"], names[argument["spec"]["dtype"]]))
    return out


ALL_IR_CASES = sorted(path.stem[3:] for path in GOLDEN.glob("ir_*.json"))


@pytest.mark.parametrize("case", ALL_IR_CASES)
def test_traced_ir_and_cache_key_equal_upstream(case, zoo, tmp_path):
    """Same kernel body traced here and by upstream → identical IR dict and identical sha256 cache key."""
    golden = golden_ir(case)
    artifact = cute.compile(zoo_kernel(case, zoo), *_carriers(golden["ir"], case), backend="portable", cache_dir=tmp_path, target=TARGET)
    assert json.loads(json.dumps(artifact.ir.to_dict())) == golden["ir"]
    assert cache_key_for(artifact.ir, TARGET, "b200") == golden["cache_key_b200_sm100a"]
    assert PortableKernelIR.from_dict(golden["ir"]).to_dict() == golden["ir"]


@pytest.mark.parametrize("case", ALL_IR_CASES)
def test_matcher_classifies_every_listing(case):
    if case.startswith("api_tile_mma"):
        # an mma on a corner tile into a discarded register accumulator has no whole-GEMM meaning: refused, not guessed
        with pytest.raises(cute.BackendNotImplementedError, match="partition at a fixed offset"):
            match(PortableKernelIR.from_dict(golden_ir(case)["ir"]))
        return
    plan = match(PortableKernelIR.from_dict(golden_ir(case)["ir"]))
    if case.startswith(("c3_", "gemm_")):
        assert plan.kind == "gemm"
    elif case.startswith(("c4_", "rmsnorm_")):
        assert plan.kind == "rmsnorm"
    elif case.startswith("layernorm_"):
        assert plan.kind == "layernorm"
    elif case.startswith("rbundle_"):
        assert plan.kind == "reduction_bundle" and [part.form for part in plan.parts] == ["all", "rows", "cols"]
    elif case.startswith("rarg_"):
        assert plan.kind == "reduction" and plan.form == "all"
    elif case.startswith("reduce_"):
        assert plan.kind == "reduction" and plan.form == {"row": "rows", "col": "cols", "total": "all"}[case.split("_")[1]]
    elif case.startswith(("c5_", "attn_")):
        assert plan.kind == "attention"
    elif case.startswith("padded_"):
        # a guarded load feeding an unguarded store: elements past the bound receive f(else_value), so the flat map runs
        # over the stored extent (not `i < bound`) and the guarded input carries its bound and fallback
        assert plan.kind == "elementwise" and plan.mode == "flat" and plan.extent == 1024
        (guarded,) = [node for node in plan.nodes if node.op == "input"]
        assert guarded.attrs["bound"] == 512 and len(guarded.operands) == 1
    elif case.startswith("sw_reduce_"):
        assert plan.kind == "reduction" and plan.form == case.split("_")[2]
    else:
        assert plan.kind == "elementwise" and plan.mode == "flat"  # every zoo body is an index bijection


def test_config_plans_carry_the_expected_shapes():
    gemm = match(PortableKernelIR.from_dict(golden_ir("c3_gemm_abt_8192_bf16")["ir"]))
    assert (gemm.m, gemm.n, gemm.k, gemm.transpose_a, gemm.transpose_b, gemm.c_dtype) == (8192, 8192, 8192, False, True, "bf16")
    norm = match(PortableKernelIR.from_dict(golden_ir("c4_rmsnorm_65536x8192_bf16")["ir"]))
    assert (norm.rows, norm.hidden, norm.gamma_is_full, norm.epsilon) == (65536, 8192, False, 1e-6)
    attn = match(PortableKernelIR.from_dict(golden_ir("c5_attn_causal_b16s4096h32d128")["ir"]))
    assert (attn.batch, attn.seq, attn.heads, attn.kv_heads, attn.head_dim, attn.causal) == (16, 4096, 32, 32, 128, True)
    fused = match(PortableKernelIR.from_dict(golden_ir("c2_fused_indexed_2p28_bf16")["ir"]))
    assert fused.extent == 2**28 and fused.inputs == (0, 1)  # the repeated load of `a` is merged
    c1 = match(PortableKernelIR.from_dict(golden_ir("c1_indexed_add_256x256_f32")["ir"]))
    assert c1.extent == 65536  # (i // 256, i % 256) on a row-major 256x256 tensor is proved to be offset i


def test_non_bijective_indexing_is_lowered_literally_and_unknown_ops_are_rejected(tmp_path):
    @cute.kernel(launch=cute.LaunchConfig(grid=(4, 1, 1), block=(64, 1, 1)))
    def reverse(src: cute.TensorSpec(shape=(256,), dtype="f32"), dst: cute.TensorSpec(shape=(256,), dtype="f32")):
        i = cute.block_idx("x") * cute.block_dim("x") + cute.thread_idx("x")
        dst[255 - i] = src[i]

    artifact = cute.compile(reverse, backend="portable", cache_dir=tmp_path)
    plan = match(artifact.ir)
    assert plan.mode == "literal"

    @cute.kernel(launch=cute.LaunchConfig(grid=(2, 2, 1), block=(16, 16, 1)))
    def add_2d_launch(a: cute.TensorSpec(shape=(32, 32), dtype="f32"), c: cute.TensorSpec(shape=(32, 32), dtype="f32")):
        col = cute.block_idx("x") * cute.block_dim("x") + cute.thread_idx("x")
        row = cute.block_idx("y") * cute.block_dim("y") + cute.thread_idx("y")
        c[row, col] = a[row, col] + 1.0

    # a 2-D launch that covers the tensor exactly, every access at the same (row, col): one shared one-to-one map,
    # so it is an elementwise map whatever the visiting order and takes the vectorised form
    covered = match(cute.compile(add_2d_launch, backend="portable", cache_dir=tmp_path).ir)
    assert covered.mode == "flat" and covered.extent == 1024

    # the same launch writing the transposed position: two different maps, lowered literally (one device thread
    # per traced thread, traced index arithmetic)
    @cute.kernel(launch=cute.LaunchConfig(grid=(2, 2, 1), block=(16, 16, 1)))
    def transpose_2d_launch(a: cute.TensorSpec(shape=(32, 32), dtype="f32"), c: cute.TensorSpec(shape=(32, 32), dtype="f32")):
        col = cute.block_idx("x") * cute.block_dim("x") + cute.thread_idx("x")
        row = cute.block_idx("y") * cute.block_dim("y") + cute.thread_idx("y")
        c[col, row] = a[row, col]

    assert match(cute.compile(transpose_2d_launch, backend="portable", cache_dir=tmp_path).ir).mode == "literal"
    lowered = cute.compile(transpose_2d_launch, backend="b200", cache_dir=tmp_path)  # lowering + nvcc need no GPU
    assert "blockIdx.y" in json.loads(lowered.lowered_module.text)["source"]

    # a grid larger than the tensor (no guard) is not a one-to-one map onto it: literal
    @cute.kernel(launch=cute.LaunchConfig(grid=(4, 2, 1), block=(16, 16, 1)))
    def oversized_2d_launch(a: cute.TensorSpec(shape=(32, 32), dtype="f32"), c: cute.TensorSpec(shape=(32, 32), dtype="f32")):
        col = cute.block_idx("x") * cute.block_dim("x") + cute.thread_idx("x")
        row = cute.block_idx("y") * cute.block_dim("y") + cute.thread_idx("y")
        c[row, col] = a[row, col] + 1.0

    assert match(cute.compile(oversized_2d_launch, backend="portable", cache_dir=tmp_path).ir).mode == "literal"

    # a 1-D launch that visits the elements in a permuted order (column-major walk of a row-major tensor) with the
    # same map for every access is still an elementwise map
    @cute.kernel(launch=cute.LaunchConfig(grid=(4, 1, 1), block=(256, 1, 1)))
    def column_major_walk(a: cute.TensorSpec(shape=(32, 32), dtype="f32"), c: cute.TensorSpec(shape=(32, 32), dtype="f32")):
        i = cute.block_idx("x") * cute.block_dim("x") + cute.thread_idx("x")
        c[i % 32, i // 32] = a[i % 32, i // 32] * 2.0

    assert match(cute.compile(column_major_walk, backend="portable", cache_dir=tmp_path).ir).mode == "flat"

    @cute.kernel
    def two_ops(a: cute.TensorSpec(shape=(64, 64), dtype="bf16"), b: cute.TensorSpec(shape=(64, 64), dtype="bf16"),
                c: cute.TensorSpec(shape=(64, 64), dtype="bf16")):
        cute.gemm(a, b, c, transpose_b=True)
        cute.rmsnorm(c, c, a)

    with pytest.raises(cute.BackendNotImplementedError, match="only op"):
        cute.compile(two_ops, backend="b200", cache_dir=tmp_path)


def test_program_tiled_gemm_lowers_to_the_whole_gemm_or_is_refused(zoo, tmp_path):
    spec = lambda rows, cols, dtype="bf16": cute.TensorSpec(shape=(rows, cols), dtype=dtype)  # noqa: E731

    carriers = [FakeCudaTensor(shape, "bfloat16") for shape in ((256, 128), (512, 128), (256, 512))]
    plan = match(cute.compile(zoo.make_tiled_gemm(256, 512, 128, 64, 128), *carriers, backend="portable", cache_dir=tmp_path).ir)
    assert (plan.kind, plan.m, plan.n, plan.k, plan.transpose_b) == ("gemm", 256, 512, 128, True)
    lowered = cute.compile(zoo.make_tiled_gemm(256, 512, 128, 64, 128), *carriers, backend="b200", cache_dir=tmp_path)
    assert lowered.lowered_module.entry_point == "bb200_gemm_bf16"

    # the grid leaves rows of C uncovered: not a whole GEMM
    @cute.kernel(launch=cute.LaunchConfig(grid=(3, 4, 1), block=(1, 1, 1)))
    def short_grid(a: spec(256, 128), b: spec(512, 128), c: spec(256, 512)):
        cute.gemm(cute.partition_program(a, (64, 128), axes=("x", "z")), cute.partition_program(b, (128, 128), axes=("y", "z")),
                  cute.partition_program(c, (64, 128), axes=("x", "y")), transpose_b=True)

    with pytest.raises(cute.BackendNotImplementedError, match="must tile axis 0"):
        cute.compile(short_grid, backend="b200", cache_dir=tmp_path)

    # programs along z each take a slice of K and overwrite C: split-K is not a GEMM
    @cute.kernel(launch=cute.LaunchConfig(grid=(4, 4, 2), block=(1, 1, 1)))
    def split_k(a: spec(256, 128), b: spec(512, 128), c: spec(256, 512)):
        cute.gemm(cute.partition_program(a, (64, 64), axes=("x", "z")), cute.partition_program(b, (128, 64), axes=("y", "z")),
                  cute.partition_program(c, (64, 128), axes=("x", "y")), transpose_b=True)

    with pytest.raises(cute.BackendNotImplementedError, match="whole K extent"):
        cute.compile(split_k, backend="b200", cache_dir=tmp_path)

    # A rows follow program x but C rows follow program y
    @cute.kernel(launch=cute.LaunchConfig(grid=(4, 4, 1), block=(1, 1, 1)))
    def crossed(a: spec(256, 128), b: spec(256, 128), c: spec(256, 256)):
        cute.gemm(cute.partition_program(a, (64, 128), axes=("x", "z")), cute.partition_program(b, (64, 128), axes=("y", "z")),
                  cute.partition_program(c, (64, 64), axes=("y", "x")), transpose_b=True)

    with pytest.raises(cute.BackendNotImplementedError, match="do not line up"):
        cute.compile(crossed, backend="b200", cache_dir=tmp_path)


def test_compile_hits_cache_and_writes_manifest(zoo, tmp_path):
    carriers = _carriers(golden_ir("c2_fused_indexed_4096_bf16")["ir"])
    kernel = zoo.make_fused_mul_add_indexed(4096)
    first = cute.compile(kernel, *carriers, backend="b200", cache_dir=tmp_path)
    second = cute.compile(kernel, *carriers, backend="b200", cache_dir=tmp_path)
    assert first.cache_key == second.cache_key and not first.from_cache and second.from_cache
    assert first.artifact_path == tmp_path / "b200" / "sm_100a" / f"{first.cache_key}.json"
    manifest = json.loads(first.artifact_path.read_text())
    assert manifest["backend_name"] == "b200" and manifest["ir"] == json.loads(json.dumps(first.ir.to_dict()))
    assert first.lowered_path.exists() and first.lowered_module.dialect == "b200.plan"
    other = cute.compile(zoo.make_fused_mul_add_indexed(8192), *[FakeCudaTensor((8192,), "bfloat16")] * 3, backend="b200", cache_dir=tmp_path)
    assert other.cache_key != first.cache_key  # shapes and launch dims are part of the key


def test_registry_and_errors(tmp_path, zoo):
    assert {"b200", "portable"} <= set(cute.registered_backends())
    with pytest.raises(cute.CompilationError, match="unknown backend 'ptx_exec'"):
        cute.compile(zoo.ssa_add, *[FakeCudaTensor((8, 8), "float32")] * 3, backend="ptx_exec", cache_dir=tmp_path)
    portable = cute.compile(zoo.ssa_add, *[FakeCudaTensor((8, 8), "float32")] * 3, backend="portable", cache_dir=tmp_path)
    with pytest.raises(cute.BackendNotImplementedError):  # IR-only artifact: nothing to launch, and no CPU runtime
        portable(*[FakeCudaTensor((8, 8), "float32")] * 3)
    with pytest.raises(cute.BackendNotImplementedError, match="sm_100a"):
        cute.compile(zoo.ssa_add, *[FakeCudaTensor((8, 8), "float32")] * 3, backend="b200", cache_dir=tmp_path,
                     target=cute.NvidiaTarget("sm_80", "8.0"))
    sentinel = object()
    cute.register_backend("custom_probe", lambda: None)
    assert "custom_probe" in cute.registered_backends() and sentinel is not None
    with pytest.raises(cute.CompilationError):
        @cute.kernel
        def branchy(a: cute.TensorSpec(shape=(8,), dtype="f32")):
            if cute.thread_idx("x") > 0:  # data-dependent Python control flow cannot be traced
                a[0] = a[0]

        cute.compile(branchy, backend="portable", cache_dir=tmp_path)


def test_host_tensors_are_containers_not_a_cpu_runtime():
    a = cute.tensor([[1, 2, 3], [4, 5, 6]], dtype="f32")
    assert a.shape == (2, 3) and a.tolist() == [[1, 2, 3], [4, 5, 6]] and a[1, 2] == 6
    assert cute.tensor([1.5, 2]).dtype == "f32" and cute.tensor([1, 2]).dtype == "index" and cute.tensor([True]).dtype == "i1"
    with pytest.raises(cute.BackendNotImplementedError):
        a + a
    with pytest.raises(cute.BackendNotImplementedError):
        cute.gemm(a, a, a)
    bf = cute.tensor([1.00390625, 1.01171875], dtype="bf16")  # ties: RNE on the upper half of the f32 pattern
    assert list(bf.device_image()) == [0x3F80, 0x3F82]
    assert cute.Float32(3).value == 3.0 and cute.Int32(2**31 + 5).value == -(2**31) + 5


def test_launcher_contract_without_a_device(zoo, tmp_path):
    """Arity/kwarg checks come first; then the launcher refuses loudly because no CUDA device exists here."""
    from baybridge_b200.backend import native

    carriers = [FakeCudaTensor((1024,), "float32") for _ in range(3)]
    artifact = cute.compile(zoo.make_indexed_binary("add", 1024), *carriers, backend="b200", cache_dir=tmp_path)
    launcher = cute.B200Backend().build_launcher(artifact.ir, TARGET, artifact.lowered_module, artifact.lowered_path)
    with pytest.raises(TypeError, match="expects 3 arguments, got 2"):
        launcher(*[cute.from_dlpack(c) for c in carriers[:2]])
    with pytest.raises(TypeError, match="optional stream="):
        launcher(*[cute.from_dlpack(c) for c in carriers], block=1)
    if not native.device_available():
        with pytest.raises(cute.BackendNotImplementedError, match="CUDA device"):
            artifact(*carriers)
    # stream= is forwarded into __dlpack__ when arguments are normalised (upstream compiler.py:63-74)
    try:
        artifact(*carriers, stream=77)
    except cute.BaybridgeError:
        pass
    assert 77 in carriers[0].dlpack_streams


def test_launch_graph_state_without_a_device():
    """Recording needs a device (no CPU stand-in); while a graph records, DLPack exporters are not handed the stream."""
    from baybridge_b200 import launch_state
    from baybridge_b200.backend import native
    from baybridge_b200.launch_graph import LaunchGraph

    graph = LaunchGraph()
    with pytest.raises(RuntimeError, match="nothing has been recorded"):
        graph.replay()
    if not native.device_available():
        with pytest.raises(cute.BackendNotImplementedError, match="CUDA device"):
            with graph.record():
                pass
    assert not native.recording()
    carrier = FakeCudaTensor((16,), "float32")
    launch_state.set_recording(True)
    try:
        cute.from_dlpack(carrier, stream=55)
    finally:
        launch_state.set_recording(False)
    assert 55 not in carrier.dlpack_streams
    cute.from_dlpack(carrier, stream=56)
    assert 56 in carrier.dlpack_streams
    graph.close()


def test_from_dlpack_handle_fields():
    handle = cute.from_dlpack(FakeCudaTensor((4, 8), "torch.float16", ptr=16384, stride=(8, 1)), assumed_align=32)
    assert (handle.shape, handle.dtype, handle.device_type, handle.device_id) == ((4, 8), "f16", 2, 0)
    assert handle.data_ptr() == 16384 and handle.stride == (8, 1) and handle.assumed_align == 32 and handle.is_contiguous
    with pytest.raises(TypeError):
        cute.from_dlpack(object())


# an upstream checkout next to this repository (or wherever BAYBRIDGE_UPSTREAM_SRC points)
REFERENCE_SRC = Path(os.environ.get("BAYBRIDGE_UPSTREAM_SRC") or Path(__file__).resolve().parents[2] / "reference" / "src")


@pytest.mark.skipif(not REFERENCE_SRC.exists(), reason="upstream checkout not present on this machine")
def test_backend_object_is_a_drop_in_for_an_unmodified_upstream_checkout(tmp_path):
    """Run in a subprocess (both packages cannot share one interpreter's idea of `baybridge`): upstream's own
    compile() accepts B200Backend() and, after install_into_upstream(), the backend name "b200"."""
    import subprocess

    script = f"""
import sys
sys.path.insert(0, {str(REFERENCE_SRC)!r}); sys.path.insert(0, {str(Path(__file__).resolve().parent.parent)!r})
import baybridge as bb
import baybridge_b200
from baybridge_b200 import B200Backend, install_into_upstream

@bb.kernel
def gemm_kernel(a: bb.TensorSpec(shape=(256, 128), dtype="bf16"), b: bb.TensorSpec(shape=(512, 128), dtype="bf16"),
                c: bb.TensorSpec(shape=(256, 512), dtype="bf16")):
    bb.gemm(a, b, c, transpose_b=True)

target = bb.NvidiaTarget(sm="sm_100a", ptx_version="8.8")
art = bb.compile(gemm_kernel, backend=B200Backend(), target=target, cache_dir={str(tmp_path)!r})
assert art.backend_name == "b200" and art.lowered_module.entry_point == "bb200_gemm_bf16", art
assert art.runtime_callable is not None
install_into_upstream(bb)
art2 = bb.compile(gemm_kernel, backend="b200", target=target, cache_dir={str(tmp_path)!r})
assert art2.cache_key == art.cache_key and art2.from_cache
print("drop-in ok")
"""
    done = subprocess.run([sys.executable, "-c", script], capture_output=True, text=True, timeout=300)
    assert done.returncode == 0 and "drop-in ok" in done.stdout, done.stderr[-2000:]


def test_debug_bounds_build_changes_only_thread_by_thread_kernels(zoo, monkeypatch, tmp_path):
    """``BB200_DEBUG_BOUNDS=1`` adds a status-word parameter and a recorded code per guarded access to literal-mode
    kernels; flat kernels (whose extent never exceeds a tensor) are rendered exactly as before."""
    carriers = [FakeCudaTensor((1000,), "float32"), FakeCudaTensor((1000,), "float32")]
    plain = json.loads(cute.B200Backend().lower(cute.compile(zoo.make_indexed_reverse(1000), *carriers, backend="portable").ir, TARGET).text)
    assert plain["mode"] == "literal" and plain["debug_bounds"] is False and "bounds_status" not in plain["source"]
    flat_ir = cute.compile(zoo.make_indexed_binary("add", 1024), *[FakeCudaTensor((1024,), "float32")] * 3, backend="portable").ir
    flat_before = json.loads(cute.B200Backend().lower(flat_ir, TARGET).text)
    monkeypatch.setenv("BB200_DEBUG_BOUNDS", "1")
    checked = json.loads(cute.B200Backend().lower(cute.compile(zoo.make_indexed_reverse(1000), *carriers, backend="portable").ir, TARGET).text)
    assert checked["debug_bounds"] is True and "int* bounds_status" in checked["source"]
    assert checked["source"].count("atomicExch(bounds_status, 301)") == 1 and checked["source"].count("atomicExch(bounds_status, 302)") == 1
    assert json.loads(cute.B200Backend().lower(flat_ir, TARGET).text) == flat_before
