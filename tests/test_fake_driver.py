"""The driver shim and the launcher against a fake ``libcuda`` — no GPU.

``libbb200.so`` opens the CUDA driver lazily with ``dlopen`` and honours ``BB200_LIBCUDA``; here that points at
``tests/fake_libcuda.c`` (built with gcc), whose entry points log every call and return the status the test plans.
The shim binds the driver once per process, so every scenario runs in a child interpreter.

Upstream tests its ctypes driver wrapper the same way — a fake library handed to ``CudaDriver``
(``tests/test_cuda_driver_runtime.py:61, 184``) — and watches stream forwarding and the error path of its
executable launcher by patching the driver (``tests/test_backend_ptx_exec.py:3062-3145``).
"""
from __future__ import annotations

import json
import os
import shutil
import subprocess
import sys
import textwrap
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
CUDA_INCLUDE = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda")) / "include"


@pytest.fixture(scope="session")
def fake_driver(tmp_path_factory) -> Path:
    compiler = shutil.which("gcc") or shutil.which("cc")
    if compiler is None or not (CUDA_INCLUDE / "cuda.h").exists():
        pytest.skip("needs gcc and cuda.h to build the fake driver")
    library = tmp_path_factory.mktemp("fake_driver") / "libcuda_fake.so"
    subprocess.run([compiler, "-shared", "-fPIC", "-O1", "-Wall", f"-I{CUDA_INCLUDE}", str(ROOT / "tests" / "fake_libcuda.c"),
                    "-o", str(library)], check=True)
    return library


def run_child(fake_driver: Path, tmp_path: Path, body: str, *, fail: str = "", devices: int = 1) -> tuple[dict, list[str]]:
    """Run ``body`` (which must assign ``result``) in a child interpreter bound to the fake driver; returns the
    child's ``result`` and the driver-call log."""
    log = tmp_path / "driver_calls.log"
    script = tmp_path / "child.py"
    script.write_text("import ctypes, json, sys\nsys.path.insert(0, %r)\n" % str(ROOT)
                      + "from baybridge_b200.backend import native\nfrom baybridge_b200.errors import CudaDriverError\n"
                      + textwrap.dedent(body) + "\nprint('RESULT ' + json.dumps(result))\n")
    env = dict(os.environ, BB200_LIBCUDA=str(fake_driver), FAKE_CUDA_LOG=str(log), FAKE_CUDA_FAIL=fail,
               FAKE_CUDA_DEVICES=str(devices), BB200_NO_REBUILD="1", CUDA_VISIBLE_DEVICES="")
    done = subprocess.run([sys.executable, str(script)], env=env, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, timeout=300)
    assert done.returncode == 0, done.stderr[-2000:]
    line = next(line for line in done.stdout.splitlines() if line.startswith("RESULT "))
    return json.loads(line[len("RESULT "):]), (log.read_text().splitlines() if log.exists() else [])


def calls(log: list[str], name: str) -> list[str]:
    return [line for line in log if line.split(" ", 1)[0] == name]


def test_init_binds_the_primary_context_of_the_requested_device(fake_driver, tmp_path):
    result, log = run_child(fake_driver, tmp_path, """
        native.call("bb200_init", 1)
        info = native.DeviceInfo()
        native.call("bb200_device_info_get", 1, ctypes.byref(info))
        result = {"name": info.name.decode(), "cc": [info.cc_major, info.cc_minor], "sms": info.sm_count, "available": native.device_available()}
    """, devices=2)
    assert result == {"name": "Fake B200 #1", "cc": [10, 0], "sms": 148, "available": True}
    order = [line.split(" ", 1)[0] for line in log]
    assert order.index("cuInit") < order.index("cuDeviceGet") < order.index("cuDevicePrimaryCtxRetain") < order.index("cuCtxSetCurrent")
    assert calls(log, "cuDevicePrimaryCtxRetain") == ["cuDevicePrimaryCtxRetain device=1"]
    assert calls(log, "cuCtxSetCurrent") == ["cuCtxSetCurrent context=0xc0de0001"]


def test_init_rejects_an_ordinal_outside_the_visible_devices(fake_driver, tmp_path):
    result, log = run_child(fake_driver, tmp_path, """
        try:
            native.call("bb200_init", 3)
            result = {"raised": False}
        except CudaDriverError as error:
            result = {"raised": True, "op": error.op, "status": error.status, "name": error.name, "text": str(error)}
    """)
    assert result["raised"] and result["op"] == "bb200_init" and result["status"] == -1
    assert result["name"] == "BB200_E_INVALID_ARGUMENT" and "out of range" in result["text"]
    assert not calls(log, "cuDevicePrimaryCtxRetain")


@pytest.mark.parametrize("entry, code, name", [("cuInit", 100, "CUDA_ERROR_NO_DEVICE"), ("cuDevicePrimaryCtxRetain", 2, "CUDA_ERROR_OUT_OF_MEMORY")])
def test_driver_failures_surface_as_cuda_driver_error(fake_driver, tmp_path, entry, code, name):
    result, _ = run_child(fake_driver, tmp_path, """
        try:
            native.call("bb200_init", 0)
            result = {"raised": False}
        except CudaDriverError as error:
            result = {"raised": True, "op": error.op, "status": error.status, "name": error.name, "text": str(error),
                      "available": native.device_available()}
    """, fail=f"{entry}={code}")
    assert result["raised"] and result["op"] == "bb200_init" and result["status"] == code
    assert name in result["text"]
    if entry == "cuInit":
        assert result["available"] is False  # a driver that cannot initialise means "no device", never a fallback


def test_module_load_get_function_and_launch_forward_their_arguments(fake_driver, tmp_path):
    result, log = run_child(fake_driver, tmp_path, """
        native.call("bb200_init", 0)
        image = b"\\x7fELF" + bytes(60)
        module, function = ctypes.c_void_p(), ctypes.c_void_p()
        native.call("bb200_module_load", image, len(image), ctypes.byref(module))
        native.call("bb200_get_function", module, b"my_kernel", ctypes.byref(function))
        native.call("bb200_function_set_dynamic_smem", function, 200 * 1024)
        value = ctypes.c_int(7)
        params = (ctypes.c_void_p * 1)(ctypes.cast(ctypes.byref(value), ctypes.c_void_p))
        stream = ctypes.c_void_p(0x1234)
        native.call("bb200_launch", function, native.U3(296, 1, 1), native.U3(192, 1, 1), native.U3(2, 1, 1), 200 * 1024, stream, params)
        native.call("bb200_launch", function, native.U3(5, 6, 7), native.U3(32, 2, 1), native.U3(1, 1, 1), 0, None, params)
        native.call("bb200_launch_dependent", function, native.U3(9, 1, 1), native.U3(256, 1, 1), native.U3(1, 1, 1), 0, stream, params)
        native.call("bb200_launch_dependent", function, native.U3(8, 1, 1), native.U3(64, 1, 1), native.U3(4, 1, 1), 1024, stream, params)
        native.call("bb200_stream_synchronize", stream)
        native.call("bb200_device_synchronize")
        native.call("bb200_module_unload", module)
        result = {"module": module.value, "function": function.value}
    """)
    assert result == {"module": 0xA001, "function": 0xA001 + 0x10000}
    assert calls(log, "cuModuleLoadData") == ["cuModuleLoadData first_bytes=7f454c46 context=0xc0de0000"]
    assert calls(log, "cuModuleGetFunction") == ["cuModuleGetFunction module=0xa001 name=my_kernel"]
    assert calls(log, "cuFuncSetAttribute") == [f"cuFuncSetAttribute function=0x1a001 attribute=8 value={200 * 1024}"]
    assert calls(log, "cuLaunchKernelEx") == [
        f"cuLaunchKernelEx function=0x1a001 grid=296,1,1 block=192,1,1 cluster=2,1,1 smem={200 * 1024} dependent=0 stream=0x1234",
        "cuLaunchKernelEx function=0x1a001 grid=5,6,7 block=32,2,1 cluster=1,1,1 smem=0 dependent=0 stream=(nil)",
        # programmatic stream serialisation reaches the driver as a launch attribute, next to the cluster when there is one
        "cuLaunchKernelEx function=0x1a001 grid=9,1,1 block=256,1,1 cluster=1,1,1 smem=0 dependent=1 stream=0x1234",
        "cuLaunchKernelEx function=0x1a001 grid=8,1,1 block=64,1,1 cluster=4,1,1 smem=1024 dependent=1 stream=0x1234",
    ]
    assert calls(log, "cuStreamSynchronize") == ["cuStreamSynchronize stream=0x1234"]
    assert calls(log, "cuCtxSynchronize") == ["cuCtxSynchronize "]
    assert calls(log, "cuModuleUnload") == ["cuModuleUnload module=0xa001"]


def test_launch_validates_before_it_reaches_the_driver(fake_driver, tmp_path):
    result, log = run_child(fake_driver, tmp_path, """
        native.call("bb200_init", 0)
        function = ctypes.c_void_p(0x77)
        params = (ctypes.c_void_p * 1)()
        outcomes = []
        for grid, block, cluster in [((0, 1, 1), (32, 1, 1), (1, 1, 1)), ((4, 1, 1), (1025, 1, 1), (1, 1, 1)), ((3, 1, 1), (32, 1, 1), (2, 1, 1))]:
            try:
                native.call("bb200_launch", function, native.U3(*grid), native.U3(*block), native.U3(*cluster), 0, None, params)
                outcomes.append("ok")
            except CudaDriverError as error:
                outcomes.append(error.name)
            try:
                native.call("bb200_launch_dependent", function, native.U3(*grid), native.U3(*block), native.U3(*cluster), 0, None, params)
                outcomes.append("ok")
            except CudaDriverError as error:
                outcomes.append(error.name)
        result = {"outcomes": outcomes}
    """)
    assert result["outcomes"] == ["BB200_E_INVALID_ARGUMENT"] * 6
    assert not calls(log, "cuLaunchKernelEx")


@pytest.mark.parametrize("entry, operation, code, name", [
    ("cuModuleLoadData", "bb200_module_load", 200, "CUDA_ERROR_INVALID_IMAGE"),
    ("cuModuleGetFunction", "bb200_get_function", 500, "CUDA_ERROR_NOT_FOUND"),
    ("cuLaunchKernelEx", "bb200_launch", 719, "CUDA_ERROR_LAUNCH_FAILED"),
    ("cuStreamSynchronize", "bb200_stream_synchronize", 719, "CUDA_ERROR_LAUNCH_FAILED"),
])
def test_each_driver_step_maps_to_cuda_driver_error(fake_driver, tmp_path, entry, operation, code, name):
    result, _ = run_child(fake_driver, tmp_path, """
        native.call("bb200_init", 0)
        image = b"\\x7fELF" + bytes(60)
        module, function = ctypes.c_void_p(0xA001), ctypes.c_void_p(0x1A001)
        params = (ctypes.c_void_p * 1)()
        steps = [
            ("bb200_module_load", lambda: native.call("bb200_module_load", image, len(image), ctypes.byref(module))),
            ("bb200_get_function", lambda: native.call("bb200_get_function", module, b"k", ctypes.byref(function))),
            ("bb200_launch", lambda: native.call("bb200_launch", function, native.U3(1, 1, 1), native.U3(32, 1, 1), native.U3(1, 1, 1), 0, None, params)),
            ("bb200_stream_synchronize", lambda: native.call("bb200_stream_synchronize", None)),
        ]
        result = {"failed": None}
        for label, step in steps:
            try:
                step()
            except CudaDriverError as error:
                result = {"failed": label, "op": error.op, "status": error.status, "text": str(error)}
                break
    """, fail=f"{entry}={code}")
    assert result["failed"] == operation and result["op"] == operation and result["status"] == code
    assert name in result["text"]


ELEMENTWISE_CHILD = """
    import numpy as np
    import baybridge_b200 as cute
    from baybridge_b200 import B200Backend
    from baybridge_b200.samples import build_zoo
    from baybridge_b200.host_values import TensorHandle

    class FakeCudaTensor:
        def __init__(self, shape, dtype, pointer, device=0):
            self.shape, self.dtype, self._pointer, self._device = tuple(shape), dtype, pointer, device
        def __dlpack__(self, stream=None):
            return "capsule"
        def __dlpack_device__(self):
            return (2, self._device)
        def data_ptr(self):
            return self._pointer

    zoo = build_zoo(cute)
    n = 1024
"""


def test_launcher_forwards_the_stream_and_synchronises_it(fake_driver, tmp_path):
    """``artifact(*handles, stream=s)`` launches on ``s`` and, being synchronous like upstream's launchers
    (``ptx_exec.py:168-171``), waits on ``s`` — not on the whole context."""
    result, log = run_child(fake_driver, tmp_path, ELEMENTWISE_CHILD + """
    tensors = [FakeCudaTensor((n,), "float32", 0x10000 * (i + 1)) for i in range(3)]
    artifact = cute.compile(zoo.make_indexed_binary("add", n), *tensors, backend="b200", cache_dir=%r)
    artifact(*tensors, stream=0x4321)
    artifact(*tensors)
    # the backend's own launcher (what upstream's compile() wraps): IR-order positional arguments and stream= only
    target = cute.NvidiaTarget(sm="sm_100a", ptx_version="8.8")
    backend = B200Backend()
    launcher = backend.build_launcher(artifact.ir, target, backend.lower(artifact.ir, target), None)
    handles = [cute.from_dlpack(t) for t in tensors]
    try:
        launcher(*handles, flavour="x")
        result = {"kwarg": "accepted"}
    except TypeError as error:
        result = {"kwarg": str(error)}
    try:
        launcher(handles[0])
    except TypeError as error:
        result["arity"] = str(error)
    """ % str(tmp_path / "cache"))
    launches = calls(log, "cuLaunchKernelEx")
    assert len(launches) == 2 and launches[0].endswith("stream=0x4321") and launches[1].endswith("stream=(nil)")
    assert calls(log, "cuStreamSynchronize") == ["cuStreamSynchronize stream=0x4321", "cuStreamSynchronize stream=(nil)"]
    assert len(calls(log, "cuModuleLoadData")) == 1  # the module is loaded once and kept
    assert "positional arguments" in result["kwarg"] and "expects 3 arguments, got 1" in result["arity"]


def test_flat_elementwise_launches_are_dependent_launches_unless_switched_off(fake_driver, tmp_path):
    """The flat elementwise kernels keep stream order themselves (``griddepcontrol.wait``), so their launcher asks for
    programmatic stream serialisation; ``B200Backend(overlap_launches=False)`` takes the plain launch, and so does a
    thread-by-thread (literal) kernel, which has no such wait."""
    _, log = run_child(fake_driver, tmp_path, ELEMENTWISE_CHILD + """
    tensors = [FakeCudaTensor((n,), "float32", 0x10000 * (i + 1)) for i in range(3)]
    cute.compile(zoo.make_indexed_binary("add", n), *tensors, backend=B200Backend(), cache_dir=%r)(*tensors)
    cute.compile(zoo.make_indexed_binary("add", n), *tensors, backend=B200Backend(overlap_launches=False), cache_dir=%r)(*tensors)
    cute.compile(zoo.make_indexed_reverse(n), *tensors[:2], backend=B200Backend(), cache_dir=%r)(*tensors[:2])
    result = {}
    """ % (str(tmp_path / "cache"), str(tmp_path / "cache"), str(tmp_path / "cache")))
    launches = calls(log, "cuLaunchKernelEx")
    assert ["dependent=1" in line for line in launches] == [True, False, False]


def test_launcher_keeps_one_module_per_device(fake_driver, tmp_path):
    _, log = run_child(fake_driver, tmp_path, ELEMENTWISE_CHILD + """
    artifact = None
    for device in (0, 1, 0):
        tensors = [FakeCudaTensor((n,), "float32", 0x10000 * (i + 1), device) for i in range(3)]
        if artifact is None:
            artifact = cute.compile(zoo.make_indexed_binary("add", n), *tensors, backend="b200", cache_dir=%r)
        artifact(*tensors)
    result = {}
    """ % str(tmp_path / "cache"), devices=2)
    loads = calls(log, "cuModuleLoadData")
    assert [line.split("context=")[1] for line in loads] == ["0xc0de0000", "0xc0de0001"]
    functions = [line.split()[1] for line in calls(log, "cuLaunchKernelEx")]
    assert functions[0] == functions[2] != functions[1]


def test_a_failed_launch_raises_and_releases_the_staged_copies(fake_driver, tmp_path):
    """Host tensors are staged through device buffers owned by the launcher; when the launch fails they are freed
    (upstream ``ptx_exec.py:174-176``) and the error reaches the caller as ``CudaDriverError``."""
    result, log = run_child(fake_driver, tmp_path, ELEMENTWISE_CHILD + """
    import warnings
    warnings.simplefilter("ignore")
    host = [cute.tensor(np.ones(n).tolist(), dtype="f32"), cute.tensor(np.ones(n).tolist(), dtype="f32"), cute.zeros((n,), dtype="f32")]
    carriers = [FakeCudaTensor((n,), "float32", 0) for _ in range(3)]
    artifact = cute.compile(zoo.make_indexed_binary("add", n), *carriers, backend="b200", cache_dir=%r)
    try:
        artifact(*host)
        result = {"raised": False}
    except CudaDriverError as error:
        result = {"raised": True, "op": error.op, "status": error.status}
    """ % str(tmp_path / "cache"), fail="cuLaunchKernelEx=719")
    assert result == {"raised": True, "op": "bb200_launch_dependent", "status": 719}
    allocated = [line.split("pointer=")[1] for line in calls(log, "cuMemAlloc.result")]
    freed = [line.split("pointer=")[1] for line in calls(log, "cuMemFree")]
    assert len(allocated) == 3 and sorted(allocated) == sorted(freed)
    assert len(calls(log, "cuMemcpyHtoDAsync")) == 3 and not calls(log, "cuMemcpyDtoHAsync")


def test_staged_host_tensors_round_trip_through_the_fake_device(fake_driver, tmp_path):
    result, log = run_child(fake_driver, tmp_path, ELEMENTWISE_CHILD + """
    import warnings
    warnings.simplefilter("ignore")
    host = [cute.tensor(np.arange(n, dtype=np.float64).tolist(), dtype="f32"), cute.tensor(np.ones(n).tolist(), dtype="f32"),
            cute.tensor(np.full(n, 5.0).tolist(), dtype="f32")]
    carriers = [FakeCudaTensor((n,), "float32", 0) for _ in range(3)]
    artifact = cute.compile(zoo.make_indexed_binary("add", n), *carriers, backend="b200", cache_dir=%r)
    artifact(*host)
    artifact(*host)
    # the fake launch computes nothing: every tensor comes back as it went in, which shows each was copied both ways
    result = {"first": host[0].tolist()[:3], "dst": host[2].tolist()[:2]}
    """ % str(tmp_path / "cache"))
    assert result == {"first": [0.0, 1.0, 2.0], "dst": [5.0, 5.0]}
    assert len(calls(log, "cuMemAlloc")) == 3  # the per-slot staging buffers are reused by the second call
    assert len(calls(log, "cuMemcpyHtoDAsync")) == 6 and len(calls(log, "cuMemcpyDtoHAsync")) == 6


def test_missing_driver_is_reported_not_worked_around(tmp_path):
    script = tmp_path / "child.py"
    script.write_text(f"import sys\nsys.path.insert(0, {str(ROOT)!r})\n" + textwrap.dedent("""
        from baybridge_b200.backend import native
        from baybridge_b200.errors import BackendNotImplementedError
        print("available", native.device_available())
        try:
            native.require_device()
        except BackendNotImplementedError as error:
            print("refused", "libcuda" in str(error))
    """))
    env = dict(os.environ, BB200_LIBCUDA=str(tmp_path / "no_such_driver.so"), BB200_NO_REBUILD="1")
    done = subprocess.run([sys.executable, str(script)], env=env, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, timeout=120)
    assert done.returncode == 0, done.stderr[-1000:]
    assert "available False" in done.stdout and "refused True" in done.stdout
