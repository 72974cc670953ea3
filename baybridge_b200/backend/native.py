"""Build and bind ``libbb200.so`` (the C ABI declared in ``include/bb200.h``).

``build_library()`` runs ``nvcc`` for sm_100a over ``csrc/*.cu`` and writes the
shared object next to the package (in-tree).  ``library()`` loads it with
``ctypes`` and declares every prototype; ``call()`` turns a non-zero status
into ``CudaDriverError`` carrying ``bb200_last_error()``.  There is no Python
or CPU substitute for anything in the library: if it is missing or cannot be
built, ``library()`` raises ``BackendNotImplementedError``.

The ctypes layer plays the role of upstream's ``cuda_driver.py:104-245``
(library discovery, prototype binding, status checking).
"""
from __future__ import annotations

import ctypes
import fcntl
import hashlib
import os
import shutil
import subprocess
import threading
from pathlib import Path
from typing import Any

from ..errors import BackendNotImplementedError, CudaDriverError
from ..launch_state import recording, set_recording  # noqa: F401 - re-exported for the launchers

PACKAGE_DIR = Path(__file__).resolve().parent.parent
CSRC_DIR = PACKAGE_DIR / "csrc"
LIBRARY_PATH = PACKAGE_DIR / "libbb200.so"
STAMP_PATH = PACKAGE_DIR / "libbb200.stamp"
GENCODE = ("-gencode", "arch=compute_100a,code=sm_100a")
NVCC_COMMON = ("-O3", "-std=c++17", "-lineinfo")

ERROR_NAMES = {
    -1: "BB200_E_INVALID_ARGUMENT", -2: "BB200_E_UNSUPPORTED_SHAPE", -3: "BB200_E_MISALIGNED",
    -4: "BB200_E_NO_DRIVER", -5: "BB200_E_NOT_SM100", -6: "BB200_E_DEVICE_TIMEOUT", -7: "BB200_E_TOO_LARGE",
}
DTYPE_CODES = {"f32": 0, "bf16": 1, "f16": 2, "i32": 3, "i64": 4, "index": 4, "i8": 5, "i1": 6}
BINARY_OP_CODES = {"add": 0, "sub": 1, "mul": 2, "div": 3, "max": 4, "min": 5}

_lock = threading.Lock()
_library: ctypes.CDLL | None = None


def nvcc_path() -> str:
    found = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(found).exists():
        raise BackendNotImplementedError("nvcc was not found; the b200 backend needs the CUDA toolkit to build its kernels")
    return found


def _sources() -> list[Path]:
    return sorted(CSRC_DIR.glob("*.cu"))


def source_digest() -> str:
    digest = hashlib.sha256()
    for path in sorted(list(CSRC_DIR.glob("*.cu")) + list(CSRC_DIR.glob("*.cuh")) + list(CSRC_DIR.glob("*.h"))
                       + [PACKAGE_DIR.parent / "include" / "bb200.h"]):
        digest.update(path.name.encode())
        digest.update(path.read_bytes())
    return digest.hexdigest()


def library_is_current() -> bool:
    return LIBRARY_PATH.exists() and STAMP_PATH.exists() and STAMP_PATH.read_text().strip() == source_digest()


def build_library(force: bool = False, verbose: bool = False) -> Path:
    """Compile ``csrc/*.cu`` into ``libbb200.so`` for sm_100a (cross-compiles without a GPU)."""
    build_dir = PACKAGE_DIR / "build"
    build_dir.mkdir(exist_ok=True)
    # one builder at a time across threads AND processes (ranks of one job share the tree): the others wait on the
    # file lock and then find the library current; the link goes to a temporary name and is renamed into place, so a
    # concurrent reader never maps a half-written file
    with _lock, open(build_dir / ".lock", "w") as lock_file:
        fcntl.flock(lock_file, fcntl.LOCK_EX)
        if not force and library_is_current():
            return LIBRARY_PATH
        objects: list[Path] = []
        procs = []
        for source in _sources():
            obj = build_dir / (source.stem + ".o")
            objects.append(obj)
            command = [nvcc_path(), *GENCODE, *NVCC_COMMON, "-Xcompiler", "-fPIC", "-c", str(source), "-o", str(obj)]
            if verbose:
                command.insert(1, "-Xptxas=-v")
            procs.append((source, subprocess.Popen(command, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        for source, proc in procs:
            output, _ = proc.communicate()
            if verbose and output:
                print(output)
            if proc.returncode:
                raise BackendNotImplementedError(f"nvcc failed on {source.name}:\n{output}")
        staged = build_dir / f"libbb200.{os.getpid()}.so"
        link = [nvcc_path(), *GENCODE, "-shared", "-cudart", "static", "-o", str(staged), *map(str, objects), "-ldl"]
        done = subprocess.run(link, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        if done.returncode:
            raise BackendNotImplementedError(f"linking libbb200.so failed:\n{done.stdout}")
        STAMP_PATH.unlink(missing_ok=True)
        os.replace(staged, LIBRARY_PATH)
        STAMP_PATH.write_text(source_digest() + "\n")
        return LIBRARY_PATH


P = ctypes.c_void_p
PP = ctypes.POINTER(ctypes.c_void_p)
I = ctypes.c_int
Z = ctypes.c_size_t
U3 = ctypes.c_uint * 3


class DeviceInfo(ctypes.Structure):
    _fields_ = [
        ("ordinal", I), ("cc_major", I), ("cc_minor", I), ("sm_count", I), ("max_smem_per_block_optin", I),
        ("l2_bytes", I), ("clock_khz", I), ("mem_clock_khz", I), ("mem_bus_bits", I),
        ("total_mem_bytes", ctypes.c_uint64), ("name", ctypes.c_char * 128),
    ]


#: every symbol ``include/bb200.h`` declares → ctypes argument types (the return type is always int,
#: except ``bb200_last_error``)
PROTOTYPES: dict[str, list[Any]] = {
    "bb200_abi_version": [],
    "bb200_last_error": [],
    "bb200_device_count": [ctypes.POINTER(I)],
    "bb200_init": [I],
    "bb200_device_info_get": [I, ctypes.POINTER(DeviceInfo)],
    "bb200_module_load": [P, Z, PP],
    "bb200_module_unload": [P],
    "bb200_get_function": [P, ctypes.c_char_p, PP],
    "bb200_function_set_dynamic_smem": [P, ctypes.c_uint],
    "bb200_launch": [P, U3, U3, U3, ctypes.c_uint, P, PP],
    "bb200_launch_dependent": [P, U3, U3, U3, ctypes.c_uint, P, PP],
    "bb200_device_synchronize": [],
    "bb200_stream_synchronize": [P],
    "bb200_stream_create": [PP],
    "bb200_stream_destroy": [P],
    "bb200_event_create": [PP],
    "bb200_event_record": [P, P],
    "bb200_event_synchronize": [P],
    "bb200_event_elapsed_ms": [P, P, ctypes.POINTER(ctypes.c_float)],
    "bb200_event_destroy": [P],
    "bb200_mem_alloc": [PP, Z],
    "bb200_mem_free": [P],
    "bb200_memcpy_h2d": [P, P, Z, P],
    "bb200_memcpy_d2h": [P, P, Z, P],
    "bb200_memset": [P, I, Z, P],
    "bb200_host_alloc_pinned": [PP, Z],
    "bb200_host_free_pinned": [P],
    "bb200_tensormap_encode_2d": [P, I, P, ctypes.c_uint64, ctypes.c_uint64, ctypes.c_uint64, ctypes.c_uint32,
                                  ctypes.c_uint32, I],
    "bb200_elementwise_binary": [I, I, P, P, P, Z, P],
    "bb200_elementwise_mul_add": [I, P, P, P, Z, P],
    "bb200_rmsnorm": [I, P, P, P, Z, Z, I, ctypes.c_float, P],
    "bb200_layernorm": [I, P, P, P, P, P, P, Z, Z, I, I, ctypes.c_float, P],
    "bb200_layernorm_gather": [I, P, P, P, P, ctypes.POINTER(P), ctypes.POINTER(P), I, Z, Z, Z, I, I, ctypes.c_float, P],
    "bb200_gemm_bf16": [P, P, P, I, I, I, I, I, I, P],
    "bb200_gemm_bf16_noalloc": [P, P, P, I, I, I, I, I, I, P],
    "bb200_rmsnorm_gather": [I, P, P, ctypes.POINTER(P), I, Z, Z, Z, I, ctypes.c_float, P],
    "bb200_gemm_bf16_gather": [P, P, ctypes.POINTER(P), I, I, I, I, I, I, I, I, P],
    "bb200_attention_fwd": [P, P, P, P, P, I, I, I, I, I, I, P],
    "bb200_attention_fwd_gather": [P, P, P, ctypes.POINTER(P), ctypes.POINTER(P), I, I, I, I, I, I, I, I, P],
    "bb200_take_device_status": [P, ctypes.POINTER(I)],
    "bb200_selftest_bounded_wait": [ctypes.c_uint, P],
    "bb200_device_status_address": [PP],
    "bb200_graph_capture_begin": [P],
    "bb200_graph_capture_end": [P, ctypes.POINTER(P)],
    "bb200_graph_launch": [P, P],
    "bb200_graph_destroy": [P],
}


def library() -> ctypes.CDLL:
    """The loaded, prototyped library; builds it first if the in-tree binary is missing or stale."""
    global _library
    if _library is not None:
        return _library
    if not LIBRARY_PATH.exists() or (not library_is_current() and os.environ.get("BB200_NO_REBUILD") != "1"):
        build_library()
    try:
        lib = ctypes.CDLL(str(LIBRARY_PATH))
    except OSError as exc:
        raise BackendNotImplementedError(f"libbb200.so could not be loaded: {exc}") from exc
    for name, argtypes in PROTOTYPES.items():
        try:
            function = getattr(lib, name)
        except AttributeError as exc:
            raise BackendNotImplementedError(f"libbb200.so does not export {name}; rebuild it") from exc
        function.argtypes = argtypes
        function.restype = ctypes.c_char_p if name == "bb200_last_error" else ctypes.c_int
    if lib.bb200_abi_version() != 1:
        raise BackendNotImplementedError("libbb200.so has a different ABI version than this package expects")
    _library = lib
    return lib


def call(name: str, *args: Any) -> None:
    """Invoke ``lib.<name>(*args)`` and raise ``CudaDriverError`` on a non-zero status."""
    lib = library()
    status = getattr(lib, name)(*args)
    if status != 0:
        message = (lib.bb200_last_error() or b"").decode("utf-8", "replace")
        raise CudaDriverError(name, status, ERROR_NAMES.get(status, "CUDA_ERROR" if status > 0 else "BB200_ERROR"), message)


def entry_point(name: str) -> Any:
    """The prototyped C function ``name``, for callers on a hot path that do not want the lookup per call."""
    return getattr(library(), name)


def call_resolved(function: Any, name: str, *args: Any) -> None:
    """``call`` for a function obtained from ``entry_point``."""
    status = function(*args)
    if status != 0:
        message = (library().bb200_last_error() or b"").decode("utf-8", "replace")
        raise CudaDriverError(name, status, ERROR_NAMES.get(status, "CUDA_ERROR" if status > 0 else "BB200_ERROR"), message)


def take_device_status(stream: ctypes.c_void_p) -> int:
    """Synchronise ``stream``, then read and clear the device status word (0 = no bounded wait gave up)."""
    status = ctypes.c_int(0)
    call("bb200_take_device_status", stream, ctypes.byref(status))
    return int(status.value)


def stream_handle(stream: Any) -> ctypes.c_void_p:
    """Accept ``None``, an int, a ``ctypes.c_void_p`` or an object with ``.cuda_stream`` (torch streams)."""
    if stream is None:
        return ctypes.c_void_p(0)
    if isinstance(stream, ctypes.c_void_p):
        return stream
    raw = getattr(stream, "cuda_stream", stream)
    if isinstance(raw, int):
        return ctypes.c_void_p(raw)
    value = getattr(raw, "value", None)
    if isinstance(value, int) or value is None:
        return ctypes.c_void_p(value or 0)
    raise TypeError(f"unsupported CUDA stream type '{type(stream).__name__}'")


def device_available() -> bool:
    """True when a CUDA driver and at least one device are usable through the library."""
    try:
        count = ctypes.c_int(0)
        return library().bb200_device_count(ctypes.byref(count)) == 0 and count.value > 0
    except BackendNotImplementedError:
        return False


_device_seen = False


def require_device() -> None:
    """Fail loudly (no fallback) when launches are impossible on this machine."""
    global _device_seen
    if _device_seen:
        return
    count = ctypes.c_int(0)
    lib = library()
    status = lib.bb200_device_count(ctypes.byref(count))
    if status != 0 or count.value < 1:
        detail = (lib.bb200_last_error() or b"").decode("utf-8", "replace") if status else "no CUDA device is visible"
        raise BackendNotImplementedError(f"the b200 backend needs a CUDA device and driver: {detail}")
    _device_seen = True
