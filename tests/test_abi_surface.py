"""The C ABI: the built library loads without a GPU and exports every symbol the header declares."""
from __future__ import annotations

import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
HEADER = ROOT / "include" / "bb200.h"


def declared_symbols() -> list[str]:
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(bb200_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_expected_families():
    names = declared_symbols()
    for required in ("bb200_init", "bb200_module_load", "bb200_launch", "bb200_stream_synchronize", "bb200_event_elapsed_ms",
                     "bb200_tensormap_encode_2d", "bb200_elementwise_binary", "bb200_elementwise_mul_add", "bb200_rmsnorm", "bb200_layernorm",
                     "bb200_gemm_bf16", "bb200_attention_fwd", "bb200_last_error"):
        assert required in names


def test_library_exports_every_declared_symbol():
    from baybridge_b200.backend import native

    library = native.library()  # builds with nvcc if the in-tree binary is missing or stale
    for name in declared_symbols():
        assert hasattr(library, name), f"libbb200.so does not export {name}"
    assert sorted(native.PROTOTYPES) == declared_symbols(), "ctypes prototypes and header are out of step"
    assert library.bb200_abi_version() == 1


def test_every_declaration_cites_what_it_replaces():
    """Each entry point's comment names the upstream interface it stands in for, or says there is none."""
    text = HEADER.read_text()
    for name in declared_symbols():
        if name in ("bb200_abi_version", "bb200_last_error"):
            continue
        position = text.index(name + "(")
        preceding = text[:position]
        comment = preceding[preceding.rindex("\n/*"):]  # the block comment above the declaration group
        # declarations that share one comment block (e.g. stream_create/destroy) sit right under it
        assert ("src/baybridge/" in comment) or ("counterpart" in comment.lower()), f"{name}: no upstream citation in its comment"


def test_calls_fail_cleanly_without_a_driver(monkeypatch):
    """On a machine without libcuda the library reports BB200_E_NO_DRIVER instead of crashing, and the
    Python layer turns that into an exception: there is no silent host fallback."""
    from baybridge_b200 import BackendNotImplementedError
    from baybridge_b200.backend import native

    if native.device_available():
        pytest.skip("a CUDA device is present")
    count = ctypes.c_int(0)
    library = native.library()
    assert library.bb200_device_count(ctypes.byref(count)) != 0
    assert b"libcuda" in library.bb200_last_error() or b"cuInit" in library.bb200_last_error()
    with pytest.raises(BackendNotImplementedError):
        native.require_device()


def test_argument_validation_needs_no_device():
    from baybridge_b200 import CudaDriverError
    from baybridge_b200.backend import native

    with pytest.raises(CudaDriverError) as info:
        native.call("bb200_rmsnorm", 1, None, None, None, 4, 16, 0, 1e-6, None)
    assert info.value.status == -1 and info.value.name == "BB200_E_INVALID_ARGUMENT"
    with pytest.raises(CudaDriverError) as info:
        native.call("bb200_gemm_bf16", ctypes.c_void_p(16), ctypes.c_void_p(16), ctypes.c_void_p(16), 8, 8, 12, 0, 1, 1, None)
    assert info.value.status == -2
    with pytest.raises(CudaDriverError) as info:
        native.call("bb200_attention_fwd", ctypes.c_void_p(16), ctypes.c_void_p(16), ctypes.c_void_p(16), ctypes.c_void_p(16),
                    ctypes.c_void_p(16), 1, 128, 4, 3, 128, 1, None)
    assert info.value.status == -1
