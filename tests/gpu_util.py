"""Helpers for the ``-m gpu`` parity tests: device tensors via torch, comparisons in ULPs and rel-L2."""
from __future__ import annotations

import ctypes

import numpy as np

from oracle import cpu_runtime as oracle

TORCH_DTYPE = {"f32": "float32", "bf16": "bfloat16", "f16": "float16", "i32": "int32", "i64": "int64", "i1": "bool"}


def torch_module():
    import torch

    return torch


def to_device(array: np.ndarray, dtype: str):
    """Host values (already representable in ``dtype``) → contiguous CUDA tensor of that dtype."""
    torch = torch_module()
    host = torch.from_numpy(np.ascontiguousarray(array, dtype=np.float32 if dtype in ("f32", "bf16", "f16") else None))
    return host.to(device="cuda", dtype=getattr(torch, TORCH_DTYPE[dtype])).contiguous()


def device_zeros(shape, dtype: str):
    torch = torch_module()
    return torch.zeros(tuple(shape), device="cuda", dtype=getattr(torch, TORCH_DTYPE[dtype]))


def to_host(tensor) -> np.ndarray:
    """CUDA tensor → float64 (or int64) numpy array with exact values."""
    torch = torch_module()
    if tensor.dtype in (torch.bfloat16, torch.float16, torch.float32):
        return tensor.detach().to(torch.float64).cpu().numpy()
    return tensor.detach().cpu().numpy()


def ulp_distance(actual: np.ndarray, expected: np.ndarray, dtype: str) -> np.ndarray:
    """Distance in units of the last place of ``dtype`` between two arrays of representable values."""
    def ordinal(values: np.ndarray) -> np.ndarray:
        if dtype == "f32":
            bits = values.astype(np.float32).view(np.int32).astype(np.int64)
            return np.where(bits < 0, -(bits & 0x7FFFFFFF), bits)
        if dtype == "bf16":
            bits = (values.astype(np.float32).view(np.uint32) >> 16).astype(np.int64)
        else:
            bits = values.astype(np.float16).view(np.uint16).astype(np.int64)
        return np.where(bits & 0x8000, -(bits & 0x7FFF), bits)

    return np.abs(ordinal(np.asarray(actual)) - ordinal(np.asarray(expected)))


def expect_rounded(actual: np.ndarray, reference_f64: np.ndarray, dtype: str, *, max_ulp: int = 0) -> None:
    """``actual`` must equal RNE(reference) in ``dtype`` up to ``max_ulp`` units in the last place."""
    expected = oracle.round_to_dtype(reference_f64, dtype)
    if max_ulp == 0:
        mismatches = int(np.count_nonzero(actual != expected))
        assert mismatches == 0, f"{mismatches} of {actual.size} elements differ from the rounded f64 reference"
        return
    worst = int(ulp_distance(actual, expected, dtype).max())
    assert worst <= max_ulp, f"worst error {worst} ulp > {max_ulp}"


def void_p(tensor) -> ctypes.c_void_p:
    return ctypes.c_void_p(tensor.data_ptr())


def current_stream() -> ctypes.c_void_p:
    return ctypes.c_void_p(torch_module().cuda.current_stream().cuda_stream)
