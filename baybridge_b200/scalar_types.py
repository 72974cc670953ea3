"""Element types of the portable IR and their host encodings.

Names, widths, aliases and the promotion rule follow upstream
``dtypes.py:7-46`` and ``:237-271``.  The host pack/unpack rule for bf16 is the
round-to-nearest-even on the upper 16 bits of the f32 pattern that upstream
uses when staging host tensors (``hip_runtime.py:246-249``), vectorised with
numpy.  The storage-only fp8/bf8 formats are named but not computed on.
"""
from __future__ import annotations

from typing import Any

import numpy as np

BIT_WIDTH = {
    "i1": 1, "i8": 8, "i32": 32, "i64": 64, "index": 64,
    "fp8": 8, "bf8": 8, "f16": 16, "bf16": 16, "f32": 32,
}
_FLOATS = frozenset({"f16", "bf16", "f32"})
_STORAGE_ONLY = frozenset({"fp8", "bf8"})
_SPELLINGS = {
    "i1": ("bool",), "index": ("int",), "i8": ("int8",), "i32": ("int32",), "i64": ("int64",),
    "f16": ("float16",), "bf16": ("bfloat16",), "f32": ("float32",),
    "fp8": ("float8_e4m3fnuz",), "bf8": ("float8_e5m2fnuz",),
}
ALIASES: dict[str, str] = {"float": "f32", "torch.float": "f32"}
for _canonical, _names in _SPELLINGS.items():
    for _name in _names:
        ALIASES[_name] = _canonical
        ALIASES[f"torch.{_name}"] = _canonical

CONSTRUCTOR_NAMES = {
    "i1": "Boolean", "i8": "Int8", "i32": "Int32", "i64": "Int64", "index": "Int",
    "f16": "Float16", "bf16": "BFloat16", "f32": "Float32",
    "fp8": "Float8E4M3FNUZ", "bf8": "BFloat8E5M2FNUZ",
}


class ElementType(str):
    """A dtype name that also knows its bit width (``element_type("bf16").width == 16``)."""

    @property
    def width(self) -> int:
        if str(self) not in BIT_WIDTH:
            raise ValueError(f"baybridge element type '{self}' does not define a bit width")
        return BIT_WIDTH[str(self)]


def element_type(dtype: str) -> ElementType:
    return ElementType(dtype)


def normalize_dtype_name(dtype: str) -> str:
    name = ALIASES.get(dtype, dtype)
    if name not in BIT_WIDTH:
        raise ValueError(f"unsupported baybridge dtype '{dtype}'")
    return name


def resolve_element_type_name(value: Any) -> str:
    if isinstance(value, str):
        return normalize_dtype_name(str(value))
    for attribute in ("__baybridge_dtype__", "dtype"):
        found = getattr(value, attribute, None)
        if isinstance(found, str):
            return normalize_dtype_name(found)
    raise TypeError("element type values must be baybridge dtype strings or scalar constructors")


def is_float_dtype(dtype: str) -> bool:
    return normalize_dtype_name(dtype) in _FLOATS


def is_integer_dtype(dtype: str) -> bool:
    name = normalize_dtype_name(dtype)
    return name not in _FLOATS and name not in _STORAGE_ONLY


def is_storage_only_dtype(dtype: str) -> bool:
    return normalize_dtype_name(dtype) in _STORAGE_ONLY


def byte_width(dtype: str) -> int:
    return (BIT_WIDTH[normalize_dtype_name(dtype)] + 7) // 8


def promote_scalar_dtype(lhs: str, rhs: str) -> str:
    """Result dtype of a scalar binary op: equal → itself, any float → f32, index wins, else wider."""
    left, right = normalize_dtype_name(lhs), normalize_dtype_name(rhs)
    for name in (left, right):
        if name in _STORAGE_ONLY:
            raise TypeError(f"baybridge dtype '{name}' is storage-only and does not support scalar arithmetic")
    if left == right:
        return left
    if left in _FLOATS or right in _FLOATS:
        return "f32"
    if "index" in (left, right):
        return "index"
    return left if BIT_WIDTH[left] >= BIT_WIDTH[right] else right


def cast_scalar_value(value: Any, dtype: str) -> bool | int | float:
    """Host-side value conversion: bool for i1, float for floats, two's-complement wrap for sized ints."""
    name = normalize_dtype_name(dtype)
    if name == "i1":
        return bool(value)
    if name in _FLOATS:
        return float(value)
    raw = int(value)
    if name == "index":
        return raw
    modulus = 1 << BIT_WIDTH[name]
    raw %= modulus
    if name in _STORAGE_ONLY:
        return raw
    return raw - modulus if raw >= modulus >> 1 else raw


# ---------------------------------------------------------------------------------------------
# host encodings (numpy)
# ---------------------------------------------------------------------------------------------
#: numpy dtype that holds the *logical* values of a host tensor (never rounded, like upstream's
#: Python-float storage) and the dtype of the packed device image.
LOGICAL_NUMPY = {
    "i1": np.bool_, "i8": np.int64, "i32": np.int64, "i64": np.int64, "index": np.int64,
    "f16": np.float64, "bf16": np.float64, "f32": np.float64, "fp8": np.int64, "bf8": np.int64,
}
DEVICE_NUMPY = {
    "i1": np.uint8, "i8": np.int8, "i32": np.int32, "i64": np.int64, "index": np.int64,
    "f16": np.float16, "bf16": np.uint16, "f32": np.float32, "fp8": np.uint8, "bf8": np.uint8,
}


def bf16_bits_from_f32(values: np.ndarray) -> np.ndarray:
    """RNE of f32 patterns onto their upper 16 bits; no NaN special case (matches upstream)."""
    bits = np.ascontiguousarray(values, dtype=np.float32).view(np.uint32).astype(np.uint64)
    rounded = (bits + (((bits >> np.uint64(16)) & np.uint64(1)) + np.uint64(0x7FFF))) >> np.uint64(16)
    return (rounded & np.uint64(0xFFFF)).astype(np.uint16)


def f32_from_bf16_bits(bits: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(bits, dtype=np.uint16).astype(np.uint32) << np.uint32(16)).view(np.float32)


def pack_for_device(values: np.ndarray, dtype: str) -> np.ndarray:
    """Logical host values → contiguous array in the device storage encoding of ``dtype``."""
    name = normalize_dtype_name(dtype)
    if name == "bf16":
        return bf16_bits_from_f32(np.asarray(values, dtype=np.float64).astype(np.float32))
    return np.ascontiguousarray(np.asarray(values).astype(DEVICE_NUMPY[name]))


def unpack_from_device(image: np.ndarray, dtype: str) -> np.ndarray:
    """Device storage image → logical host values (float64 / int64 / bool)."""
    name = normalize_dtype_name(dtype)
    if name == "bf16":
        return f32_from_bf16_bits(image).astype(np.float64)
    return np.asarray(image).astype(LOGICAL_NUMPY[name])
