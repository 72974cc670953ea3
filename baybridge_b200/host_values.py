"""Host-side values that cross the ``compile`` / artifact-call boundary.

* ``RuntimeTensor`` — a host tensor (upstream ``runtime.py:376-646``).  Here it
  is a *container only*: a numpy array of logical values (never rounded to the
  tensor dtype, like upstream's list of Python floats) that the b200 launcher
  stages to the device and copies back.  It does not execute kernels: this
  package has no CPU runtime, so arithmetic on host tensors raises.
* ``RuntimeScalar`` and the ``Float32`` … constructors (``runtime.py:184-322,
  1130-1175``).
* ``TensorHandle`` / ``from_dlpack`` — a borrowed device tensor described by
  shape, dtype, strides, device and raw address (``runtime.py:49-124,
  733-761``).  ``normalize_runtime_argument`` and ``infer_runtime_spec`` mirror
  ``runtime.py:797-855``.
"""
from __future__ import annotations

from dataclasses import dataclass, replace
from typing import Any

import numpy as np

from .errors import BackendNotImplementedError
from .launch_state import recording
from .portable_ir import Layout, row_major_stride
from .scalar_types import (
    LOGICAL_NUMPY,
    cast_scalar_value,
    element_type,
    normalize_dtype_name,
    pack_for_device,
    unpack_from_device,
)

DLPACK_CPU = 1
DLPACK_CUDA = 2


def _no_cpu_runtime(what: str) -> BackendNotImplementedError:
    return BackendNotImplementedError(
        f"{what} would execute on the host; baybridge_b200 has no CPU runtime — compile the kernel with backend='b200'"
    )


# ---------------------------------------------------------------------------------------------
# scalars
# ---------------------------------------------------------------------------------------------
@dataclass(frozen=True)
class RuntimeScalar:
    value: bool | int | float
    dtype: str

    def __post_init__(self) -> None:
        object.__setattr__(self, "dtype", normalize_dtype_name(self.dtype))
        object.__setattr__(self, "value", cast_scalar_value(self.value, self.dtype))

    @property
    def element_type(self):
        return element_type(self.dtype)

    def to(self, target: Any) -> "RuntimeScalar":
        return RuntimeScalar(self.value, resolve_scalar_target_dtype(target))

    def __float__(self) -> float:
        return float(self.value)

    def __int__(self) -> int:
        return int(self.value)

    def __bool__(self) -> bool:
        return bool(self.value)

    def __index__(self) -> int:
        return int(self.value)


def resolve_scalar_target_dtype(target: Any) -> str:
    if isinstance(target, RuntimeScalar):
        return target.dtype
    if isinstance(target, str):
        return normalize_dtype_name(target)
    tagged = getattr(target, "__baybridge_dtype__", None)
    if isinstance(tagged, str):
        return normalize_dtype_name(tagged)
    raise TypeError("scalar conversion target must be a baybridge scalar constructor or dtype string")


def _scalar_constructor(name: str, dtype: str):
    def constructor(value: Any = 0):
        # under tracing a constructor call is a cast / typed literal (upstream runtime.py:1143-1156)
        from .trace import ScalarValue, active_builder

        builder = active_builder()
        if builder is None:
            return RuntimeScalar(value.value if isinstance(value, RuntimeScalar) else value, dtype)
        if isinstance(value, ScalarValue):
            return value.to(dtype)
        raw = value.value if isinstance(value, RuntimeScalar) else cast_scalar_value(value, dtype)
        return builder.constant(raw, dtype=dtype)

    constructor.__name__ = constructor.__qualname__ = name
    constructor.__baybridge_dtype__ = dtype
    return constructor


Boolean = _scalar_constructor("Boolean", "i1")
Int8 = _scalar_constructor("Int8", "i8")
Int32 = _scalar_constructor("Int32", "i32")
Int64 = _scalar_constructor("Int64", "i64")
Int = _scalar_constructor("Int", "index")
Float16 = _scalar_constructor("Float16", "f16")
BFloat16 = _scalar_constructor("BFloat16", "bf16")
Float32 = _scalar_constructor("Float32", "f32")


# ---------------------------------------------------------------------------------------------
# host tensors
# ---------------------------------------------------------------------------------------------
def _nested_shape(data: Any) -> tuple[int, ...]:
    if not isinstance(data, (list, tuple)):
        return ()
    if not data:
        raise ValueError("tensor data must be a non-empty nested list")
    inner = _nested_shape(data[0])
    if any(_nested_shape(item) != inner for item in data[1:]):
        raise ValueError("tensor data must have a regular rectangular shape")
    return (len(data),) + inner


def _leaves(data: Any, sink: list[Any]) -> None:
    if isinstance(data, (list, tuple)):
        for item in data:
            _leaves(item, sink)
    else:
        sink.append(data)


def _dtype_from_leaves(leaves: list[Any]) -> str:
    """Inference order of upstream ``runtime.py:1010-1025``: typed scalars, then float > bool > int."""
    typed = [leaf for leaf in leaves if isinstance(leaf, RuntimeScalar)]
    if any(leaf.dtype.startswith("f") for leaf in typed):
        return "f32"
    if any(leaf.dtype == "i1" for leaf in typed):
        return "i1"
    if typed:
        return typed[0].dtype
    for python_type, name in ((float, "f32"), (bool, "i1"), (int, "index")):
        if any(isinstance(leaf, python_type) for leaf in leaves):
            return name
    return type(leaves[0]).__name__ if leaves else "unknown"


class RuntimeTensor:
    """Host tensor: logical values + shape/stride/offset view metadata."""

    def __init__(
        self,
        storage: Any,
        shape: tuple[int, ...],
        *,
        dtype: str,
        stride: tuple[int, ...] | None = None,
        offset: int = 0,
    ):
        if not isinstance(storage, np.ndarray):
            storage = np.asarray(
                [item.value if isinstance(item, RuntimeScalar) else item for item in storage],
                dtype=LOGICAL_NUMPY.get(dtype, np.float64),
            )
        self._storage = storage.reshape(-1)
        self.shape = tuple(int(extent) for extent in shape)
        self.dtype = dtype
        self.stride = tuple(stride) if stride is not None else row_major_stride(self.shape)
        self.offset = int(offset)

    # -- construction -------------------------------------------------------------------------
    @classmethod
    def from_data(cls, data: Any, *, dtype: str | None = None) -> "RuntimeTensor":
        if isinstance(data, np.ndarray):
            name = dtype or {"f": "f32", "b": "i1", "i": "index", "u": "index"}[data.dtype.kind]
            return cls(np.array(data, dtype=LOGICAL_NUMPY.get(name, np.float64)).reshape(-1), data.shape, dtype=name)
        shape = _nested_shape(data)
        leaves: list[Any] = []
        _leaves(data, leaves)
        return cls(leaves, shape, dtype=dtype or _dtype_from_leaves(leaves))

    @classmethod
    def zeros(cls, shape: tuple[int, ...], *, dtype: str = "f32") -> "RuntimeTensor":
        shape = tuple(shape)
        return cls(np.zeros(int(np.prod(shape, dtype=np.int64)), dtype=LOGICAL_NUMPY.get(dtype, np.float64)), shape, dtype=dtype)

    # -- metadata -----------------------------------------------------------------------------
    @property
    def ndim(self) -> int:
        return len(self.shape)

    @property
    def element_type(self):
        return element_type(self.dtype)

    @property
    def type(self) -> str:
        return f"Tensor(shape={self.shape}, dtype={self.dtype}, stride={self.stride})"

    @property
    def layout(self) -> Layout:
        return Layout(shape=self.shape, stride=self.stride)

    @property
    def is_dense(self) -> bool:
        return self.offset == 0 and self.stride == row_major_stride(self.shape) and self._storage.size == self.numel

    @property
    def numel(self) -> int:
        return int(np.prod(self.shape, dtype=np.int64)) if self.shape else 1

    def __len__(self) -> int:
        return self.shape[0] if self.shape else 0

    def __repr__(self) -> str:
        return f"RuntimeTensor(shape={self.shape}, dtype={self.dtype})"

    # -- element access (host bookkeeping only) ---------------------------------------------------
    def _linear(self, index: Any) -> int:
        coords = index if isinstance(index, tuple) else (index,)
        if len(coords) != self.ndim:
            raise IndexError(f"tensor of rank {self.ndim} indexed with {len(coords)} coordinates")
        return self.offset + sum(int(c) * s for c, s in zip(coords, self.stride))

    def __getitem__(self, index: Any) -> Any:
        return self._storage[self._linear(index)].item()

    def __setitem__(self, index: Any, value: Any) -> None:
        self._storage[self._linear(index)] = value.value if isinstance(value, RuntimeScalar) else value

    def as_numpy(self) -> np.ndarray:
        """Logical values as an ndarray of ``shape`` (a view when the tensor is dense)."""
        if self.is_dense:
            return self._storage.reshape(self.shape)
        window = np.lib.stride_tricks.as_strided(
            self._storage[self.offset:], shape=self.shape, strides=tuple(s * self._storage.itemsize for s in self.stride)
        )
        return np.array(window)

    def tolist(self) -> Any:
        return self.as_numpy().tolist()

    # -- device staging ---------------------------------------------------------------------------
    def device_image(self) -> np.ndarray:
        """Contiguous array in the device encoding of ``dtype`` (bf16 → RNE'd uint16 patterns)."""
        if not self.is_dense:
            raise BackendNotImplementedError("b200 currently requires contiguous runtime tensors without offsets")
        return pack_for_device(self._storage, self.dtype)

    def absorb_device_image(self, image: np.ndarray) -> None:
        self._storage[...] = unpack_from_device(image.reshape(-1), self.dtype)

    # -- whole-tensor DSL methods: trace-only in this package ---------------------------------------
    def load(self) -> "RuntimeTensor":
        raise _no_cpu_runtime("Tensor.load()")

    def store(self, value: Any) -> None:
        raise _no_cpu_runtime("Tensor.store()")

    def _arith(self, *_: Any) -> "RuntimeTensor":
        raise _no_cpu_runtime("host tensor arithmetic")

    __add__ = __radd__ = __sub__ = __rsub__ = __mul__ = __rmul__ = __truediv__ = __rtruediv__ = _arith


Tensor = RuntimeTensor
Shape = tuple


def tensor(data: Any, *, dtype: str | None = None) -> RuntimeTensor:
    return RuntimeTensor.from_data(data, dtype=dtype)


def zeros(shape: tuple[int, ...], *, dtype: str = "f32") -> RuntimeTensor:
    return RuntimeTensor.zeros(shape, dtype=dtype)


def full(shape: tuple[int, ...], fill_value: Any, *, dtype: str = "f32") -> RuntimeTensor:
    result = RuntimeTensor.zeros(shape, dtype=dtype)
    result._storage[...] = fill_value.value if isinstance(fill_value, RuntimeScalar) else fill_value
    return result


def clone(value: RuntimeTensor) -> RuntimeTensor:
    return RuntimeTensor(value._storage.copy(), value.shape, dtype=value.dtype, stride=value.stride, offset=value.offset)


# ---------------------------------------------------------------------------------------------
# borrowed device tensors
# ---------------------------------------------------------------------------------------------
@dataclass(frozen=True)
class TensorHandle:
    capsule: Any
    shape: tuple[int, ...]
    dtype: str
    device_type: int
    device_id: int
    source: Any | None = None
    stride: tuple[int, ...] | None = None
    assumed_align: int | None = None
    dynamic_layout_leading_dim: int | None = None
    raw_address: int | None = None

    def __post_init__(self) -> None:
        object.__setattr__(self, "shape", tuple(int(extent) for extent in self.shape))
        object.__setattr__(self, "dtype", normalize_dtype_name(str(self.dtype)))
        if self.stride is not None:
            object.__setattr__(self, "stride", tuple(int(step) for step in self.stride))

    def mark_layout_dynamic(self, leading_dim: int | None = None) -> "TensorHandle":
        if leading_dim is not None and not 0 <= leading_dim < len(self.shape):
            raise ValueError(f"leading_dim must be within [0, {len(self.shape)})")
        return replace(self, dynamic_layout_leading_dim=leading_dim)

    def data_ptr(self) -> int:
        if self.raw_address is not None:
            return int(self.raw_address)
        getter = getattr(self.source, "data_ptr", None)
        return int(getter()) if callable(getter) else 0

    def __dlpack__(self, stream: Any | None = None):
        exporter = getattr(self.source, "__dlpack__", None)
        if exporter is not None:
            if stream is not None:
                try:
                    return exporter(stream=stream)
                except TypeError:
                    pass
            return exporter()
        if self.capsule is None:
            raise TypeError("tensor handle does not carry a DLPack capsule")
        return self.capsule

    def __dlpack_device__(self) -> tuple[int, int]:
        probe = getattr(self.source, "__dlpack_device__", None)
        if probe is not None:
            return tuple(probe())
        return int(self.device_type), int(self.device_id)

    @property
    def is_contiguous(self) -> bool:
        return self.stride is None or self.stride == row_major_stride(self.shape)


def _export_capsule(value: Any, stream: Any | None) -> Any:
    if stream is None or recording():  # a recording stream cannot wait for the exporter's pending work
        return value.__dlpack__()
    try:
        return value.__dlpack__(stream=stream)
    except TypeError:
        return value.__dlpack__()


def from_dlpack(value: Any, assumed_align: int | None = None, stream: Any | None = None) -> TensorHandle:
    if not (hasattr(value, "__dlpack__") and hasattr(value, "__dlpack_device__")):
        raise TypeError("from_dlpack expects an object implementing __dlpack__ and __dlpack_device__")
    device_type, device_id = value.__dlpack_device__()
    stride = getattr(value, "stride", None)
    if callable(stride):
        stride = stride()
    return TensorHandle(
        capsule=_export_capsule(value, stream),
        shape=tuple(getattr(value, "shape", ())),
        dtype=str(getattr(value, "dtype", "unknown")),
        device_type=int(device_type),
        device_id=int(device_id),
        source=value,
        stride=tuple(int(step) for step in stride) if stride is not None else None,
        assumed_align=assumed_align,
        raw_address=int(value.data_ptr()) if hasattr(value, "data_ptr") else None,
    )


def _is_dlpack(value: Any) -> bool:
    return hasattr(value, "__dlpack__") and hasattr(value, "__dlpack_device__")


def _is_nested_numbers(value: Any) -> bool:
    if not isinstance(value, list) or not value:
        return False
    if isinstance(value[0], list):
        return all(_is_nested_numbers(item) for item in value)
    return all(isinstance(item, (bool, int, float, RuntimeScalar)) for item in value)


def infer_runtime_spec(value: Any) -> tuple[str, tuple[int, ...] | None]:
    """(dtype, shape) of a sample argument; shape ``None`` = scalar; dtype ``python_object`` = opaque."""
    if isinstance(value, RuntimeScalar):
        return value.dtype, None
    if isinstance(value, (RuntimeTensor, TensorHandle)):
        return value.dtype, value.shape
    if _is_dlpack(value):
        dtype, shape = getattr(value, "dtype", None), getattr(value, "shape", None)
        if dtype is not None and shape is not None:
            try:
                return normalize_dtype_name(str(dtype)), tuple(int(extent) for extent in tuple(shape))
            except (TypeError, ValueError):
                pass
    if _is_nested_numbers(value):
        converted = tensor(value)
        return converted.dtype, converted.shape
    for python_type, name in ((bool, "i1"), (int, "index"), (float, "f32")):
        if isinstance(value, python_type):
            return name, None
    return "python_object", None


def normalize_runtime_argument(value: Any, stream: Any | None = None) -> Any:
    """DLPack exporters → ``TensorHandle``, nested number lists → ``RuntimeTensor``, containers recursively."""
    if isinstance(value, (RuntimeScalar, RuntimeTensor, TensorHandle)):
        return value
    if _is_dlpack(value):
        return from_dlpack(value, stream=stream)
    if _is_nested_numbers(value):
        return tensor(value)
    if isinstance(value, list):
        return [normalize_runtime_argument(item, stream=stream) for item in value]
    if isinstance(value, tuple):
        return tuple(normalize_runtime_argument(item, stream=stream) for item in value)
    if isinstance(value, dict):
        return {key: normalize_runtime_argument(item, stream=stream) for key, item in value.items()}
    return value

