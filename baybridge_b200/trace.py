"""Tracer: symbolic scalar/tensor proxies and the IR builder they record into.

A kernel body is executed once on ``ScalarValue`` / ``TensorValue`` proxies;
every overloaded operator appends one ``Operation`` to the active
``IRBuilder``.  Op names, result dtypes, attribute dictionaries and the
``<hint>_<n>`` temporary naming (one counter per kernel) reproduce upstream
``tracing.py:17-711`` so the emitted IR serialises identically.  Unlike
upstream's one-method-per-operator classes, the operator surface here is
generated from the tables below.
"""
from __future__ import annotations

from contextlib import contextmanager
from contextvars import ContextVar
from dataclasses import dataclass, replace
from typing import Any, Iterator

from .errors import CompilationError
from .host_values import RuntimeScalar, resolve_scalar_target_dtype
from .portable_ir import (
    AddressSpace,
    KernelArgument,
    LaunchConfig,
    Layout,
    Operation,
    PortableKernelIR,
    ScalarSpec,
    TensorSpec,
)
from .scalar_types import byte_width, element_type, is_float_dtype, promote_scalar_dtype

import enum


class ReductionOp(str, enum.Enum):
    """Reduction operators of ``Tensor.reduce`` (upstream ``runtime.py:325-333``)."""

    ADD = "add"
    MUL = "mul"
    MAX = "max"
    MIN = "min"
    AND = "and"
    OR = "or"
    XOR = "xor"

    @classmethod
    def coerce(cls, value: "ReductionOp | str") -> "ReductionOp":
        if isinstance(value, cls):
            return value
        try:
            return cls(str(value).lower())
        except ValueError:
            names = ", ".join(member.value for member in cls)
            raise ValueError(f"unsupported reduction op '{value}', expected one of: {names}") from None


def reduction_axes(profile: Any, rank: int) -> tuple[tuple[int, ...], tuple[int, ...]]:
    """``0`` reduces every axis; otherwise a length-``rank`` sequence where ``None`` marks a kept axis."""
    if isinstance(profile, int) and not isinstance(profile, bool) and profile == 0:
        return tuple(range(rank)), ()
    if not isinstance(profile, (tuple, list)):
        raise TypeError("reduction_profile must be 0 or a tuple/list describing kept axes with None")
    if len(profile) != rank:
        raise ValueError(f"reduction_profile must have length {rank} for tensor rank {rank}")
    keep = tuple(axis for axis, item in enumerate(profile) if item is None)
    return tuple(axis for axis in range(rank) if axis not in keep), keep


_ACTIVE: ContextVar["IRBuilder | None"] = ContextVar("baybridge_b200_builder", default=None)

ScalarLike = Any  # ScalarValue | RuntimeScalar | bool | int | float


def active_builder() -> "IRBuilder | None":
    return _ACTIVE.get()


def require_builder() -> "IRBuilder":
    builder = _ACTIVE.get()
    if builder is None:
        raise CompilationError("baybridge operations can only be used while tracing a @kernel or @jit function")
    return builder


@contextmanager
def tracing(builder: "IRBuilder") -> Iterator["IRBuilder"]:
    token = _ACTIVE.set(builder)
    try:
        yield builder
    finally:
        _ACTIVE.reset(token)


def coerce_scalar(value: ScalarLike, preferred_dtype: str | None = None) -> "ScalarValue":
    """Literals and host scalars become ``constant`` ops (typed by ``preferred_dtype`` when given)."""
    if isinstance(value, ScalarValue):
        return value
    if isinstance(value, RuntimeScalar):
        return require_builder().constant(value.value, dtype=preferred_dtype or value.dtype)
    return require_builder().constant(value, dtype=preferred_dtype)


def broadcast_shapes(lhs: tuple[int, ...], rhs: tuple[int, ...]) -> tuple[int, ...]:
    rank = max(len(lhs), len(rhs))
    result = []
    for left, right in zip((1,) * (rank - len(lhs)) + lhs, (1,) * (rank - len(rhs)) + rhs):
        if left != right and 1 not in (left, right):
            raise ValueError(f"tensor shapes are not broadcast-compatible: {lhs} and {rhs}")
        result.append(right if left == 1 else left)
    return tuple(result)


# ---------------------------------------------------------------------------------------------
# scalar proxy
# ---------------------------------------------------------------------------------------------
@dataclass(frozen=True, eq=False)
class ScalarValue:
    name: str
    spec: ScalarSpec

    def __hash__(self) -> int:
        return hash((self.name, self.spec.dtype))

    def __bool__(self) -> bool:
        raise CompilationError(
            "dynamic Python control flow on traced baybridge scalars is not supported; use predication or runtime execution"
        )

    # arithmetic: literals are typed by promotion defaults (int → index, float → f32)
    def _arith(self, op: str, other: ScalarLike, swapped: bool) -> "ScalarValue":
        builder = require_builder()
        peer = coerce_scalar(other)
        lhs, rhs = (peer, self) if swapped else (self, peer)
        dtype = promote_scalar_dtype(lhs.spec.dtype, rhs.spec.dtype)
        return builder.emit_scalar(op, lhs, rhs, spec=ScalarSpec(dtype), name_hint=op)

    # division family: a literal peer adopts this scalar's dtype
    def _divide(self, op: str, other: ScalarLike, swapped: bool) -> "ScalarValue":
        builder = require_builder()
        peer = coerce_scalar(other, preferred_dtype=self.spec.dtype)
        lhs, rhs = (peer, self) if swapped else (self, peer)
        if op == "div":
            dtype = promote_scalar_dtype(lhs.spec.dtype, rhs.spec.dtype)
        else:
            if is_float_dtype(self.spec.dtype) or is_float_dtype(peer.spec.dtype):
                raise TypeError(f"{op} is only supported for integer/index scalars")
            dtype = "index"
        return builder.emit_scalar(op, lhs, rhs, spec=ScalarSpec(dtype), name_hint=op)

    def _compare(self, op: str, other: ScalarLike) -> "ScalarValue":
        builder = require_builder()
        peer = coerce_scalar(other, preferred_dtype=self.spec.dtype)
        return builder.emit_scalar(op, self, peer, spec=ScalarSpec("i1"), name_hint=op)

    def _logic(self, op: str, other: ScalarLike) -> "ScalarValue":
        peer = coerce_scalar(other, preferred_dtype=self.spec.dtype)
        if self.spec.dtype == "i1" and peer.spec.dtype == "i1":
            return require_builder().emit_scalar(op, self, peer, spec=ScalarSpec("i1"), name_hint=op)
        if is_float_dtype(self.spec.dtype) or is_float_dtype(peer.spec.dtype):
            raise TypeError(f"{op} requires integer baybridge scalars")
        dtype = promote_scalar_dtype(self.spec.dtype, peer.spec.dtype)
        return require_builder().emit_scalar("bit" + op, self, peer, spec=ScalarSpec(dtype), name_hint="bit" + op)

    def _unary(self, op: str) -> "ScalarValue":
        return require_builder().emit_scalar(op, self, spec=ScalarSpec(self.spec.dtype), name_hint=op)

    def __neg__(self) -> "ScalarValue":
        return self._unary("neg")

    def __abs__(self) -> "ScalarValue":
        if self.spec.dtype == "i1":
            raise TypeError("scalar abs requires non-boolean baybridge scalars")
        return self._unary("abs")

    def __invert__(self) -> "ScalarValue":
        if is_float_dtype(self.spec.dtype):
            raise TypeError("bitwise invert is only supported for integer baybridge scalars")
        return self._unary("bitnot")

    def to(self, target: object) -> "ScalarValue":
        dtype = resolve_scalar_target_dtype(target)
        if dtype == self.spec.dtype:
            return self
        return require_builder().emit_scalar(
            "cast",
            self,
            spec=ScalarSpec(dtype),
            attrs={"source_dtype": self.spec.dtype, "target_dtype": dtype},
            name_hint="cast",
        )


def _install_scalar_operators() -> None:
    def arith(op: str, swapped: bool):
        return lambda self, other: self._arith(op, other, swapped)

    def divide(op: str, swapped: bool):
        return lambda self, other: self._divide(op, other, swapped)

    for dunder, op in (("add", "add"), ("sub", "sub"), ("mul", "mul")):
        setattr(ScalarValue, f"__{dunder}__", arith(op, False))
        setattr(ScalarValue, f"__r{dunder}__", arith(op, True))
    for dunder, op in (("truediv", "div"), ("floordiv", "floordiv"), ("mod", "mod")):
        setattr(ScalarValue, f"__{dunder}__", divide(op, False))
        setattr(ScalarValue, f"__r{dunder}__", divide(op, True))
    for dunder in ("lt", "le", "gt", "ge"):
        setattr(ScalarValue, f"__{dunder}__", (lambda op: lambda self, other: self._compare(op, other))(f"cmp_{dunder}"))
    for dunder in ("eq", "ne"):
        def equality(self, other, _op=f"cmp_{dunder}"):
            if not isinstance(other, (ScalarValue, RuntimeScalar, bool, int, float)):
                raise TypeError("comparisons are only supported against baybridge scalar values")
            return self._compare(_op, other)
        setattr(ScalarValue, f"__{dunder}__", equality)
    for dunder in ("and", "or", "xor"):
        setattr(ScalarValue, f"__{dunder}__", (lambda op: lambda self, other: self._logic(op, other))(dunder))


_install_scalar_operators()


# ---------------------------------------------------------------------------------------------
# tensor proxy
# ---------------------------------------------------------------------------------------------
def _register_spec(shape: tuple[int, ...], dtype: str) -> TensorSpec:
    return TensorSpec(shape=shape, dtype=dtype, address_space=AddressSpace.REGISTER)


@dataclass(frozen=True, eq=False)
class TensorValue:
    name: str
    spec: TensorSpec

    def __hash__(self) -> int:
        return hash((self.name, self.spec.shape, self.spec.dtype))

    @property
    def shape(self) -> tuple[int, ...]:
        return self.spec.shape

    @property
    def ndim(self) -> int:
        return len(self.spec.shape)

    @property
    def dtype(self) -> str:
        return self.spec.dtype

    @property
    def element_type(self):
        return element_type(self.spec.dtype)

    @property
    def type(self) -> str:
        return f"Tensor(shape={self.spec.shape}, dtype={self.spec.dtype})"

    @property
    def layout(self) -> Layout:
        return self.spec.resolved_layout()

    # element access → scalar load/store ops
    def __getitem__(self, index: Any) -> ScalarValue:
        from .dsl import load

        return load(self, index)

    def __setitem__(self, index: Any, value: ScalarValue) -> None:
        from .dsl import store

        store(value, self, index)

    # whole-tensor SSA
    def load(self) -> "TensorValue":
        builder = require_builder()
        staged = builder.make_tensor(
            f"{self.name}_load_{builder.next_temp()}", _register_spec(self.spec.shape, self.spec.dtype)
        )
        builder.emit_void("copy", self, staged)
        return staged

    def store(self, value: "TensorValue | ScalarValue") -> None:
        if not isinstance(value, TensorValue):
            raise CompilationError("whole-tensor store requires a baybridge tensor value while tracing")
        if self.spec.shape != value.spec.shape:
            raise ValueError(f"tensor shapes must match, got {self.spec.shape} and {value.spec.shape}")
        if self.spec.dtype != value.spec.dtype:
            raise ValueError(f"tensor dtypes must match, got {self.spec.dtype} and {value.spec.dtype}")
        require_builder().emit_void("copy", value, self)

    def fill(self, value: ScalarLike) -> None:
        builder = require_builder()
        scalar = value if isinstance(value, ScalarValue) else builder.constant(value, dtype=self.spec.dtype)
        if scalar.spec.dtype != self.spec.dtype:
            raise ValueError(f"fill expects dtype {self.spec.dtype}, got {scalar.spec.dtype}")
        builder.emit_void("fill", self, scalar)

    def reduce(self, op: "ReductionOp | str", init_value: ScalarLike, *, reduction_profile: Any = 0):
        """Reduce over the axes ``reduction_profile`` does not keep; returns a scalar when none is kept."""
        reduction = ReductionOp.coerce(op)
        _, keep = reduction_axes(reduction_profile, self.ndim)
        builder = require_builder()
        init = init_value if isinstance(init_value, ScalarValue) else builder.constant(init_value, dtype=self.spec.dtype)
        if init.spec.dtype != self.spec.dtype:
            raise ValueError(f"reduce expects init value dtype {self.spec.dtype}, got {init.spec.dtype}")
        name = f"reduce_{reduction.value}"
        attrs = {"reduction_profile": list(reduction_profile) if isinstance(reduction_profile, (tuple, list)) else reduction_profile}
        if not keep:
            return builder.emit_scalar(name, self, init, spec=ScalarSpec(self.spec.dtype), attrs=attrs, name_hint=name)
        kept_shape = tuple(self.spec.shape[axis] for axis in keep)
        return builder.emit_tensor(name, self, init, spec=_register_spec(kept_shape, self.spec.dtype), attrs=attrs, name_hint=name)

    def broadcast_to(self, shape: tuple[int, ...]) -> "TensorValue":
        target = tuple(int(extent) for extent in shape)
        if target == self.spec.shape:
            return self
        source = self.spec.resolved_layout()
        if len(target) < len(source.shape):
            raise ValueError(f"cannot broadcast rank-{len(source.shape)} tensor to rank-{len(target)} shape {target}")
        pad = len(target) - len(source.shape)
        stride = []
        for have, want, step in zip((1,) * pad + source.shape, target, (0,) * pad + source.stride):
            if have != want and have != 1:
                raise ValueError(f"cannot broadcast shape {source.shape} to {target}")
            stride.append(step if have == want else 0)
        return require_builder().emit_tensor(
            "broadcast_to",
            self,
            spec=TensorSpec(target, self.spec.dtype, Layout(target, tuple(stride), source.swizzle), self.spec.address_space),
            attrs={"target_shape": list(target)},
            name_hint=f"{self.name}_broadcast",
        )

    def _elementwise(self, op: str, other: Any, result_dtype: str | None) -> "TensorValue":
        builder = require_builder()
        if isinstance(other, TensorValue):
            shape = broadcast_shapes(self.spec.shape, other.spec.shape)
            lhs, rhs = self.broadcast_to(shape), other.broadcast_to(shape)
            if self.spec.dtype != other.spec.dtype:
                raise ValueError(f"tensor dtypes must match, got {self.spec.dtype} and {other.spec.dtype}")
            operands: tuple[Any, ...] = (lhs, rhs)
        else:
            scalar = other if isinstance(other, ScalarValue) else builder.constant(other, dtype=self.spec.dtype)
            if scalar.spec.dtype != self.spec.dtype:
                raise ValueError(f"{op} scalar dtype must match {self.spec.dtype}, got {scalar.spec.dtype}")
            shape, operands = self.spec.shape, (self, scalar)
        return builder.emit_tensor(op, *operands, spec=_register_spec(shape, result_dtype or self.spec.dtype), name_hint=op)

    def _unary(self, op: str) -> "TensorValue":
        return require_builder().emit_tensor(op, self, spec=_register_spec(self.spec.shape, self.spec.dtype), name_hint=op)

    def __neg__(self) -> "TensorValue":
        if self.spec.dtype == "i1":
            raise TypeError("tensor neg requires non-boolean baybridge tensors")
        return self._unary("tensor_neg")

    def __abs__(self) -> "TensorValue":
        if self.spec.dtype == "i1":
            raise TypeError("tensor abs requires non-boolean baybridge tensors")
        return self._unary("tensor_abs")

    def __invert__(self) -> "TensorValue":
        if is_float_dtype(self.spec.dtype):
            raise TypeError("tensor bitnot requires integer baybridge tensors")
        return self._unary("tensor_bitnot")


def _install_tensor_operators() -> None:
    for dunder in ("add", "sub", "mul"):
        setattr(TensorValue, f"__{dunder}__", (lambda op: lambda self, other: self._elementwise(op, other, None))(f"tensor_{dunder}"))
    TensorValue.__truediv__ = lambda self, other: self._elementwise("tensor_div", other, None)
    for dunder in ("and", "or", "xor"):
        def bitwise(self, other, _name=dunder):
            if is_float_dtype(self.spec.dtype):
                raise TypeError(f"tensor bit{_name} requires integer baybridge tensors")
            return self._elementwise(f"tensor_bit{_name}", other, None)
        setattr(TensorValue, f"__{dunder}__", bitwise)
    for dunder in ("lt", "le", "gt", "ge", "eq", "ne"):
        def compare(self, other, _op=f"cmp_{dunder}", _strict=dunder in ("eq", "ne")):
            if _strict and not isinstance(other, (TensorValue, ScalarValue, RuntimeScalar, int, float)):
                raise TypeError("tensor comparisons are only supported against baybridge tensor/scalar values")
            return self._elementwise(_op, other, "i1")
        setattr(TensorValue, f"__{dunder}__", compare)


_install_tensor_operators()


# ---------------------------------------------------------------------------------------------
# builder
# ---------------------------------------------------------------------------------------------
class IRBuilder:
    """Accumulates arguments and operations for one kernel and numbers its temporaries."""

    def __init__(self, kernel_name: str, *, launch: LaunchConfig | None = None):
        self.kernel_name = kernel_name
        self.launch = launch or LaunchConfig()
        self.arguments: list[KernelArgument] = []
        self.operations: list[Operation] = []
        self.metadata: dict[str, object] = {
            "dialect": "baybridge.portable",
            "stage": "portable_ir",
            "launch": self.launch.to_dict(),
        }
        self._temp_index = 0
        self._dynamic_shared_mem_bytes = 0

    def next_temp(self) -> int:
        self._temp_index += 1
        return self._temp_index

    def next_temp_preview(self) -> int:
        """The number the next temporary will get, without taking it."""
        return self._temp_index + 1

    def bind_argument(self, name: str, spec: TensorSpec | ScalarSpec) -> TensorValue | ScalarValue:
        is_tensor = isinstance(spec, TensorSpec)
        self.arguments.append(KernelArgument(name=name, kind="tensor" if is_tensor else "scalar", spec=spec))
        return TensorValue(name, spec) if is_tensor else ScalarValue(name, spec)

    def _record(self, op: str, inputs: tuple[Any, ...], outputs: tuple[str, ...], attrs: dict[str, object]) -> None:
        self.operations.append(Operation(op, tuple(value.name for value in inputs), outputs, attrs))

    def _result(self, kind: str, op: str, inputs, spec, attrs, name_hint: str) -> str:
        name = f"{name_hint}_{self.next_temp()}"
        merged: dict[str, object] = {"result": {"kind": kind, **spec.to_dict()}}
        merged.update(attrs or {})
        self._record(op, inputs, (name,), merged)
        return name

    def emit_scalar(self, op: str, *inputs: Any, spec: ScalarSpec, attrs: dict[str, object] | None = None,
                    name_hint: str = "scalar") -> ScalarValue:
        return ScalarValue(self._result("scalar", op, inputs, spec, attrs, name_hint), spec)

    def emit_tensor(self, op: str, *inputs: Any, spec: TensorSpec, attrs: dict[str, object] | None = None,
                    name_hint: str = "tmp") -> TensorValue:
        return TensorValue(self._result("tensor", op, inputs, spec, attrs, name_hint), spec)

    def emit_void(self, op: str, *inputs: Any, attrs: dict[str, object] | None = None) -> None:
        self._record(op, inputs, (), dict(attrs or {}))

    def constant(self, value: Any, *, dtype: str | None = None) -> ScalarValue:
        if isinstance(value, RuntimeScalar):
            dtype = dtype or value.dtype
            value = value.value
        if dtype is None:
            for python_type, name in ((bool, "i1"), (int, "index"), (float, "f32")):
                if isinstance(value, python_type):
                    dtype = name
                    break
            else:
                raise TypeError(f"unsupported scalar literal type: {type(value).__name__}")
        return self.emit_scalar("constant", spec=ScalarSpec(dtype), attrs={"value": value}, name_hint="cst")

    def make_tensor(self, name: str, spec: TensorSpec, *, dynamic_shared: bool = False,
                    byte_alignment: int | None = None, byte_offset: int | None = None) -> TensorValue:
        attrs: dict[str, object] = {
            "shape": list(spec.shape),
            "dtype": spec.dtype,
            "address_space": spec.address_space.value,
            "layout": spec.resolved_layout().to_dict(),
        }
        if dynamic_shared:
            if spec.address_space is not AddressSpace.SHARED:
                raise ValueError("dynamic shared tensors must use baybridge.AddressSpace.SHARED")
            alignment = max(1, int(byte_alignment or byte_width(spec.dtype)))
            offset = self.reserve_dynamic_shared(
                spec.numel * byte_width(spec.dtype), byte_alignment=alignment, byte_offset=byte_offset
            )
            attrs.update(dynamic_shared=True, byte_offset=offset, byte_alignment=alignment)
        self.operations.append(Operation("make_tensor", (), (name,), attrs))
        return TensorValue(name, spec)

    def reserve_dynamic_shared(self, size_bytes: int, *, byte_alignment: int | None = None,
                               byte_offset: int | None = None) -> int:
        if size_bytes < 0:
            raise ValueError("dynamic shared reservation size must be >= 0")
        alignment = max(1, int(byte_alignment or 1))
        if byte_offset is None:
            offset = -(-self._dynamic_shared_mem_bytes // alignment) * alignment
        else:
            offset = int(byte_offset)
            if offset < 0:
                raise ValueError("dynamic shared reservation offset must be >= 0")
            if offset % alignment:
                raise ValueError("dynamic shared reservation offset must respect the requested alignment")
        self._dynamic_shared_mem_bytes = max(self._dynamic_shared_mem_bytes, offset + size_bytes)
        return offset

    def finalize(self) -> PortableKernelIR:
        launch = self.launch
        if self._dynamic_shared_mem_bytes > launch.shared_mem_bytes:
            launch = replace(launch, shared_mem_bytes=self._dynamic_shared_mem_bytes)
        metadata = dict(self.metadata)
        metadata["launch"] = launch.to_dict()
        if self._dynamic_shared_mem_bytes:
            metadata["inferred_shared_mem_bytes"] = self._dynamic_shared_mem_bytes
        return PortableKernelIR(self.kernel_name, tuple(self.arguments), tuple(self.operations), launch, metadata)
