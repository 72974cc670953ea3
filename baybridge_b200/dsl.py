"""The DSL entry points a kernel body calls.

This is the slice of upstream ``frontend.py`` / ``math.py`` that the b200 hot
path exercises: ``kernel``/``jit`` decorators and launch objects
(``frontend.py:756-864``), topology builtins (``:2038-2117``), scalar
``load``/``store`` with optional predicates (``:2931-3019``), whole-tensor
``copy`` (``:3357-3415``), ``where`` (``:2538-2600``), the ``math`` namespace
(``math.py:13-76``), and the explicit ops ``gemm``/``mma`` (``frontend.py:3684-3740,
4052-4091``), ``rmsnorm`` (``:3828-3874``) and ``attention`` (``:3877-3968``).

Upstream entry points are dual-mode (emit IR while tracing, otherwise execute
on the CPU).  Here they are trace-only; calling one with host tensors outside
``compile`` raises, because results are only ever produced by the b200 device
kernels.  The exception is *launching*: ``kernel(args).launch(grid=..,
block=..)`` and calling a ``@jit`` wrapper outside a trace compile for the
``b200`` backend (memoised) and run on the device.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable

from .errors import BackendNotImplementedError, CompilationError
from .host_values import RuntimeScalar, RuntimeTensor, normalize_runtime_argument
from .portable_ir import AddressSpace, LaunchConfig, ScalarSpec, TensorSpec
from .scalar_types import byte_width
from .trace import ScalarValue, TensorValue, active_builder, broadcast_shapes, coerce_scalar, require_builder


# ---------------------------------------------------------------------------------------------
# kernel definitions and launches
# ---------------------------------------------------------------------------------------------
@dataclass(frozen=True)
class KernelDefinition:
    fn: Callable[..., Any]
    kind: str  # "kernel" (device body) | "jit" (host wrapper)
    launch: LaunchConfig

    @property
    def __name__(self) -> str:  # type: ignore[override]
        return self.fn.__name__

    def __call__(self, *args: Any, **kwargs: Any) -> Any:
        args = tuple(normalize_runtime_argument(arg) for arg in args)
        kwargs = {name: normalize_runtime_argument(value) for name, value in kwargs.items()}
        if self.kind == "kernel":
            return KernelLaunch(self, args, kwargs)
        if active_builder() is not None:
            return self.fn(*args, **kwargs)
        # a @jit wrapper called eagerly: compile for the device and run
        from .driver import run_on_device

        return run_on_device(self, args, kwargs)

    def set_name_prefix(self, prefix: str) -> None:
        del prefix


class TraceKernelLaunch(CompilationError):
    """Raised by ``.launch()`` under tracing so ``compile`` can re-trace the launched kernel."""

    def __init__(self, definition: KernelDefinition, args: tuple[Any, ...], kwargs: dict[str, Any], launch: LaunchConfig):
        super().__init__("kernel launch tracing is being handled by baybridge compile")
        self.definition, self.args, self.kwargs, self.launch = definition, args, kwargs, launch


@dataclass(frozen=True)
class KernelLaunch:
    definition: KernelDefinition
    args: tuple[Any, ...]
    kwargs: dict[str, Any]

    def launch(self, *, grid, block, cluster=(1, 1, 1), shared_mem_bytes: int = 0, cooperative: bool = False,
               stream: Any | None = None) -> None:
        config = LaunchConfig(tuple(grid), tuple(block), tuple(cluster), shared_mem_bytes, cooperative)
        if active_builder() is not None:
            raise TraceKernelLaunch(self.definition, self.args, self.kwargs, config)
        from .driver import run_on_device

        run_on_device(KernelDefinition(self.definition.fn, "kernel", config), self.args, self.kwargs, stream=stream)


def _decorator(kind: str):
    def decorate(fn: Callable[..., Any] | None = None, *, launch: LaunchConfig | None = None):
        chosen = launch or LaunchConfig()
        if fn is None:
            return lambda inner: KernelDefinition(fn=inner, kind=kind, launch=chosen)
        return KernelDefinition(fn=fn, kind=kind, launch=chosen)

    decorate.__name__ = kind
    return decorate


kernel = _decorator("kernel")
jit = _decorator("jit")


# ---------------------------------------------------------------------------------------------
# topology builtins
# ---------------------------------------------------------------------------------------------
def _topology(op: str):
    def builtin(axis: str = "x") -> ScalarValue:
        if axis not in ("x", "y", "z"):
            raise ValueError("axis must be one of: x, y, z")
        return require_builder().emit_scalar(op, spec=ScalarSpec("index"), attrs={"axis": axis}, name_hint=f"{op}_{axis}")

    builtin.__name__ = op
    return builtin


program_id = _topology("program_id")
block_idx = _topology("block_idx")
thread_idx = _topology("thread_idx")
block_dim = _topology("block_dim")
grid_dim = _topology("grid_dim")


def lane_id() -> ScalarValue:
    return require_builder().emit_scalar("lane_id", spec=ScalarSpec("index"), name_hint="lane_id")


class _ArchNamespace:
    """``cute.arch.thread_idx()`` … return (x, y, z) triples; each component is its own IR op."""

    @staticmethod
    def _triple(builtin) -> tuple[ScalarValue, ScalarValue, ScalarValue]:
        return builtin("x"), builtin("y"), builtin("z")

    def thread_idx(self):
        return self._triple(thread_idx)

    def block_idx(self):
        return self._triple(block_idx)

    def block_dim(self):
        return self._triple(block_dim)

    def grid_dim(self):
        return self._triple(grid_dim)

    @staticmethod
    def lane_id():
        return lane_id()


arch = _ArchNamespace()


def dim(tensor: TensorValue | RuntimeTensor, axis: int) -> ScalarValue | int:
    rank = tensor.ndim
    if not 0 <= axis < rank:
        raise ValueError(f"axis {axis} is out of range for tensor rank {rank}")
    if isinstance(tensor, RuntimeTensor):
        return tensor.shape[axis]
    return require_builder().emit_scalar(
        "tensor_dim",
        tensor,
        spec=ScalarSpec("index"),
        attrs={"axis": axis, "value": tensor.spec.shape[axis]},
        name_hint=f"{tensor.name}_dim_{axis}",
    )


# ---------------------------------------------------------------------------------------------
# scalar element access
# ---------------------------------------------------------------------------------------------
def _index_operands(tensor: TensorValue, index: Any, what: str) -> tuple[ScalarValue, ...]:
    if not isinstance(tensor, TensorValue):
        raise BackendNotImplementedError(
            f"{what} on a host tensor would execute on the host; baybridge_b200 has no CPU runtime"
        )
    builder = require_builder()
    operands = []
    for item in index if isinstance(index, tuple) else (index,):
        if isinstance(item, ScalarValue):
            operands.append(item)
        elif isinstance(item, int) and not isinstance(item, bool):
            operands.append(builder.constant(item))
        else:
            raise TypeError("indices must be ScalarValue, int, or tuples of those values")
    if len(operands) != tensor.ndim:
        raise ValueError(f"{what} expects {tensor.ndim} indices for tensor rank {tensor.ndim}")
    return tuple(operands)


def _checked_predicate(predicate: ScalarValue | None) -> ScalarValue | None:
    if predicate is not None and predicate.spec.dtype != "i1":
        raise ValueError("predicate values must have dtype i1")
    return predicate


def load(tensor: TensorValue, index: Any, *, predicate: ScalarValue | None = None,
         else_value: ScalarValue | int | float | None = None) -> ScalarValue:
    operands = _index_operands(tensor, index, "load")
    guard = _checked_predicate(predicate)
    builder = require_builder()
    dtype = tensor.spec.dtype
    if guard is None:
        return builder.emit_scalar(
            "load", tensor, *operands, spec=ScalarSpec(dtype), attrs={"rank": len(operands)}, name_hint=f"{tensor.name}_val"
        )
    fallback = else_value if else_value is not None else 0
    if not isinstance(fallback, ScalarValue):
        fallback = builder.constant(fallback, dtype=dtype)
    if fallback.spec.dtype != dtype:
        raise ValueError(f"else_value dtype mismatch: value has {fallback.spec.dtype}, tensor expects {dtype}")
    return builder.emit_scalar(
        "masked_load", tensor, *operands, guard, fallback,
        spec=ScalarSpec(dtype), attrs={"rank": len(operands)}, name_hint=f"{tensor.name}_val",
    )


def store(value: ScalarValue, tensor: TensorValue, index: Any, *, predicate: ScalarValue | None = None) -> None:
    operands = _index_operands(tensor, index, "store")
    if not isinstance(value, ScalarValue):
        raise TypeError("traced store values must be baybridge scalar expressions")
    if value.spec.dtype != tensor.spec.dtype:
        raise ValueError(f"store dtype mismatch: value has {value.spec.dtype}, tensor expects {tensor.spec.dtype}")
    guard = _checked_predicate(predicate)
    builder = require_builder()
    if guard is None:
        builder.emit_void("store", value, tensor, *operands, attrs={"rank": len(operands)})
    else:
        builder.emit_void("masked_store", value, tensor, *operands, guard, attrs={"rank": len(operands)})


class ReductionOp:
    """Reduction kinds of a reducing copy (upstream ``frontend.py:76-84``); the IR carries the lower-case string."""
    ADD, INC, DEC, MIN, MAX, AND, OR, XOR = "add", "inc", "dec", "min", "max", "and", "or", "xor"


class CtaGroup:
    """Upstream ``nvgpu.tcgen05.CtaGroup``: recorded on copy ops as the strings ``"one"`` / ``"two"``."""
    ONE, TWO = "one", "two"


@dataclass(frozen=True)
class CopyReduceBulkTensorTileS2GOp:
    """``dst = dst (op) src`` element by element (upstream ``frontend.py:115-121``): the traced op is ``copy_reduce``."""
    reduction_kind: Any = ReductionOp.ADD
    cta_group: Any = None

    def __post_init__(self) -> None:
        kind = str(getattr(self.reduction_kind, "value", self.reduction_kind)).lower()
        if kind not in ("add", "inc", "dec", "min", "max", "and", "or", "xor"):
            raise ValueError(f"unsupported cpasync reduction op '{self.reduction_kind}'")
        object.__setattr__(self, "reduction_kind", kind)


@dataclass(frozen=True)
class CopyAtom:
    """A copy op bound to an element type (upstream ``make_copy_atom``, ``frontend.py:3123-3127``)."""
    op: Any
    value_type: str
    num_bits_per_copy: int

    @property
    def vector_bytes(self) -> int:
        return self.num_bits_per_copy // 8


def make_copy_atom(op: Any, value_type: Any, *, num_bits_per_copy: int | None = None) -> CopyAtom:
    from .scalar_types import resolve_element_type_name

    resolved = resolve_element_type_name(value_type)
    if num_bits_per_copy is None:
        num_bits_per_copy = 8 * byte_width(resolved)
    return CopyAtom(op=op, value_type=resolved, num_bits_per_copy=int(num_bits_per_copy))


def copy(*args: Any, vector_bytes: int | None = None) -> None:
    """Whole-tensor copy op, ``copy(src, dst)`` or ``copy(copy_atom, src, dst)`` (upstream ``frontend.py:3358-3414``).
    ``vector_bytes`` and the atom's attributes are recorded exactly as upstream records them; an atom built on
    ``CopyReduceBulkTensorTileS2GOp`` traces the read-modify-write op ``copy_reduce``."""
    atom = None
    if len(args) == 2:
        src, dst = args
    elif len(args) == 3 and isinstance(args[0], CopyAtom):
        atom, src, dst = args
    else:
        raise TypeError("copy expects (src, dst) or (copy_atom, src, dst)")
    if not (isinstance(src, TensorValue) and isinstance(dst, TensorValue)):
        raise BackendNotImplementedError("copy on host tensors would execute on the host; baybridge_b200 has no CPU runtime")
    if atom is not None and vector_bytes is None:
        vector_bytes = atom.vector_bytes
    attrs: dict[str, Any] = {"vector_bytes": vector_bytes}
    if atom is None:
        require_builder().emit_void("copy", src, dst, attrs=attrs)
        return
    if not isinstance(atom.op, CopyReduceBulkTensorTileS2GOp):
        raise BackendNotImplementedError(f"copy atoms over {type(atom.op).__name__} are outside the b200 hot path")
    attrs.update(copy_variant="cpasync_tma_s2g_reduce", cta_group=atom.op.cta_group, reduction=atom.op.reduction_kind)
    require_builder().emit_void("copy_reduce", src, dst, attrs=attrs)


def make_tensor(name: str, shape: tuple[int, ...] | None = None, dtype: str | None = None, *,
                layout=None, address_space: AddressSpace | str = AddressSpace.REGISTER) -> TensorValue:
    if not isinstance(name, str):
        raise TypeError("make_tensor expects a tensor name")
    if shape is None or dtype is None:
        raise TypeError("make_tensor(name, ...) requires shape=... and dtype=...")
    builder = require_builder()
    taken = {argument.name for argument in builder.arguments}
    for operation in builder.operations:
        taken.update(operation.outputs)
    unique = f"{name}_{builder.next_temp()}" if name in taken else name
    return builder.make_tensor(unique, TensorSpec(tuple(shape), dtype, layout, address_space))


# ---------------------------------------------------------------------------------------------
# register tensors filled with a constant (``frontend.py:2803-2854`` upstream)
# ---------------------------------------------------------------------------------------------
def empty_like(value: TensorValue, dtype: str | None = None) -> TensorValue:
    if not isinstance(value, TensorValue):
        raise BackendNotImplementedError("empty_like on a host tensor would execute on the host; baybridge_b200 has no CPU runtime")
    return make_tensor("empty_like", tuple(value.spec.shape), dtype or value.spec.dtype, layout=value.spec.layout,
                       address_space=AddressSpace.REGISTER)


def full_like(value: TensorValue, fill_value: Any, dtype: str | None = None) -> TensorValue:
    target = empty_like(value, dtype=dtype)
    target.fill(fill_value)
    return target


def zeros_like(value: TensorValue, dtype: str | None = None) -> TensorValue:
    return full_like(value, 0, dtype=dtype or value.spec.dtype)


def ones_like(value: TensorValue, dtype: str | None = None) -> TensorValue:
    return full_like(value, 1, dtype=dtype or value.spec.dtype)


def full(shape: tuple[int, ...], fill_value: Any, *, dtype: str = "f32") -> TensorValue | RuntimeTensor:
    """Inside a traced body: a register tensor filled with ``fill_value``.  Outside: a host tensor container."""
    builder = active_builder()
    if builder is None:
        from .host_values import full as host_full

        return host_full(shape, fill_value, dtype=dtype)
    tensor = builder.make_tensor(f"full_{builder.next_temp_preview()}",
                                 TensorSpec(tuple(int(extent) for extent in shape), str(dtype), None, AddressSpace.REGISTER))
    tensor.fill(fill_value)
    return tensor


# ---------------------------------------------------------------------------------------------
# tile views and barriers
# ---------------------------------------------------------------------------------------------
_DEFAULT_AXES = {1: ("x",), 2: ("y", "x"), 3: ("z", "y", "x")}


def partition(tensor: TensorValue, tile: tuple[int, ...], *, offset: tuple[Any, ...] | None = None,
              policy: str = "blocked") -> TensorValue:
    """A ``tile``-shaped view of ``tensor`` starting at ``offset`` (default: the origin); the view keeps
    the source's strides.  Recorded as a ``partition`` op (``frontend.py:3553-3607`` upstream)."""
    if not isinstance(tensor, TensorValue):
        raise BackendNotImplementedError("partition on a host tensor would execute on the host; baybridge_b200 has no CPU runtime")
    shape = tensor.spec.shape
    if len(tile) != len(shape):
        raise ValueError(f"partition expects a tile rank of {len(shape)}")
    if any(step <= 0 for step in tile):
        raise ValueError("partition tile dimensions must be > 0")
    if any(step > extent for step, extent in zip(tile, shape)):
        raise ValueError("partition tile dimensions cannot exceed the source tensor shape")
    builder = require_builder()
    operands: list[ScalarValue] = []
    if offset is not None:
        if len(offset) != len(shape):
            raise ValueError(f"offset expects {len(shape)} values for tensor rank {len(shape)}")
        for axis, item in enumerate(offset):
            if isinstance(item, ScalarValue):
                operands.append(item)
                continue
            if not isinstance(item, int) or isinstance(item, bool):
                raise TypeError("partition offsets must be ScalarValue or int")
            if item < 0:
                raise ValueError("partition offsets must be >= 0")
            if item + tile[axis] > shape[axis]:
                raise ValueError("static partition offsets plus tile dimensions must stay within the source tensor shape")
            operands.append(builder.constant(item))
    source_layout = tensor.spec.resolved_layout()
    view_layout = type(source_layout)(shape=tuple(tile), stride=source_layout.stride, swizzle=source_layout.swizzle)
    view_spec = TensorSpec(tuple(tile), tensor.spec.dtype, view_layout, tensor.spec.address_space)
    return builder.emit_tensor("partition", tensor, *operands, spec=view_spec,
                               attrs={"tile": list(tile), "policy": policy}, name_hint=f"{tensor.name}_part")


def _axes_for(rank: int, axes: tuple[str, ...] | None) -> tuple[str, ...]:
    if axes is None:
        if rank not in _DEFAULT_AXES:
            raise ValueError("default execution axes are only defined for ranks 1, 2, and 3")
        axes = _DEFAULT_AXES[rank]
    if len(axes) != rank:
        raise ValueError(f"axes must have length {rank} for tensor rank {rank}")
    for axis in axes:
        if axis not in ("x", "y", "z"):
            raise ValueError("axis must be one of: x, y, z")
    return tuple(axes)


def partition_program(tensor: TensorValue, tile: tuple[int, ...], *, axes: tuple[str, ...] | None = None,
                      policy: str = "blocked") -> TensorValue:
    """The tile owned by this program: ``offset[d] = program_id(axes[d]) * tile[d]``."""
    offsets = tuple(program_id(axis) * step for axis, step in zip(_axes_for(len(tile), axes), tile))
    return partition(tensor, tile, offset=offsets, policy=policy)


def partition_thread(tensor: TensorValue, tile: tuple[int, ...], *, axes: tuple[str, ...] | None = None,
                     policy: str = "blocked") -> TensorValue:
    """The tile owned by this thread: ``offset[d] = thread_idx(axes[d]) * tile[d]``."""
    offsets = tuple(thread_idx(axis) * step for axis, step in zip(_axes_for(len(tile), axes), tile))
    return partition(tensor, tile, offset=offsets, policy=policy)


def barrier(*, kind: str = "block", **attrs: Any) -> None:
    if kind not in {"block", "grid", "warp"}:
        raise ValueError("barrier kind must be 'block', 'grid', or 'warp'")
    require_builder().emit_void("barrier", attrs={"kind": kind, **attrs})


# ---------------------------------------------------------------------------------------------
# select and math
# ---------------------------------------------------------------------------------------------
def where(predicate: Any, true_value: Any, false_value: Any, *, loc: Any = None, ip: Any = None) -> Any:
    del loc, ip
    builder = require_builder()
    if isinstance(predicate, ScalarValue):
        if predicate.spec.dtype != "i1":
            raise ValueError("where requires an i1 predicate")
        if isinstance(true_value, ScalarValue):
            chosen = true_value
        else:
            hint = false_value.spec.dtype if isinstance(false_value, ScalarValue) else None
            chosen = builder.constant(true_value, dtype=hint)
        other = false_value if isinstance(false_value, ScalarValue) else builder.constant(false_value, dtype=chosen.spec.dtype)
        if chosen.spec.dtype != other.spec.dtype:
            raise ValueError("where requires the true and false branches to have the same dtype")
        return builder.emit_scalar("select", predicate, chosen, other, spec=ScalarSpec(chosen.spec.dtype), name_hint="select")
    if isinstance(predicate, TensorValue):
        if predicate.spec.dtype != "i1":
            raise ValueError("where requires an i1 predicate tensor")
        # the branch dtype follows the tensor branch (the true one first), scalars and literals adapt to it
        # (upstream frontend.py:2571-2625)
        required = next((v.spec.dtype for v in (true_value, false_value) if isinstance(v, TensorValue)), None)

        def branch(value: Any, wanted: str | None) -> Any:
            if isinstance(value, TensorValue):
                if value.spec.shape != predicate.spec.shape:
                    value = value.broadcast_to(predicate.spec.shape)
                if wanted is not None and value.spec.dtype != wanted:
                    raise ValueError(f"where tensor branch dtype must match {wanted}, got {value.spec.dtype}")
                return value
            if not isinstance(value, ScalarValue):
                value = builder.constant(value) if wanted is None else builder.constant(value, dtype=wanted)
            if wanted is not None and value.spec.dtype != wanted:
                raise ValueError(f"where scalar branch dtype must match {wanted}, got {value.spec.dtype}")
            return value

        chosen = branch(true_value, required)
        other = branch(false_value, chosen.spec.dtype)
        if chosen.spec.dtype != other.spec.dtype:
            raise ValueError("where requires the true and false branches to have the same dtype")
        if not isinstance(chosen, TensorValue) and not isinstance(other, TensorValue):
            raise TypeError("where with a traced tensor predicate requires at least one tensor branch")
        return builder.emit_tensor(
            "tensor_select", predicate, chosen, other,
            spec=TensorSpec(predicate.spec.shape, chosen.spec.dtype, address_space=AddressSpace.REGISTER),
            name_hint="tensor_select",
        )
    raise BackendNotImplementedError("where on host values would execute on the host; baybridge_b200 has no CPU runtime")


def _float_only(value: Any, op: str, what: str) -> None:
    if not value.spec.dtype.startswith("f"):
        raise TypeError(f"{op} requires a floating-point {what}")


def _unary_math(op: str):
    def apply(value: Any) -> Any:
        if isinstance(value, ScalarValue):
            _float_only(value, op, "scalar")
            return require_builder().emit_scalar(op, value, spec=ScalarSpec(value.spec.dtype), name_hint=op)
        if isinstance(value, TensorValue):
            _float_only(value, op, "tensor")
            return require_builder().emit_tensor(
                op, value, spec=TensorSpec(value.spec.shape, value.spec.dtype, address_space=AddressSpace.REGISTER), name_hint=op
            )
        raise BackendNotImplementedError(f"{op} on host values would execute on the host; baybridge_b200 has no CPU runtime")

    apply.__name__ = op[len("math_"):]
    return apply


def _tensor_pair(lhs: Any, rhs: Any, op: str) -> TensorValue:
    builder = require_builder()
    if isinstance(lhs, TensorValue) and isinstance(rhs, TensorValue):
        if lhs.spec.dtype != rhs.spec.dtype:
            raise TypeError(f"{op} requires matching tensor dtypes")
        shape = broadcast_shapes(lhs.spec.shape, rhs.spec.shape)
        operands = (lhs.broadcast_to(shape), rhs.broadcast_to(shape))
        dtype = lhs.spec.dtype
    else:
        tensor = lhs if isinstance(lhs, TensorValue) else rhs
        scalar = rhs if isinstance(lhs, TensorValue) else lhs
        if not isinstance(scalar, ScalarValue):
            scalar = builder.constant(scalar, dtype=tensor.spec.dtype)
        if scalar.spec.dtype != tensor.spec.dtype:
            raise TypeError(f"{op} requires matching tensor/scalar dtypes")
        operands = (tensor, scalar) if isinstance(lhs, TensorValue) else (scalar, tensor)
        shape, dtype = tensor.spec.shape, tensor.spec.dtype
    return builder.emit_tensor(op, *operands, spec=TensorSpec(shape, dtype, address_space=AddressSpace.REGISTER), name_hint=op)


def _extrema(scalar_op: str, tensor_op: str):
    def apply(lhs: Any, rhs: Any) -> Any:
        if isinstance(lhs, TensorValue) or isinstance(rhs, TensorValue):
            tensor = lhs if isinstance(lhs, TensorValue) else rhs
            if tensor.spec.dtype not in ("f32", "i32"):
                raise TypeError(f"{tensor_op} requires tensor dtype f32 or i32")
            return _tensor_pair(lhs, rhs, tensor_op)
        if isinstance(lhs, ScalarValue) or isinstance(rhs, ScalarValue):
            left = lhs if isinstance(lhs, ScalarValue) else coerce_scalar(lhs, rhs.spec.dtype)
            right = rhs if isinstance(rhs, ScalarValue) else coerce_scalar(rhs, left.spec.dtype)
            if left.spec.dtype not in ("f32", "i32"):
                raise TypeError(f"{scalar_op} requires scalar dtype f32 or i32")
            if left.spec.dtype != right.spec.dtype:
                raise TypeError(f"{scalar_op} requires matching scalar dtypes")
            return require_builder().emit_scalar(scalar_op, left, right, spec=ScalarSpec(left.spec.dtype), name_hint=scalar_op)
        pick = max if scalar_op == "max" else min
        unwrap = lambda v: v.value if isinstance(v, RuntimeScalar) else v  # noqa: E731
        return pick(unwrap(lhs), unwrap(rhs))

    apply.__name__ = "maximum" if scalar_op == "max" else "minimum"
    return apply


def _atan2(lhs: Any, rhs: Any) -> Any:
    if isinstance(lhs, ScalarValue) and isinstance(rhs, ScalarValue):
        _float_only(lhs, "math_atan2", "scalar")
        _float_only(rhs, "math_atan2", "scalar")
        if lhs.spec.dtype != rhs.spec.dtype:
            raise TypeError("math_atan2 requires matching scalar dtypes")
        return require_builder().emit_scalar("math_atan2", lhs, rhs, spec=ScalarSpec(lhs.spec.dtype), name_hint="math_atan2")
    if isinstance(lhs, TensorValue) or isinstance(rhs, TensorValue):
        for value in (lhs, rhs):
            if isinstance(value, TensorValue):
                _float_only(value, "math_atan2", "tensor")
        return _tensor_pair(lhs, rhs, "math_atan2")
    raise BackendNotImplementedError("atan2 on host values would execute on the host; baybridge_b200 has no CPU runtime")


UNARY_MATH = ("round", "floor", "ceil", "trunc", "acos", "asin", "atan", "sqrt", "rsqrt", "exp", "sin", "cos",
              "exp2", "log", "log2", "log10", "erf")


class _MathNamespace:
    atan2 = staticmethod(_atan2)
    maximum = staticmethod(_extrema("max", "tensor_max"))
    minimum = staticmethod(_extrema("min", "tensor_min"))


for _name in UNARY_MATH:
    setattr(_MathNamespace, _name, staticmethod(_unary_math(f"math_{_name}")))
math = _MathNamespace()
maximum, minimum, atan2 = math.maximum, math.minimum, math.atan2
(round, floor, ceil, trunc, acos, asin, atan, sqrt, rsqrt, exp, sin, cos, exp2, log, log2, log10, erf) = (
    getattr(math, _name) for _name in UNARY_MATH
)


# ---------------------------------------------------------------------------------------------
# explicit ops: GEMM, RMSNorm, attention
# ---------------------------------------------------------------------------------------------
def _all_traced(values: tuple[Any, ...], what: str) -> None:
    if all(isinstance(value, RuntimeTensor) for value in values):
        raise BackendNotImplementedError(
            f"baybridge.{what} on host tensors would execute on the host; baybridge_b200 has no CPU runtime — "
            "compile the kernel with backend='b200'"
        )
    if not all(isinstance(value, TensorValue) for value in values):
        raise TypeError(f"baybridge.{what} expects all arguments to be runtime tensors or all to be traced tensors")


def mma(a: TensorValue, b: TensorValue, c: TensorValue | None = None, *, tile: tuple[int, ...] | None = None,
        accumulate: bool = True, accumulator_dtype: str | None = None, transpose_a: bool = False,
        transpose_b: bool = False) -> TensorValue:
    if a.spec.dtype != b.spec.dtype and {a.spec.dtype, b.spec.dtype} != {"fp8", "bf8"}:
        raise ValueError(f"mma currently requires matching operand dtypes, got {a.spec.dtype} and {b.spec.dtype}")
    if c is None:
        default = "f32" if a.spec.dtype in ("f16", "bf16", "f32", "fp8", "bf8") else a.spec.dtype
        c = make_tensor("acc", shape=a.spec.shape, dtype=accumulator_dtype or default, address_space="register")
    elif accumulator_dtype is not None and accumulator_dtype != c.spec.dtype:
        raise ValueError(
            f"mma accumulator_dtype={accumulator_dtype} does not match explicit accumulator tensor dtype {c.spec.dtype}"
        )
    require_builder().emit_void(
        "mma", a, b, c,
        attrs={"tile": list(tile) if tile else None, "accumulate": accumulate,
               "transpose_a": transpose_a, "transpose_b": transpose_b},
    )
    return c


def gemm(a: Any, b: Any, c: Any, *, transpose_a: bool = False, transpose_b: bool = False) -> Any:
    """``C[m, n] = sum_k A[m, k] * B[k, n]`` with optional operand transposes; C is overwritten."""
    _all_traced((a, b, c), "gemm")
    if not (a.ndim == b.ndim == c.ndim == 2):
        raise ValueError("traced baybridge.gemm currently requires rank-2 tensors")
    k, m = a.spec.shape if transpose_a else a.spec.shape[::-1]
    n, kb = b.spec.shape if transpose_b else b.spec.shape[::-1]
    if kb != k or c.spec.shape != (m, n):
        raise ValueError(f"gemm shape mismatch: {a.spec.shape} x {b.spec.shape} -> {c.spec.shape}")
    return mma(a, b, c, tile=(m, n, k), accumulator_dtype=c.spec.dtype, transpose_a=transpose_a, transpose_b=transpose_b)


def rmsnorm(x: Any, out: Any, gamma: Any, *, epsilon: float = 1e-5) -> Any:
    """``out = x * rsqrt(mean(x**2 over the last axis) + epsilon) * gamma``."""
    _all_traced((x, out, gamma), "rmsnorm")
    if x.spec.shape != out.spec.shape:
        raise ValueError("baybridge.rmsnorm requires x and out to have matching shapes")
    if x.ndim < 1:
        raise ValueError("baybridge.rmsnorm requires rank >= 1 tensors")
    hidden = x.spec.shape[-1]
    if gamma.spec.shape not in {(hidden,), x.spec.shape}:
        raise ValueError(f"baybridge.rmsnorm expects gamma shape {(hidden,)} or {x.spec.shape}, got {gamma.spec.shape}")
    if gamma.spec.dtype != x.spec.dtype or out.spec.dtype != x.spec.dtype:
        raise ValueError("baybridge.rmsnorm requires matching tensor dtypes")
    require_builder().emit_void("rmsnorm", x, out, gamma, attrs={"epsilon": float(epsilon)})
    return out


def layernorm(x: Any, residual: Any, out: Any, out_resid: Any, weight: Any, bias: Any, *, epsilon: float = 1e-5) -> Any:
    """``out_resid = x + residual``; ``out = (out_resid - mean) / sqrt(var + epsilon) * weight + bias`` over the last axis."""
    _all_traced((x, residual, out, out_resid, weight, bias), "layernorm")
    if not (x.spec.shape == residual.spec.shape == out.spec.shape == out_resid.spec.shape):
        raise ValueError("baybridge.layernorm requires x, residual, out, and out_resid to have matching shapes")
    if x.ndim < 1:
        raise ValueError("baybridge.layernorm requires rank >= 1 tensors")
    hidden = x.spec.shape[-1]
    for name, value in (("weight", weight), ("bias", bias)):
        if value.spec.shape not in {(hidden,), x.spec.shape}:
            raise ValueError(f"baybridge.layernorm expects {name} shape {(hidden,)} or {x.spec.shape}, got {value.spec.shape}")
    if any(value.spec.dtype != x.spec.dtype for value in (residual, out, out_resid, weight, bias)):
        raise ValueError("baybridge.layernorm requires matching tensor dtypes")
    require_builder().emit_void("layernorm", x, residual, out, out_resid, weight, bias, attrs={"epsilon": float(epsilon)})
    return out


def attention(q: Any, k: Any, v: Any, out: Any, lse: Any, *, causal: bool = False) -> Any:
    """Softmax attention on ``[batch, seq, heads, head_dim]`` tensors, scale ``1/sqrt(head_dim)``;
    ``lse`` (``[batch, heads, 1, seq]`` or ``[batch, heads, seq]``) receives the natural-log row sums."""
    _all_traced((q, k, v, out, lse), "attention")
    if not (q.ndim == k.ndim == v.ndim == out.ndim == 4):
        raise ValueError("baybridge.attention requires rank-4 q, k, v, and out tensors")
    if q.spec.shape != out.spec.shape:
        raise ValueError("baybridge.attention requires q and out to have matching shapes")
    bsz, seqlen, heads, head_dim = q.spec.shape
    kv_batch, kv_len, kv_heads, kv_dim = k.spec.shape
    if v.spec.shape != k.spec.shape:
        raise ValueError("baybridge.attention requires k and v to have matching shapes")
    if (kv_batch, kv_len, kv_dim) != (bsz, seqlen, head_dim):
        raise ValueError("baybridge.attention requires compatible q/k/v shapes")
    if heads % kv_heads:
        raise ValueError("baybridge.attention requires q heads to be divisible by kv heads")
    if lse.spec.shape not in {(bsz, heads, 1, seqlen), (bsz, heads, seqlen)}:
        raise ValueError(
            f"baybridge.attention expects lse shape {(bsz, heads, 1, seqlen)} or {(bsz, heads, seqlen)}, got {lse.spec.shape}"
        )
    if any(value.spec.dtype != q.spec.dtype for value in (k, v, out)):
        raise ValueError("baybridge.attention requires matching q/k/v/out dtypes")
    require_builder().emit_void("attention", q, k, v, out, lse, attrs={"causal": bool(causal)})
    return out
