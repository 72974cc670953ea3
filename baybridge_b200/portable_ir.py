"""Portable kernel IR: the wire format between the tracer and a backend.

The serialised form (``to_dict()``) is byte-compatible with upstream
``ir.py:47-197`` and ``runtime.py:22-46`` so that a cache key computed from an
IR traced here equals the key upstream computes for the same kernel, and a
backend object written against one package accepts IR from the other.  All
records are immutable; ``RECORD.to_dict()`` is the only serialisation.
"""
from __future__ import annotations

import enum
from dataclasses import dataclass, field
from typing import Any, Iterable


def _ints(value: Any) -> tuple[int, ...]:
    """Flatten nested int tuples/lists (CuTe-style hierarchical shapes) to a flat tuple."""
    if isinstance(value, bool) or not isinstance(value, (int, tuple, list)):
        raise TypeError("layout shapes and strides must contain only integers or nested tuples/lists of integers")
    if isinstance(value, int):
        return (value,)
    return tuple(leaf for item in value for leaf in _ints(item))


def row_major_stride(shape: Iterable[int]) -> tuple[int, ...]:
    stride: list[int] = []
    running = 1
    for extent in reversed(tuple(shape)):
        stride.append(running)
        running *= extent
    return tuple(reversed(stride))


def _dim3(value: Any, what: str) -> tuple[int, int, int]:
    if len(value) != 3:
        raise ValueError(f"{what} must have exactly 3 dimensions")
    dims = tuple(int(item) for item in value)
    if min(dims) <= 0:
        raise ValueError(f"{what} dimensions must be > 0")
    return dims  # type: ignore[return-value]


@dataclass(frozen=True)
class LaunchConfig:
    grid: tuple[int, int, int] = (1, 1, 1)
    block: tuple[int, int, int] = (1, 1, 1)
    cluster: tuple[int, int, int] = (1, 1, 1)
    shared_mem_bytes: int = 0
    cooperative: bool = False

    def __post_init__(self) -> None:
        for name in ("grid", "block", "cluster"):
            object.__setattr__(self, name, _dim3(getattr(self, name), name))
        if self.shared_mem_bytes < 0:
            raise ValueError("shared_mem_bytes must be >= 0")

    @property
    def threads(self) -> int:
        gx, gy, gz = self.grid
        bx, by, bz = self.block
        return gx * gy * gz * bx * by * bz

    def to_dict(self) -> dict[str, Any]:
        record: dict[str, Any] = {name: list(getattr(self, name)) for name in ("grid", "block", "cluster")}
        record["shared_mem_bytes"] = self.shared_mem_bytes
        if self.cooperative:
            record["cooperative"] = True
        return record


@dataclass(frozen=True)
class Layout:
    shape: tuple[int, ...]
    stride: tuple[int, ...]
    swizzle: str | None = None

    def __post_init__(self) -> None:
        object.__setattr__(self, "shape", _ints(self.shape))
        object.__setattr__(self, "stride", _ints(self.stride))
        if len(self.shape) != len(self.stride):
            raise ValueError("layout shape and stride must have the same rank")
        if any(extent <= 0 for extent in self.shape):
            raise ValueError("layout shape dimensions must be > 0")
        if any(step < 0 for step in self.stride):
            raise ValueError("layout strides must be >= 0")

    @classmethod
    def row_major(cls, shape: Iterable[int], swizzle: str | None = None) -> "Layout":
        shape = tuple(shape)
        return cls(shape, row_major_stride(shape), swizzle)

    @classmethod
    def ordered(cls, shape: Iterable[int], order: Iterable[int], swizzle: str | None = None) -> "Layout":
        shape, order = tuple(shape), tuple(order)
        if sorted(order) != list(range(len(shape))):
            raise ValueError("layout order must be a permutation of the shape axes")
        stride = [0] * len(shape)
        running = 1
        for axis in order:
            stride[axis] = running
            running *= shape[axis]
        return cls(shape, tuple(stride), swizzle)

    def __call__(self, coord: int | tuple[int, ...]) -> int:
        """Offset of a coordinate; a bare int is a column-major-enumerated linear coordinate."""
        if isinstance(coord, int):
            digits, rest = [], coord
            for extent in self.shape[:-1]:
                digits.append(rest % extent)
                rest //= extent
            digits.append(rest)
            index = tuple(digits)
        else:
            index = _ints(coord)
        if len(index) != len(self.shape):
            raise ValueError(f"layout expects {len(self.shape)} coordinates, got {len(index)}")
        return sum(i * s for i, s in zip(index, self.stride))

    @property
    def is_row_major(self) -> bool:
        return self.stride == row_major_stride(self.shape)

    def __repr__(self) -> str:
        return f"{self.shape}:{self.stride}"

    def to_dict(self) -> dict[str, Any]:
        return {"shape": list(self.shape), "stride": list(self.stride), "swizzle": self.swizzle}


class AddressSpace(str, enum.Enum):
    GLOBAL = "global"
    SHARED = "shared"
    REGISTER = "register"
    LOCAL = "local"

    @classmethod
    def coerce(cls, value: "AddressSpace | str") -> "AddressSpace":
        try:
            return value if isinstance(value, cls) else cls(value)
        except ValueError:
            names = ", ".join(member.value for member in cls)
            raise ValueError(f"unsupported address_space '{value}', expected one of: {names}") from None


@dataclass(frozen=True)
class TensorSpec:
    shape: tuple[int, ...]
    dtype: str
    layout: Layout | None = None
    address_space: AddressSpace | str = AddressSpace.GLOBAL

    def __post_init__(self) -> None:
        object.__setattr__(self, "address_space", AddressSpace.coerce(self.address_space))

    def resolved_layout(self) -> Layout:
        return self.layout if self.layout is not None else Layout.row_major(self.shape)

    @property
    def numel(self) -> int:
        total = 1
        for extent in self.shape:
            total *= extent
        return total

    def to_dict(self) -> dict[str, Any]:
        return {
            "shape": list(self.shape),
            "dtype": self.dtype,
            "layout": self.resolved_layout().to_dict(),
            "address_space": self.address_space.value,
        }


@dataclass(frozen=True)
class ScalarSpec:
    dtype: str

    def to_dict(self) -> dict[str, Any]:
        return {"dtype": self.dtype}


@dataclass(frozen=True)
class KernelArgument:
    name: str
    kind: str  # "tensor" | "scalar"
    spec: TensorSpec | ScalarSpec

    def to_dict(self) -> dict[str, Any]:
        return {"name": self.name, "kind": self.kind, "spec": self.spec.to_dict()}


@dataclass(frozen=True)
class Operation:
    op: str
    inputs: tuple[str, ...] = ()
    outputs: tuple[str, ...] = ()
    attrs: dict[str, Any] = field(default_factory=dict)

    def to_dict(self) -> dict[str, Any]:
        return {"op": self.op, "inputs": list(self.inputs), "outputs": list(self.outputs), "attrs": self.attrs}


@dataclass(frozen=True)
class PortableKernelIR:
    name: str
    arguments: tuple[KernelArgument, ...]
    operations: tuple[Operation, ...]
    launch: LaunchConfig = field(default_factory=LaunchConfig)
    metadata: dict[str, Any] = field(default_factory=dict)

    def to_dict(self) -> dict[str, Any]:
        return {
            "name": self.name,
            "arguments": [argument.to_dict() for argument in self.arguments],
            "operations": [operation.to_dict() for operation in self.operations],
            "launch": self.launch.to_dict(),
            "metadata": self.metadata,
        }

    @classmethod
    def from_dict(cls, record: dict[str, Any]) -> "PortableKernelIR":
        """Rebuild an IR from its serialised form (used for golden listings and cached manifests)."""

        def spec_of(argument: dict[str, Any]) -> TensorSpec | ScalarSpec:
            raw = argument["spec"]
            if argument["kind"] != "tensor":
                return ScalarSpec(dtype=raw["dtype"])
            layout = raw.get("layout")
            return TensorSpec(
                shape=tuple(raw["shape"]),
                dtype=raw["dtype"],
                layout=Layout(tuple(layout["shape"]), tuple(layout["stride"]), layout.get("swizzle")) if layout else None,
                address_space=raw.get("address_space", "global"),
            )

        launch = record.get("launch", {})
        return cls(
            name=record["name"],
            arguments=tuple(KernelArgument(a["name"], a["kind"], spec_of(a)) for a in record["arguments"]),
            operations=tuple(
                Operation(o["op"], tuple(o["inputs"]), tuple(o["outputs"]), dict(o["attrs"])) for o in record["operations"]
            ),
            launch=LaunchConfig(
                grid=tuple(launch.get("grid", (1, 1, 1))),
                block=tuple(launch.get("block", (1, 1, 1))),
                cluster=tuple(launch.get("cluster", (1, 1, 1))),
                shared_mem_bytes=int(launch.get("shared_mem_bytes", 0)),
                cooperative=bool(launch.get("cooperative", False)),
            ),
            metadata=dict(record.get("metadata", {})),
        )
