"""Portable-IR pattern matcher of the b200 backend.

``match(ir)`` classifies a traced kernel as one of

* ``GemmPlan`` / ``RmsNormPlan`` / ``AttentionPlan`` — a single explicit op whose
  operands are kernel arguments (the "single explicit op" rule of upstream
  ``hipkittens_ref.py:88-275`` and ``hipkittens_exec.py:631-894``), or
* ``ElementwisePlan`` — a load / scalar-expression / store body, in the indexed
  scalar form or the tensor-SSA form,

and raises ``BackendNotImplementedError`` for anything else (no CPU fallback).

Unlike upstream's positional matcher (``ptx_bridge.py:542-586`` requires an
exact op sequence), elementwise matching here is dataflow based: every value is
resolved through the op graph, repeated loads of one tensor are merged, and the
index of every access is analysed symbolically.  When every access provably hits
linear offset ``i`` for the global thread id ``i`` — e.g. ``g[i // C, i % C]``
on a row-major ``[R, C]`` tensor — the kernel is a *flat map* and may be
re-gridded into 128-bit vector steps.  Otherwise it is lowered *literally*: one
device thread per traced thread with the traced index arithmetic and a bounds
guard on every access (the guard upstream's PTX emits, ``ptx_bridge.py:5846``).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

from ..errors import BackendNotImplementedError
from ..portable_ir import row_major_stride

FLOAT_DTYPES = ("f32", "bf16", "f16")
STORAGE_DTYPES = ("f32", "bf16", "f16", "i32", "i64", "index", "i8", "i1")

UNARY_OPS = {
    "neg", "abs", "bitnot", "cast",
    "math_round", "math_floor", "math_ceil", "math_trunc", "math_acos", "math_asin", "math_atan", "math_sqrt",
    "math_rsqrt", "math_exp", "math_sin", "math_cos", "math_exp2", "math_log", "math_log2", "math_log10", "math_erf",
}
BINARY_OPS = {
    "add", "sub", "mul", "div", "floordiv", "mod", "max", "min", "math_atan2",
    "cmp_lt", "cmp_le", "cmp_gt", "cmp_ge", "cmp_eq", "cmp_ne",
    "and", "or", "xor", "bitand", "bitor", "bitxor",
}
TENSOR_OP_ALIASES = {
    "tensor_add": "add", "tensor_sub": "sub", "tensor_mul": "mul", "tensor_div": "div", "tensor_max": "max",
    "tensor_min": "min", "tensor_neg": "neg", "tensor_abs": "abs", "tensor_bitand": "bitand", "tensor_bitor": "bitor",
    "tensor_bitxor": "bitxor", "tensor_bitnot": "bitnot", "tensor_select": "select",
}
TOPOLOGY_OPS = {"thread_idx", "block_idx", "program_id", "block_dim", "grid_dim"}


def _unsupported(message: str) -> BackendNotImplementedError:
    return BackendNotImplementedError(f"b200: {message}")


# ---------------------------------------------------------------------------------------------
# plans
# ---------------------------------------------------------------------------------------------
@dataclass(frozen=True)
class GemmPlan:
    a: int  # positions in ir.arguments
    b: int
    c: int
    m: int
    n: int
    k: int
    transpose_a: bool
    transpose_b: bool
    operand_dtype: str
    c_dtype: str
    kind: str = "gemm"

    @property
    def flops(self) -> int:
        return 2 * self.m * self.n * self.k


@dataclass(frozen=True)
class RmsNormPlan:
    x: int
    out: int
    gamma: int
    rows: int
    hidden: int
    gamma_is_full: bool
    epsilon: float
    dtype: str
    kind: str = "rmsnorm"


@dataclass(frozen=True)
class LayerNormPlan:
    x: int
    residual: int
    out: int
    out_resid: int
    weight: int
    bias: int
    rows: int
    hidden: int
    weight_is_full: bool
    bias_is_full: bool
    epsilon: float
    dtype: str
    kind: str = "layernorm"


@dataclass(frozen=True)
class AttentionPlan:
    q: int
    k: int
    v: int
    out: int
    lse: int
    batch: int
    seq: int
    heads: int
    kv_heads: int
    head_dim: int
    causal: bool
    dtype: str
    kind: str = "attention"


@dataclass(frozen=True)
class Node:
    """One value of the per-element expression graph."""

    name: str
    op: str  # "input" | "scalar_arg" | "constant" | "index" | unary/binary op | "select"
    dtype: str
    operands: tuple[str, ...] = ()
    attrs: dict[str, Any] = field(default_factory=dict)


@dataclass(frozen=True)
class ElementwisePlan:
    """``mode == "flat"``: ``nodes`` computes, for linear element ``i < extent``, the values stored by
    ``stores`` = ((tensor argument position, value name), …); ``inputs`` are the tensor argument
    positions that are read (each exactly once per element).

    ``mode == "literal"``: ``nodes`` additionally contains the traced index arithmetic; loads and
    stores carry explicit per-axis index operands and optional predicates, and the launch is the
    traced launch."""

    mode: str
    nodes: tuple[Node, ...]
    inputs: tuple[int, ...]
    stores: tuple[tuple[Any, ...], ...]
    scalars: tuple[int, ...]
    extent: int
    kind: str = "elementwise"
    # flat mode only: tensor positions read through ``uniform_input`` nodes (one fixed element, e.g. a one-element
    # tensor used as a scalar) or ``broadcast_input`` nodes (a smaller tensor broadcast over the element space)
    gathers: tuple[int, ...] = ()


@dataclass(frozen=True)
class ReductionPlan:
    """``dst = fold(op, init, value over the reduced axes)`` where ``value`` is the per-element expression
    ``nodes`` computes from ``inputs`` (all of ``source_shape``).  ``form``: ``rows`` (trailing axes reduced:
    ``[outer, inner] -> [outer]``), ``cols`` (leading axes reduced: ``[outer, inner] -> [inner]``) or ``all``
    (scalar result stored at ``dst_offset`` of ``dst``)."""

    nodes: tuple[Node, ...]
    inputs: tuple[int, ...]
    scalars: tuple[int, ...]
    value: str
    op: str
    init: Any
    form: str
    outer: int
    inner: int
    dst: int
    dst_offset: int
    source_shape: tuple[int, ...]
    dtype: str
    kind: str = "reduction"


@dataclass(frozen=True)
class ReductionBundlePlan:
    """Several folds in one kernel body (e.g. the total, the row folds and the column folds of one loaded tensor):
    each part is an independent ``ReductionPlan`` over the kernel's arguments, run one after the other."""

    parts: tuple[ReductionPlan, ...]
    kind: str = "reduction_bundle"


# ---------------------------------------------------------------------------------------------
# explicit single-op kernels
# ---------------------------------------------------------------------------------------------
def _argument_positions(ir) -> dict[str, int]:
    return {argument.name: position for position, argument in enumerate(ir.arguments)}


def _tensor_arg(ir, positions: dict[str, int], name: str, what: str):
    if name not in positions or ir.arguments[positions[name]].kind != "tensor":
        raise _unsupported(f"{what} operands must be kernel tensor arguments (got '{name}')")
    spec = ir.arguments[positions[name]].spec
    if not spec.resolved_layout().is_row_major or spec.address_space.value != "global":
        raise _unsupported(f"{what} operand '{name}' must be a row-major global tensor")
    return positions[name], spec


def _match_gemm(ir, op) -> GemmPlan:
    positions = _argument_positions(ir)
    (a, a_spec), (b, b_spec), (c, c_spec) = (_tensor_arg(ir, positions, name, "gemm") for name in op.inputs)
    if not (len(a_spec.shape) == len(b_spec.shape) == len(c_spec.shape) == 2):
        raise _unsupported("gemm requires rank-2 operands")
    transpose_a, transpose_b = bool(op.attrs.get("transpose_a")), bool(op.attrs.get("transpose_b"))
    k, m = a_spec.shape if transpose_a else a_spec.shape[::-1]
    n, kb = b_spec.shape if transpose_b else b_spec.shape[::-1]
    if kb != k or c_spec.shape != (m, n):
        raise _unsupported(f"gemm shape mismatch: {a_spec.shape} x {b_spec.shape} -> {c_spec.shape}")
    tile = op.attrs.get("tile")
    if tile is not None and tuple(tile) != (m, n, k):
        raise _unsupported("mma with a tile smaller than the operands (a sub-tile of a larger kernel) is not a whole-GEMM op")
    if a_spec.dtype != "bf16" or b_spec.dtype != "bf16":
        raise _unsupported(f"gemm operands must be bf16 (got {a_spec.dtype}, {b_spec.dtype})")
    if c_spec.dtype not in ("bf16", "f32"):
        raise _unsupported(f"gemm output must be bf16 or f32 (got {c_spec.dtype})")
    return GemmPlan(a, b, c, m, n, k, transpose_a, transpose_b, "bf16", c_spec.dtype)


_PROGRAM_AXIS = {"x": 0, "y": 1, "z": 2}
TOPOLOGY_OPS = frozenset({"program_id", "block_idx", "thread_idx", "block_dim", "grid_dim", "lane_id"})


def _match_tiled_gemm(ir, mma_op) -> GemmPlan:
    """A GEMM written per program: each program takes ``partition`` views of A, B and C at offsets
    ``program_id(axis) * tile`` and issues one ``mma`` on them.  When the launch grid tiles C exactly and
    every program reads the whole K extent, the grid of programs computes one whole GEMM (programs or
    threads that repeat a tile rewrite the same values), so the kernel lowers to the GEMM on the full
    tensors.  Anything else about the body (other ops, nested views, partial K) is refused."""
    grid = tuple(ir.launch.grid)
    positions = _argument_positions(ir)
    scalars: dict[str, tuple[int | None, int]] = {}  # name -> (program axis or None, multiplier / constant)
    views: dict[str, tuple[str, list[tuple[str, int]]]] = {}  # view name -> (argument, per-dim ("all"|axis, tile))
    for op in ir.operations:
        if op is mma_op or op.op == "barrier":
            continue
        if op.op in ("program_id", "block_idx"):
            scalars[op.outputs[0]] = (_PROGRAM_AXIS[op.attrs["axis"]], 1)
        elif op.op == "constant" and isinstance(op.attrs.get("value"), int) and not isinstance(op.attrs.get("value"), bool):
            scalars[op.outputs[0]] = (None, int(op.attrs["value"]))
        elif op.op == "mul" and all(name in scalars for name in op.inputs):
            (axis_l, value_l), (axis_r, value_r) = (scalars[name] for name in op.inputs)
            if axis_l is not None and axis_r is not None:
                raise _unsupported("a product of two program ids is not a tile offset")
            scalars[op.outputs[0]] = (axis_l if axis_l is not None else axis_r, value_l * value_r)
        elif op.op == "partition":
            source, offsets = op.inputs[0], op.inputs[1:]
            spec = _tensor_arg(ir, positions, source, "tiled gemm")[1]
            tile = tuple(op.attrs["tile"])
            dims: list[tuple[str, int]] = []
            for axis_index, (extent, step) in enumerate(zip(spec.shape, tile)):
                program_axis, factor = scalars.get(offsets[axis_index], (None, None)) if offsets else (None, 0)
                if factor is None:
                    raise _unsupported(f"partition offset '{offsets[axis_index]}' is not a constant or a program id times a constant")
                if program_axis is None or grid[program_axis] == 1:
                    # a fixed offset (a program id along an axis of extent 1 is always 0)
                    if (factor if program_axis is None else 0) != 0 or step != extent:
                        raise _unsupported("a partition at a fixed offset must cover the whole axis to be part of a whole GEMM")
                    dims.append(("all", step))
                else:
                    if factor != step or grid[program_axis] * step != extent:
                        raise _unsupported(
                            f"programs along {'xyz'[program_axis]} must tile axis {axis_index} of '{source}' exactly "
                            f"(extent {extent}, tile {step}, offset step {factor}, grid {grid[program_axis]})")
                    dims.append(("xyz"[program_axis], step))
            views[op.outputs[0]] = (source, dims)
        else:
            raise _unsupported(f"'{op.op}' next to an mma on partitioned tiles is not lowered")
    operands = []
    for name in mma_op.inputs:
        if name in views:
            operands.append(views[name])
        elif name in positions:
            spec = _tensor_arg(ir, positions, name, "tiled gemm")[1]
            operands.append((name, [("all", extent) for extent in spec.shape]))
        else:
            raise _unsupported(f"mma operand '{name}' is neither a kernel argument nor a partition of one")
    if any(len(dims) != 2 for _, dims in operands):
        raise _unsupported("gemm requires rank-2 operands")
    (a_name, a_dims), (b_name, b_dims), (c_name, c_dims) = operands
    transpose_a, transpose_b = bool(mma_op.attrs.get("transpose_a")), bool(mma_op.attrs.get("transpose_b"))
    a_k, a_m = a_dims if transpose_a else a_dims[::-1]
    b_n, b_k = b_dims if transpose_b else b_dims[::-1]
    c_m, c_n = c_dims
    if a_k[0] != "all" or b_k[0] != "all":
        raise _unsupported("every program must read the whole K extent (split-K over programs is not lowered)")
    if a_m != c_m or b_n != c_n:
        raise _unsupported("the A / B tiles of a program do not line up with its C tile")
    if c_m[0] != "all" and c_m[0] == c_n[0]:
        raise _unsupported("rows and columns of C are tiled along the same program axis")
    tile = mma_op.attrs.get("tile")
    if tile is not None and tuple(tile) != (c_m[1], c_n[1], a_k[1]):
        raise _unsupported("the mma tile does not match the partitioned operands")
    full = PortableKernelIRView(ir, a_name, b_name, c_name)
    return _match_gemm(full, full.operation(transpose_a, transpose_b))


class PortableKernelIRView:
    """The whole-tensor GEMM a tiled kernel amounts to, in the shape ``_match_gemm`` reads."""

    def __init__(self, ir, a: str, b: str, c: str):
        self.arguments, self._names = ir.arguments, (a, b, c)

    def operation(self, transpose_a: bool, transpose_b: bool):
        from ..portable_ir import Operation

        return Operation("mma", self._names, (), {"tile": None, "transpose_a": transpose_a, "transpose_b": transpose_b})


def _match_rmsnorm(ir, op) -> RmsNormPlan:
    positions = _argument_positions(ir)
    (x, x_spec), (out, out_spec), (gamma, gamma_spec) = (_tensor_arg(ir, positions, name, "rmsnorm") for name in op.inputs)
    if x_spec.shape != out_spec.shape or not x_spec.shape:
        raise _unsupported("rmsnorm requires x and out of equal, non-scalar shape")
    hidden = x_spec.shape[-1]
    if gamma_spec.shape not in ((hidden,), x_spec.shape):
        raise _unsupported(f"rmsnorm gamma shape must be {(hidden,)} or {x_spec.shape}")
    if not (x_spec.dtype == out_spec.dtype == gamma_spec.dtype) or x_spec.dtype not in FLOAT_DTYPES:
        raise _unsupported("rmsnorm requires x, out and gamma of one dtype among f32/bf16/f16")
    vector = 4 if x_spec.dtype == "f32" else 8
    if hidden % vector:
        raise _unsupported(f"rmsnorm hidden size {hidden} must be a multiple of {vector} for {x_spec.dtype}")
    full = gamma_spec.shape == x_spec.shape and len(x_spec.shape) > 1
    return RmsNormPlan(x, out, gamma, x_spec.numel // hidden, hidden, full, float(op.attrs.get("epsilon", 1e-5)), x_spec.dtype)


def _match_layernorm(ir, op) -> LayerNormPlan:
    positions = _argument_positions(ir)
    (x, xs), (res, rs), (out, os_), (out_resid, ors), (weight, ws), (bias, bs) = (
        _tensor_arg(ir, positions, name, "layernorm") for name in op.inputs
    )
    if not (xs.shape == rs.shape == os_.shape == ors.shape) or not xs.shape:
        raise _unsupported("layernorm requires x, residual, out and out_resid of equal, non-scalar shape")
    hidden = xs.shape[-1]
    for label, spec in (("weight", ws), ("bias", bs)):
        if spec.shape not in ((hidden,), xs.shape):
            raise _unsupported(f"layernorm {label} shape must be {(hidden,)} or {xs.shape}")
    if len({spec.dtype for spec in (xs, rs, os_, ors, ws, bs)}) != 1 or xs.dtype not in FLOAT_DTYPES:
        raise _unsupported("layernorm requires all tensors of one dtype among f32/bf16/f16")
    vector = 4 if xs.dtype == "f32" else 8
    if hidden % vector or hidden > 4096 * vector:
        raise _unsupported(f"layernorm hidden size {hidden} must be a multiple of {vector} and at most {4096 * vector}")
    full = lambda spec: spec.shape == xs.shape and len(xs.shape) > 1  # noqa: E731
    return LayerNormPlan(x, res, out, out_resid, weight, bias, xs.numel // hidden, hidden, full(ws), full(bs),
                         float(op.attrs.get("epsilon", 1e-5)), xs.dtype)


def _match_attention(ir, op) -> AttentionPlan:
    positions = _argument_positions(ir)
    (q, q_spec), (k, k_spec), (v, v_spec), (out, out_spec), (lse, lse_spec) = (
        _tensor_arg(ir, positions, name, "attention") for name in op.inputs
    )
    if not (len(q_spec.shape) == len(k_spec.shape) == len(v_spec.shape) == len(out_spec.shape) == 4):
        raise _unsupported("attention requires rank-4 q, k, v and out")
    batch, seq, heads, head_dim = q_spec.shape
    if out_spec.shape != q_spec.shape or k_spec.shape != v_spec.shape:
        raise _unsupported("attention requires q/out and k/v of matching shapes")
    kv_batch, kv_seq, kv_heads, kv_dim = k_spec.shape
    if (kv_batch, kv_seq, kv_dim) != (batch, seq, head_dim) or heads % kv_heads:
        raise _unsupported("attention requires compatible q/k/v shapes and heads divisible by kv heads")
    if lse_spec.shape not in ((batch, heads, 1, seq), (batch, heads, seq)) or lse_spec.dtype != "f32":
        raise _unsupported("attention lse must be f32 of shape [batch, heads, 1, seq] or [batch, heads, seq]")
    if any(spec.dtype != "bf16" for spec in (q_spec, k_spec, v_spec, out_spec)):
        raise _unsupported("attention operands must be bf16")
    if head_dim not in (64, 128) and seq > 8192:
        raise _unsupported(f"attention with head_dim {head_dim} (not 64/128) is limited to seq <= 8192 (got {seq})")
    return AttentionPlan(q, k, v, out, lse, batch, seq, heads, kv_heads, head_dim, bool(op.attrs.get("causal")), "bf16")


# ---------------------------------------------------------------------------------------------
# symbolic index analysis
# ---------------------------------------------------------------------------------------------
@dataclass(frozen=True)
class Digit:
    """``(v // div) % mod`` of a launch variable ``v`` (``mod is None`` = no wrap).  For a one-dimensional
    launch the only variable is ``"i"``, the global linear thread id; a multi-dimensional launch has one
    variable per axis, ``block_idx.a * block_dim.a + thread_idx.a`` for ``a`` in x, y, z."""

    div: int
    mod: int | None
    var: str = "i"


class Sym:
    """Integer-valued expression ``const + Σ coef · digit`` (``None`` terms = not analysable)."""

    __slots__ = ("terms", "const")

    def __init__(self, terms: dict[Digit, int] | None = None, const: int = 0):
        self.terms = {digit: coef for digit, coef in (terms or {}).items() if coef}
        self.const = const

    @property
    def is_const(self) -> bool:
        return not self.terms

    def single_digit(self) -> Digit | None:
        if self.const == 0 and len(self.terms) == 1:
            (digit, coef), = self.terms.items()
            if coef == 1:
                return digit
        return None

    def plus(self, other: "Sym", sign: int = 1) -> "Sym":
        merged = dict(self.terms)
        for digit, coef in other.terms.items():
            merged[digit] = merged.get(digit, 0) + sign * coef
        return Sym(merged, self.const + sign * other.const)

    def scaled(self, factor: int) -> "Sym":
        return Sym({digit: coef * factor for digit, coef in self.terms.items()}, self.const * factor)

    def same_as(self, other: "Sym") -> bool:
        return self.const == other.const and self.terms == other.terms

    def bijection_extent(self, extents: dict[str, int]) -> int | None:
        """If the expression is a mixed-radix number whose digits are exactly the digits of the launch
        variables (``extents``: variable → number of values), it maps the launched threads one-to-one onto
        ``[0, N)``: returns N, else None.  Variables of extent 1 may be absent."""
        if self.const != 0 or not self.terms:
            return None
        by_var: dict[str, list[Digit]] = {}
        for digit in self.terms:
            by_var.setdefault(digit.var, []).append(digit)
        ranges: dict[Digit, int] = {}
        for var, extent in extents.items():
            digits = sorted(by_var.pop(var, []), key=lambda d: d.div)
            if not digits:
                if extent != 1:
                    return None  # threads that differ only in this variable would collide
                continue
            expected_div = 1
            for position, digit in enumerate(digits):  # the digits must tile the variable's range exactly
                if digit.div != expected_div:
                    return None
                if position == len(digits) - 1:
                    if extent % digit.div or (digit.mod is not None and digit.div * digit.mod != extent):
                        return None
                    ranges[digit] = extent // digit.div
                else:
                    if digit.mod is None:
                        return None
                    ranges[digit] = digit.mod
                    expected_div = digit.div * digit.mod
        if by_var:
            return None
        weight = 1
        for digit, coef in sorted(self.terms.items(), key=lambda item: item[1]):
            if coef != weight:
                return None
            weight *= ranges[digit]
        return weight

    def equals_linear_id(self, threads: int) -> bool:
        """True iff the expression equals ``i`` for every ``0 <= i < threads`` (digits tile exactly)."""
        if self.const != 0 or not self.terms or any(digit.var != "i" for digit in self.terms):
            return False
        expected_div = 1
        ordered = sorted(self.terms.items(), key=lambda item: item[0].div)
        for position, (digit, coef) in enumerate(ordered):
            if digit.div != expected_div or coef != expected_div:
                return False
            last = position == len(ordered) - 1
            if digit.mod is None:
                return last
            if last:
                return digit.div * digit.mod >= threads
            expected_div = digit.div * digit.mod
        return False


class _Elementwise:
    """Walks the op list once, building the per-element expression graph and the access list."""

    def __init__(self, ir):
        self.ir = ir
        self.positions = _argument_positions(ir)
        self.launch = ir.launch
        self.nodes: dict[str, Node] = {}
        self.order: list[str] = []
        self.sym: dict[str, Sym | None] = {}
        self.accesses: list[dict[str, Any]] = []  # loads and stores in program order
        self.bound: int | None = None  # i < bound predicate shared by all masked accesses
        self.flat_ok = True
        self.flat_reason = ""
        one_d = self.launch.grid[1:] == (1, 1) and self.launch.block[1:] == (1, 1)
        self.one_d = one_d

    # -- node helpers ---------------------------------------------------------------------------
    def add(self, node: Node) -> None:
        self.nodes[node.name] = node
        self.order.append(node.name)

    def not_flat(self, reason: str) -> None:
        if self.flat_ok:
            self.flat_ok, self.flat_reason = False, reason

    def dtype_of(self, name: str) -> str:
        return self.nodes[name].dtype

    # -- scalar (indexed) form ------------------------------------------------------------------
    def topology(self, op) -> None:
        axis = op.attrs["axis"]
        name = op.outputs[0]
        index = "xyz".index(axis)
        if op.op == "block_dim":
            value = self.launch.block[index]
            self.add(Node(name, "constant", "index", attrs={"value": value}))
            self.sym[name] = Sym(const=value)
            return
        if op.op == "grid_dim":
            value = self.launch.grid[index]
            self.add(Node(name, "constant", "index", attrs={"value": value}))
            self.sym[name] = Sym(const=value)
            return
        kind = "thread_idx" if op.op == "thread_idx" else "block_idx"
        self.add(Node(name, "index", "index", attrs={"builtin": kind, "axis": axis}))
        extent = (self.launch.block if kind == "thread_idx" else self.launch.grid)[index]
        if extent == 1:
            self.sym[name] = Sym(const=0)
        elif axis == "x" and self.one_d:
            block = self.launch.block[0]
            # i = block_idx.x * block + thread_idx.x  ⇒  thread_idx.x = i % block, block_idx.x = i // block
            self.sym[name] = Sym({Digit(1, block): 1}) if kind == "thread_idx" else Sym({Digit(block, None): 1})
        else:
            # one independent variable per axis: v_a = block_idx.a * block_dim.a + thread_idx.a
            block = self.launch.block[index]
            self.sym[name] = Sym({Digit(1, block, axis): 1}) if kind == "thread_idx" else Sym({Digit(block, None, axis): 1})

    def scalar_arith(self, op) -> None:
        name = op.outputs[0]
        dtype = op.attrs["result"]["dtype"]
        base = op.op
        attrs = {k: v for k, v in op.attrs.items() if k != "result"}
        self.add(Node(name, base, dtype, tuple(op.inputs), attrs))
        syms = [self.sym.get(operand) for operand in op.inputs]
        result: Sym | None = None
        if dtype in ("index", "i32", "i64") and all(s is not None for s in syms):
            if base == "add":
                result = syms[0].plus(syms[1])
            elif base == "sub":
                result = syms[0].plus(syms[1], -1)
            elif base == "mul":
                if syms[0].is_const:
                    result = syms[1].scaled(syms[0].const)
                elif syms[1].is_const:
                    result = syms[0].scaled(syms[1].const)
            elif base in ("floordiv", "mod") and syms[1].is_const and syms[1].const > 0:
                divisor = syms[1].const
                if syms[0].is_const:
                    result = Sym(const=syms[0].const // divisor if base == "floordiv" else syms[0].const % divisor)
                else:
                    result = self._divmod(syms[0], divisor, base)
        self.sym[name] = result

    @staticmethod
    def _divmod(value: Sym, divisor: int, op: str) -> Sym | None:
        # reassemble "i // d" style sums (e.g. block_idx*block + thread_idx) into a single digit first
        digit = value.single_digit()
        if digit is None and value.const == 0 and value.terms:
            variables = {d.var for d in value.terms}
            if len(variables) == 1:
                (var,) = variables
                renamed = Sym({Digit(d.div, d.mod): coef for d, coef in value.terms.items()})
                if renamed.equals_linear_id(1 << 62):
                    digit = Digit(1, None, var)
        if digit is None:
            return None
        if op == "floordiv":
            if digit.mod is None:
                return Sym({Digit(digit.div * divisor, None, digit.var): 1})
            if digit.mod % divisor == 0:
                return Sym({Digit(digit.div * divisor, digit.mod // divisor, digit.var): 1})
            return None
        if digit.mod is None or digit.mod % divisor == 0:
            return Sym({Digit(digit.div, divisor, digit.var): 1})
        if divisor % digit.mod == 0:
            return Sym({digit: 1})
        return None

    def access(self, op) -> None:
        rank = op.attrs["rank"]
        masked = op.op.startswith("masked_")
        is_load = op.op.endswith("load")
        operands = list(op.inputs)
        value = None if is_load else operands.pop(0)
        tensor = operands.pop(0)
        indices = operands[:rank]
        predicate = operands[rank] if masked else None
        fallback = operands[rank + 1] if masked and is_load else None
        if tensor not in self.positions or self.ir.arguments[self.positions[tensor]].kind != "tensor":
            raise _unsupported(f"{op.op} on '{tensor}', which is not a kernel tensor argument")
        spec = self.ir.arguments[self.positions[tensor]].spec
        if spec.dtype not in STORAGE_DTYPES or spec.address_space.value != "global":
            raise _unsupported(f"tensor '{tensor}' has unsupported dtype/address space {spec.dtype}/{spec.address_space.value}")
        stride = spec.resolved_layout().stride
        offset: Sym | None = Sym()
        for index_name, step in zip(indices, stride):
            part = self.sym.get(index_name)
            if part is None:
                offset = None
                break
            offset = offset.plus(part.scaled(step))
        uniform = is_load and not masked and offset is not None and offset.is_const and 0 <= offset.const < spec.numel
        record = {
            "kind": ("uniform" if uniform else "load") if is_load else "store", "tensor": self.positions[tensor], "indices": tuple(indices),
            "predicate": predicate, "fallback": fallback, "value": value, "offset": offset, "numel": spec.numel,
            "result": op.outputs[0] if is_load else None, "dtype": spec.dtype, "shape": spec.shape, "stride": stride,
        }
        self.accesses.append(record)
        if is_load:
            # the fallback of a guarded load is an operand: it must stay alive wherever the load's value is used
            self.add(Node(op.outputs[0], "load", spec.dtype, (fallback,) if fallback is not None else (),
                          attrs={"access": len(self.accesses) - 1}))
        if predicate is not None:
            bound = self._predicate_bound(predicate)
            if bound is None:
                self.not_flat("a predicate that is not `linear_id < constant`")
            elif self.bound is not None and self.bound != bound:
                self.not_flat("accesses guarded by different bounds")
            else:
                self.bound = bound

    def _predicate_bound(self, name: str) -> int | None:
        node = self.nodes.get(name)
        if node is None or node.op != "cmp_lt":
            return None
        lhs, rhs = (self.sym.get(operand) for operand in node.operands)
        if lhs is None or rhs is None or not rhs.is_const:
            return None
        return rhs.const if lhs.equals_linear_id(1 << 62) else None

    # -- classification -------------------------------------------------------------------------
    def finish_scalar(self) -> ElementwisePlan:
        if not any(access["kind"] == "store" for access in self.accesses):
            raise _unsupported("the kernel body stores nothing")
        threads = self.launch.threads
        scalars = tuple(position for position, argument in enumerate(self.ir.arguments) if argument.kind == "scalar")
        # a load at a fixed position (a one-element tensor used as a scalar) is the same value for every element; it
        # stays out of the index proofs as long as the kernel never writes that tensor
        written = {access["tensor"] for access in self.accesses if access["kind"] == "store"}
        if any(access["kind"] == "uniform" and access["tensor"] in written for access in self.accesses):
            self.not_flat("a fixed-position load from a tensor the kernel also writes")
        indexed = [access for access in self.accesses if access["kind"] != "uniform"]
        # the flat form runs `i < bound` only, which is the kernel's behaviour only when every store carries that guard:
        # a masked load feeding an unguarded store writes `f(fallback)` to the elements at and past the bound
        self.padded = False
        if self.bound is not None and any(access["kind"] == "store" and access["predicate"] is None for access in indexed):
            # zero padding: guarded loads, unguarded stores.  Still one flat map over the stored extent when no store is
            # guarded, every guarded tensor is read nowhere unguarded, and each holds the elements below the bound;
            # past the bound the load yields its fallback value
            guarded = {access["tensor"] for access in indexed if access["kind"] == "load" and access["predicate"] is not None}
            clean = (all(access["predicate"] is None for access in indexed if access["kind"] == "store")
                     and all(access["predicate"] is not None for access in indexed if access["tensor"] in guarded)
                     and all(access["fallback"] is not None and access["numel"] >= min(self.bound, threads)
                             for access in indexed if access["tensor"] in guarded))
            if clean:
                self.padded = True
            else:
                self.not_flat("guarded and unguarded accesses that do not form a zero-padding map")
        identity = self.flat_ok and self.one_d and all(
            access["offset"] is not None and access["offset"].equals_linear_id(threads) for access in indexed)
        if identity:
            return self._flat_plan(threads, scalars)
        # Any launch shape: if every access uses the same offset expression and that expression maps the
        # launched threads one-to-one onto [0, numel) of every tensor, the body is an elementwise map and the
        # order in which threads visit the elements does not matter.
        if self.flat_ok and self.bound is None and self._is_permutation_map(threads):
            return self._flat_plan(threads, scalars)
        if self.one_d:
            self.not_flat("an access whose offset is not provably the linear thread id")
        else:
            self.not_flat("a multi-dimensional launch whose accesses are not provably one shared one-to-one map")
        return self._literal_plan(scalars)

    def _is_permutation_map(self, threads: int) -> bool:
        accesses = [access for access in self.accesses if access["kind"] != "uniform"]
        first = accesses[0]["offset"]
        if first is None or any(access["predicate"] is not None for access in accesses):
            return False
        if any(access["offset"] is None or not access["offset"].same_as(first) for access in accesses):
            return False
        if self.one_d:
            extents = {"i": threads}
        else:
            extents = {axis: self.launch.grid[k] * self.launch.block[k] for k, axis in enumerate("xyz")}
        covered = first.bijection_extent(extents)
        return covered is not None and covered == threads and all(access["numel"] == covered for access in accesses)

    def _flat_plan(self, threads: int, scalars: tuple[int, ...]) -> ElementwisePlan:
        padded = getattr(self, "padded", False)
        if padded:  # the stored extent; guarded inputs may be shorter and are read below the bound only
            extent = min([threads] + [access["numel"] for access in self.accesses
                                      if access["kind"] == "store" or (access["kind"] == "load" and access["predicate"] is None)])
        else:
            extent = min([threads] + [access["numel"] for access in self.accesses if access["kind"] != "uniform"]
                         + ([self.bound] if self.bound is not None else []))
        current: dict[int, str] = {}  # tensor position → value name that a later load must observe
        alias: dict[str, str] = {}
        inputs: list[int] = []
        first_load: dict[int, str] = {}
        stores: dict[int, str] = {}
        for access in self.accesses:
            tensor = access["tensor"]
            if access["kind"] == "uniform":
                continue
            if access["kind"] == "load":
                if tensor in current:
                    alias[access["result"]] = current[tensor]  # store→load forwarding inside one thread
                elif tensor in first_load:
                    alias[access["result"]] = first_load[tensor]  # CSE of repeated loads
                else:
                    first_load[tensor] = access["result"]
                    inputs.append(tensor)
            else:
                current[tensor] = access["value"]
                stores[tensor] = access["value"]

        def resolve(name: str) -> str:
            while name in alias:
                name = alias[name]
            return name

        # with every access inside `i < extent`, masked loads never take their fallback
        live = _live_set(self.nodes, [resolve(value) for value in stores.values()], resolve)
        nodes: list[Node] = []
        for name in self.order:
            if name not in live:
                continue
            node = self.nodes[name]
            if node.op == "load":
                access = self.accesses[node.attrs["access"]]
                if access["kind"] == "uniform":
                    nodes.append(Node(name, "uniform_input", node.dtype, attrs={"tensor": access["tensor"], "offset": access["offset"].const}))
                elif padded and access["predicate"] is not None:
                    nodes.append(Node(name, "input", node.dtype, (resolve(access["fallback"]),),
                                      attrs={"tensor": access["tensor"], "bound": int(self.bound)}))
                else:
                    nodes.append(Node(name, "input", node.dtype, attrs={"tensor": access["tensor"]}))
            elif node.op == "index":
                raise _unsupported("a stored value depends on the thread index itself (iota-style bodies are not lowered yet)")
            else:
                nodes.append(Node(name, node.op, node.dtype, tuple(resolve(operand) for operand in node.operands), node.attrs))
        return ElementwisePlan(
            mode="flat", nodes=tuple(nodes), inputs=tuple(inputs),
            stores=tuple((tensor, resolve(value)) for tensor, value in stores.items()),
            scalars=tuple(s for s in scalars if self.ir.arguments[s].name in live), extent=extent,
            gathers=tuple(dict.fromkeys(node.attrs["tensor"] for node in nodes if node.op == "uniform_input")),
        )

    def _literal_plan(self, scalars: tuple[int, ...]) -> ElementwisePlan:
        nodes: list[Node] = []
        stores: list[tuple[Any, ...]] = []
        for access in self.accesses:
            if access["kind"] == "uniform":
                access["kind"] = "load"  # literal lowering treats it like any other indexed load
        for name in self.order:
            node = self.nodes[name]
            if node.op == "load":
                access = self.accesses[node.attrs["access"]]
                nodes.append(Node(name, "load", node.dtype, access["indices"], {
                    "tensor": access["tensor"], "predicate": access["predicate"], "fallback": access["fallback"],
                    "shape": access["shape"], "stride": access["stride"]}))
            else:
                nodes.append(node)
        for access in self.accesses:
            if access["kind"] == "store":
                stores.append((access["tensor"], access["value"], access["indices"], access["predicate"],
                               access["shape"], access["stride"]))
        inputs = tuple(dict.fromkeys(access["tensor"] for access in self.accesses if access["kind"] == "load"))
        return ElementwisePlan(mode="literal", nodes=tuple(nodes), inputs=inputs, stores=tuple(stores), scalars=scalars,
                               extent=self.launch.threads)


def _live_set(nodes: dict[str, Node], roots: list[str], resolve) -> set[str]:
    live: set[str] = set()
    stack = list(roots)
    while stack:
        name = resolve(stack.pop())
        if name in live:
            continue
        live.add(name)
        node = nodes.get(name)
        if node is not None:
            stack.extend(node.operands)
    return live


def _match_scalar_elementwise(ir) -> ElementwisePlan:
    walker = _Elementwise(ir)
    for position, argument in enumerate(ir.arguments):
        if argument.kind == "scalar":
            walker.add(Node(argument.name, "scalar_arg", argument.spec.dtype, attrs={"position": position}))
            walker.sym[argument.name] = None
    for op in ir.operations:
        if op.op in TOPOLOGY_OPS:
            walker.topology(op)
        elif op.op == "constant":
            dtype = op.attrs["result"]["dtype"]
            walker.add(Node(op.outputs[0], "constant", dtype, attrs={"value": op.attrs["value"]}))
            value = op.attrs["value"]
            walker.sym[op.outputs[0]] = Sym(const=int(value)) if dtype in ("index", "i32", "i64") and not isinstance(value, float) else None
        elif op.op == "tensor_dim":
            walker.add(Node(op.outputs[0], "constant", "index", attrs={"value": op.attrs["value"]}))
            walker.sym[op.outputs[0]] = Sym(const=int(op.attrs["value"]))
        elif op.op in ("load", "store", "masked_load", "masked_store"):
            walker.access(op)
        elif op.op in UNARY_OPS or op.op in BINARY_OPS or op.op == "select":
            walker.scalar_arith(op)
        else:
            raise _unsupported(f"op '{op.op}' is not part of an elementwise load/op/store body")
    return walker.finish_scalar()


# ---------------------------------------------------------------------------------------------
# tensor-SSA form
# ---------------------------------------------------------------------------------------------
def _match_ssa_elementwise(ir) -> ElementwisePlan:
    positions = _argument_positions(ir)
    nodes: list[Node] = []
    known: dict[str, str] = {}  # SSA tensor/scalar name → node name holding its per-element value
    shapes: dict[str, tuple[int, ...]] = {}
    dtypes: dict[str, str] = {}
    register_buffers: dict[str, dict[str, Any]] = {}
    inputs: list[int] = []
    stores: dict[int, str] = {}
    shape: tuple[int, ...] | None = None
    reductions: list[dict[str, Any]] = []  # in program order; each is completed by the copy/store of its result
    constants: dict[str, Any] = {}

    def element_shape(candidate: tuple[int, ...]) -> None:
        nonlocal shape
        if shape is None:
            shape = tuple(candidate)
        elif tuple(candidate) != shape:
            raise _unsupported(f"tensor-SSA values of different shapes ({shape} vs {tuple(candidate)}) without an explicit broadcast")

    def global_tensor(name: str):
        spec = ir.arguments[positions[name]].spec
        if not spec.resolved_layout().is_row_major or spec.address_space.value != "global" or spec.dtype not in STORAGE_DTYPES:
            raise _unsupported(f"tensor '{name}' must be a row-major global tensor of a supported dtype")
        return spec

    for argument in ir.arguments:
        if argument.kind == "scalar":
            nodes.append(Node(argument.name, "scalar_arg", argument.spec.dtype, attrs={"position": positions[argument.name]}))
            known[argument.name] = argument.name
            dtypes[argument.name] = argument.spec.dtype

    consumed = {name for op in ir.operations for name in op.inputs}
    for op in ir.operations:
        if op.op in TOPOLOGY_OPS and not (set(op.outputs) & consumed):
            continue  # a topology query whose value is never used has no effect
        pending = {record["result"]: record for record in reductions if "dst" not in record}
        if reductions and not (op.op in ("constant", "make_tensor") or op.op.startswith("reduce_")
                               or (op.op in ("copy", "store") and op.inputs[0] in pending)
                               or (op.op == "copy" and op.inputs[0] in positions and op.inputs[1] not in positions)):
            raise _unsupported(f"op '{op.op}' after a reduction is not lowered (only further reductions and the stores of their results are)")
        if op.op.startswith("reduce_"):
            source, init = op.inputs
            if source in positions and ir.arguments[positions[source]].kind == "tensor" and source not in known:
                # a fold taken straight from the kernel argument: an implicit whole-tensor load
                spec = global_tensor(source)
                node = f"{source}__elem"
                if positions[source] not in inputs:
                    inputs.append(positions[source])
                    nodes.append(Node(node, "input", spec.dtype, attrs={"tensor": positions[source]}))
                known[source], dtypes[source], shapes[source] = node, spec.dtype, tuple(spec.shape)
            if source not in known or init not in constants:
                raise _unsupported("a reduction must consume a tensor value and a literal init value")
            profile = op.attrs.get("reduction_profile", 0)
            source_shape = tuple(shapes.get(source, shape or ()))
            rank = len(source_shape)
            keep = () if profile == 0 else tuple(axis for axis, item in enumerate(profile) if item is None)
            reductions.append({"value": known[source], "op": op.op[len("reduce_"):], "init": constants[init], "keep": keep,
                               "shape": source_shape, "result": op.outputs[0], "dtype": op.attrs["result"]["dtype"], "rank": rank})
        elif op.op == "copy" and op.inputs[0] in pending:
            source, destination = op.inputs
            reduction = pending[source]
            if destination not in positions:
                raise _unsupported("the result of a reduction must be stored straight into a kernel tensor argument")
            spec = global_tensor(destination)
            kept_shape = tuple(reduction["shape"][axis] for axis in reduction["keep"])
            if tuple(spec.shape) != kept_shape or spec.dtype != reduction["dtype"]:
                raise _unsupported("reduction result and destination differ in shape or dtype")
            reduction["dst"], reduction["dst_offset"] = positions[destination], 0
        elif op.op == "store" and op.inputs[0] in pending:
            value, destination, *indices = op.inputs
            reduction = pending[value]
            if destination not in positions or any(i not in constants for i in indices):
                raise _unsupported("a scalar reduction result must be stored at a constant index of a kernel tensor argument")
            spec = global_tensor(destination)
            if spec.dtype != reduction["dtype"]:
                raise _unsupported("reduction result and destination differ in dtype")
            offset = sum(int(constants[i]) * step for i, step in zip(indices, spec.resolved_layout().stride))
            if not 0 <= offset < spec.numel:
                raise _unsupported("scalar reduction result stored out of bounds")
            reduction["dst"], reduction["dst_offset"] = positions[destination], offset
        elif op.op == "make_tensor":
            if op.attrs.get("address_space") != "register":
                raise _unsupported("tensor-SSA bodies may only stage through register tensors")
            register_buffers[op.outputs[0]] = op.attrs
        elif op.op == "copy":
            source, destination = op.inputs
            if source in positions and ir.arguments[positions[source]].kind == "tensor":
                spec = global_tensor(source)
                if destination in positions:  # global → global copy
                    element_shape(spec.shape)
                    node = f"{source}__elem"
                    if positions[source] not in inputs:
                        inputs.append(positions[source])
                        nodes.append(Node(node, "input", spec.dtype, attrs={"tensor": positions[source]}))
                    global_tensor(destination)
                    stores[positions[destination]] = node
                    continue
                if destination not in register_buffers:
                    raise _unsupported(f"copy into unknown tensor '{destination}'")
                tensor_position = positions[source]
                if tensor_position in stores:
                    known[destination] = stores[tensor_position]  # reads observe the earlier whole-tensor store
                else:
                    node = f"{source}__elem"
                    if tensor_position not in inputs:
                        inputs.append(tensor_position)
                        nodes.append(Node(node, "input", spec.dtype, attrs={"tensor": tensor_position}))
                    known[destination] = node
                dtypes[destination], shapes[destination] = spec.dtype, spec.shape
            elif source in known:
                if destination in positions:
                    spec = global_tensor(destination)
                    element_shape(spec.shape)
                    if tuple(shapes.get(source, spec.shape)) != tuple(spec.shape):
                        raise _unsupported("whole-tensor store of a value whose shape differs from the destination")
                    stores[positions[destination]] = known[source]
                elif destination in register_buffers:
                    known[destination] = known[source]
                    dtypes[destination], shapes[destination] = dtypes[source], shapes.get(source, ())
                else:
                    raise _unsupported(f"copy into unknown tensor '{destination}'")
            else:
                raise _unsupported(f"copy from unknown value '{source}'")
        elif op.op == "copy_reduce":
            # dst = dst (op) src over whole global tensors (upstream frontend.py:1957-1979); the launch only distributes the
            # elements, each is combined once (the executable upstream backend's reading, ptx_bridge.py:1391-1428, 2028-2070)
            source, destination = op.inputs
            for name in (source, destination):
                if name not in positions or ir.arguments[positions[name]].kind != "tensor":
                    raise _unsupported("copy_reduce operands must be kernel tensor arguments")
            source_spec, destination_spec = global_tensor(source), global_tensor(destination)
            if source_spec.shape != destination_spec.shape or source_spec.dtype != destination_spec.dtype:
                raise _unsupported(f"copy_reduce requires matching shapes and dtypes, got {source_spec.shape}/{source_spec.dtype} "
                                   f"and {destination_spec.shape}/{destination_spec.dtype}")
            combine = {"add": "add", "max": "max", "min": "min", "and": "bitand", "or": "bitor", "xor": "bitxor"}.get(
                str(op.attrs.get("reduction", "")).lower())
            if combine is None:
                raise _unsupported(f"copy_reduce reduction '{op.attrs.get('reduction')}' is not lowered (add/max/min/and/or/xor are)")
            if combine.startswith("bit") and destination_spec.dtype not in ("i32", "i64", "i8", "i1"):
                raise _unsupported(f"bitwise copy_reduce on {destination_spec.dtype} tensors")
            element_shape(destination_spec.shape)
            current = []
            for name, spec in ((destination, destination_spec), (source, source_spec)):
                position = positions[name]
                if position in stores:
                    current.append(stores[position])  # the value an earlier whole-tensor store left there
                    continue
                node = f"{name}__elem"
                if position not in inputs:
                    inputs.append(position)
                    nodes.append(Node(node, "input", spec.dtype, attrs={"tensor": position}))
                current.append(node)
            combined = f"{destination}__reduced_{len(nodes)}"
            nodes.append(Node(combined, combine, destination_spec.dtype, tuple(current)))
            stores[positions[destination]] = combined
        elif op.op == "fill":
            buffer, value = op.inputs
            if buffer not in register_buffers or value not in known:
                raise _unsupported("fill of something that is not a register tensor, or with an unknown value")
            known[buffer] = known[value]
            dtypes[buffer], shapes[buffer] = register_buffers[buffer]["dtype"], tuple(register_buffers[buffer]["shape"])
        elif op.op == "broadcast_to":
            (source,) = op.inputs
            target = tuple(op.attrs["target_shape"])
            if source not in known:
                raise _unsupported(f"broadcast of unknown value '{source}'")
            origin = next((node for node in nodes if node.name == known[source]), None)
            if origin is not None and origin.op == "input":
                source_shape = tuple(shapes[source])
                padded = (1,) * (len(target) - len(source_shape)) + source_shape
                if len(padded) != len(target) or any(extent not in (1, wanted) for extent, wanted in zip(padded, target)):
                    raise _unsupported(f"shape {source_shape} does not broadcast to {target}")
                nodes.append(Node(op.outputs[0], "broadcast_input", origin.dtype,
                                  attrs={"tensor": origin.attrs["tensor"], "source_shape": padded, "target_shape": target}))
                known[op.outputs[0]] = op.outputs[0]
            elif origin is not None and origin.op in ("constant", "scalar_arg", "uniform_input"):
                known[op.outputs[0]] = known[source]  # one value for every element already
            else:
                raise _unsupported("broadcast of a computed tensor value is not lowered (broadcast the loaded operand instead)")
            dtypes[op.outputs[0]], shapes[op.outputs[0]] = dtypes[source], target
        elif op.op == "load":
            tensor, *indices = op.inputs
            if tensor not in positions or any(index not in constants for index in indices):
                raise _unsupported("a scalar load inside a tensor-SSA body must read a kernel tensor at constant indices")
            spec = global_tensor(tensor)
            offset = sum(int(constants[index]) * step for index, step in zip(indices, spec.resolved_layout().stride))
            if not 0 <= offset < spec.numel:
                raise _unsupported("scalar load out of bounds")
            if positions[tensor] in stores:
                raise _unsupported("a scalar load from a tensor the kernel has already stored to")
            nodes.append(Node(op.outputs[0], "uniform_input", spec.dtype, attrs={"tensor": positions[tensor], "offset": offset}))
            known[op.outputs[0]] = op.outputs[0]
            dtypes[op.outputs[0]] = spec.dtype
        elif op.op == "constant":
            dtype = op.attrs["result"]["dtype"]
            nodes.append(Node(op.outputs[0], "constant", dtype, attrs={"value": op.attrs["value"]}))
            known[op.outputs[0]] = op.outputs[0]
            dtypes[op.outputs[0]] = dtype
            constants[op.outputs[0]] = op.attrs["value"]
        elif op.op in TENSOR_OP_ALIASES or op.op in UNARY_OPS or op.op in BINARY_OPS or op.op == "select":
            base = TENSOR_OP_ALIASES.get(op.op, op.op)
            result = op.attrs["result"]
            if op.op == "tensor_bitnot" and result.get("dtype") == "i1":
                base = "lognot"  # upstream inverts an i1 TENSOR logically (runtime.py:615-625); scalars and integers take ~
            if result.get("kind") != "tensor":
                raise _unsupported(f"scalar op '{op.op}' inside a tensor-SSA body")
            element_shape(tuple(result["shape"]))
            operands = []
            for operand in op.inputs:
                if operand not in known:
                    raise _unsupported(f"op '{op.op}' consumes unknown value '{operand}'")
                operands.append(known[operand])
            nodes.append(Node(op.outputs[0], base, result["dtype"], tuple(operands),
                              {k: v for k, v in op.attrs.items() if k != "result"}))
            known[op.outputs[0]] = op.outputs[0]
            dtypes[op.outputs[0]], shapes[op.outputs[0]] = result["dtype"], tuple(result["shape"])
        else:
            raise _unsupported(f"op '{op.op}' is not part of a tensor-SSA elementwise body")
    if reductions:
        if stores:
            raise _unsupported("whole-tensor stores next to reductions in one kernel are not lowered")
        parts = tuple(_reduction_plan(ir, record, nodes, inputs) for record in reductions)
        return parts[0] if len(parts) == 1 else ReductionBundlePlan(parts)
    if not stores or shape is None:
        raise _unsupported("the kernel body stores nothing")
    by_name = {node.name: node for node in nodes}
    live = _live_set(by_name, list(stores.values()), lambda name: name)
    extent = 1
    for dim in shape:
        extent *= dim
    kept = tuple(node for node in nodes if node.name in live)
    gathers = tuple(dict.fromkeys(node.attrs["tensor"] for node in kept if node.op in ("uniform_input", "broadcast_input")))
    if set(gathers) & set(stores):
        raise _unsupported("a broadcast or fixed-position read of a tensor the kernel also writes")
    dense = tuple(position for position in inputs if f"{ir.arguments[position].name}__elem" in live)
    for position in dense:  # a loaded tensor used directly must have the element shape
        if tuple(ir.arguments[position].spec.shape) != shape:
            raise _unsupported(f"tensor '{ir.arguments[position].name}' of shape {ir.arguments[position].spec.shape} is used without a broadcast to {shape}")
    return ElementwisePlan(
        mode="flat", nodes=kept, inputs=dense, stores=tuple(stores.items()),
        scalars=tuple(node.attrs["position"] for node in kept if node.op == "scalar_arg"), extent=extent, gathers=gathers,
    )


def _reduction_plan(ir, reduction: dict[str, Any], nodes: list[Node], inputs: list[int]) -> ReductionPlan:
    if "dst" not in reduction:
        raise _unsupported("the result of the reduction is never stored")
    if reduction["dtype"] not in ("f32", "bf16", "f16", "i32"):
        raise _unsupported(f"reductions over {reduction['dtype']} tensors are not lowered")
    if reduction["op"] in ("and", "or", "xor") and reduction["dtype"] != "i32":
        raise _unsupported("bitwise reductions need i32 tensors")
    shape, keep, rank = reduction["shape"], reduction["keep"], reduction["rank"]
    total = 1
    for extent in shape:
        total *= extent
    kept = 1
    for axis in keep:
        kept *= shape[axis]
    if not keep:
        form, outer, inner = "all", 1, total
    elif keep == tuple(range(len(keep))):
        form, outer, inner = "rows", kept, total // kept
    elif keep == tuple(range(rank - len(keep), rank)):
        form, outer, inner = "cols", total // kept, kept
    else:
        raise _unsupported(f"reduction keeping axes {keep} of a rank-{rank} tensor is neither a row nor a column reduction")
    by_name = {node.name: node for node in nodes}
    live = _live_set(by_name, [reduction["value"]], lambda name: name)
    kept_nodes = tuple(node for node in nodes if node.name in live)
    if any(node.op in ("broadcast_input", "uniform_input") for node in kept_nodes):
        raise _unsupported("a reduction whose mapped value reads a broadcast or fixed-position operand is not lowered")
    return ReductionPlan(
        nodes=kept_nodes,
        inputs=tuple(p for p in inputs if f"{ir.arguments[p].name}__elem" in live),
        scalars=tuple(node.attrs["position"] for node in kept_nodes if node.op == "scalar_arg"),
        value=reduction["value"], op=reduction["op"], init=reduction["init"], form=form, outer=outer, inner=inner,
        dst=reduction["dst"], dst_offset=reduction["dst_offset"], source_shape=tuple(shape), dtype=reduction["dtype"],
    )


# ---------------------------------------------------------------------------------------------
# entry point
# ---------------------------------------------------------------------------------------------
def adopt(ir):
    """IR objects built by an upstream checkout are rebuilt from their serialised form, which is
    identical by construction, so the rest of the backend can rely on this package's record types."""
    from ..portable_ir import PortableKernelIR

    return ir if isinstance(ir, PortableKernelIR) else PortableKernelIR.from_dict(ir.to_dict())


EXPLICIT = {"mma": _match_gemm, "rmsnorm": _match_rmsnorm, "layernorm": _match_layernorm, "attention": _match_attention}


def match(ir):
    """Classify ``ir`` (a ``PortableKernelIR`` from this package or from upstream) into a plan."""
    ir = adopt(ir)
    operations = ir.operations
    if not operations:
        raise _unsupported("the kernel body is empty")
    explicit = [op for op in operations if op.op in EXPLICIT]
    if explicit:
        if len(explicit) == 1 and explicit[0].op == "mma" and any(op.op == "partition" for op in operations):
            return _match_tiled_gemm(ir, explicit[0])
        if len(operations) != 1:
            raise _unsupported(
                f"'{explicit[0].op}' must be the only op of the kernel (found {len(operations)} ops); "
                "fusing explicit ops with other work is not lowered"
            )
        return EXPLICIT[explicit[0].op](ir, explicit[0])
    names = {op.op for op in operations}
    if any(name.startswith("reduce_") for name in names):
        return _match_ssa_elementwise(ir)
    if names & {"copy", "copy_reduce", "make_tensor", "fill"}:  # whole-tensor form (scalar loads at fixed positions are allowed inside it)
        return _match_ssa_elementwise(ir)
    if names & {"load", "store", "masked_load", "masked_store"}:
        return _match_scalar_elementwise(ir)
    if "copy" in names:
        return _match_ssa_elementwise(ir)
    raise _unsupported("no load/store or whole-tensor copy found; not an elementwise, gemm, rmsnorm or attention kernel")
