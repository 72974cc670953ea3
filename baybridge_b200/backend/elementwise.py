"""Lower an ``ElementwisePlan`` to a specialised sm_100a kernel.

The memory side of every elementwise kernel is the hand-written skeleton in
``csrc/bb200_elementwise.cuh`` (128-bit streaming loads/stores, grid mapping,
tail handling, dtype conversion).  What differs between traced kernels is only
the register-resident scalar expression, so ``render()`` emits that expression
as a small ``Body`` struct and instantiates the skeleton with it; ``nvcc``
turns the translation unit into a cubin for sm_100a, cached on disk under the
hash of its source.  No PTX JIT, no Triton, no interpreter on the device.

Arithmetic: values are widened exactly on load, evaluated in the plan's
compute type and rounded once (RNE) at the store — mirroring upstream's CPU
runtime, which computes in Python floats and never rounds intermediates
(``runtime.py:459-462``).  f32 tensors use f64 arithmetic whenever more than
one rounding could otherwise occur, which makes the result equal to the f64
reference rounded to f32; 16-bit tensors compute in f32.
"""
from __future__ import annotations

import hashlib
import os
import subprocess
from dataclasses import dataclass
from pathlib import Path

from ..errors import BackendNotImplementedError
from .matcher import ElementwisePlan, Node
from .native import CSRC_DIR, GENCODE, NVCC_COMMON, PACKAGE_DIR, nvcc_path

STORAGE_CTYPE = {
    "f32": "float", "bf16": "__nv_bfloat16", "f16": "__half", "i32": "int32_t", "i64": "int64_t",
    "index": "int64_t", "i8": "int8_t", "i1": "uint8_t",
}
STORAGE_BYTES = {"f32": 4, "bf16": 2, "f16": 2, "i32": 4, "i64": 8, "index": 8, "i8": 1, "i1": 1}
FLOATS = ("f32", "bf16", "f16")
THREADS = 256
# 16-byte vectors per thread and stream.  One: with 8 CTAs of 256 threads resident per SM the loads in flight already cover
# the memory latency, and small CTAs (2048 bf16 elements) leave the shortest tail — measured with back-to-back launches,
# unroll 1 / 2 / 4 / 8: bf16 a*b+a 2^28 elements 228.5 / 229.1 / 232.9 / 230.4 us, 2^25 31.1 / 31.0 / 31.8 / 31.3, 2^24 16.9 / 16.8 /
# 17.4 / 17.4; f32 add 2^27 227.6 / 230.6 / 231.3 / 230.2, 2^24 30.4 / 30.9 / 31.2 / 31.6
UNROLL = 1

JIT_CACHE_ENV = "BAYBRIDGE_B200_KERNEL_CACHE"

_SINGLE_ROUNDING_OPS = {"add", "sub", "mul", "div", "max", "min", "neg", "abs", "select", "math_sqrt",
                        "cmp_lt", "cmp_le", "cmp_gt", "cmp_ge", "cmp_eq", "cmp_ne", "and", "or", "xor"}


def kernel_cache_dir() -> Path:
    configured = os.environ.get(JIT_CACHE_ENV)
    return Path(configured).expanduser() if configured else PACKAGE_DIR / "_kernel_cache"


def choose_compute_type(plan: ElementwisePlan, tensor_dtypes: list[str]) -> str:
    """``double`` when an f32 result could be rounded more than once in f32 arithmetic, else ``float``."""
    if not any(dtype == "f32" for dtype in tensor_dtypes):
        return "float"
    rounding_ops = [node for node in plan.nodes if node.dtype in FLOATS and node.op not in ("input", "load", "constant", "scalar_arg")]
    if len(rounding_ops) <= 1 and all(node.op in _SINGLE_ROUNDING_OPS for node in rounding_ops):
        return "float"
    return "double"


@dataclass(frozen=True)
class RenderedKernel:
    source: str
    entry: str
    mode: str
    vec: int
    tensor_order: tuple[int, ...]  # IR argument positions of the pointer parameters, in order
    scalar_order: tuple[int, ...]  # IR argument positions of the scalar parameters, in order
    scalar_ctypes: tuple[str, ...]
    compute: str
    relaxed: tuple[int, ...] = ()  # tensor positions only read element by element: no 16-byte alignment needed
    debug_bounds: bool = False     # literal mode: a trailing `int* bounds_status` parameter records out-of-range accesses


def _ident(name: str) -> str:
    return "v_" + "".join(ch if ch.isalnum() else "_" for ch in name)


def _float_literal(value: float, compute: str) -> str:
    value = float(value)
    if value != value:
        return "(%s)NAN" % compute
    if value in (float("inf"), float("-inf")):
        return ("-" if value < 0 else "") + "(%s)INFINITY" % compute
    text = value.hex()  # exact; C++17 hexadecimal floating literal
    return f"({compute}){text}" if compute == "double" else f"(float){text}"


def _repr_type(dtype: str, compute: str) -> str:
    if dtype in FLOATS:
        return compute
    if dtype == "i1":
        return "bool"
    return {"i32": "int32_t", "i8": "int32_t"}.get(dtype, "int64_t")


_MATH = {
    "math_sqrt": "sqrt", "math_exp": "exp", "math_exp2": "exp2", "math_log": "log", "math_log2": "log2",
    "math_log10": "log10", "math_sin": "sin", "math_cos": "cos", "math_acos": "acos", "math_asin": "asin",
    "math_atan": "atan", "math_erf": "erf", "math_floor": "floor", "math_ceil": "ceil", "math_trunc": "trunc",
    "math_round": "rint",  # Python round() is round-half-to-even
}
_INFIX = {"add": "+", "sub": "-", "mul": "*", "cmp_lt": "<", "cmp_le": "<=", "cmp_gt": ">", "cmp_ge": ">=",
          "cmp_eq": "==", "cmp_ne": "!=", "bitand": "&", "bitor": "|", "bitxor": "^"}


def _expression(node: Node, compute: str, dtype_of) -> str:
    """C++ expression for one node in terms of its operands' identifiers."""
    op = node.op
    args = [_ident(name) for name in node.operands]
    rtype = _repr_type(node.dtype, compute)
    fn_suffix = "f" if compute == "float" else ""
    if op == "constant":
        value = node.attrs["value"]
        if node.dtype in FLOATS:
            return _float_literal(value, compute)
        if node.dtype == "i1":
            return "true" if value else "false"
        return f"({rtype}){int(value)}LL"
    if op in _INFIX:
        operand_is_float = dtype_of(node.operands[0]) in FLOATS or dtype_of(node.operands[1]) in FLOATS
        cast = compute if operand_is_float else ("int64_t" if not op.startswith("cmp") and not op.startswith("bit") else "")
        lhs, rhs = (f"({cast}){a}" if cast else a for a in args)
        return f"({rtype})({lhs} {_INFIX[op]} {rhs})"
    if op == "div":
        return f"(({compute}){args[0]} / ({compute}){args[1]})"
    if op == "floordiv":
        return f"bb200::floordiv_i64((int64_t){args[0]}, (int64_t){args[1]})"
    if op == "mod":
        return f"bb200::floormod_i64((int64_t){args[0]}, (int64_t){args[1]})"
    if op == "max":
        return f"({args[0]} >= {args[1]} ? {args[0]} : {args[1]})"  # "lhs if lhs >= rhs else rhs"
    if op == "min":
        return f"({args[0]} <= {args[1]} ? {args[0]} : {args[1]})"
    if op in ("and", "or", "xor"):
        return f"(bool)({args[0]} {'&&' if op == 'and' else '||' if op == 'or' else '!='} {args[1]})"
    if op == "neg":
        return f"(-{args[0]})"
    if op == "abs":
        return f"fabs{fn_suffix}({args[0]})" if node.dtype in FLOATS else f"({args[0]} < 0 ? -{args[0]} : {args[0]})"
    if op == "bitnot":
        return f"(~{args[0]})"
    if op == "lognot":
        return f"(!{args[0]})"
    if op == "cast":
        if node.dtype == "i1":
            return f"({args[0]} != 0)"
        if node.dtype in FLOATS:
            return f"({compute}){args[0]}"
        return f"({rtype}){args[0]}"  # float → int truncates toward zero like Python int()
    if op == "select":
        return f"({args[0]} ? {args[1]} : {args[2]})"
    if op == "math_rsqrt":
        one = "1.0f" if compute == "float" else "1.0"
        return f"({one} / sqrt{fn_suffix}({args[0]}))"  # upstream: 1.0 / math.sqrt(x)
    if op == "math_atan2":
        return f"atan2{fn_suffix}({args[0]}, {args[1]})"
    if op in _MATH:
        return f"{_MATH[op]}{fn_suffix}({args[0]})"
    raise BackendNotImplementedError(f"b200: elementwise op '{op}' has no device lowering")


def _narrow(dtype: str, compute: str, expr: str) -> str:
    storage = STORAGE_CTYPE[dtype]
    if dtype in FLOATS:
        return f"bb200::Conv<{compute}, {storage}>::narrow({expr})"
    if dtype == "i1":
        return f"(uint8_t)(({expr}) ? 1 : 0)"
    return f"({storage})({expr})"


def _widen(dtype: str, compute: str, expr: str) -> str:
    storage = STORAGE_CTYPE[dtype]
    if dtype in FLOATS:
        return f"bb200::Conv<{compute}, {storage}>::widen({expr})"
    if dtype == "i1":
        return f"(({expr}) != 0)"
    return f"({_repr_type(dtype, compute)})({expr})"


def gather_read(tensor: int, offset: str) -> str:
    """A read of a small operand that many elements share (kept in cache, so the read-only path is used)."""
    return f"__ldg(p{tensor} + {offset})"


def broadcast_offset(source_shape, target_shape, index: str) -> str:
    """Offset into a row-major tensor of ``source_shape`` (same rank as ``target_shape``, extent 1 on the broadcast
    axes) for the element whose linear index in the row-major ``target_shape`` space is ``index``."""
    terms = []
    suffix = 1       # elements per step of this axis in the target space
    stride = 1       # stride of this axis in the source tensor
    for source_extent, target_extent in zip(reversed(tuple(source_shape)), reversed(tuple(target_shape))):
        if source_extent != 1:
            digit = f"(({index} / {suffix}ULL) % {target_extent}ULL)" if suffix > 1 else f"({index} % {target_extent}ULL)"
            terms.append(f"{digit} * {stride}ULL" if stride > 1 else digit)
            stride *= source_extent
        suffix *= target_extent
    return " + ".join(terms) if terms else "0"


MAX_FANOUT = 8  # destinations per stored tensor in the fan-out form (one per GPU of a box)


#: status-word codes of the bounds-checking debug build (kernels' wait codes start at 100, the self-test uses 99)
BOUNDS_LOAD_CODE, BOUNDS_STORE_CODE = 301, 302


def debug_bounds_enabled() -> bool:
    """``BB200_DEBUG_BOUNDS=1`` at compile() time: thread-by-thread ("literal") kernels record an access whose traced
    index falls outside its tensor in the device status word instead of skipping it silently, and the synchronising
    launcher raises.  The role ``compute-sanitizer`` would play, without a tool attached; the fast flat form needs no
    such check (its extent never exceeds a tensor)."""
    return os.environ.get("BB200_DEBUG_BOUNDS", "0") not in ("", "0")


def render(plan: ElementwisePlan, ir, entry: str = "bb200_elementwise_kernel", fanout: int = 0,
           debug_bounds: bool = False) -> RenderedKernel:
    """``fanout == 0``: the ordinary kernel.  ``fanout >= 1`` (flat plans only): every stored tensor is written to
    ``fanout`` destination buffers at ``shard_offset + i`` instead of to its argument — the form a rank uses to put
    its output shard straight into every rank's gathered output (peer memory) while it computes.  The pointer
    parameter of a stored tensor becomes a by-value table of ``MAX_FANOUT`` pointers, and ``size_t shard_offset``
    follows ``n`` in the signature."""
    arguments = ir.arguments
    if fanout:
        if plan.mode != "flat" or not 1 <= fanout <= MAX_FANOUT:
            raise BackendNotImplementedError("b200: the fan-out form needs a flat elementwise plan and 1..8 destinations")
        if {store[0] for store in plan.stores} & (set(plan.inputs) | set(getattr(plan, "gathers", ()))):
            raise BackendNotImplementedError("b200: the fan-out form does not take kernels that update a tensor in place")
    tensors_used = list(dict.fromkeys(list(plan.inputs) + list(getattr(plan, "gathers", ())) + [store[0] for store in plan.stores]))
    tensor_dtypes = [arguments[position].spec.dtype for position in tensors_used]
    compute = choose_compute_type(plan, tensor_dtypes)
    by_name = {node.name: node for node in plan.nodes}

    def dtype_of(name: str) -> str:
        return by_name[name].dtype

    scalar_order = tuple(plan.scalars)
    scalar_ctypes = tuple(
        # float scalars travel as double so the f64 compute path sees the caller's exact Python float
        {"f32": "double", "f16": "double", "bf16": "double", "i1": "int32_t", "i32": "int32_t", "i8": "int32_t"}.get(
            arguments[position].spec.dtype, "int64_t")
        for position in scalar_order
    )
    pointer_params = []
    written = {store[0] for store in plan.stores}
    for position in tensors_used:
        ctype = STORAGE_CTYPE[arguments[position].spec.dtype]
        const = "" if position in written else "const "
        if fanout and position in written:
            pointer_params.append(f"bb200::Destinations<{ctype}> q{position}")
        else:
            pointer_params.append(f"{const}{ctype}* __restrict__ p{position}")
    scalar_params = [f"{ctype} s{position}" for position, ctype in zip(scalar_order, scalar_ctypes)]

    def scalar_value(node: Node) -> str:
        position = node.attrs["position"]
        return _widen(node.dtype, compute, f"s{position}") if node.dtype not in FLOATS else f"({compute})s{position}"

    lines = [
        "// generated by baybridge_b200.backend.elementwise from a traced kernel body; the memory access",
        "// pattern, grid mapping and conversions come from the hand-written skeleton included below.",
        '#include "bb200_elementwise.cuh"',
        "#include <math.h>",
        "",
    ]
    if plan.mode == "flat":
        vec = 16 // min(STORAGE_BYTES[dtype] for dtype in tensor_dtypes)
        body = ["struct Body {", f"  static constexpr int VEC = {vec};"]
        for param in pointer_params + scalar_params + (["size_t shard_offset"] if fanout else []):
            body.append(f"  {param};")
        # Broadcast operands in the vector path.  A vector step covers VEC consecutive elements of one row when the
        # innermost extent is a multiple of VEC: an operand that is dense along that axis (a row vector) is then one
        # 16-byte load at its own offset, and one that is broadcast along it (a column vector) is one value per step.
        row_like = {}   # node name -> (tensor, ctype, offset expression of the step's first element)
        per_step = {}
        for node in plan.nodes:
            if node.op != "broadcast_input" or node.attrs["target_shape"][-1] % vec:
                continue
            tensor, ctype = node.attrs["tensor"], STORAGE_CTYPE[arguments[node.attrs["tensor"]].spec.dtype]
            offset = broadcast_offset(node.attrs["source_shape"], node.attrs["target_shape"], "base")
            if node.attrs["source_shape"][-1] == node.attrs["target_shape"][-1]:
                row_like[node.name] = (tensor, ctype, offset)
            elif node.attrs["source_shape"][-1] == 1:
                per_step[node.name] = (tensor, ctype, offset)
        body.append("  struct Regs {")
        for position in plan.inputs:
            body.append(f"    bb200::Pack<{STORAGE_CTYPE[arguments[position].spec.dtype]}, VEC> r{position};")
        for name, (tensor, ctype, _) in row_like.items():
            body.append(f"    bb200::Pack<{ctype}, VEC> g{_ident(name)};")
        for name, (tensor, ctype, _) in per_step.items():
            body.append(f"    {ctype} g{_ident(name)};")
        if not plan.inputs and not row_like and not per_step:
            body.append("    int unused;")
        body.append("  };")
        body.append("  __device__ __forceinline__ void load(size_t base, Regs& r) const {")
        bounds = {node.attrs["tensor"]: node.attrs["bound"] for node in plan.nodes if node.op == "input" and "bound" in node.attrs}
        for position in plan.inputs:
            ctype = STORAGE_CTYPE[arguments[position].spec.dtype]
            if position in bounds:
                body.append(f"    r.r{position} = bb200::load_stream_guarded<{ctype}, VEC>(p{position}, base, (size_t){bounds[position]}ULL);")
            else:
                body.append(f"    r.r{position} = bb200::load_stream<{ctype}, VEC>(p{position} + base);")
        for name, (tensor, ctype, offset) in row_like.items():
            body.append(f"    r.g{_ident(name)} = bb200::load_shared_operand<{ctype}, VEC>(p{tensor} + {offset});")
        for name, (tensor, ctype, offset) in per_step.items():
            body.append(f"    r.g{_ident(name)} = __ldg(p{tensor} + {offset});")
        body.append("  }")

        def element_code(read, write, indent: str, index: str, staged: bool) -> list[str]:
            """``index``: C expression of the element's linear index (only broadcast operands need it); ``staged``: the
            vector path, where row-like and per-step broadcast operands were fetched by ``load``."""
            code = []
            for node in plan.nodes:
                ident, rtype = _ident(node.name), _repr_type(node.dtype, compute)
                if staged and node.name in row_like:
                    code.append(f"{indent}const {rtype} {ident} = {_widen(node.dtype, compute, f'r.g{ident}.v[j]')};")
                elif staged and node.name in per_step:
                    code.append(f"{indent}const {rtype} {ident} = {_widen(node.dtype, compute, f'r.g{ident}')};")
                elif node.op == "input" and "bound" in node.attrs:
                    # defined below the bound only; past it the traced fallback value stands in (and nothing is read)
                    loaded = _widen(node.dtype, compute, read(node.attrs["tensor"]))
                    code.append(f"{indent}const {rtype} {ident} = (size_t)({index}) < (size_t){node.attrs['bound']}ULL ? {loaded} : "
                                f"({rtype}){_ident(node.operands[0])};")
                elif node.op == "input":
                    code.append(f"{indent}const {rtype} {ident} = {_widen(node.dtype, compute, read(node.attrs['tensor']))};")
                elif node.op == "uniform_input":
                    code.append(f"{indent}const {rtype} {ident} = {_widen(node.dtype, compute, gather_read(node.attrs['tensor'], str(int(node.attrs['offset']))))};")
                elif node.op == "broadcast_input":
                    offset = broadcast_offset(node.attrs["source_shape"], node.attrs["target_shape"], index)
                    code.append(f"{indent}const {rtype} {ident} = {_widen(node.dtype, compute, gather_read(node.attrs['tensor'], offset))};")
                elif node.op == "scalar_arg":
                    code.append(f"{indent}const {rtype} {ident} = {scalar_value(node)};")
                else:
                    code.append(f"{indent}const {rtype} {ident} = {_expression(node, compute, dtype_of)};")
            for position, value in plan.stores:
                dtype = arguments[position].spec.dtype
                code.append(f"{indent}{write(position)} = {_narrow(dtype, compute, _ident(value))};")
            return code

        body.append("  __device__ __forceinline__ void compute_store(size_t base, const Regs& r) const {")
        for position, _ in plan.stores:
            body.append(f"    bb200::Pack<{STORAGE_CTYPE[arguments[position].spec.dtype]}, VEC> o{position};")
        body.append("#pragma unroll")
        body.append("    for (int j = 0; j < VEC; ++j) {")
        body.extend(element_code(lambda p: f"r.r{p}.v[j]", lambda p: f"o{p}.v[j]", "      ", "(base + j)", True))
        body.append("    }")
        for position, _ in plan.stores:
            ctype = STORAGE_CTYPE[arguments[position].spec.dtype]
            if fanout:
                body.append("#pragma unroll")
                body.append(f"    for (int d = 0; d < {fanout}; ++d) bb200::store_stream<{ctype}, VEC>(q{position}.p[d] + shard_offset + base, o{position});")
            else:
                body.append(f"    bb200::store_stream<{ctype}, VEC>(p{position} + base, o{position});")
        body.append("  }")
        body.append("  __device__ __forceinline__ void scalar(size_t i) const {")
        if fanout:
            for position, _ in plan.stores:
                body.append(f"    {STORAGE_CTYPE[arguments[position].spec.dtype]} w{position};")
            body.extend(element_code(lambda p: f"p{p}[i]", lambda p: f"w{p}", "    ", "i", False))
            for position, _ in plan.stores:
                body.append(f"    for (int d = 0; d < {fanout}; ++d) q{position}.p[d][shard_offset + i] = w{position};")
        else:
            body.extend(element_code(lambda p: f"p{p}[i]", lambda p: f"p{p}[i]", "    ", "i", False))
        body.append("  }")
        body.append("};")
        lines.extend(body)
        signature = ", ".join(pointer_params + scalar_params + ["size_t n"] + (["size_t shard_offset"] if fanout else []) + ["int vector_ok"])
        init = ", ".join([(f"q{position}" if fanout and position in written else f"p{position}") for position in tensors_used]
                         + [f"s{position}" for position in scalar_order] + (["shard_offset"] if fanout else []))
        lines += [
            "",
            f'extern "C" __global__ void __launch_bounds__({THREADS}) {entry}({signature}) {{',
            f"  Body body{{{init}}};",
            f"  bb200::flat_map<{UNROLL}>(body, n, vector_ok != 0);",
            "}",
        ]
        vector_read = {entry_[0] for entry_ in row_like.values()}
        relaxed = tuple(position for position in getattr(plan, "gathers", ()) if position not in vector_read)
        return RenderedKernel("\n".join(lines) + "\n", entry, "flat", vec, tuple(tensors_used), scalar_order, scalar_ctypes, compute,
                              relaxed)

    # ---- literal mode: one device thread per traced thread, traced index arithmetic, guarded accesses
    signature = ", ".join(pointer_params + scalar_params + (["int* bounds_status"] if debug_bounds else []))
    code = [f'extern "C" __global__ void {entry}({signature}) {{']

    def guarded_offset(indices, shape, stride) -> tuple[str, str]:
        terms = " + ".join(f"(int64_t){_ident(i)} * {step}LL" for i, step in zip(indices, stride)) or "0"
        inside = " && ".join(f"(int64_t){_ident(i)} >= 0 && (int64_t){_ident(i)} < {extent}LL" for i, extent in zip(indices, shape)) or "true"
        return terms, inside

    for node in plan.nodes:
        ident, rtype = _ident(node.name), _repr_type(node.dtype, compute)
        if node.op == "index":
            builtin = "threadIdx" if node.attrs["builtin"] == "thread_idx" else "blockIdx"
            code.append(f"  const int64_t {ident} = (int64_t){builtin}.{node.attrs['axis']};")
        elif node.op == "scalar_arg":
            code.append(f"  const {rtype} {ident} = {scalar_value(node)};")
        elif node.op == "load":
            tensor = node.attrs["tensor"]
            offset, inside = guarded_offset(node.operands, node.attrs["shape"], node.attrs["stride"])
            fallback = _ident(node.attrs["fallback"]) if node.attrs["fallback"] else f"({rtype})0"
            predicate = f"{_ident(node.attrs['predicate'])} && " if node.attrs["predicate"] else ""
            code.append(f"  {rtype} {ident} = {fallback};")
            code.append(f"  if ({predicate}{inside}) {ident} = {_widen(node.dtype, compute, f'p{tensor}[{offset}]')};")
            if debug_bounds:
                code.append(f"  else if ({predicate}true) atomicExch(bounds_status, {BOUNDS_LOAD_CODE});")
        else:
            code.append(f"  const {rtype} {ident} = {_expression(node, compute, dtype_of)};")
    for tensor, value, indices, predicate, shape, stride in plan.stores:
        offset, inside = guarded_offset(indices, shape, stride)
        guard = f"{_ident(predicate)} && " if predicate else ""
        dtype = arguments[tensor].spec.dtype
        code.append(f"  if ({guard}{inside}) p{tensor}[{offset}] = {_narrow(dtype, compute, _ident(value))};")
        if debug_bounds:
            code.append(f"  else if ({guard}true) atomicExch(bounds_status, {BOUNDS_STORE_CODE});")
    code.append("}")
    # literal bodies interleave loads and stores in program order only when a store feeds a later
    # load of the same tensor; such bodies are rejected below rather than silently reordered
    store_targets = {store[0] for store in plan.stores}
    if store_targets & set(plan.inputs):
        raise BackendNotImplementedError(
            "b200: a kernel that both loads and stores one tensor at non-identity indices is not lowered "
            "(other threads' stores could be observed)"
        )
    lines.extend(code)
    return RenderedKernel("\n".join(lines) + "\n", entry, "literal", 1, tuple(tensors_used), scalar_order, scalar_ctypes, compute,
                          debug_bounds=debug_bounds)


def _skeleton_digest() -> str:
    return hashlib.sha256((CSRC_DIR / "bb200_elementwise.cuh").read_bytes()).hexdigest()


def compile_cubin(source: str) -> Path:
    """``nvcc -cubin`` for sm_100a, cached by the hash of (source, skeleton header, flags)."""
    key = hashlib.sha256("\n".join([source, _skeleton_digest(), " ".join(GENCODE + NVCC_COMMON + ("-fmad=false",))]).encode()).hexdigest()[:32]
    directory = kernel_cache_dir()
    cubin = directory / f"{key}.cubin"
    if cubin.exists() and cubin.stat().st_size:
        return cubin
    directory.mkdir(parents=True, exist_ok=True)
    unit = directory / f"{key}.cu"
    unit.write_text(source)
    scratch = directory / f"{key}.{os.getpid()}.tmp"
    # -fmad=false: the CPU runtime rounds after every multiply and add; a fused multiply-add would round once
    command = [nvcc_path(), *GENCODE, *NVCC_COMMON, "-fmad=false", "-cubin", "-I", str(CSRC_DIR), str(unit), "-o", str(scratch)]
    done = subprocess.run(command, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if done.returncode:
        scratch.unlink(missing_ok=True)
        raise BackendNotImplementedError(f"b200: nvcc rejected the generated elementwise kernel:\n{done.stdout}\n--- source ---\n{source}")
    os.replace(scratch, cubin)
    return cubin
