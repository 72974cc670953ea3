"""CPU oracle for the b200 hot path — TEST INFRASTRUCTURE, NOT A PRODUCT PATH.

Only ``tests/``, ``__graft_entry__.smoke()`` and the ``cpu_baseline`` /
``--impl reference`` legs of ``bench.py`` may import this module; nothing under
``baybridge_b200/`` does, and the product raises when its CUDA library is
missing rather than falling back to this code.

What it restates (numpy float64, following upstream's CPU reference runtime):

* ``run_kernel_ir``   — the sequential thread-emulation loop of upstream
  ``frontend.py:783-821`` applied to a traced kernel body: every IR op of the
  scalar form (``frontend.py:2038-2117, 2931-3019``; operators
  ``tracing.py:27-249``; math ``math.py:13-76``) and of the tensor-SSA form
  (``runtime.py:464-532``) is evaluated for all emulated threads at once.
  Values are Python-float (f64) semantics and are NEVER rounded to the tensor
  dtype, exactly like ``RuntimeTensor.__setitem__`` (``runtime.py:459-462``).
* ``gemm``            — ``frontend.py:3709-3716`` (C is overwritten, f64 accumulate).
* ``rmsnorm``         — ``frontend.py:3845-3852``;  ``layernorm`` — ``frontend.py:3775-3793``.
* ``attention``       — ``frontend.py:3903-3937`` including masked scores
  contributing weight 0 and ``lse = -inf`` when the row norm is 0.

Pinned: ``tests/test_oracle_golden.py`` checks every function here against the
fixtures in ``tests/golden/`` that were produced by running upstream's own CPU
runtime (``tests/golden/make_golden.py``); summation order differs from
upstream's scalar loops only in the last bits (asserted ≤ 1e-12 relative).
"""
from __future__ import annotations

import math
from typing import Any

import numpy as np

F64 = np.float64


# ---------------------------------------------------------------------------------------------
# rounding helpers shared with the tests (the reference rule for bf16 staging is RNE on the
# upper half of the f32 pattern, upstream hip_runtime.py:246-249)
# ---------------------------------------------------------------------------------------------
def bf16_round(x: np.ndarray) -> np.ndarray:
    x32 = np.ascontiguousarray(x, dtype=np.float32)
    bits = x32.view(np.uint32).astype(np.uint64)
    rounded = ((bits + (((bits >> np.uint64(16)) & np.uint64(1)) + np.uint64(0x7FFF))) >> np.uint64(16)) << np.uint64(16)
    return (rounded & np.uint64(0xFFFFFFFF)).astype(np.uint32).view(np.float32).reshape(x32.shape)


def round_to_dtype(x: np.ndarray, dtype: str) -> np.ndarray:
    """One round-to-nearest-even from f64 to the storage dtype, returned as f64."""
    x = np.asarray(x, dtype=F64)
    if dtype == "f32":
        return x.astype(np.float32).astype(F64)
    if dtype == "f16":
        return x.astype(np.float16).astype(F64)
    if dtype == "bf16":
        # f64 → bf16 directly (going through f32 first could double-round): 8 significant bits,
        # quantum never below the subnormal step 2**-133
        _, exponent = np.frexp(x)
        quantum = np.ldexp(1.0, np.maximum(exponent - 8, -133))
        rounded = np.rint(x / quantum) * quantum  # rint rounds half to even
        return np.where(np.isfinite(x), rounded, x)
    if dtype in ("i32", "i64", "index", "i8"):
        return np.asarray(x).astype(np.int64).astype(F64)
    if dtype == "i1":
        return (np.asarray(x) != 0).astype(F64)
    raise ValueError(dtype)


# ---------------------------------------------------------------------------------------------
# traced-kernel interpreter
# ---------------------------------------------------------------------------------------------
_SCALAR_BINARY = {
    "add": np.add, "sub": np.subtract, "mul": np.multiply,
    "max": lambda a, b: np.where(a >= b, a, b), "min": lambda a, b: np.where(a <= b, a, b),
    "cmp_lt": np.less, "cmp_le": np.less_equal, "cmp_gt": np.greater, "cmp_ge": np.greater_equal,
    "cmp_eq": np.equal, "cmp_ne": np.not_equal,
    "and": np.logical_and, "or": np.logical_or, "xor": np.logical_xor,
    "bitand": np.bitwise_and, "bitor": np.bitwise_or, "bitxor": np.bitwise_xor,
    "math_atan2": np.arctan2,
}
_erf = np.vectorize(math.erf, otypes=[F64])
_UNARY = {
    "neg": np.negative, "abs": np.abs, "bitnot": np.invert,
    "math_sqrt": np.sqrt, "math_rsqrt": lambda v: 1.0 / np.sqrt(v), "math_exp": np.exp, "math_exp2": np.exp2,
    "math_log": np.log, "math_log2": np.log2, "math_log10": np.log10, "math_sin": np.sin, "math_cos": np.cos,
    "math_acos": np.arccos, "math_asin": np.arcsin, "math_atan": np.arctan, "math_erf": _erf,
    # upstream uses Python's math.floor/ceil/trunc/round, which return ints
    "math_floor": np.floor, "math_ceil": np.ceil, "math_trunc": np.trunc, "math_round": np.rint,
}
_TENSOR_ALIAS = {
    "tensor_add": "add", "tensor_sub": "sub", "tensor_mul": "mul", "tensor_div": "div",
    "tensor_max": "max", "tensor_min": "min", "tensor_neg": "neg", "tensor_abs": "abs",
    "tensor_bitand": "bitand", "tensor_bitor": "bitor", "tensor_bitxor": "bitxor", "tensor_bitnot": "bitnot",
}


def _as_index(value: np.ndarray) -> np.ndarray:
    return np.asarray(value).astype(np.int64)


def run_kernel_ir(ir: dict[str, Any], arguments: dict[str, Any]) -> None:
    """Execute a traced elementwise kernel on host arrays, in place.

    ``ir`` is ``PortableKernelIR.to_dict()``; ``arguments`` maps IR argument
    names to float64/int64 ndarrays (tensors, shaped like their spec; mutated in
    place) or Python numbers (scalars).  All ``grid × block`` emulated threads
    are evaluated together; an out-of-range unmasked access raises IndexError
    just as upstream's list indexing would.
    """
    launch = ir["launch"]
    grid, block = launch["grid"], launch["block"]
    # thread enumeration order of upstream: block z,y,x outer, thread z,y,x inner (x fastest)
    bz, by, bx, tz, ty, tx = np.meshgrid(
        *(np.arange(n, dtype=np.int64) for n in (grid[2], grid[1], grid[0], block[2], block[1], block[0])), indexing="ij"
    )
    topo = {
        ("block_idx", "x"): bx, ("block_idx", "y"): by, ("block_idx", "z"): bz,
        ("program_id", "x"): bx, ("program_id", "y"): by, ("program_id", "z"): bz,
        ("thread_idx", "x"): tx, ("thread_idx", "y"): ty, ("thread_idx", "z"): tz,
    }
    threads = bx.size
    env: dict[str, Any] = {}
    tensors: dict[str, np.ndarray] = {}
    for argument in ir["arguments"]:
        value = arguments[argument["name"]]
        if argument["kind"] == "tensor":
            tensors[argument["name"]] = value
        env[argument["name"]] = value

    def flat_offset(name: str, indices: list[np.ndarray]) -> np.ndarray:
        array = tensors[name]
        offset = np.zeros(threads, dtype=np.int64)
        for axis, index in enumerate(indices):
            index = np.broadcast_to(_as_index(index).reshape(-1) if np.ndim(index) else _as_index(index), (threads,))
            offset = offset * array.shape[axis] + index
            if ((index < 0) | (index >= array.shape[axis])).any():
                raise IndexError(f"{name}: index out of range on axis {axis}")
        return offset

    def lane(value: Any) -> np.ndarray:
        return np.broadcast_to(np.asarray(value).reshape(-1) if np.ndim(value) else np.asarray(value), (threads,))

    # Whole-tensor values (tensor-SSA form) by name.  Every emulated thread runs the same whole-tensor statement, so a
    # per-thread scalar that meets a whole tensor (``src.load() + alpha[0]``) must be the same for all threads and is
    # used as that one value.
    whole_values: set[str] = set(tensors)

    def operand(name: str, whole: bool) -> Any:
        value = env[name]
        if whole and threads > 1 and name not in whole_values and np.ndim(value) == 1 and np.shape(value)[0] == threads:
            array = np.asarray(value)
            if not np.all(array == array[0]):
                raise NotImplementedError("oracle: a whole-tensor op consumes a scalar that differs between threads")
            return array[0]
        return value

    for operation in ir["operations"]:
        op, ins, outs, attrs = operation["op"], operation["inputs"], operation["outputs"], operation["attrs"]
        result: Any = None
        whole = op not in ("load", "store", "masked_load", "masked_store") and any(name in whole_values for name in ins)

        def arg(position: int) -> Any:
            return operand(ins[position], whole)

        if op in ("block_idx", "program_id", "thread_idx"):
            result = topo[(op, attrs["axis"])]
        elif op == "block_dim":
            result = np.int64(block["xyz".index(attrs["axis"])])
        elif op == "grid_dim":
            result = np.int64(grid["xyz".index(attrs["axis"])])
        elif op == "constant":
            result = attrs["value"]
        elif op == "tensor_dim":
            result = np.int64(attrs["value"])
        elif op == "cast":
            source = arg(0)
            target = attrs["target_dtype"]
            result = np.asarray(source).astype(F64) if target.startswith(("f", "bf")) else _as_index(source)
        elif op in ("floordiv", "mod"):
            lhs, rhs = _as_index(arg(0)), _as_index(arg(1))
            result = lhs // rhs if op == "floordiv" else lhs % rhs
        elif op == "div":
            result = np.asarray(arg(0), dtype=F64) / np.asarray(arg(1), dtype=F64)
        elif op in ("bitand", "bitor", "bitxor"):  # Python int semantics (two's complement, unbounded)
            result = _SCALAR_BINARY[op](_as_index(arg(0)), _as_index(arg(1)))
        elif op == "bitnot":
            result = np.invert(_as_index(arg(0)))
        elif op in _SCALAR_BINARY:
            result = _SCALAR_BINARY[op](np.asarray(arg(0)), np.asarray(arg(1)))
        elif op in _UNARY:
            result = _UNARY[op](np.asarray(arg(0)))
        elif op == "select":
            result = np.where(np.asarray(arg(0)).astype(bool), arg(1), arg(2))
        elif op == "tensor_select":  # frontend.py:2626-2640: element-wise choice, scalar branches broadcast
            result = np.where(np.asarray(arg(0)).astype(bool), arg(1), arg(2))
        elif op == "load":
            result = tensors[ins[0]].reshape(-1)[flat_offset(ins[0], [env[n] for n in ins[1:]])]
        elif op == "masked_load":
            rank = attrs["rank"]
            mask = lane(env[ins[1 + rank]]).astype(bool)
            fallback = lane(env[ins[2 + rank]])
            indices = [np.where(mask, lane(env[n]), 0) for n in ins[1:1 + rank]]
            result = np.where(mask, tensors[ins[0]].reshape(-1)[flat_offset(ins[0], indices)], fallback)
        elif op in ("store", "masked_store"):
            rank = attrs["rank"]
            value = lane(env[ins[0]])
            if op == "store":
                offset = flat_offset(ins[1], [env[n] for n in ins[2:2 + rank]])
                tensors[ins[1]].reshape(-1)[offset] = value  # later threads win, as in the sequential loop
            else:
                mask = lane(env[ins[2 + rank]]).astype(bool)
                indices = [np.where(mask, lane(env[n]), 0) for n in ins[2:2 + rank]]
                offset = flat_offset(ins[1], indices)
                tensors[ins[1]].reshape(-1)[offset[mask]] = value[mask]
        # ---- tensor-SSA ------------------------------------------------------------------------
        elif op == "make_tensor":
            env[outs[0]] = np.zeros(attrs["shape"], dtype=F64)
            whole_values.add(outs[0])
            continue
        elif op == "copy_reduce":
            # frontend.py:1957-1979: dst[i] = dst[i] (op) src[i]; the statement runs once per emulated thread, so kinds
            # that are not idempotent (add, xor) are applied `threads` times, exactly as the sequential launch loop does
            kind = str(attrs["reduction"]).lower()
            source, target = tensors[ins[0]], tensors[ins[1]]
            combine = {"add": np.add, "max": np.maximum, "min": np.minimum,
                       "and": np.bitwise_and, "or": np.bitwise_or, "xor": np.bitwise_xor}[kind]
            integer = kind in ("and", "or", "xor")
            for _ in range(threads if kind in ("add", "xor") else 1):
                if integer:
                    target[...] = combine(_as_index(target), _as_index(source))
                else:
                    target[...] = combine(target, source)
            continue
        elif op == "copy":
            source = env[ins[0]]
            if ins[1] in tensors:
                tensors[ins[1]][...] = source
            else:
                env[ins[1]] = np.array(source, dtype=F64)
                whole_values.add(ins[1])
            continue
        elif op == "fill":
            env[ins[0]] = np.full(np.shape(env[ins[0]]), env[ins[1]], dtype=F64)
            continue
        elif op == "broadcast_to":
            result = np.broadcast_to(env[ins[0]], attrs["target_shape"])
        elif op.startswith("reduce_"):
            # upstream runtime.py:484-505: fold of every element of the reduced axes, starting from the init value
            profile = attrs.get("reduction_profile", 0)
            source = np.asarray(env[ins[0]])
            keep = () if profile == 0 else tuple(axis for axis, item in enumerate(profile) if item is None)
            kept_shape = tuple(source.shape[axis] for axis in keep)
            folded_view = np.moveaxis(source, keep, range(len(keep))).reshape(kept_shape + (-1,))
            kind = op[len("reduce_"):]
            integer = kind in ("and", "or", "xor")
            ufunc = {"add": np.add, "mul": np.multiply, "max": np.maximum, "min": np.minimum,
                     "and": np.bitwise_and, "or": np.bitwise_or, "xor": np.bitwise_xor}[kind]
            data = folded_view.astype(np.int64) if integer else folded_view.astype(F64)
            init = np.int64(env[ins[1]]) if integer else F64(env[ins[1]])
            result = ufunc(init, ufunc.reduce(data, axis=-1))
        elif op in _TENSOR_ALIAS:
            base = _TENSOR_ALIAS[op]
            operands = [np.asarray(arg(i)) for i in range(len(ins))]
            if base in ("bitand", "bitor", "bitxor", "bitnot"):
                operands = [_as_index(v) for v in operands]
            if base == "bitnot" and attrs.get("result", {}).get("dtype") == "i1":
                result = np.logical_not(operands[0].astype(bool))  # runtime.py:615-625: `not value` on i1 tensors, `~int` otherwise
            elif base == "div":
                result = operands[0] / operands[1]
            elif base in _UNARY:
                result = _UNARY[base](operands[0])
            else:
                result = _SCALAR_BINARY[base](*operands)
        else:
            raise NotImplementedError(f"oracle: op '{op}' is outside the elementwise path")
        if outs:
            env[outs[0]] = result
            if whole or op == "broadcast_to" or op in _TENSOR_ALIAS:
                whole_values.add(outs[0])


# ---------------------------------------------------------------------------------------------
# explicit ops
# ---------------------------------------------------------------------------------------------
def gemm(a: np.ndarray, b: np.ndarray, *, transpose_a: bool = False, transpose_b: bool = False) -> np.ndarray:
    """``C[m,n] = Σ_k A'[m,k]·B'[k,n]`` in f64; returns C (the caller's C contents are irrelevant)."""
    lhs = np.asarray(a, dtype=F64).T if transpose_a else np.asarray(a, dtype=F64)
    rhs = np.asarray(b, dtype=F64).T if transpose_b else np.asarray(b, dtype=F64)
    if lhs.shape[1] != rhs.shape[0]:
        raise ValueError(f"gemm shape mismatch: {a.shape} x {b.shape}")
    return lhs @ rhs


def rmsnorm(x: np.ndarray, gamma: np.ndarray, epsilon: float = 1e-5) -> np.ndarray:
    x = np.asarray(x, dtype=F64)
    gamma = np.asarray(gamma, dtype=F64)
    hidden = x.shape[-1]
    if gamma.shape not in {(hidden,), x.shape}:
        raise ValueError(f"rmsnorm expects gamma shape {(hidden,)} or {x.shape}, got {gamma.shape}")
    mean_square = np.sum(x * x, axis=-1, keepdims=True) / float(hidden)
    return x * (1.0 / np.sqrt(mean_square + float(epsilon))) * gamma


def layernorm(x: np.ndarray, residual: np.ndarray, weight: np.ndarray, bias: np.ndarray,
              epsilon: float = 1e-5) -> tuple[np.ndarray, np.ndarray]:
    """Upstream ``frontend.py:3754-3793``: returns (out, out_resid); biased variance, f64 throughout."""
    mixed = np.asarray(x, dtype=F64) + np.asarray(residual, dtype=F64)
    mean = mixed.sum(axis=-1, keepdims=True) / float(mixed.shape[-1])
    variance = ((mixed - mean) ** 2).sum(axis=-1, keepdims=True) / float(mixed.shape[-1])
    out = ((mixed - mean) / np.sqrt(variance + float(epsilon))) * np.asarray(weight, dtype=F64) + np.asarray(bias, dtype=F64)
    return out, mixed


def attention(q: np.ndarray, k: np.ndarray, v: np.ndarray, *, causal: bool = False) -> tuple[np.ndarray, np.ndarray]:
    """q/out ``[B,S,H,D]``, k/v ``[B,S,Hkv,D]`` → (out ``[B,S,H,D]``, lse ``[B,H,1,S]``), all f64."""
    q, k, v = (np.asarray(t, dtype=F64) for t in (q, k, v))
    bsz, seqlen, heads, head_dim = q.shape
    kv_heads = k.shape[2]
    if heads % kv_heads:
        raise ValueError("attention requires q heads to be divisible by kv heads")
    group = heads // kv_heads
    scale = 1.0 / math.sqrt(float(head_dim))
    out = np.empty_like(q)
    lse = np.empty((bsz, heads, 1, seqlen), dtype=F64)
    future = np.triu(np.ones((seqlen, seqlen), dtype=bool), k=1) if causal else None
    for batch in range(bsz):
        for head in range(heads):
            kv = head // group
            scores = (q[batch, :, head, :] @ k[batch, :, kv, :].T) * scale
            if future is not None:
                scores = np.where(future, -np.inf, scores)
            row_max = scores.max(axis=1, keepdims=True)
            weights = np.where(np.isneginf(scores), 0.0, np.exp(scores - row_max))
            norm = weights.sum(axis=1, keepdims=True)
            with np.errstate(divide="ignore"):
                lse[batch, head, 0, :] = np.where(norm[:, 0] == 0.0, -np.inf, np.log(norm[:, 0]) + row_max[:, 0])
            out[batch, :, head, :] = (weights / norm) @ v[batch, :, kv, :]
    return out, lse


def rel_l2(actual: np.ndarray, expected: np.ndarray) -> float:
    actual = np.asarray(actual, dtype=F64).reshape(-1)
    expected = np.asarray(expected, dtype=F64).reshape(-1)
    denom = float(np.linalg.norm(expected))
    return float(np.linalg.norm(actual - expected)) / (denom if denom else 1.0)
