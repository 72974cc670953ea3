"""The conformance sweep: one table of small kernels shared by the fixture generator and the tests.

Every entry names a kernel factory of ``baybridge_b200/samples.py`` and the tensors it runs on.  The generator
(``make_golden.py``) builds each kernel against UPSTREAM's package, runs it on upstream's CPU reference runtime and
stores inputs and outputs as ``vec_sw_<name>.npz`` plus the traced listing as ``ir_sw_<name>.json``; the tests build
the same kernel against this package, compare the traced IR and cache key byte for byte, run it on the GPU and
compare with the stored outputs.  The families follow upstream's executable-backend conformance kernels
(``tests/test_backend_ptx_exec.py:430-2330``): whole-tensor binary / unary / compare / select / broadcast /
scalar-parameter / one-element-tensor forms, copies, reducing copies and reductions, each under the serial
(one thread), parallel (one block) and multiblock (2-D grid) launch shapes.

Inputs come from ``numpy.random.default_rng(crc32(name))`` and are representable in the tensor dtype.
"""
from __future__ import annotations

import zlib
from dataclasses import dataclass
from typing import Any

import numpy as np

SHAPE = (4, 8)
FLOAT_MATH = ("sqrt", "rsqrt", "sin", "cos", "exp2", "exp", "log2", "log", "log10", "round", "floor", "ceil", "trunc",
              "atan", "asin", "acos", "erf")
LIBM_OPS = {"rsqrt", "sin", "cos", "exp2", "exp", "log2", "log", "log10", "atan", "asin", "acos", "erf", "atan2"}


@dataclass(frozen=True)
class Argument:
    name: str
    shape: tuple[int, ...] | None  # None: a scalar parameter
    dtype: str                      # f32 / f16 / bf16 / i32 / i1, or the scalar's dtype
    role: str                       # "in", "out" or "inout"
    fill: Any = "uniform"           # value distribution of an input tensor, or the scalar's value


@dataclass(frozen=True)
class Case:
    name: str
    factory: str
    factory_args: tuple
    arguments: tuple[Argument, ...]
    max_ulp: int = 0                # 0: bit-exact against the f64 reference rounded once to the storage dtype

    def kernel(self, zoo):
        return getattr(zoo, self.factory)(*self.factory_args)

    def inputs(self) -> dict[str, np.ndarray]:
        rng = np.random.default_rng(zlib.crc32(self.name.encode()))
        return {a.name: _draw(rng, a) for a in self.arguments if a.shape is not None}

    @property
    def outputs(self) -> tuple[str, ...]:
        return tuple(a.name for a in self.arguments if a.role in ("out", "inout"))


def _draw(rng, argument: Argument) -> np.ndarray:
    shape, dtype, fill = argument.shape, argument.dtype, argument.fill
    if argument.role == "out":
        return np.zeros(shape, dtype=bool if dtype == "i1" else np.int64 if dtype.startswith("i") else np.float64)
    if dtype == "i1":
        return rng.integers(0, 2, shape).astype(bool)
    if dtype.startswith("i"):
        if fill == "bits":
            return rng.integers(0, 1 << 20, shape).astype(np.int64)
        if fill == "nonzero":
            return (rng.integers(1, 9, shape) * rng.choice([-1, 1], shape)).astype(np.int64)
        if fill == "multiples":  # of the matching "nonzero" divisor drawn next from the same stream: see _fix_division
            return rng.integers(-9, 10, shape).astype(np.int64)
        if fill == "small":
            return rng.integers(1, 3, shape).astype(np.int64)
        return rng.integers(-50, 51, shape).astype(np.int64)
    low, high = {"uniform": (-2.0, 2.0), "positive": (0.25, 3.0), "unit": (-0.95, 0.95), "near_one": (0.9, 1.1),
                 "nonzero": (0.5, 2.5)}[fill]
    values = rng.uniform(low, high, shape).astype(np.float32)
    if dtype == "f16":
        values = values.astype(np.float16).astype(np.float32)
    elif dtype == "bf16":
        bits = values.view(np.uint32).astype(np.uint64)
        values = ((((bits + (((bits >> 16) & 1) + 0x7FFF)) >> 16) << 16).astype(np.uint32)).view(np.float32)
    return values.astype(np.float64)


def _tensor(name: str, dtype: str, role: str = "in", fill: Any = "uniform", shape: tuple[int, ...] = SHAPE) -> Argument:
    return Argument(name, shape, dtype, role, fill)


def _fill_for(op: str, position: int = 0) -> str:
    if op in ("sqrt", "rsqrt", "log", "log2", "log10"):
        return "positive"
    if op in ("asin", "acos"):
        return "unit"
    if op == "div" and position == 1:
        return "nonzero"
    return "uniform"


def build_cases() -> list[Case]:
    cases: list[Case] = []

    def add(name: str, factory: str, factory_args: tuple, arguments: list[Argument], op: str = "") -> None:
        cases.append(Case(name, factory, factory_args, tuple(arguments), max_ulp=1 if op in LIBM_OPS else 0))

    every = ("serial", "parallel", "multiblock")
    # ---- dense binary ------------------------------------------------------------------------------------------
    for launch in every:
        for op in ("add", "sub", "mul", "div", "max", "min", "atan2"):
            add(f"dense_{op}_f32_{launch}", "make_dense_binary", (op, launch),
                [_tensor("lhs", "f32"), _tensor("rhs", "f32", fill=_fill_for(op, 1)), _tensor("dst", "f32", "out")], op)
    for op in ("add", "sub", "mul", "max", "min", "bitand", "bitor", "bitxor"):
        fill = "bits" if op.startswith("bit") else "uniform"
        add(f"dense_{op}_i32_serial", "make_dense_binary", (op, "serial"),
            [_tensor("lhs", "i32", fill=fill), _tensor("rhs", "i32", fill=fill), _tensor("dst", "i32", "out")])
    for launch in ("parallel", "multiblock"):
        for op in ("add", "bitxor"):
            fill = "bits" if op.startswith("bit") else "uniform"
            add(f"dense_{op}_i32_{launch}", "make_dense_binary", (op, launch),
                [_tensor("lhs", "i32", fill=fill), _tensor("rhs", "i32", fill=fill), _tensor("dst", "i32", "out")])
    for op, launch in (("bitand", "serial"), ("bitor", "serial"), ("bitxor", "serial"), ("bitxor", "parallel"), ("bitand", "multiblock")):
        add(f"dense_{op}_i1_{launch}", "make_dense_binary", (op, launch),
            [_tensor("lhs", "i1"), _tensor("rhs", "i1"), _tensor("dst", "i1", "out")])
    add("dense_add_f16_serial", "make_dense_binary", ("add", "serial"),
        [_tensor("lhs", "f16"), _tensor("rhs", "f16"), _tensor("dst", "f16", "out")])
    add("dense_mul_bf16_parallel", "make_dense_binary", ("mul", "parallel"),
        [_tensor("lhs", "bf16"), _tensor("rhs", "bf16"), _tensor("dst", "bf16", "out")])
    # ---- compare → i1 ----------------------------------------------------------------------------------------------
    for launch in every:
        add(f"dense_cmp_lt_f32_{launch}", "make_dense_binary", ("cmp_lt", launch),
            [_tensor("lhs", "f32"), _tensor("rhs", "f32"), _tensor("dst", "i1", "out")])
        add(f"dense_cmp_eq_i32_{launch}", "make_dense_binary", ("cmp_eq", launch),
            [_tensor("lhs", "i32", fill="small"), _tensor("rhs", "i32", fill="small"), _tensor("dst", "i1", "out")])
    # ---- broadcast (a row or a column vector against the full shape) -------------------------------------------------
    row, column = (1, SHAPE[1]), (SHAPE[0], 1)
    for index, op in enumerate(("add", "sub", "mul", "div", "atan2", "max")):
        vector = row if index % 2 == 0 else column
        launch = every[index % 3]
        add(f"broadcast_{op}_f32_{launch}", "make_dense_binary", (op, launch),
            [_tensor("lhs", "f32"), _tensor("rhs", "f32", fill=_fill_for(op, 1), shape=vector), _tensor("dst", "f32", "out")], op)
    for index, op in enumerate(("add", "sub", "mul", "bitand", "bitor", "bitxor", "min")):
        vector = column if index % 2 == 0 else row
        fill = "bits" if op.startswith("bit") else "uniform"
        add(f"broadcast_{op}_i32_{every[index % 3]}", "make_dense_binary", (op, every[index % 3]),
            [_tensor("lhs", "i32", fill=fill), _tensor("rhs", "i32", fill=fill, shape=vector), _tensor("dst", "i32", "out")])
    add("broadcast_cmp_eq_i32_serial", "make_dense_binary", ("cmp_eq", "serial"),
        [_tensor("lhs", "i32", fill="small"), _tensor("rhs", "i32", fill="small", shape=row), _tensor("dst", "i1", "out")])
    add("broadcast_bitor_i1_multiblock", "make_dense_binary", ("bitor", "multiblock"),
        [_tensor("lhs", "i1"), _tensor("rhs", "i1", shape=column), _tensor("dst", "i1", "out")])
    # ---- unary --------------------------------------------------------------------------------------------------------
    for op in FLOAT_MATH + ("neg", "abs"):
        add(f"dense_{op}_f32_serial", "make_dense_unary", (op, "serial"),
            [_tensor("src", "f32", fill=_fill_for(op)), _tensor("dst", "f32", "out")], op)
    for index, op in enumerate(FLOAT_MATH + ("neg", "abs")):
        launch = ("parallel", "multiblock")[index % 2]
        add(f"dense_{op}_f32_{launch}", "make_dense_unary", (op, launch),
            [_tensor("src", "f32", fill=_fill_for(op)), _tensor("dst", "f32", "out")], op)
    for op, dtype, launch in (("neg", "i32", "serial"), ("abs", "i32", "parallel"), ("bitnot", "i32", "serial"), ("bitnot", "i32", "multiblock"),
                              ("neg", "f16", "serial"), ("abs", "f16", "multiblock"), ("bitnot", "i1", "serial"), ("bitnot", "i1", "parallel")):
        add(f"dense_{op}_{dtype}_{launch}", "make_dense_unary", (op, launch),
            [_tensor("src", dtype, fill="bits" if op == "bitnot" and dtype == "i32" else "uniform"), _tensor("dst", dtype, "out")])
    # ---- scalar kernel parameter ----------------------------------------------------------------------------------------
    for index, op in enumerate(("add", "sub", "mul", "div", "atan2", "max", "min")):
        add(f"scalar_{op}_f32_{every[index % 3]}", "make_dense_scalar_binary", (op, "f32", every[index % 3]),
            [_tensor("src", "f32"), Argument("alpha", None, "f32", "in", 0.75), _tensor("dst", "f32", "out")], op)
    for index, op in enumerate(("add", "sub", "mul", "bitand", "bitor", "bitxor")):
        add(f"scalar_{op}_i32_{every[index % 3]}", "make_dense_scalar_binary", (op, "i32", every[index % 3]),
            [_tensor("src", "i32", fill="bits" if op.startswith("bit") else "uniform"), Argument("alpha", None, "i32", "in", 5),
             _tensor("dst", "i32", "out")])
    add("scalar_cmp_lt_f32_serial", "make_dense_scalar_binary", ("cmp_lt", "f32", "serial"),
        [_tensor("src", "f32"), Argument("alpha", None, "f32", "in", 0.25), _tensor("dst", "i1", "out")])
    add("scalar_cmp_lt_f32_multiblock", "make_dense_scalar_binary", ("cmp_lt", "f32", "multiblock"),
        [_tensor("src", "f32"), Argument("alpha", None, "f32", "in", 0.25), _tensor("dst", "i1", "out")])
    # ---- one-element tensor used as a scalar --------------------------------------------------------------------------------
    for index, op in enumerate(("add", "sub", "mul", "div", "atan2")):
        add(f"tensor_scalar_{op}_f32_{every[index % 3]}", "make_dense_tensor_scalar_binary", (op, every[index % 3]),
            [_tensor("src", "f32"), _tensor("alpha", "f32", fill="nonzero", shape=(1,)), _tensor("dst", "f32", "out")], op)
    for index, op in enumerate(("add", "sub", "mul", "bitand", "bitor", "bitxor")):
        fill = "bits" if op.startswith("bit") else "uniform"
        add(f"tensor_scalar_{op}_i32_{every[(index + 1) % 3]}", "make_dense_tensor_scalar_binary", (op, every[(index + 1) % 3]),
            [_tensor("src", "i32", fill=fill), _tensor("alpha", "i32", fill=fill, shape=(1,)), _tensor("dst", "i32", "out")])
    add("tensor_scalar_cmp_eq_i32_parallel", "make_dense_tensor_scalar_binary", ("cmp_eq", "parallel"),
        [_tensor("src", "i32", fill="small"), _tensor("alpha", "i32", fill="small", shape=(1,)), _tensor("dst", "i1", "out")])
    # ---- select ---------------------------------------------------------------------------------------------------------------
    for launch in every:
        add(f"select_f32_{launch}", "make_dense_select", ("tensor", launch),
            [_tensor("pred", "i1"), _tensor("lhs", "f32"), _tensor("rhs", "f32"), _tensor("dst", "f32", "out")])
        add(f"select_scalar_f32_{launch}", "make_dense_select", ("scalar", launch),
            [_tensor("pred", "i1"), _tensor("src", "f32"), Argument("alpha", None, "f32", "in", -1.5), _tensor("dst", "f32", "out")])
        add(f"select_tensor_scalar_i32_{launch}", "make_dense_select", ("tensor_scalar", launch),
            [_tensor("pred", "i1"), _tensor("src", "i32"), _tensor("alpha", "i32", shape=(1,)), _tensor("dst", "i32", "out")])
    add("select_i32_serial", "make_dense_select", ("tensor", "serial"),
        [_tensor("pred", "i1"), _tensor("lhs", "i32"), _tensor("rhs", "i32"), _tensor("dst", "i32", "out")])
    add("select_i1_parallel", "make_dense_select", ("tensor", "parallel"),
        [_tensor("pred", "i1"), _tensor("lhs", "i1"), _tensor("rhs", "i1"), _tensor("dst", "i1", "out")])
    # ---- copies and reducing copies ---------------------------------------------------------------------------------------------
    for launch in every:
        add(f"copy_f32_{launch}", "make_dense_copy", (launch,), [_tensor("src", "f32"), _tensor("dst", "f32", "out")])
        add(f"copy_i32_{launch}", "make_dense_copy", (launch,), [_tensor("src", "i32"), _tensor("dst", "i32", "out")])
    # add and xor are applied once per emulated thread by the CPU runtime, so only the one-thread launch pins them; the
    # idempotent kinds (max, min, and, or) give the same result under every launch shape
    line = (128,)
    for kind, dtype, grid, block, shape in (
            ("add", "f32", 1, 1, line), ("xor", "i32", 1, 1, line), ("add", "i32", 1, 1, SHAPE), ("add", "f32", 1, 1, SHAPE),
            ("max", "f32", 1, 1, line), ("max", "f32", 2, 64, line), ("max", "f32", 1, 128, line), ("max", "f32", 1, 1, SHAPE),
            ("or", "i32", 1, 1, line), ("or", "i32", 1, 128, line), ("or", "i32", 2, 64, SHAPE), ("min", "f32", 2, 64, line),
            ("and", "i32", 1, 128, line), ("min", "i32", 1, 1, SHAPE), ("max", "bf16", 2, 64, line)):
        rank = "2d" if len(shape) == 2 else "1d"
        fill = "bits" if kind in ("and", "or", "xor") else "uniform"
        add(f"copy_reduce_{kind}_{dtype}_{rank}_g{grid}b{block}", "make_copy_reduce", (kind, grid, block),
            [_tensor("src", dtype, fill=fill, shape=shape), _tensor("dst", dtype, "inout", fill=fill, shape=shape)])
    # ---- reductions ------------------------------------------------------------------------------------------------------------------
    inits = {"add": 0.0, "mul": 1.0, "max": -99.0, "min": 99.0}
    for index, op in enumerate(("add", "mul", "max", "min")):
        launch = ("serial", "parallel")[index % 2]
        add(f"reduce_all_{op}_f32_{launch}", "make_reduce", (op, inits[op], "all", launch),
            [_tensor("src", "f32", fill="near_one" if op == "mul" else "uniform", shape=(256,)), _tensor("dst", "f32", "out", shape=(1,))])
    int_inits = {"add": 0, "mul": 1, "max": -999, "min": 999, "and": -1, "or": 0, "xor": 0}
    for index, op in enumerate(("add", "mul", "max", "min", "and", "or", "xor")):
        launch = ("parallel", "serial")[index % 2]
        fill = "bits" if op in ("and", "or", "xor") else "small" if op == "mul" else "uniform"
        add(f"reduce_all_{op}_i32_{launch}", "make_reduce", (op, int_inits[op], "all", launch),
            [_tensor("src", "i32", fill=fill, shape=(24,) if op == "mul" else (256,)), _tensor("dst", "i32", "out", shape=(1,))])
    wide = (6, 40)
    for axis in ("rows", "cols"):
        kept = (wide[0],) if axis == "rows" else (wide[1],)
        for index, op in enumerate(("add", "mul", "max", "min")):
            launch = every[index % 3]
            add(f"reduce_{axis}_{op}_f32_{launch}", "make_reduce", (op, inits[op], axis, launch),
                [_tensor("src", "f32", fill="near_one" if op == "mul" else "uniform", shape=wide), _tensor("dst", "f32", "out", shape=kept)])
        for index, op in enumerate(("add", "max", "min", "and", "or", "xor")):
            launch = every[(index + 1) % 3]
            fill = "bits" if op in ("and", "or", "xor") else "uniform"
            add(f"reduce_{axis}_{op}_i32_{launch}", "make_reduce", (op, int_inits[op], axis, launch),
                [_tensor("src", "i32", fill=fill, shape=wide), _tensor("dst", "i32", "out", shape=kept)])
    names = [case.name for case in cases]
    assert len(names) == len(set(names)), "duplicate sweep case names"
    return cases


CASES = build_cases()
BY_NAME = {case.name: case for case in CASES}

#: cases whose fixture upstream could not produce or whose kernel this backend declines; filled in by hand with the reason
EXCLUDED: dict[str, str] = {}
