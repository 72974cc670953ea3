#!/usr/bin/env python3
"""Time upstream's own CPU reference runtime on a reduced case of one workload — TEST INFRASTRUCTURE.

    python oracle/ref_runtime.py --workload fused_mul_add --size 65536 --steps 3 --warmup 1

Runs in a process of its own (``bench.py`` starts it as a subprocess): it imports the unmodified
upstream package from ``oracle/_ref/`` (put there by ``oracle/make_ref.py``), builds the workload's
kernel from ``baybridge_b200/samples.py`` against the *upstream* DSL, and calls the compiled artifact
through upstream's public API, ``compile(kernel, *args, backend="portable")(*args)``, which executes

* the sequential launch loop of ``frontend.py:783-821`` for traced elementwise kernels
  (``indexed_add``: one Python call per emulated thread; ``fused_mul_add``: the tensor-SSA form,
  ``runtime.py:464-532``),
* ``gemm`` ``frontend.py:3709-3716``, ``rmsnorm`` ``:3845-3852``, ``attention`` ``:3903-3937``.

The runtime is single-threaded interpreted Python over lists of floats, so only the 256x256 indexed add
runs at full size; the other workloads are timed at ``--size`` and reported with their work per step so
the caller can quote a per-unit rate.  Prints one JSON line: ``{"workload", "seconds": [per step...],
"work_per_step", "unit_of_work", "sample", "cores": 1}``.
"""
from __future__ import annotations

import argparse
import json
import math
import sys
import time
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
REF = HERE / "_ref"


def bf16_round(x: np.ndarray) -> np.ndarray:
    bits = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    bias = ((bits >> 16) & 1) + 0x7FFF
    return (((bits + bias) >> 16) << 16).astype(np.uint32).view(np.float32)


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--workload", required=True, choices=["indexed_add", "fused_mul_add", "gemm", "rmsnorm", "attention"])
    parser.add_argument("--size", type=int, default=0, help="elements / M=N=K / rows / sequence length of the reduced case")
    parser.add_argument("--steps", type=int, default=1)
    parser.add_argument("--warmup", type=int, default=0)
    args = parser.parse_args()
    if not (REF / "baybridge" / "__init__.py").exists():
        raise SystemExit("oracle/_ref/baybridge is missing: run oracle/make_ref.py where an upstream checkout exists")
    sys.path.insert(0, str(REF))
    sys.path.insert(1, str(HERE.parent))
    import baybridge as bb  # upstream, unmodified

    from baybridge_b200.samples import build_zoo

    zoo = build_zoo(bb)

    def tensor(array: np.ndarray, dtype: str):
        return bb.tensor(np.asarray(array, dtype=np.float64).tolist(), dtype=dtype)

    name = args.workload
    if name == "indexed_add":
        rows = cols = args.size or 256
        rng = np.random.default_rng(1001)
        a, b = (rng.uniform(-1, 1, (rows, cols)).astype(np.float32) for _ in range(2))
        kernel, operands = zoo.make_indexed_add_2d(rows, cols), [tensor(a, "f32"), tensor(b, "f32"), bb.zeros((rows, cols), dtype="f32")]
        work, unit, sample = 3.0 * rows * cols * 4, "bytes", f"f32 {rows}x{cols}, one emulated thread per element"
    elif name == "fused_mul_add":
        n = args.size or 2**16
        rng = np.random.default_rng(1002)
        a, b = (bf16_round(rng.standard_normal(n, dtype=np.float32)) for _ in range(2))
        kernel, operands = zoo.fused_mul_add_ssa, [tensor(a, "bf16"), tensor(b, "bf16"), bb.zeros((n,), dtype="bf16")]
        work, unit, sample = 6.0 * n, "bytes", f"{n} of 2^28 elements, tensor-SSA form"
    elif name == "gemm":
        size = args.size or 64
        rng = np.random.default_rng(1003)
        a, b = (bf16_round((rng.standard_normal((size, size)) / math.sqrt(size)).astype(np.float32)) for _ in range(2))
        kernel, operands = zoo.gemm_abt, [tensor(a, "bf16"), tensor(b, "bf16"), bb.zeros((size, size), dtype="bf16")]
        work, unit, sample = 2.0 * size**3, "flop", f"M=N=K={size} (of 8192)"
    elif name == "rmsnorm":
        rows, hidden = args.size or 8, 8192
        rng = np.random.default_rng(1004)
        x = bf16_round(rng.standard_normal((rows, hidden), dtype=np.float32))
        w = bf16_round((1 + 0.1 * rng.standard_normal(hidden)).astype(np.float32))
        kernel, operands = zoo.make_rmsnorm(1e-6), [tensor(x, "bf16"), bb.zeros((rows, hidden), dtype="bf16"), tensor(w, "bf16")]
        work, unit, sample = 2.0 * rows * hidden * 2 + hidden * 2, "bytes", f"{rows} of 65536 rows x {hidden}"
    else:
        seq, heads, dim = args.size or 64, 2, 128
        rng = np.random.default_rng(1005)
        q, k, v = (bf16_round(rng.standard_normal((1, seq, heads, dim), dtype=np.float32)) for _ in range(3))
        kernel = zoo.attention_causal
        operands = [tensor(q, "bf16"), tensor(k, "bf16"), tensor(v, "bf16"), bb.zeros((1, seq, heads, dim), dtype="bf16"),
                    bb.zeros((1, heads, 1, seq), dtype="f32")]
        work, unit, sample = 4.0 * heads * dim * seq * (seq + 1) / 2, "flop", f"B1 H{heads} S{seq} D{dim} causal (of B16 H32 S4096)"
    artifact = bb.compile(kernel, *operands, backend="portable")
    for _ in range(args.warmup):
        artifact(*operands)
    seconds = []
    for _ in range(max(1, args.steps)):
        started = time.perf_counter()
        artifact(*operands)
        seconds.append(time.perf_counter() - started)
    print(json.dumps({"workload": name, "seconds": seconds, "work_per_step": work, "unit_of_work": unit, "sample": sample,
                      "cores": 1}), flush=True)


if __name__ == "__main__":
    main()
