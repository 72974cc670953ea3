"""The 512 x 256 CTA-pair GEMM tile, forced on shapes the launcher would give to other kernels.

The launcher picks a kernel from the problem's shape and reads ``BB200_GEMM_PAIR`` once per process, so the forced runs
happen in a child interpreter (``BB200_GEMM_PAIR=2``): one full tile, ragged edges in m, n and k, several row blocks, both
output dtypes — each through the C ABI against the oracle, like the other GEMM tests.
"""
from __future__ import annotations

import os
import subprocess
import sys
import textwrap
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent

CHILD = textwrap.dedent("""
    import ctypes, sys
    import numpy as np
    sys.path.insert(0, %(root)r); sys.path.insert(0, %(tests)r)
    import torch
    from baybridge_b200.backend import native
    from gpu_util import current_stream, device_zeros, to_device, to_host, void_p
    from oracle import cpu_runtime as oracle
    failures = []
    for m, n, k in [(512, 256, 64), (512, 512, 1024), (1000, 520, 264), (1536, 768, 320), (640, 1032, 200), (2048, 2048, 512)]:
        rng = np.random.default_rng(m * 7 + n)
        a = oracle.bf16_round((rng.standard_normal((m, k)) / np.sqrt(k)).astype(np.float32))
        b = oracle.bf16_round((rng.standard_normal((n, k)) / np.sqrt(k)).astype(np.float32))
        reference = oracle.gemm(a, b, transpose_b=True)
        for c_dtype, bar in (("bf16", 1e-2), ("f32", 1e-5)):
            d_a, d_b, d_c = to_device(a, "bf16"), to_device(b, "bf16"), device_zeros((m, n), c_dtype)
            native.call("bb200_gemm_bf16", void_p(d_a), void_p(d_b), void_p(d_c), m, n, k, 0, 1, native.DTYPE_CODES[c_dtype], current_stream())
            torch.cuda.synchronize()
            status = native.take_device_status(current_stream())
            error = oracle.rel_l2(to_host(d_c), reference)
            if status or not error <= bar:
                failures.append((m, n, k, c_dtype, status, error))
    print("FAILURES", failures)
    sys.exit(1 if failures else 0)
""")


def test_wide_pair_tile_matches_the_oracle_on_forced_shapes(tmp_path):
    script = tmp_path / "wide_child.py"
    script.write_text(CHILD % {"root": str(ROOT), "tests": str(ROOT / "tests")})
    done = subprocess.run([sys.executable, str(script)], env=dict(os.environ, BB200_GEMM_PAIR="2"), stdout=subprocess.PIPE,
                          stderr=subprocess.STDOUT, text=True, timeout=600)
    assert done.returncode == 0, done.stdout[-3000:]
