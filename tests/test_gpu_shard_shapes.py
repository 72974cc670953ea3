"""The per-rank shard shapes of the five configurations (2-, 4- and 8-way splits of the outer axis), each run on one
GPU through the benchmark's own workload objects and compared with the oracle on sampled units — the same check
``bench.py`` applies to the gathered output of a multi-GPU run, here without needing more than one GPU."""
from __future__ import annotations

import argparse

import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def context():
    import bench

    args = argparse.Namespace(scaling="strong", kernel_only=False, e2e_steps=1, no_cpu_baseline=True, small=False, steps=1, warmup=1,
                              gpus=1, workload="all", impl="b200")
    return bench.Context(args)


@pytest.mark.parametrize("ways", [2, 4, 8])
@pytest.mark.parametrize("name", ["fused_mul_add", "gemm", "rmsnorm", "attention", "indexed_add"])
def test_shard_shape_matches_the_oracle(context, name, ways):
    import bench

    workload = bench.WORKLOADS[name]()
    workload.extent //= ways  # one rank's share of the outer axis; everything else stays at the configuration's size
    try:
        workload.prepare(context)
        workload.step_in_place()
        context.torch.cuda.synchronize()
        record = workload.check(workload.outputs)
    finally:
        bench.release(context, workload)
    assert record["ok"], record
    assert record["samples"] >= 1
