"""Multi-rank host logic on CPU: world-size-2 (and 3, ragged) gloo process groups."""
from __future__ import annotations

import os
import socket

import numpy as np
import pytest
from conftest import golden_ir

from baybridge_b200.backend.matcher import match
from baybridge_b200.portable_ir import PortableKernelIR
from baybridge_b200.sharding import local_slices, shard_bounds, shard_spec


def test_shard_bounds_partition_exactly():
    for total in (0, 1, 7, 8, 65536, 2**28 + 3):
        for world in (1, 2, 3, 4, 8):
            cursor = 0
            sizes = []
            for rank in range(world):
                start, stop = shard_bounds(total, world, rank)
                assert start == cursor and stop >= start
                sizes.append(stop - start)
                cursor = stop
            assert cursor == total and max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard_bounds(8, 2, 2)


def test_shard_specs_of_the_five_configs():
    def spec_of(case):
        ir = PortableKernelIR.from_dict(golden_ir(case)["ir"])
        return shard_spec(match(ir), ir)

    c1 = spec_of("c1_indexed_add_256x256_f32")
    assert c1.extent == 256 and c1.outputs == (2,) and not c1.replicated
    c2 = spec_of("c2_fused_indexed_2p28_bf16")
    assert c2.extent == 2**28 and {p for p, _ in c2.sharded} == {0, 1, 2}
    c3 = spec_of("c3_gemm_abt_8192_bf16")
    assert c3.extent == 8192 and c3.sharded == ((0, 0), (2, 0)) and c3.replicated == (1,)
    assert spec_of("gemm_atb_48x40x64_bf16").sharded == ((0, 1), (2, 0))  # A stored [k, m]: split its columns
    c4 = spec_of("c4_rmsnorm_65536x8192_bf16")
    assert c4.extent == 65536 and c4.replicated == (2,) and c4.outputs == (1,)
    c5 = spec_of("c5_attn_causal_b16s4096h32d128")
    assert c5.extent == 16 and c5.outputs == (3, 4)
    assert local_slices(c5, 8, 3)[0] == (0, slice(6, 8))
    norm = spec_of("layernorm_2x4x128_bf16")   # rank-3 input: the leading axis splits, weight and bias are replicated
    assert norm.extent == 2 and norm.sharded == ((0, 0), (1, 0), (2, 0), (3, 0)) and norm.replicated == (4, 5) and norm.outputs == (2, 3)
    rows = spec_of("reduce_row_sumsq_16x96_f32")
    assert rows.extent == 16 and rows.sharded == ((0, 0), (1, 0)) and rows.outputs == (1,)
    for case in ("reduce_col_max_24x64_bf16", "reduce_total_sum_8x96_f32"):  # folds over the leading axis run whole on one GPU
        whole = spec_of(case)
        assert whole.extent == 1 and not whole.sharded and whole.replicated == (0, 1) and whole.outputs == (1,)


def _free_port() -> int:
    with socket.socket() as probe:
        probe.bind(("127.0.0.1", 0))
        return probe.getsockname()[1]


def _worker(rank: int, world: int, port: int, rows: int, failures) -> None:
    import torch
    import torch.distributed as dist

    from baybridge_b200.sharding import all_gather_rows, max_over_ranks
    from oracle import cpu_runtime as oracle

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rng = np.random.default_rng(5)  # every rank derives the same global arrays, then keeps its shard only
        x = rng.standard_normal((rows, 64))
        w = 1 + 0.1 * rng.standard_normal(64)
        start, stop = shard_bounds(rows, world, rank)
        local = torch.from_numpy(oracle.rmsnorm(x[start:stop], w, 1e-6))  # stands in for the per-rank kernel
        gathered = all_gather_rows(local)
        expected = oracle.rmsnorm(x, w, 1e-6)
        if gathered.shape != expected.shape or not np.array_equal(gathered.numpy(), expected):
            failures.put(f"rank {rank}: gathered output differs")
        slowest = max_over_ranks(1.0 + rank)
        if slowest != float(world):
            failures.put(f"rank {rank}: max over ranks gave {slowest}")
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,rows", [(2, 64), (3, 65)])  # the second case is ragged: shards of 22, 22, 21 rows
def test_shard_run_allgather_over_gloo(world, rows):
    """Host-side multi-rank plumbing only: shard bounds, the (ragged) all-gather of row shards and the max-over-ranks
    reduction, over gloo on CPU.  No kernel runs here — the oracle fills in each rank's rows; the kernels' own
    multi-rank results are compared with the oracle on GPUs by ``bench.py`` (``parity`` of the gathered output)."""
    import torch.multiprocessing as mp

    context = mp.get_context("spawn")
    failures = context.Queue()
    port = _free_port()
    workers = [context.Process(target=_worker, args=(rank, world, port, rows, failures)) for rank in range(world)]
    for worker in workers:
        worker.start()
    for worker in workers:
        worker.join(timeout=120)
        assert worker.exitcode == 0, "a rank failed or hung"
    assert failures.empty(), failures.get()
