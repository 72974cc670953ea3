#!/usr/bin/env python3
"""Benchmark of the b200 hot path.  Prints ONE JSON line (rank 0).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

Workloads (``--workload``; default ``fused_mul_add``, the bandwidth config the headline metric is
quoted on):

    fused_mul_add   c = a*b + a, bf16, 2^28 elements per GPU          HBM GB/s   (6 B / element)
    rmsnorm         bf16 [65536, 8192] per GPU, eps 1e-6               HBM GB/s   (4 B / element + weight)
    gemm            C = A·B^T, bf16, M=N=K=8192 per GPU, bf16 out      TFLOP/s    (2·M·N·K)
    attention       causal fwd, bf16, B16 H32 S4096 D128 per GPU      TFLOP/s    (4·B·H·D·S(S+1)/2)

A step is one pass of the kernel over one batch of seeded synthetic input resident in HBM.  With
N > 1 (launched under torchrun, one rank per GPU) every rank owns an equal shard of an N-times
larger problem (weak scaling, no data-path collective); the NCCL all-gather of the output shards
is timed separately and reported under ``allgather``.  Timing: CUDA events on the launching
stream, bracketed by barrier + synchronize, max over ranks.  The working sets (1.6 GB / 2.1 GB /
0.4 GB / 2.1 GB) exceed the 126 MB L2 except for GEMM, whose timed loop flushes L2 between steps
outside the event pairs.

``--impl reference`` times the CPU port of upstream's reference runtime (``oracle/``) on a bounded
sample of the same workload, on rank 0 only.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import math
import os
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
for entry in (str(ROOT), str(ROOT / "tests")):
    if entry not in sys.path:
        sys.path.insert(0, entry)

L2_FLUSH_BYTES = 256 << 20
E2E_CHUNKS = int(os.environ.get("BB200_BENCH_E2E_CHUNKS", "16"))  # chunks of the host pipeline (copy-in / kernel / copy-out overlap)
# dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant kernel at the full-size
# workload, from one-pass `ncu --metrics dram__bytes_read.sum,dram__bytes_write.sum --clock-control none`
# captures of this script (commands and figures in profiles/); None for other sizes.
MEASURED_DRAM_TRAFFIC = {
    ("fused_mul_add", 2**28): 1.07e9 + 497.2e6,
    ("rmsnorm", 65536): 1.07e9 + 1.02e9,
    ("gemm", 8192): 1.43e9 + 126.8e6,
    ("attention", 16): 1.61e9 + 523.8e6,
    ("layernorm", 32768): 1.07e9 + 1.02e9,
    ("reduce_rows", 65536): 1.07e9 + 2.0e6,
    ("reduce_cols", 65536): 1.07e9 + 1.8e6,
}
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def load_peaks() -> tuple[dict, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            return json.loads(path.read_text()), "measured"
        except ValueError:
            pass
    return dict(FALLBACK_PEAKS), "fallback"


# ---------------------------------------------------------------------------------------------
# clocks: sampled through NVML while the timed region runs (read-only queries)
# ---------------------------------------------------------------------------------------------
class ClockSampler:
    REASONS = {
        0x1: "gpu_idle", 0x2: "applications_clocks_setting", 0x4: "sw_power_cap", 0x8: "hw_slowdown",
        0x10: "sync_boost", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown", 0x80: "hw_power_brake_slowdown",
        0x100: "display_clock_setting",
    }

    def __init__(self, device_index: int, period_s: float = 0.004):
        self.samples: list[tuple[int, int, int]] = []
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        self._period = period_s
        try:
            import pynvml

            pynvml.nvmlInit()
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            physical = device_index
            if visible:
                entries = [item.strip() for item in visible.split(",") if item.strip()]
                if device_index < len(entries) and entries[device_index].isdigit():
                    physical = int(entries[device_index])
            self._nvml = pynvml
            self._handle = pynvml.nvmlDeviceGetHandleByIndex(physical)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self._handle, pynvml.NVML_CLOCK_SM))
        except Exception:  # NVML missing: the line reports clocks as unavailable
            self._nvml = None

    def _loop(self) -> None:
        nvml = self._nvml
        while not self._stop.is_set():
            try:
                mhz = int(nvml.nvmlDeviceGetClockInfo(self._handle, nvml.NVML_CLOCK_SM))
                reasons = int(nvml.nvmlDeviceGetCurrentClocksEventReasons(self._handle))
                util = int(nvml.nvmlDeviceGetUtilizationRates(self._handle).gpu)
                self.samples.append((mhz, reasons, util))
            except Exception:
                pass
            self._stop.wait(self._period)

    def __enter__(self):
        if self._nvml is not None:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2)

    def summary(self) -> dict:
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0}
        clocks = sorted(sample[0] for sample in self.samples)
        mask = 0
        for _, reasons, _ in self.samples:
            mask |= reasons
        names = sorted(name for bit, name in self.REASONS.items() if mask & bit and name != "gpu_idle")
        return {"sm_mhz": clocks[len(clocks) // 2], "sm_max_mhz": self.max_mhz, "reasons": names, "samples": len(clocks)}


# ---------------------------------------------------------------------------------------------
# workloads
# ---------------------------------------------------------------------------------------------
class Workload:
    name = ""
    unit = ""
    dtype = "bf16"
    bound = "hbm"
    needs_l2_flush = False

    def work_per_step(self) -> float:  # algorithmic bytes (hbm) or flops (tensor) one rank processes per step
        raise NotImplementedError

    def setup(self, torch, cute, zoo, rank: int, cache_dir: str) -> None:
        raise NotImplementedError

    def step(self) -> None:
        raise NotImplementedError

    def output(self):
        raise NotImplementedError

    def e2e_setup(self, cute, zoo, cache_dir: str) -> None:
        raise NotImplementedError

    def e2e_step(self, torch) -> None:
        """Host → device → kernel → host through the public host pipeline (copies overlapped in chunks)."""
        self.pipeline.run()

    def config(self) -> dict:
        raise NotImplementedError

    def shrink(self) -> None:
        raise NotImplementedError

    def size_key(self) -> int:
        raise NotImplementedError


class FusedMulAdd(Workload):
    name, unit, bound = "fused_mul_add", "GB/s", "hbm"
    n = 2**28

    def shrink(self):
        self.n = 2**26  # 400 MB working set

    def size_key(self):
        return self.n

    def work_per_step(self) -> float:
        return 6.0 * self.n  # read a, read b, write c at 2 B each

    def setup(self, torch, cute, zoo, rank, cache_dir):
        generator = torch.Generator(device="cuda").manual_seed(1002 + rank)
        self.a = torch.randn(self.n, device="cuda", dtype=torch.float32, generator=generator).to(torch.bfloat16)
        self.b = torch.randn(self.n, device="cuda", dtype=torch.float32, generator=generator).to(torch.bfloat16)
        self.c = torch.empty_like(self.a)
        from baybridge_b200 import B200Backend

        self.artifact = cute.compile(zoo.make_fused_mul_add_indexed(self.n), self.a, self.b, self.c,
                                     backend=B200Backend(synchronize=False), cache_dir=cache_dir)
        self.args = tuple(cute.from_dlpack(t) for t in (self.a, self.b, self.c))
        self.stream = torch.cuda.current_stream().cuda_stream
        self.a_host = self.a.cpu().pin_memory()
        self.b_host = self.b.cpu().pin_memory()
        self.c_host = torch.empty_like(self.a_host).pin_memory()
        self.h2d_bytes = 2 * self.n * 2
        self.d2h_bytes = self.n * 2

    def step(self):
        self.artifact(*self.args, stream=self.stream)

    def output(self):
        return self.c

    def e2e_setup(self, cute, zoo, cache_dir):
        from baybridge_b200.host_pipeline import HostPipeline

        self.pipeline = HostPipeline(lambda rows: zoo.make_fused_mul_add_indexed(rows), [self.a_host, self.b_host, self.c_host],
                                     chunks=E2E_CHUNKS, cache_dir=cache_dir)

    def fused_gather_ms(self, torch, dist, cute, zoo, barrier) -> float | None:
        """The same step with the output all-gather fused into the kernel: every rank's kernel stores its shard into the
        gathered buffer of every rank (peer stores over NVLink), then one barrier.  Checked against the NCCL result."""
        from baybridge_b200.fused_gather import FusedGather

        fused, gathered = FusedGather.over_group(zoo.make_fused_mul_add_indexed(self.n), [self.a, self.b, self.c])
        buffer = gathered[2]
        stream = torch.cuda.current_stream().cuda_stream
        for _ in range(3):
            fused.run(self.a, self.b, self.c, stream=stream)
            fused.barrier()
        barrier()
        reference = torch.empty_like(buffer)
        dist.all_gather_into_tensor(reference, self.c)
        if not torch.equal(buffer, reference):
            raise RuntimeError("fused kernel + gather differs from kernel followed by the NCCL all-gather")
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = 10
        barrier()
        begin.record()
        for _ in range(reps):
            fused.run(self.a, self.b, self.c, stream=stream)
            fused.barrier()
        end.record()
        barrier()
        return begin.elapsed_time(end) / reps

    def config(self):
        return {"workload": f"fused_mul_add c=a*b+a bf16 {self.n} (2^{self.n.bit_length() - 1}) elements per GPU (6 B/element), indexed IR form",
                "l2": "working set 1.6 GB > 126 MB L2, no flush"}

    # CPU port leg -------------------------------------------------------------------------------
    sample_n = 2**24

    def cpu_sample(self):
        rng = np.random.default_rng(1002)
        from oracle import cpu_runtime as oracle

        a = oracle.bf16_round(rng.standard_normal(self.sample_n, dtype=np.float32)).astype(np.float64)
        b = oracle.bf16_round(rng.standard_normal(self.sample_n, dtype=np.float32)).astype(np.float64)
        ir = {
            "launch": {"grid": [1, 1, 1], "block": [1, 1, 1]},
            "arguments": [{"name": n, "kind": "tensor"} for n in "abc"],
            "operations": [
                {"op": "make_tensor", "inputs": [], "outputs": ["a_load_1"], "attrs": {"shape": [self.sample_n]}},
                {"op": "copy", "inputs": ["a", "a_load_1"], "outputs": [], "attrs": {}},
                {"op": "make_tensor", "inputs": [], "outputs": ["b_load_2"], "attrs": {"shape": [self.sample_n]}},
                {"op": "copy", "inputs": ["b", "b_load_2"], "outputs": [], "attrs": {}},
                {"op": "tensor_mul", "inputs": ["a_load_1", "b_load_2"], "outputs": ["t3"], "attrs": {}},
                {"op": "tensor_add", "inputs": ["t3", "a_load_1"], "outputs": ["t4"], "attrs": {}},
                {"op": "copy", "inputs": ["t4", "c"], "outputs": [], "attrs": {}},
            ],
        }
        arguments = {"a": a, "b": b, "c": np.zeros(self.sample_n)}
        return (lambda: oracle.run_kernel_ir(ir, arguments)), 6.0 * self.sample_n, f"{self.sample_n} of {self.n} elements, numpy f64 port of the tensor-SSA CPU runtime path"


class RmsNorm(Workload):
    name, unit, bound = "rmsnorm", "GB/s", "hbm"
    rows, hidden = 65536, 8192

    def shrink(self):
        self.rows = 8192  # 268 MB working set

    def size_key(self):
        return self.rows

    def work_per_step(self) -> float:
        return 2.0 * self.rows * self.hidden * 2 + self.hidden * 2

    def setup(self, torch, cute, zoo, rank, cache_dir):
        generator = torch.Generator(device="cuda").manual_seed(1004 + rank)
        self.x = torch.randn((self.rows, self.hidden), device="cuda", dtype=torch.float32, generator=generator).to(torch.bfloat16)
        self.w = (1 + 0.1 * torch.randn((self.hidden,), device="cuda", dtype=torch.float32, generator=generator)).to(torch.bfloat16)
        self.out = torch.empty_like(self.x)
        from baybridge_b200 import B200Backend

        self.artifact = cute.compile(zoo.make_rmsnorm(1e-6), self.x, self.out, self.w,
                                     backend=B200Backend(synchronize=False), cache_dir=cache_dir)
        self.args = tuple(cute.from_dlpack(t) for t in (self.x, self.out, self.w))
        self.stream = torch.cuda.current_stream().cuda_stream
        self.x_host = self.x.cpu().pin_memory()
        self.out_host = torch.empty_like(self.x_host).pin_memory()
        self.h2d_bytes = self.rows * self.hidden * 2
        self.d2h_bytes = self.rows * self.hidden * 2

    def step(self):
        self.artifact(*self.args, stream=self.stream)

    def output(self):
        return self.out

    def e2e_setup(self, cute, zoo, cache_dir):
        from baybridge_b200.host_pipeline import HostPipeline

        self.w_host = self.w.cpu().pin_memory()
        self.pipeline = HostPipeline(lambda rows: zoo.make_rmsnorm(1e-6), [self.x_host, self.out_host, self.w_host],
                                     chunks=E2E_CHUNKS, cache_dir=cache_dir)

    def fused_gather_ms(self, torch, dist, cute, zoo, barrier) -> float | None:
        """RMSNorm with the all-gather of its output fused into the kernel (peer stores of every vector), then one barrier."""
        from baybridge_b200.fused_gather import FusedGatherRmsNorm

        fused, full = FusedGatherRmsNorm.over_group(zoo.make_rmsnorm(1e-6), [self.x, self.out, self.w])
        stream = torch.cuda.current_stream().cuda_stream
        for _ in range(3):
            fused.run(self.x, self.w, stream=stream)
            fused.barrier()
        barrier()
        reference = torch.empty_like(full)
        dist.all_gather_into_tensor(reference, self.out)
        if not torch.equal(full, reference):
            raise RuntimeError("fused RMSNorm + gather differs from RMSNorm followed by the NCCL all-gather")
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = 10
        barrier()
        begin.record()
        for _ in range(reps):
            fused.run(self.x, self.w, stream=stream)
            fused.barrier()
        end.record()
        barrier()
        return begin.elapsed_time(end) / reps

    def config(self):
        return {"workload": f"rmsnorm bf16 [{self.rows}, {self.hidden}] per GPU, weight [{self.hidden}], eps 1e-6",
                "l2": "working set 2.1 GB > 126 MB L2, no flush"}

    def cpu_sample(self):
        from oracle import cpu_runtime as oracle

        rng = np.random.default_rng(1004)
        rows = 512
        x = oracle.bf16_round(rng.standard_normal((rows, self.hidden), dtype=np.float32)).astype(np.float64)
        w = oracle.bf16_round((1 + 0.1 * rng.standard_normal(self.hidden)).astype(np.float32)).astype(np.float64)
        return (lambda: oracle.rmsnorm(x, w, 1e-6)), 2.0 * rows * self.hidden * 2 + self.hidden * 2, f"{rows} of {self.rows} rows, numpy f64 port"


class Gemm(Workload):
    name, unit, bound = "gemm", "TFLOP/s", "tensor"
    m = n = k = 8192
    needs_l2_flush = True

    def shrink(self):
        self.m = self.n = self.k = 4096

    def size_key(self):
        return self.m

    def work_per_step(self) -> float:
        return 2.0 * self.m * self.n * self.k

    def setup(self, torch, cute, zoo, rank, cache_dir):
        generator = torch.Generator(device="cuda").manual_seed(1003 + rank)
        scale = 1.0 / math.sqrt(self.k)
        self.a = (torch.randn((self.m, self.k), device="cuda", dtype=torch.float32, generator=generator) * scale).to(torch.bfloat16)
        self.b = (torch.randn((self.n, self.k), device="cuda", dtype=torch.float32, generator=generator) * scale).to(torch.bfloat16)
        self.c = torch.empty((self.m, self.n), device="cuda", dtype=torch.bfloat16)
        from baybridge_b200 import B200Backend

        self.artifact = cute.compile(zoo.gemm_abt, self.a, self.b, self.c, backend=B200Backend(synchronize=False), cache_dir=cache_dir)
        self.args = tuple(cute.from_dlpack(t) for t in (self.a, self.b, self.c))
        self.stream = torch.cuda.current_stream().cuda_stream
        self.a_host = self.a.cpu().pin_memory()
        self.b_host = self.b.cpu().pin_memory()
        self.c_host = torch.empty((self.m, self.n), dtype=torch.bfloat16).pin_memory()
        self.h2d_bytes = (self.m * self.k + self.n * self.k) * 2
        self.d2h_bytes = self.m * self.n * 2

    def step(self):
        self.artifact(*self.args, stream=self.stream)

    def output(self):
        return self.c

    def e2e_setup(self, cute, zoo, cache_dir):
        from baybridge_b200.host_pipeline import HostPipeline

        self.pipeline = HostPipeline(lambda rows: zoo.gemm_abt, [self.a_host, self.b_host, self.c_host],
                                     chunks=E2E_CHUNKS, cache_dir=cache_dir)

    def config(self):
        return {"workload": f"gemm C=A·B^T bf16 M=N=K={self.m} per GPU, fp32 accumulate, bf16 out",
                "l2": "384 MB working set; 256 MB L2 flush write between timed steps (outside the event pairs)"}

    def cpu_sample(self):
        from oracle import cpu_runtime as oracle

        rng = np.random.default_rng(1003)
        size = 2048
        a = oracle.bf16_round((rng.standard_normal((size, size)) / math.sqrt(size)).astype(np.float32)).astype(np.float64)
        b = oracle.bf16_round((rng.standard_normal((size, size)) / math.sqrt(size)).astype(np.float32)).astype(np.float64)
        return (lambda: oracle.gemm(a, b, transpose_b=True)), 2.0 * size**3, f"M=N=K={size} (of 8192), numpy f64 BLAS port"


    def fused_gather_ms(self, torch, dist, cute, zoo, barrier) -> float | None:
        """The same GEMM with the all-gather of C fused into its epilogue (peer stores of every tile), then one barrier."""
        from baybridge_b200.fused_gather import FusedGatherGemm

        fused, full = FusedGatherGemm.over_group(zoo.gemm_abt, [self.a, self.b, self.c])
        stream = torch.cuda.current_stream().cuda_stream
        for _ in range(3):
            fused.run(self.a, self.b, stream=stream)
            fused.barrier()
        barrier()
        reference = torch.empty_like(full)
        dist.all_gather_into_tensor(reference, self.c)
        if not torch.equal(full, reference):
            raise RuntimeError("fused GEMM + gather differs from the GEMM followed by the NCCL all-gather")
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = 10
        barrier()
        begin.record()
        for _ in range(reps):
            fused.run(self.a, self.b, stream=stream)
            fused.barrier()
        end.record()
        barrier()
        return begin.elapsed_time(end) / reps


class Attention(Workload):
    name, unit, bound = "attention", "TFLOP/s", "tensor"
    batch, heads, seq, dim = 16, 32, 4096, 128

    def shrink(self):
        self.batch = 2

    def size_key(self):
        return self.batch

    def work_per_step(self) -> float:
        return 4.0 * self.batch * self.heads * self.dim * self.seq * (self.seq + 1) / 2

    def setup(self, torch, cute, zoo, rank, cache_dir):
        generator = torch.Generator(device="cuda").manual_seed(1005 + rank)
        shape = (self.batch, self.seq, self.heads, self.dim)
        self.q, self.k, self.v = (torch.randn(shape, device="cuda", dtype=torch.float32, generator=generator).to(torch.bfloat16) for _ in range(3))
        self.o = torch.empty_like(self.q)
        self.lse = torch.empty((self.batch, self.heads, 1, self.seq), device="cuda", dtype=torch.float32)
        from baybridge_b200 import B200Backend

        self.artifact = cute.compile(zoo.attention_causal, self.q, self.k, self.v, self.o, self.lse,
                                     backend=B200Backend(synchronize=False), cache_dir=cache_dir)
        self.args = tuple(cute.from_dlpack(t) for t in (self.q, self.k, self.v, self.o, self.lse))
        self.stream = torch.cuda.current_stream().cuda_stream
        self.hosts = [t.cpu().pin_memory() for t in (self.q, self.k, self.v)]
        self.o_host = torch.empty_like(self.hosts[0]).pin_memory()
        self.h2d_bytes = 3 * self.q.numel() * 2
        self.d2h_bytes = self.q.numel() * 2

    def step(self):
        self.artifact(*self.args, stream=self.stream)

    def output(self):
        return self.o

    def e2e_setup(self, cute, zoo, cache_dir):
        import torch

        from baybridge_b200.host_pipeline import HostPipeline

        self.lse_host = torch.empty((self.batch, self.heads, 1, self.seq), dtype=torch.float32).pin_memory()
        self.pipeline = HostPipeline(lambda rows: zoo.attention_causal, [*self.hosts, self.o_host, self.lse_host],
                                     chunks=min(E2E_CHUNKS, self.batch), cache_dir=cache_dir)

    def fused_gather_ms(self, torch, dist, cute, zoo, barrier) -> float | None:
        """Attention with the all-gather of out (and lse) fused into the epilogue (peer stores of whole rows), then one barrier."""
        from baybridge_b200.fused_gather import FusedGatherAttention

        fused, (out_full, lse_full) = FusedGatherAttention.over_group(zoo.attention_causal, [self.q, self.k, self.v, self.o, self.lse])
        stream = torch.cuda.current_stream().cuda_stream
        for _ in range(3):
            fused.run(self.q, self.k, self.v, stream=stream)
            fused.barrier()
        barrier()
        reference, reference_lse = torch.empty_like(out_full), torch.empty_like(lse_full)
        dist.all_gather_into_tensor(reference, self.o)
        dist.all_gather_into_tensor(reference_lse, self.lse)
        if not (torch.equal(out_full, reference) and torch.equal(lse_full, reference_lse)):
            raise RuntimeError("fused attention + gather differs from attention followed by the NCCL all-gather")
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = 10
        barrier()
        begin.record()
        for _ in range(reps):
            fused.run(self.q, self.k, self.v, stream=stream)
            fused.barrier()
        end.record()
        barrier()
        return begin.elapsed_time(end) / reps

    def config(self):
        return {"workload": f"causal attention fwd bf16 B{self.batch} H{self.heads} S{self.seq} D{self.dim} per GPU (layout [B,S,H,D]), causal FLOPs",
                "l2": "working set 2.1 GB > 126 MB L2, no flush"}

    def cpu_sample(self):
        from oracle import cpu_runtime as oracle

        rng = np.random.default_rng(1005)
        bsz, seq, heads = 1, 1024, 4
        q, k, v = (oracle.bf16_round(rng.standard_normal((bsz, seq, heads, self.dim), dtype=np.float32)).astype(np.float64) for _ in range(3))
        flops = 4.0 * bsz * heads * self.dim * seq * (seq + 1) / 2
        return (lambda: oracle.attention(q, k, v, causal=True)), flops, f"B{bsz} H{heads} S{seq} D{self.dim}, numpy f64 port"


class LayerNorm(Workload):
    """LayerNorm with fused residual add: reads x, residual, weight, bias; writes out and x + residual."""
    name, unit, bound = "layernorm", "GB/s", "hbm"
    rows, hidden = 32768, 8192

    def shrink(self):
        self.rows = 4096  # 268 MB working set

    def size_key(self):
        return self.rows

    def work_per_step(self) -> float:
        return 4.0 * self.rows * self.hidden * 2 + 2 * self.hidden * 2

    def setup(self, torch, cute, zoo, rank, cache_dir):
        generator = torch.Generator(device="cuda").manual_seed(1006 + rank)
        make = lambda: torch.randn((self.rows, self.hidden), device="cuda", dtype=torch.float32, generator=generator).to(torch.bfloat16)  # noqa: E731
        self.x, self.residual = make(), make()
        self.w = (1 + 0.1 * torch.randn((self.hidden,), device="cuda", dtype=torch.float32, generator=generator)).to(torch.bfloat16)
        self.b = (0.1 * torch.randn((self.hidden,), device="cuda", dtype=torch.float32, generator=generator)).to(torch.bfloat16)
        self.out, self.out_resid = torch.empty_like(self.x), torch.empty_like(self.x)
        from baybridge_b200 import B200Backend

        tensors = (self.x, self.residual, self.out, self.out_resid, self.w, self.b)
        self.artifact = cute.compile(zoo.layernorm_kernel, *tensors, backend=B200Backend(synchronize=False), cache_dir=cache_dir)
        self.args = tuple(cute.from_dlpack(t) for t in tensors)
        self.stream = torch.cuda.current_stream().cuda_stream
        self.host = [t.cpu().pin_memory() for t in tensors]
        self.h2d_bytes = 2 * self.rows * self.hidden * 2
        self.d2h_bytes = 2 * self.rows * self.hidden * 2

    def step(self):
        self.artifact(*self.args, stream=self.stream)

    def output(self):
        return self.out

    def e2e_setup(self, cute, zoo, cache_dir):
        from baybridge_b200.host_pipeline import HostPipeline

        self.pipeline = HostPipeline(lambda rows: zoo.layernorm_kernel, self.host, chunks=E2E_CHUNKS, cache_dir=cache_dir)

    def fused_gather_ms(self, torch, dist, cute, zoo, barrier) -> float | None:
        """LayerNorm with the all-gather of out and out_resid fused into the kernel (peer stores of every vector), then one
        barrier.  The separate NCCL figure next to it gathers `out` alone."""
        from baybridge_b200.fused_gather import FusedGatherLayerNorm

        fused, (out_full, resid_full) = FusedGatherLayerNorm.over_group(
            zoo.layernorm_kernel, [self.x, self.residual, self.out, self.out_resid, self.w, self.b])
        stream = torch.cuda.current_stream().cuda_stream
        for _ in range(3):
            fused.run(self.x, self.residual, self.w, self.b, stream=stream)
            fused.barrier()
        barrier()
        reference, reference_resid = torch.empty_like(out_full), torch.empty_like(resid_full)
        dist.all_gather_into_tensor(reference, self.out)
        dist.all_gather_into_tensor(reference_resid, self.out_resid)
        if not (torch.equal(out_full, reference) and torch.equal(resid_full, reference_resid)):
            raise RuntimeError("fused LayerNorm + gather differs from LayerNorm followed by the NCCL all-gather")
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = 10
        barrier()
        begin.record()
        for _ in range(reps):
            fused.run(self.x, self.residual, self.w, self.b, stream=stream)
            fused.barrier()
        end.record()
        barrier()
        return begin.elapsed_time(end) / reps

    def config(self):
        return {"workload": f"layernorm with residual add, bf16 [{self.rows}, {self.hidden}] per GPU, weight/bias [{self.hidden}], eps 1e-5",
                "l2": "working set 2.1 GB > 126 MB L2, no flush"}

    def cpu_sample(self):
        from oracle import cpu_runtime as oracle

        rng = np.random.default_rng(1006)
        rows = 256
        x = oracle.bf16_round(rng.standard_normal((rows, self.hidden), dtype=np.float32)).astype(np.float64)
        r = oracle.bf16_round(rng.standard_normal((rows, self.hidden), dtype=np.float32)).astype(np.float64)
        w = oracle.bf16_round((1 + 0.1 * rng.standard_normal(self.hidden)).astype(np.float32)).astype(np.float64)
        b = oracle.bf16_round((0.1 * rng.standard_normal(self.hidden)).astype(np.float32)).astype(np.float64)
        return (lambda: oracle.layernorm(x, r, w, b, 1e-5)), 4.0 * rows * self.hidden * 2, f"{rows} of {self.rows} rows, numpy f64 port"


class _Reduction(Workload):
    """A traced `Tensor.reduce` over one axis of a bf16 matrix: every element is read once."""
    unit, bound = "GB/s", "hbm"
    rows, cols = 65536, 8192
    kernel_name = ""
    kept_axis = 0

    def shrink(self):
        self.rows = 8192

    def size_key(self):
        return self.rows

    def work_per_step(self) -> float:
        kept = self.rows if self.kept_axis == 0 else self.cols
        return self.rows * self.cols * 2.0 + kept * 2.0

    def setup(self, torch, cute, zoo, rank, cache_dir):
        generator = torch.Generator(device="cuda").manual_seed(1007 + rank)
        self.src = torch.rand((self.rows, self.cols), device="cuda", dtype=torch.float32, generator=generator).mul_(2).sub_(1).to(torch.bfloat16)
        kept = self.rows if self.kept_axis == 0 else self.cols
        self.dst = torch.empty((kept,), device="cuda", dtype=torch.bfloat16)
        from baybridge_b200 import B200Backend

        self.artifact = cute.compile(getattr(zoo, self.kernel_name), self.src, self.dst, backend=B200Backend(synchronize=False),
                                     cache_dir=cache_dir)
        self.args = tuple(cute.from_dlpack(t) for t in (self.src, self.dst))
        self.stream = torch.cuda.current_stream().cuda_stream
        self.host = [self.src.cpu().pin_memory(), self.dst.cpu().pin_memory()]
        self.h2d_bytes = self.rows * self.cols * 2
        self.d2h_bytes = kept * 2

    def step(self):
        self.artifact(*self.args, stream=self.stream)

    def output(self):
        return self.dst

    def e2e_setup(self, cute, zoo, cache_dir):
        from baybridge_b200.host_pipeline import HostPipeline

        self.pipeline = HostPipeline(lambda rows: getattr(zoo, self.kernel_name), self.host, chunks=E2E_CHUNKS if self.kept_axis == 0 else 1,
                                     cache_dir=cache_dir)

    def cpu_sample(self):
        from oracle import cpu_runtime as oracle

        rng = np.random.default_rng(1007)
        rows = 2048
        src = oracle.bf16_round(rng.uniform(-1, 1, (rows, self.cols)).astype(np.float32)).astype(np.float64)
        run = (lambda: (src * src).sum(axis=1)) if self.kept_axis == 0 else (lambda: np.maximum(src.max(axis=0), -1000.0))
        return run, rows * self.cols * 2.0, f"{rows} of {self.rows} rows, numpy f64 restatement of the traced fold"


class RowReduce(_Reduction):
    name, kernel_name, kept_axis = "reduce_rows", "row_sum_of_squares", 0

    def config(self):
        return {"workload": f"row reduction dst[r] = sum_c src[r,c]^2, bf16 [{self.rows}, {self.cols}] per GPU (traced Tensor.reduce)",
                "l2": "working set 1.07 GB > 126 MB L2, no flush"}


class ColumnReduce(_Reduction):
    name, kernel_name, kept_axis = "reduce_cols", "column_max", 1

    def config(self):
        return {"workload": f"column reduction dst[c] = max_r src[r,c], bf16 [{self.rows}, {self.cols}] per GPU (traced Tensor.reduce)",
                "l2": "working set 1.07 GB > 126 MB L2, no flush"}


class IndexedAdd(Workload):
    """Config 1: 256x256 f32 indexed add.  786 KB of traffic, all of it L2-resident after the first launch: what this
    measures is launch latency, reported per call and per launch of a recorded launch graph (`launch_latency`)."""
    name, unit, bound, dtype = "indexed_add", "GB/s", "hbm", "f32"
    rows = cols = 256

    def shrink(self):
        pass

    def size_key(self):
        return self.rows

    def work_per_step(self) -> float:
        return 3.0 * self.rows * self.cols * 4

    def setup(self, torch, cute, zoo, rank, cache_dir):
        generator = torch.Generator(device="cuda").manual_seed(1001 + rank)
        self.a = torch.rand((self.rows, self.cols), device="cuda", dtype=torch.float32, generator=generator).mul_(2).sub_(1)
        self.b = torch.rand((self.rows, self.cols), device="cuda", dtype=torch.float32, generator=generator).mul_(2).sub_(1)
        self.c = torch.zeros_like(self.a)
        from baybridge_b200 import B200Backend

        self.kernel = zoo.make_indexed_add_2d(self.rows, self.cols)
        self.artifact = cute.compile(self.kernel, self.a, self.b, self.c, backend=B200Backend(synchronize=False), cache_dir=cache_dir)
        self.blocking = cute.compile(self.kernel, self.a, self.b, self.c, backend="b200", cache_dir=cache_dir)  # upstream-style: sync per launch
        self.args = tuple(cute.from_dlpack(t) for t in (self.a, self.b, self.c))
        self.stream = torch.cuda.current_stream().cuda_stream
        self.host = [self.a.cpu().pin_memory(), self.b.cpu().pin_memory(), self.c.cpu().pin_memory()]
        self.h2d_bytes = 2 * self.rows * self.cols * 4
        self.d2h_bytes = self.rows * self.cols * 4

    def step(self):
        self.artifact(*self.args, stream=self.stream)

    def output(self):
        return self.c

    def e2e_setup(self, cute, zoo, cache_dir):
        from baybridge_b200.host_pipeline import HostPipeline

        self.pipeline = HostPipeline(lambda rows: zoo.make_indexed_add_2d(rows, self.cols), self.host, chunks=1, cache_dir=cache_dir)

    def config(self):
        return {"workload": f"indexed add c[r,c]=a[r,c]+b[r,c] f32 {self.rows}x{self.cols} per GPU (grid {self.rows} x block {self.cols})",
                "l2": "786 KB working set is L2-resident: launch-latency bound, no roofline claimed"}

    def cpu_sample(self):
        rng = np.random.default_rng(1001)
        a = rng.uniform(-1, 1, (self.rows, self.cols)).astype(np.float32).astype(np.float64)
        b = rng.uniform(-1, 1, (self.rows, self.cols)).astype(np.float32).astype(np.float64)
        return (lambda: (a + b).astype(np.float32)), self.work_per_step(), "full size, numpy f64 port of the per-thread CPU runtime loop"

    def extras(self, torch) -> dict:
        """Microseconds per launch three ways: upstream-style (synchronise after every launch), asynchronous launches,
        and the same launches recorded once into a launch graph and replayed."""
        from baybridge_b200.launch_graph import LaunchGraph

        calls = 2000
        torch.cuda.synchronize()
        started = time.perf_counter()
        for _ in range(calls):
            self.blocking(*self.args)
        blocking_us = (time.perf_counter() - started) / calls * 1e6
        started = time.perf_counter()
        for _ in range(calls):
            self.artifact(*self.args, stream=self.stream)
        torch.cuda.synchronize()
        eager_us = (time.perf_counter() - started) / calls * 1e6
        per_graph, replays = 200, 20
        graph = LaunchGraph()
        with graph.record() as recording_stream:
            for _ in range(per_graph):
                self.artifact(*self.args, stream=recording_stream)
        for _ in range(3):
            graph.replay(stream=self.stream)
        torch.cuda.synchronize()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        started = time.perf_counter()
        begin.record()
        for _ in range(replays):
            graph.replay(stream=self.stream)
        end.record()
        torch.cuda.synchronize()
        graph_wall_us = (time.perf_counter() - started) / (per_graph * replays) * 1e6
        graph_us = begin.elapsed_time(end) * 1e3 / (per_graph * replays)
        graph.close()
        return {"launch_latency": {"synchronising_call_us": blocking_us, "asynchronous_call_us": eager_us,
                                   "graph_replay_us_per_launch": graph_us, "graph_replay_wall_us_per_launch": graph_wall_us,
                                   "launches_per_graph": per_graph, "calls": calls}}


WORKLOADS = {cls.name: cls for cls in (FusedMulAdd, RmsNorm, Gemm, Attention, LayerNorm, RowReduce, ColumnReduce, IndexedAdd)}
METRIC = {
    "fused_mul_add": "elementwise HBM GB/s (fused c=a*b+a, bf16)", "rmsnorm": "RMSNorm HBM GB/s (bf16)",
    "gemm": "BF16 GEMM TFLOP/s", "attention": "causal attention forward TFLOP/s (bf16)",
    "layernorm": "LayerNorm + residual HBM GB/s (bf16)", "reduce_rows": "row reduction HBM GB/s (bf16)",
    "reduce_cols": "column reduction HBM GB/s (bf16)",
    "indexed_add": "indexed add 256x256 f32: effective GB/s of a launch-latency-bound call",
}


# ---------------------------------------------------------------------------------------------
# CPU legs
# ---------------------------------------------------------------------------------------------
def time_cpu(workload: Workload, budget_s: float = 10.0, min_runs: int = 2) -> dict:
    run, work, sample = workload.cpu_sample()
    run()  # warm-up
    durations = []
    started = time.perf_counter()
    while len(durations) < min_runs or (time.perf_counter() - started < budget_s and len(durations) < 50):
        t0 = time.perf_counter()
        run()
        durations.append(time.perf_counter() - t0)
    median = sorted(durations)[len(durations) // 2]
    scale = 1e9 if workload.unit == "GB/s" else 1e12
    threads = 1 if workload.name in ("fused_mul_add", "rmsnorm", "indexed_add") else (os.cpu_count() or 1)
    return {"value": work / median / scale, "unit": workload.unit, "cores": threads, "kind": "port",
            "sample": sample, "seconds_per_sample": median, "runs": len(durations)}


def reference_arm(args, workload: Workload) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    run, work, sample = workload.cpu_sample()
    for _ in range(min(args.warmup, 2)):
        run()
    steps = max(1, min(args.steps, 20))
    started = time.perf_counter()
    for _ in range(steps):
        run()
    elapsed = time.perf_counter() - started
    scale = 1e9 if workload.unit == "GB/s" else 1e12
    value = work * steps / elapsed / scale
    threads = 1 if workload.name in ("fused_mul_add", "rmsnorm", "indexed_add") else (os.cpu_count() or 1)
    line = {
        "impl": "reference", "metric": METRIC[workload.name], "value": value, "unit": workload.unit,
        "n_gpus": args.gpus, "steps": steps, "warmup": min(args.warmup, 2), "ms_per_step": elapsed / steps * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f64 (CPU runtime arithmetic)",
        "data": "synthetic", "config": workload.config(),
        "cpu_baseline": {"value": value, "unit": workload.unit, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": workload.unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------------
def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=50)
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--workload", default="fused_mul_add", choices=sorted(WORKLOADS))
    parser.add_argument("--impl", default="b200", choices=["b200", "reference"])
    parser.add_argument("--no-cpu-baseline", action="store_true")
    parser.add_argument("--e2e-steps", type=int, default=3)
    parser.add_argument("--small", action="store_true",
                        help="reduced problem (still larger than L2) for profiler captures; never a bench value")
    args = parser.parse_args()
    workload = WORKLOADS[args.workload]()
    if args.small:
        workload.shrink()
    if args.impl == "reference":
        reference_arm(args, workload)
        return

    import torch

    import baybridge_b200 as cute
    from baybridge_b200.backend import b200 as backend_module
    from baybridge_b200.backend import native
    from kernel_zoo import build_zoo

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; the b200 backend has no CPU path")
    torch.cuda.set_device(local_rank)
    distributed = world > 1
    if distributed:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    warmup = max(args.warmup, 3)
    steps = max(args.steps, 1)
    zoo = build_zoo(cute)
    cache_dir = str(ROOT / ".bench_cache" / f"rank{rank}")
    workload.setup(torch, cute, zoo, rank, cache_dir)
    flush = torch.empty(L2_FLUSH_BYTES, device="cuda", dtype=torch.uint8) if workload.needs_l2_flush else None

    def barrier() -> None:
        if distributed:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(warmup):
        workload.step()
    barrier()

    peaks, peak_source = load_peaks()
    launches_before = backend_module.LAUNCH_COUNTER["launches"]
    with ClockSampler(local_rank) as sampler:
        if flush is None:
            # back-to-back launches, one event pair around the K steps
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            barrier()
            start.record()
            for _ in range(steps):
                workload.step()
            stop.record()
            barrier()
            total_ms = start.elapsed_time(stop)
        else:
            # an event pair per step so the L2 flush between steps is not timed
            pairs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
            barrier()
            for begin, end in pairs:
                flush.fill_(1)
                begin.record()
                workload.step()
                end.record()
            barrier()
            total_ms = sum(begin.elapsed_time(end) for begin, end in pairs)
        launches = backend_module.LAUNCH_COUNTER["launches"] - launches_before
        # keep the device busy a little longer so NVML has samples under this load even when K is small
        deadline = time.perf_counter() + 0.25
        while time.perf_counter() < deadline:
            for _ in range(10):
                workload.step()
            torch.cuda.synchronize()
    clocks = sampler.summary()

    if distributed:
        slowest = torch.tensor([total_ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(slowest, op=dist.ReduceOp.MAX)
        total_ms = float(slowest.item())
    ms_per_step = total_ms / steps
    scale = 1e9 if workload.unit == "GB/s" else 1e12
    per_rank = workload.work_per_step() / (ms_per_step * 1e-3) / scale
    value = per_rank * world

    # end to end: pinned host inputs → device, kernel through the public host pipeline, result → host
    workload.e2e_setup(cute, zoo, cache_dir)
    workload.h2d_bytes, workload.d2h_bytes = workload.pipeline.h2d_bytes, workload.pipeline.d2h_bytes
    for _ in range(2):
        workload.e2e_step(torch)
    barrier()
    e2e_started = time.perf_counter()
    for _ in range(args.e2e_steps):
        workload.e2e_step(torch)
    e2e_seconds = (time.perf_counter() - e2e_started) / args.e2e_steps
    if distributed:
        worst = torch.tensor([e2e_seconds], device="cuda", dtype=torch.float64)
        dist.all_reduce(worst, op=dist.ReduceOp.MAX)
        e2e_seconds = float(worst.item())
    e2e_value = workload.work_per_step() * world / e2e_seconds / scale

    allgather = None
    if distributed:
        out = workload.output()
        gathered = torch.empty((world,) + tuple(out.shape), device="cuda", dtype=out.dtype)
        for _ in range(2):
            dist.all_gather_into_tensor(gathered, out)
        barrier()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        reps = 5
        for _ in range(reps):
            dist.all_gather_into_tensor(gathered, out)
        end.record()
        barrier()
        gather_ms = torch.tensor([begin.elapsed_time(end) / reps], device="cuda", dtype=torch.float64)
        dist.all_reduce(gather_ms, op=dist.ReduceOp.MAX)
        total_bytes = out.numel() * out.element_size() * world
        allgather = {"ms": float(gather_ms.item()), "output_bytes_total": total_bytes,
                     "bus_gbs": total_bytes * (world - 1) / world / (float(gather_ms.item()) * 1e-3) / 1e9,
                     "kernel_plus_allgather_ms": ms_per_step + float(gather_ms.item())}

        fused = None
        if hasattr(workload, "fused_gather_ms"):
            try:  # an extra measurement: a box without symmetric-memory support must not lose the bench line
                fused = workload.fused_gather_ms(torch, dist, cute, zoo, barrier)
            except Exception as error:  # noqa: BLE001
                allgather["fused_unavailable"] = f"{type(error).__name__}: {error}"[:200]
        ready = torch.tensor([0.0 if fused is None else 1.0], device="cuda", dtype=torch.float64)
        dist.all_reduce(ready, op=dist.ReduceOp.MIN)
        if float(ready.item()) < 1.0:
            fused = None
        if fused is not None:
            fused_ms = torch.tensor([fused], device="cuda", dtype=torch.float64)
            dist.all_reduce(fused_ms, op=dist.ReduceOp.MAX)
            allgather["fused_kernel_and_gather_ms"] = float(fused_ms.item())
            allgather["fused_speedup_vs_kernel_plus_allgather"] = allgather["kernel_plus_allgather_ms"] / float(fused_ms.item())

    if rank == 0:
        if workload.bound == "hbm":
            peak, peak_unit = float(peaks["hbm_gbs"]), "GB/s"
        else:
            peak, peak_unit = float(peaks["bf16_tflops"]), "TFLOP/s"
        roofline = {
            "bound": workload.bound, "achieved": per_rank, "peak": peak, "unit": peak_unit, "frac": per_rank / peak,
            "peak_source": f"{peak_source} ({'hbm_gbs' if workload.bound == 'hbm' else 'bf16_tflops burst'})",
            "traffic": MEASURED_DRAM_TRAFFIC.get((workload.name, workload.size_key())), "kernel_ms": ms_per_step,
        }
        if workload.bound == "tensor":
            roofline["frac_of_sustained_peak"] = per_rank / float(peaks.get("bf16_tflops_sustained", peak))
        else:
            roofline["algorithmic_bytes"] = workload.work_per_step()
        line = {
            "metric": METRIC[workload.name], "value": value, "unit": workload.unit, "n_gpus": world, "steps": steps,
            "warmup": warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": workload.dtype, "data": "synthetic", "config": workload.config(),
            "roofline": roofline, "clocks": clocks,
            "e2e": {"value": e2e_value, "unit": workload.unit, "h2d_bytes_per_step": workload.h2d_bytes,
                    "d2h_bytes_per_step": workload.d2h_bytes, "ms_per_step": e2e_seconds * 1e3},
            "gpu_launches": launches,
        }
        if allgather is not None:
            line["allgather"] = allgather
        if hasattr(workload, "extras"):
            line.update(workload.extras(torch))
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = time_cpu(workload)
        info = native.DeviceInfo()
        if native.library().bb200_device_info_get(local_rank, ctypes.byref(info)) == 0:
            line["device"] = {"name": info.name.decode(), "sm_count": info.sm_count}
        print(json.dumps(line), flush=True)
    if distributed:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
