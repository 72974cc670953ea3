#!/usr/bin/env python3
"""Benchmark of the b200 hot path.  Prints ONE JSON line (rank 0).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME|all] [--scaling strong|weak]
                    [--impl reference]

Workloads (the five configurations the headline metric is quoted on, plus the neighbouring ops):

    fused_mul_add   c = a*b + a, bf16, 2^28 elements                  HBM GB/s   (6 B / element)
    gemm            C = A·B^T, bf16, M=N=K=8192, bf16 out             TFLOP/s    (2·M·N·K)
    rmsnorm         bf16 [65536, 8192], eps 1e-6                       HBM GB/s   (4 B / element + weight)
    attention       causal fwd, bf16, B16 H32 S4096 D128               TFLOP/s    (4·B·H·D·S(S+1)/2)
    indexed_add     f32 256x256, one thread per element                launch latency
    layernorm, reduce_rows, reduce_cols                                HBM GB/s

``--workload all`` (the default) puts ``fused_mul_add`` in the top-level keys of the line and the other
four configurations under ``"workloads"``; a single name makes that workload the whole line.

A step is one pass of the kernel over its seeded synthetic input resident in HBM.  With N > 1
(launched under torchrun, one rank per GPU) the ONE global problem is sharded over its outer axis
(``--scaling strong``, the default: elements / rows of A and C / rows / batches split N ways, B and the
norm weight replicated); ``--scaling weak`` keeps the full configuration on every rank instead.  Every
rank generates the same global arrays from the workload's seed and keeps its slice.  Three step forms are
timed, each as the max over ranks of CUDA-event time on the launching stream:

    value               kernel on the shard only
    value_with_gather   kernel, then the NCCL all-gather of the output shards
    value_fused         the kernel that stores its shard into every rank's gathered buffer + one barrier

and sampled rows of the GATHERED output are compared with the CPU oracle (``"parity"``).  L2 between timed
steps: a working set of 1 GiB or more per rank is simply larger than the 126 MB L2; a smaller one is timed over
several copies of its tensors used in rotation, so that at least 1 GiB of other data passes through L2 before a
copy is touched again; the GEMM and every step form that contains a collective instead get a 256 MB L2 flush
write before each step, outside that step's event pair.

``--impl reference`` times upstream's own CPU reference runtime (``oracle/ref_runtime.py`` over the copy in
``oracle/_ref``; the numpy port in ``oracle/cpu_runtime.py`` when that copy is absent) on a bounded sample
of the same workloads, on rank 0 only.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import math
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

L2_FLUSH_BYTES = 256 << 20
ROTATE_BELOW_BYTES = 1 << 30  # smaller working sets are timed over rotating copies that add up to at least this much
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
CONFIGS = ("fused_mul_add", "gemm", "rmsnorm", "attention", "indexed_add")


def load_peaks() -> tuple[dict, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            return json.loads(path.read_text()), "measured"
        except ValueError:
            pass
    return dict(FALLBACK_PEAKS), "fallback"


def load_traffic() -> dict:
    """DRAM bytes per launch of each workload's dominant kernel, from profiler captures recorded in a tracked file
    (with the command, date and commit of each capture)."""
    path = ROOT / "profiles" / "traffic.json"
    try:
        entries = json.loads(path.read_text())["captures"]
    except (OSError, ValueError, KeyError):
        return {}
    return {(entry["workload"], int(entry["size_key"])): entry for entry in entries}


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
# run context
# ---------------------------------------------------------------------------------------------
class Context:
    def __init__(self, args):
        import torch

        import baybridge_b200 as cute
        from baybridge_b200.samples import build_zoo

        self.torch, self.cute, self.args = torch, cute, args
        self.zoo = build_zoo(cute)
        self.rank = int(os.environ.get("RANK", "0"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.weak = args.scaling == "weak"
        if not torch.cuda.is_available():
            raise SystemExit("bench.py needs a CUDA device; the b200 backend has no CPU path")
        torch.cuda.set_device(self.local_rank)
        self.dist = None
        if self.world > 1:
            import torch.distributed as dist

            dist.init_process_group("nccl", device_id=torch.device("cuda", self.local_rank))
            self.dist = dist
        self.cache_dir = str(ROOT / ".bench_cache" / f"rank{self.rank}")
        self.flush = torch.empty(L2_FLUSH_BYTES, device="cuda", dtype=torch.uint8)
        self.stream = torch.cuda.current_stream().cuda_stream
        self.peaks, self.peak_source = load_peaks()
        self.traffic = load_traffic()
        self.placement = host_placement(self.local_rank) if os.environ.get("BB200_BENCH_NUMA", "1") != "0" else {}

    def barrier(self) -> None:
        if self.dist is not None:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def slowest(self, value: float) -> float:
        """Max over ranks: the slowest rank defines a multi-GPU step."""
        if self.dist is None:
            return float(value)
        cell = self.torch.tensor([float(value)], device="cuda", dtype=self.torch.float64)
        self.dist.all_reduce(cell, op=self.dist.ReduceOp.MAX)
        return float(cell.item())

    def everyone(self, flag: bool) -> bool:
        if self.dist is None:
            return bool(flag)
        cell = self.torch.tensor([1.0 if flag else 0.0], device="cuda", dtype=self.torch.float64)
        self.dist.all_reduce(cell, op=self.dist.ReduceOp.MIN)
        return float(cell.item()) >= 1.0

    def per_rank(self, value: float) -> list[float]:
        if self.dist is None:
            return [float(value)]
        mine = self.torch.tensor([float(value)], device="cuda", dtype=self.torch.float64)
        cells = self.torch.empty(self.world, device="cuda", dtype=self.torch.float64)
        self.dist.all_gather_into_tensor(cells, mine)
        return [float(v) for v in cells.tolist()]

    def time_ms(self, step, steps: int, flush: bool) -> float:
        """Device milliseconds per step of ``step()`` on the current stream, max over ranks.  With ``flush`` every step
        has its own event pair and a write of a buffer larger than L2 before it, outside the pair."""
        torch = self.torch
        if flush:
            pairs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
            self.barrier()
            for begin, end in pairs:
                self.flush.fill_(1)
                begin.record()
                step()
                end.record()
            self.barrier()
            total = sum(begin.elapsed_time(end) for begin, end in pairs)
        else:
            begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            self.barrier()
            begin.record()
            for _ in range(steps):
                step()
            end.record()
            self.barrier()
            total = begin.elapsed_time(end)
        return self.slowest(total) / steps


def host_placement(device_index: int) -> dict:
    """Where this rank's host side sits relative to its GPU: the GPU's NUMA node (sysfs), the CPUs and memory nodes the
    process may use, and — when the GPU's node is among the allowed memory nodes — a preferred-node memory policy set
    before the pinned buffers are allocated, so the copies do not cross the socket interconnect.  Read-only apart from
    this process's own memory policy."""
    record: dict = {}
    try:
        import torch

        bus = torch.cuda.get_device_properties(device_index).pci_bus_id
        domain = getattr(torch.cuda.get_device_properties(device_index), "pci_domain_id", 0)
        device = getattr(torch.cuda.get_device_properties(device_index), "pci_device_id", 0)
        node_file = Path(f"/sys/bus/pci/devices/{domain:04x}:{bus:02x}:{device:02x}.0/numa_node")
        record["gpu_numa_node"] = int(node_file.read_text().strip()) if node_file.exists() else None
    except Exception as error:  # noqa: BLE001
        record["gpu_numa_node"] = None
        record["gpu_numa_error"] = f"{type(error).__name__}: {error}"[:120]
    try:
        status = Path("/proc/self/status").read_text()
        for key, label in (("Cpus_allowed_list", "cpus_allowed"), ("Mems_allowed_list", "mems_allowed")):
            record[label] = next(line.split(":", 1)[1].strip() for line in status.splitlines() if line.startswith(key))
    except Exception:  # noqa: BLE001
        pass
    node = record.get("gpu_numa_node")
    record["preferred_node_policy"] = "not attempted"
    if node is not None and node >= 0:
        allowed: set[int] = set()
        for part in str(record.get("mems_allowed", "")).split(","):
            if "-" in part:
                low, high = part.split("-")
                allowed.update(range(int(low), int(high) + 1))
            elif part.strip().isdigit():
                allowed.add(int(part))
        if node in allowed and len(allowed) > 1:
            try:
                libc = ctypes.CDLL(None, use_errno=True)
                mask = ctypes.c_ulong(1 << node)
                MPOL_PREFERRED, SYS_set_mempolicy = 1, 238  # x86-64
                result = libc.syscall(SYS_set_mempolicy, MPOL_PREFERRED, ctypes.byref(mask), ctypes.c_ulong(64))
                record["preferred_node_policy"] = "set" if result == 0 else f"refused (errno {ctypes.get_errno()})"
            except Exception as error:  # noqa: BLE001
                record["preferred_node_policy"] = f"unavailable ({type(error).__name__})"
        else:
            record["preferred_node_policy"] = "single memory node allowed" if len(allowed) <= 1 else "gpu node not allowed"
    return record


def spread(total: int, world: int, per_rank: int, width: int) -> list[tuple[int, int]]:
    """Sample ranges ``[start, stop)`` of ``width`` units over ``range(total)``: the first and the last units of every
    rank's shard (where an off-by-one in the shard offsets would show) and evenly spaced ones in between."""
    shard = total // world
    width = max(1, min(width, shard))
    ranges = []
    for rank in range(world):
        base = rank * shard
        starts = {0, shard - width}
        for index in range(1, max(per_rank - 1, 1)):
            starts.add(((shard - width) * index // max(per_rank - 1, 1)) // width * width)
        ranges += [(base + start, base + start + width) for start in sorted(starts)]
    return ranges


def host64(tensor) -> np.ndarray:
    return tensor.detach().to("cpu").double().numpy()


# ---------------------------------------------------------------------------------------------
# workloads
# ---------------------------------------------------------------------------------------------
class Workload:
    name = metric = unit = ""
    dtype, bound, seed = "bf16", "hbm", 0
    extent = 0            # length of the sharded outer axis at the configuration's size
    axis_name = "rows"
    always_flush = False   # time every step behind an L2 flush write (event pair per step)
    l2_resident = False    # the configuration is smaller than L2 by design and is reported as such
    input_names: tuple[str, ...] = ()
    output_names: tuple[str, ...] = ()
    order: tuple[str, ...] = ()   # kernel argument order over inputs, replicated operands and outputs
    e2e_chunks = 16
    tolerance = 0.0
    reference_size = 0      # reduced size for upstream's CPU runtime in the cpu_baseline leg (one run)
    reference_arm_size = 0  # smaller still for the --impl reference arm, which runs K steps

    # ---- description ------------------------------------------------------------------------------------
    def shrink(self) -> None:
        raise NotImplementedError

    def work(self, extent: int) -> float:
        """Algorithmic bytes (hbm) or flops (tensor) of ``extent`` units of the outer axis."""
        raise NotImplementedError

    def bytes_resident(self, extent: int) -> float:
        return self.work(extent)

    def generate(self, torch, piece: int) -> dict:
        """The sharded inputs of configuration-sized piece ``piece`` on the device, seeded: every rank gets the same."""
        raise NotImplementedError

    def replicated(self, torch) -> dict:
        return {}

    def alloc_outputs(self, torch, extent: int) -> dict:
        raise NotImplementedError

    def kernel(self, zoo, extent: int):
        raise NotImplementedError

    def describe(self, extent: int) -> str:
        raise NotImplementedError

    def size_key(self) -> int:
        return self.extent

    # ---- set-up -----------------------------------------------------------------------------------------
    def prepare(self, ctx: Context) -> None:
        torch, world = ctx.torch, ctx.world
        self.ctx = ctx
        self.total = self.extent * (world if ctx.weak else 1)
        if self.total % world:
            raise SystemExit(f"{self.name}: {self.total} {self.axis_name} do not split over {world} ranks")
        self.local = self.total // world
        low = ctx.rank * self.local
        self.rep = self.replicated(torch)
        self.sample_ranges = self.choose_samples(world)
        self.sample_inputs: list[dict] = []
        self.inputs: dict = {}
        for piece in range(world if ctx.weak else 1):
            tensors = self.generate(torch, piece)
            base = piece * self.extent
            if ctx.rank == 0 and not ctx.args.kernel_only:
                for sample in self.sample_ranges:
                    if base <= sample[0] < base + self.extent:
                        self.sample_inputs.append(self.take_sample(tensors, base, sample))
            start, stop = max(low, base), min(low + self.local, base + self.extent)
            if start < stop:
                self.inputs = {name: tensor[start - base:stop - base].clone() for name, tensor in tensors.items()}
            del tensors
        torch.cuda.empty_cache()
        self.outputs = self.alloc_outputs(torch, self.local)
        everything = {**self.inputs, **self.rep, **self.outputs}
        self.tensors = [everything[name] for name in self.order]
        from baybridge_b200 import B200Backend

        self.kernel_object = self.kernel(ctx.zoo, self.local)
        self.artifact = ctx.cute.compile(self.kernel_object, *self.tensors, backend=B200Backend(synchronize=False),
                                         cache_dir=ctx.cache_dir)
        self.handles = tuple(ctx.cute.from_dlpack(t) for t in self.tensors)
        resident = self.bytes_resident(self.local)
        self.flush = self.always_flush
        # kernel-only timing of a small working set: rotate over copies of every tensor so no step finds its data in L2
        copies = 1 if (self.flush or self.l2_resident or resident >= ROTATE_BELOW_BYTES) else min(16, -(-ROTATE_BELOW_BYTES // int(resident)) + 1)
        self.rotation_keep = [[tensor.clone() for tensor in self.tensors] for _ in range(copies - 1)]
        self.rotation = [self.handles] + [tuple(ctx.cute.from_dlpack(t) for t in clones) for clones in self.rotation_keep]
        self.launches = 0

    def step(self) -> None:
        """The timed step: the compiled artifact on the next copy of the tensors (copy 0 is the one that is gathered and checked)."""
        self.artifact(*self.rotation[self.launches % len(self.rotation)], stream=self.ctx.stream)
        self.launches += 1

    def step_in_place(self) -> None:
        self.artifact(*self.handles, stream=self.ctx.stream)

    # ---- parity against the CPU oracle on sampled units of the global problem -----------------------------
    def choose_samples(self, world: int) -> list[tuple]:
        raise NotImplementedError

    def take_sample(self, tensors: dict, base: int, sample: tuple) -> dict:
        start, stop = sample
        return {name: host64(tensor[start - base:stop - base]) for name, tensor in tensors.items()}

    def oracle_sample(self, oracle, sample: tuple, inputs: dict) -> dict:
        """name → float64 oracle result for one sample."""
        raise NotImplementedError

    def output_sample(self, full: dict, sample: tuple) -> dict:
        start, stop = sample
        return {name: host64(full[name][start:stop]) for name in self.output_names}

    def units_in(self, sample: tuple) -> int:
        return sample[1] - sample[0]

    def check(self, full: dict) -> dict:
        """Compare the gathered outputs (name → device tensor over the whole outer axis) with the oracle on the samples."""
        from oracle import cpu_runtime as oracle

        worst, worst_lse, units, exact, compared = 0.0, 0.0, 0, 0, 0
        ok = True
        for sample, inputs in zip(self.sample_ranges, self.sample_inputs):
            expected = self.oracle_sample(oracle, sample, inputs)
            actual = self.output_sample(full, sample)
            for name, reference in expected.items():
                got = actual[name]
                if name == "lse":
                    worst_lse = max(worst_lse, float(np.abs(got - reference).max()))
                    ok &= worst_lse <= 1e-2
                elif self.tolerance == 0.0:
                    mismatches = int(np.count_nonzero(got != oracle.round_to_dtype(reference, self.dtype)))
                    ok &= mismatches == 0
                    worst += mismatches
                else:
                    error = oracle.rel_l2(got, reference)
                    worst = max(worst, error)
                    ok &= error <= self.tolerance
                    exact += int(np.count_nonzero(got == oracle.round_to_dtype(reference, self.dtype)))
                    compared += got.size
            units += self.units_in(sample)
        record = {"against": "oracle/cpu_runtime.py on sampled units of the gathered global output",
                  f"checked_{self.axis_name}": units, "samples": len(self.sample_ranges), "ok": bool(ok)}
        if self.tolerance == 0.0:
            record.update(bar="bit-exact", mismatches=int(worst))
        else:
            record.update(bar=f"rel-L2 <= {self.tolerance:g}", rel_l2=worst)
            if compared:
                record["fraction_equal_to_rounded_reference"] = exact / compared
        if "lse" in self.output_names:
            record.update(lse_bar="abs <= 1e-2", lse_max_abs_error=worst_lse)
        return record

    # ---- the kernel fused with the all-gather ---------------------------------------------------------------
    def fused(self, ctx: Context):
        """→ (run, barrier, {output name: gathered tensor})."""
        raise NotImplementedError

    # ---- end to end -----------------------------------------------------------------------------------------
    def make_pipeline(self, ctx: Context):
        from baybridge_b200.host_pipeline import HostPipeline

        torch = ctx.torch
        host = {name: tensor.cpu().pin_memory() for name, tensor in {**self.inputs, **self.rep}.items()}
        host.update({name: torch.empty(tensor.shape, dtype=tensor.dtype).pin_memory() for name, tensor in self.outputs.items()})
        self.host = host
        chunks = max(1, min(self.e2e_chunks, self.local))
        if ctx.world > 1:
            chunks = max(min(4, chunks), chunks // ctx.world)  # about the bytes per chunk of the single-GPU pipeline
        chunks = int(os.environ.get("BB200_BENCH_E2E_CHUNKS", chunks))
        return HostPipeline(lambda extent: self.kernel(ctx.zoo, extent), [host[name] for name in self.order], chunks=chunks,
                            cache_dir=ctx.cache_dir)

    # ---- CPU legs ---------------------------------------------------------------------------------------------
    def port_sample(self):
        """→ (callable, work, description, cores) for the numpy port of the CPU runtime."""
        raise NotImplementedError


class FusedMulAdd(Workload):
    name, unit, bound, seed = "fused_mul_add", "GB/s", "hbm", 1002
    metric = "elementwise HBM GB/s (fused c=a*b+a, bf16)"
    extent, axis_name = 2**28, "elements"
    input_names, output_names, order = ("a", "b"), ("c",), ("a", "b", "c")
    tolerance = 2e-3
    reference_size, reference_arm_size = 2**20, 2**16

    def shrink(self):
        self.extent = 2**26  # 400 MB working set

    def work(self, extent):
        return 6.0 * extent  # read a, read b, write c at 2 B each

    def generate(self, torch, piece):
        generator = torch.Generator(device="cuda").manual_seed(self.seed + piece)
        return {name: torch.randn(self.extent, device="cuda", dtype=torch.float32, generator=generator).to(torch.bfloat16)
                for name in ("a", "b")}

    def alloc_outputs(self, torch, extent):
        return {"c": torch.empty(extent, device="cuda", dtype=torch.bfloat16)}

    def kernel(self, zoo, extent):
        return zoo.make_fused_mul_add_indexed(extent)

    def describe(self, extent):
        return f"fused_mul_add c=a*b+a bf16, {extent} elements per GPU (6 B/element), indexed IR form"

    def choose_samples(self, world):
        return spread(self.total, world, 4, 4096)

    def oracle_sample(self, oracle, sample, inputs):
        # the tensor-SSA listing of the same body, traced here for the sample's length and run by the oracle's interpreter
        n = sample[1] - sample[0]
        ir = self.ctx.cute.compile(self.ctx.zoo.fused_mul_add_ssa, *[_ShapeOnly((n,), "bfloat16")] * 3, backend="portable").ir.to_dict()
        arguments = {"a": inputs["a"], "b": inputs["b"], "c": np.zeros(n)}
        oracle.run_kernel_ir(ir, arguments)
        return {"c": arguments["c"]}

    def fused(self, ctx):
        from baybridge_b200.fused_gather import FusedGather

        fused, gathered = FusedGather.over_group(self.kernel_object, self.tensors)
        return (lambda: fused.run(*self.tensors, stream=ctx.stream)), fused.barrier, {"c": gathered[2]}

    def port_sample(self):
        from oracle import cpu_runtime as oracle

        n = 2**24
        rng = np.random.default_rng(self.seed)
        a, b = (oracle.bf16_round(rng.standard_normal(n, dtype=np.float32)).astype(np.float64) for _ in range(2))
        return (lambda: a * b + a), 6.0 * n, f"{n} of 2^28 elements, numpy f64 restatement of the tensor-SSA CPU runtime path", 1


class Gemm(Workload):
    name, unit, bound, seed = "gemm", "TFLOP/s", "tensor", 1003
    metric = "BF16 GEMM TFLOP/s"
    extent, axis_name = 8192, "rows"   # rows of A and C; N and K stay at the configuration's size
    n = k = 8192
    always_flush = True
    input_names, output_names, order = ("a",), ("c",), ("a", "b", "c")
    tolerance = 1e-2
    reference_size, reference_arm_size = 128, 48

    def shrink(self):
        self.extent = self.n = self.k = 4096

    def size_key(self):
        return self.n

    def work(self, extent):
        return 2.0 * extent * self.n * self.k

    def bytes_resident(self, extent):
        return 2.0 * (extent * self.k + self.n * self.k + extent * self.n)

    def generate(self, torch, piece):
        generator = torch.Generator(device="cuda").manual_seed(self.seed + 1 + piece)
        scale = 1.0 / math.sqrt(self.k)
        return {"a": (torch.randn((self.extent, self.k), device="cuda", dtype=torch.float32, generator=generator) * scale).to(torch.bfloat16)}

    def replicated(self, torch):
        generator = torch.Generator(device="cuda").manual_seed(self.seed)
        scale = 1.0 / math.sqrt(self.k)
        return {"b": (torch.randn((self.n, self.k), device="cuda", dtype=torch.float32, generator=generator) * scale).to(torch.bfloat16)}

    def alloc_outputs(self, torch, extent):
        return {"c": torch.empty((extent, self.n), device="cuda", dtype=torch.bfloat16)}

    def kernel(self, zoo, extent):
        return zoo.gemm_abt

    def describe(self, extent):
        return f"gemm C=A·B^T bf16, A [{extent}, {self.k}] per GPU, B [{self.n}, {self.k}] replicated, fp32 accumulate, bf16 out"

    def choose_samples(self, world):
        return spread(self.total, world, 2, 4)

    def oracle_sample(self, oracle, sample, inputs):
        if not hasattr(self, "_b_host"):
            self._b_host = host64(self.rep["b"])
        return {"c": oracle.gemm(inputs["a"], self._b_host, transpose_b=True)}

    def fused(self, ctx):
        from baybridge_b200.fused_gather import FusedGatherGemm

        fused, full = FusedGatherGemm.over_group(self.kernel_object, self.tensors)
        return (lambda: fused.run(self.inputs["a"], self.rep["b"], stream=ctx.stream)), fused.barrier, {"c": full}

    def library_ms(self, ctx) -> float:
        """``torch.matmul`` (cuBLAS) on the same operands, timed the same way: a reported comparison, never the kernel."""
        torch = ctx.torch
        a, b = self.inputs["a"], self.rep["b"]
        out = torch.empty_like(self.outputs["c"])
        step = lambda: torch.matmul(a, b.t(), out=out)  # noqa: E731
        for _ in range(3):
            step()
        return ctx.time_ms(step, 10, True)

    def port_sample(self):
        from oracle import cpu_runtime as oracle

        size = 2048
        rng = np.random.default_rng(self.seed)
        a, b = (oracle.bf16_round((rng.standard_normal((size, size)) / math.sqrt(size)).astype(np.float32)).astype(np.float64) for _ in range(2))
        return (lambda: oracle.gemm(a, b, transpose_b=True)), 2.0 * size**3, f"M=N=K={size} (of 8192), numpy f64 BLAS port", os.cpu_count() or 1


class RmsNorm(Workload):
    name, unit, bound, seed = "rmsnorm", "GB/s", "hbm", 1004
    metric = "RMSNorm HBM GB/s (bf16)"
    extent, hidden = 65536, 8192
    input_names, output_names, order = ("x",), ("out",), ("x", "out", "w")
    tolerance = 2e-3
    reference_size, reference_arm_size = 32, 8

    def shrink(self):
        self.extent = 8192  # 268 MB working set

    def work(self, extent):
        return 2.0 * extent * self.hidden * 2 + self.hidden * 2

    def generate(self, torch, piece):
        generator = torch.Generator(device="cuda").manual_seed(self.seed + 1 + piece)
        return {"x": torch.randn((self.extent, self.hidden), device="cuda", dtype=torch.float32, generator=generator).to(torch.bfloat16)}

    def replicated(self, torch):
        generator = torch.Generator(device="cuda").manual_seed(self.seed)
        return {"w": (1 + 0.1 * torch.randn((self.hidden,), device="cuda", dtype=torch.float32, generator=generator)).to(torch.bfloat16)}

    def alloc_outputs(self, torch, extent):
        return {"out": torch.empty((extent, self.hidden), device="cuda", dtype=torch.bfloat16)}

    def kernel(self, zoo, extent):
        return zoo.make_rmsnorm(1e-6)

    def describe(self, extent):
        return f"rmsnorm bf16 [{extent}, {self.hidden}] per GPU, weight [{self.hidden}] replicated, eps 1e-6"

    def choose_samples(self, world):
        return spread(self.total, world, 4, 8)

    def oracle_sample(self, oracle, sample, inputs):
        return {"out": oracle.rmsnorm(inputs["x"], host64(self.rep["w"]), 1e-6)}

    def fused(self, ctx):
        from baybridge_b200.fused_gather import FusedGatherRmsNorm

        fused, full = FusedGatherRmsNorm.over_group(self.kernel_object, self.tensors)
        return (lambda: fused.run(self.inputs["x"], self.rep["w"], stream=ctx.stream)), fused.barrier, {"out": full}

    def port_sample(self):
        from oracle import cpu_runtime as oracle

        rows = 512
        rng = np.random.default_rng(self.seed)
        x = oracle.bf16_round(rng.standard_normal((rows, self.hidden), dtype=np.float32)).astype(np.float64)
        w = oracle.bf16_round((1 + 0.1 * rng.standard_normal(self.hidden)).astype(np.float32)).astype(np.float64)
        return (lambda: oracle.rmsnorm(x, w, 1e-6)), self.work(rows), f"{rows} of 65536 rows, numpy f64 port", 1


class Attention(Workload):
    name, unit, bound, seed = "attention", "TFLOP/s", "tensor", 1005
    metric = "causal attention forward TFLOP/s (bf16)"
    extent, axis_name = 16, "batches"
    heads, seq, dim = 32, 4096, 128
    input_names, output_names, order = ("q", "k", "v"), ("out", "lse"), ("q", "k", "v", "out", "lse")
    tolerance = 1e-2
    reference_size, reference_arm_size = 128, 48

    def shrink(self):
        self.extent = 2

    def work(self, extent):
        return 4.0 * extent * self.heads * self.dim * self.seq * (self.seq + 1) / 2

    def bytes_resident(self, extent):
        return 4.0 * extent * self.seq * self.heads * self.dim * 2

    def generate(self, torch, piece):
        generator = torch.Generator(device="cuda").manual_seed(self.seed + piece)
        shape = (self.extent, self.seq, self.heads, self.dim)
        return {name: torch.randn(shape, device="cuda", dtype=torch.float32, generator=generator).to(torch.bfloat16) for name in "qkv"}

    def alloc_outputs(self, torch, extent):
        return {"out": torch.empty((extent, self.seq, self.heads, self.dim), device="cuda", dtype=torch.bfloat16),
                "lse": torch.empty((extent, self.heads, 1, self.seq), device="cuda", dtype=torch.float32)}

    def kernel(self, zoo, extent):
        return zoo.attention_causal

    def describe(self, extent):
        return (f"causal attention fwd bf16, B{extent} per GPU, H{self.heads} S{self.seq} D{self.dim} "
                "(layout [B,S,H,D]), causal FLOPs")

    def choose_samples(self, world):
        """(batch, head, prefix length): causal rows below the prefix length depend on keys below it only.  Every rank's
        first and last batch with a 1024-row prefix, and one whole sequence."""
        shard = self.total // world
        samples = []
        for rank in range(world):
            for batch in sorted({rank * shard, rank * shard + shard - 1}):
                samples.append((batch, (7 * batch + 3) % self.heads, min(1024, self.seq)))
        samples.append((self.total - 1, self.heads - 1, self.seq))
        return samples

    def take_sample(self, tensors, base, sample):
        batch, head, prefix = sample
        return {name: host64(tensors[name][batch - base, :prefix, head, :])[None, :, None, :] for name in "qkv"}

    def oracle_sample(self, oracle, sample, inputs):
        out, lse = oracle.attention(inputs["q"], inputs["k"], inputs["v"], causal=True)
        return {"out": out, "lse": lse}

    def output_sample(self, full, sample):
        batch, head, prefix = sample
        return {"out": host64(full["out"][batch, :prefix, head, :])[None, :, None, :],
                "lse": host64(full["lse"][batch, head, :, :prefix])[None, None]}

    def units_in(self, sample):
        return 1

    def check(self, full):
        record = super().check(full)
        record["checked_query_rows"] = sum(sample[2] for sample in self.sample_ranges)
        return record

    def fused(self, ctx):
        from baybridge_b200.fused_gather import FusedGatherAttention

        fused, (out_full, lse_full) = FusedGatherAttention.over_group(self.kernel_object, self.tensors)
        run = lambda: fused.run(self.inputs["q"], self.inputs["k"], self.inputs["v"], stream=ctx.stream)  # noqa: E731
        return run, fused.barrier, {"out": out_full, "lse": lse_full}

    def port_sample(self):
        from oracle import cpu_runtime as oracle

        bsz, seq, heads = 1, 1024, 4
        rng = np.random.default_rng(self.seed)
        q, k, v = (oracle.bf16_round(rng.standard_normal((bsz, seq, heads, self.dim), dtype=np.float32)).astype(np.float64) for _ in range(3))
        flops = 4.0 * bsz * heads * self.dim * seq * (seq + 1) / 2
        return (lambda: oracle.attention(q, k, v, causal=True)), flops, f"B{bsz} H{heads} S{seq} D{self.dim}, numpy f64 port", os.cpu_count() or 1


class IndexedAdd(Workload):
    """256x256 f32 indexed add.  786 KB of traffic, L2-resident after the first launch: what this measures is launch
    latency, reported per call and per launch of a recorded launch graph (``launch_latency``); no roofline is claimed."""
    name, unit, bound, dtype, seed = "indexed_add", "GB/s", "hbm", "f32", 1001
    metric = "indexed add 256x256 f32: effective GB/s of a launch-latency-bound call"
    extent, cols = 256, 256
    input_names, output_names, order = ("a", "b"), ("c",), ("a", "b", "c")
    e2e_chunks = 1
    l2_resident = True
    tolerance = 0.0
    reference_size = reference_arm_size = 256

    def shrink(self):
        pass

    def work(self, extent):
        return 3.0 * extent * self.cols * 4

    def generate(self, torch, piece):
        generator = torch.Generator(device="cuda").manual_seed(self.seed + piece)
        return {name: torch.rand((self.extent, self.cols), device="cuda", dtype=torch.float32, generator=generator).mul_(2).sub_(1)
                for name in ("a", "b")}

    def alloc_outputs(self, torch, extent):
        return {"c": torch.zeros((extent, self.cols), device="cuda", dtype=torch.float32)}

    def kernel(self, zoo, extent):
        return zoo.make_indexed_add_2d(extent, self.cols)

    def describe(self, extent):
        return f"indexed add c[r,c]=a[r,c]+b[r,c] f32, {extent}x{self.cols} per GPU, one thread per element (block 256)"

    def choose_samples(self, world):
        shard = self.total // world
        return [(rank * shard, (rank + 1) * shard) for rank in range(world)]  # every row

    def oracle_sample(self, oracle, sample, inputs):
        rows = sample[1] - sample[0]
        carriers = [_ShapeOnly((rows, self.cols), "float32")] * 3
        ir = self.ctx.cute.compile(self.ctx.zoo.make_indexed_add_2d(rows, self.cols), *carriers, backend="portable").ir.to_dict()
        names = [argument["name"] for argument in ir["arguments"]]
        arguments = {names[0]: inputs["a"], names[1]: inputs["b"], names[2]: np.zeros((rows, self.cols))}
        oracle.run_kernel_ir(ir, arguments)
        return {"c": arguments[names[2]]}

    def fused(self, ctx):
        from baybridge_b200.fused_gather import FusedGather

        fused, gathered = FusedGather.over_group(self.kernel_object, self.tensors)
        full = gathered[2].view(self.total, self.cols)
        return (lambda: fused.run(*self.tensors, stream=ctx.stream)), fused.barrier, {"c": full}

    def port_sample(self):
        rng = np.random.default_rng(self.seed)
        a, b = (rng.uniform(-1, 1, (256, 256)).astype(np.float32).astype(np.float64) for _ in range(2))
        return (lambda: (a + b).astype(np.float32)), self.work(256), "full size, numpy f64 restatement of the per-thread CPU runtime loop", 1

    def extras(self, ctx) -> dict:
        """Microseconds per launch three ways: upstream-style (synchronise after every launch), asynchronous launches,
        and the same launches recorded once into a launch graph and replayed."""
        from baybridge_b200.launch_graph import LaunchGraph

        torch = ctx.torch
        blocking = ctx.cute.compile(self.kernel_object, *self.tensors, backend="b200", cache_dir=ctx.cache_dir)
        calls = 2000
        torch.cuda.synchronize()
        started = time.perf_counter()
        for _ in range(calls):
            blocking(*self.handles)
        blocking_us = (time.perf_counter() - started) / calls * 1e6
        started = time.perf_counter()
        for _ in range(calls):
            self.artifact(*self.handles, stream=ctx.stream)
        torch.cuda.synchronize()
        eager_us = (time.perf_counter() - started) / calls * 1e6
        per_graph, replays = 200, 20
        graph = LaunchGraph()
        with graph.record() as recording_stream:
            for _ in range(per_graph):
                self.artifact(*self.handles, stream=recording_stream)
        for _ in range(3):
            graph.replay(stream=ctx.stream)
        torch.cuda.synchronize()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        for _ in range(replays):
            graph.replay(stream=ctx.stream)
        end.record()
        torch.cuda.synchronize()
        graph_us = begin.elapsed_time(end) * 1e3 / (per_graph * replays)
        graph.close()
        return {"launch_latency": {"synchronising_call_us": blocking_us, "asynchronous_call_us": eager_us,
                                   "graph_replay_us_per_launch": graph_us, "launches_per_graph": per_graph, "calls": calls}}


class LayerNorm(Workload):
    """LayerNorm with fused residual add: reads x, residual, weight, bias; writes out and x + residual."""
    name, unit, bound, seed = "layernorm", "GB/s", "hbm", 1006
    metric = "LayerNorm + residual HBM GB/s (bf16)"
    extent, hidden = 32768, 8192
    input_names, output_names = ("x", "residual"), ("out", "out_resid")
    order = ("x", "residual", "out", "out_resid", "w", "b")
    tolerance = 2e-3

    def shrink(self):
        self.extent = 4096

    def work(self, extent):
        return 4.0 * extent * self.hidden * 2 + 2 * self.hidden * 2

    def generate(self, torch, piece):
        generator = torch.Generator(device="cuda").manual_seed(self.seed + 1 + piece)
        return {name: torch.randn((self.extent, self.hidden), device="cuda", dtype=torch.float32, generator=generator).to(torch.bfloat16)
                for name in ("x", "residual")}

    def replicated(self, torch):
        generator = torch.Generator(device="cuda").manual_seed(self.seed)
        return {"w": (1 + 0.1 * torch.randn((self.hidden,), device="cuda", dtype=torch.float32, generator=generator)).to(torch.bfloat16),
                "b": (0.1 * torch.randn((self.hidden,), device="cuda", dtype=torch.float32, generator=generator)).to(torch.bfloat16)}

    def alloc_outputs(self, torch, extent):
        return {name: torch.empty((extent, self.hidden), device="cuda", dtype=torch.bfloat16) for name in self.output_names}

    def kernel(self, zoo, extent):
        return zoo.layernorm_kernel

    def describe(self, extent):
        return f"layernorm with residual add, bf16 [{extent}, {self.hidden}] per GPU, weight/bias [{self.hidden}], eps 1e-5"

    def choose_samples(self, world):
        return spread(self.total, world, 4, 8)

    def oracle_sample(self, oracle, sample, inputs):
        out, mixed = oracle.layernorm(inputs["x"], inputs["residual"], host64(self.rep["w"]), host64(self.rep["b"]), 1e-5)
        return {"out": out, "out_resid": mixed}

    def fused(self, ctx):
        from baybridge_b200.fused_gather import FusedGatherLayerNorm

        fused, (out_full, resid_full) = FusedGatherLayerNorm.over_group(self.kernel_object, self.tensors)
        run = lambda: fused.run(self.inputs["x"], self.inputs["residual"], self.rep["w"], self.rep["b"], stream=ctx.stream)  # noqa: E731
        return run, fused.barrier, {"out": out_full, "out_resid": resid_full}

    def port_sample(self):
        from oracle import cpu_runtime as oracle

        rows = 256
        rng = np.random.default_rng(self.seed)
        x, r = (oracle.bf16_round(rng.standard_normal((rows, self.hidden), dtype=np.float32)).astype(np.float64) for _ in range(2))
        w = oracle.bf16_round((1 + 0.1 * rng.standard_normal(self.hidden)).astype(np.float32)).astype(np.float64)
        b = oracle.bf16_round((0.1 * rng.standard_normal(self.hidden)).astype(np.float32)).astype(np.float64)
        return (lambda: oracle.layernorm(x, r, w, b, 1e-5)), self.work(rows), f"{rows} of 32768 rows, numpy f64 port", 1


class _Reduction(Workload):
    """A traced ``Tensor.reduce`` over one axis of a bf16 matrix: every element is read once."""
    unit, bound, seed = "GB/s", "hbm", 1007
    extent, cols = 65536, 8192
    kernel_name = ""
    kept_axis = 0
    input_names, output_names, order = ("src",), ("dst",), ("src", "dst")
    tolerance = 2e-3

    def shrink(self):
        self.extent = 8192

    def work(self, extent):
        return extent * self.cols * 2.0 + (extent if self.kept_axis == 0 else self.cols) * 2.0

    def generate(self, torch, piece):
        generator = torch.Generator(device="cuda").manual_seed(self.seed + piece)
        return {"src": torch.rand((self.extent, self.cols), device="cuda", dtype=torch.float32, generator=generator).mul_(2).sub_(1).to(torch.bfloat16)}

    def alloc_outputs(self, torch, extent):
        return {"dst": torch.empty((extent if self.kept_axis == 0 else self.cols,), device="cuda", dtype=torch.bfloat16)}

    def kernel(self, zoo, extent):
        return getattr(zoo, self.kernel_name)

    def port_sample(self):
        from oracle import cpu_runtime as oracle

        rows = 2048
        rng = np.random.default_rng(self.seed)
        src = oracle.bf16_round(rng.uniform(-1, 1, (rows, self.cols)).astype(np.float32)).astype(np.float64)
        run = (lambda: (src * src).sum(axis=1)) if self.kept_axis == 0 else (lambda: src.max(axis=0))
        return run, rows * self.cols * 2.0, f"{rows} of 65536 rows, numpy f64 restatement of the traced fold", 1


class RowReduce(_Reduction):
    name, kernel_name, kept_axis = "reduce_rows", "row_sum_of_squares", 0
    metric = "row reduction HBM GB/s (bf16)"

    def describe(self, extent):
        return f"row reduction dst[r] = sum_c src[r,c]^2, bf16 [{extent}, {self.cols}] per GPU (traced Tensor.reduce)"

    def choose_samples(self, world):
        return spread(self.total, world, 4, 8)

    def oracle_sample(self, oracle, sample, inputs):
        return {"dst": (inputs["src"] * inputs["src"]).sum(axis=1)}

    def fused(self, ctx):
        raise NotImplementedError("no fused gather form for reductions")


class ColumnReduce(_Reduction):
    """Folds over the sharded axis: it does not shard without an exchange step, so it runs on one GPU only."""
    name, kernel_name, kept_axis = "reduce_cols", "column_max", 1
    metric = "column reduction HBM GB/s (bf16)"
    e2e_chunks = 1

    def describe(self, extent):
        return f"column reduction dst[c] = max_r src[r,c], bf16 [{extent}, {self.cols}] (traced Tensor.reduce)"

    def choose_samples(self, world):
        if world > 1:
            raise SystemExit("reduce_cols folds over the outer axis and does not shard; run it with --gpus 1")
        return [(0, self.extent)]

    def take_sample(self, tensors, base, sample):
        return {"max": host64(tensors["src"].float().max(dim=0).values)}  # a fold of exact values: order-free

    def oracle_sample(self, oracle, sample, inputs):
        return {"dst": inputs["max"]}

    def output_sample(self, full, sample):
        return {"dst": host64(full["dst"])}


WORKLOADS = {cls.name: cls for cls in (FusedMulAdd, Gemm, RmsNorm, Attention, IndexedAdd, LayerNorm, RowReduce, ColumnReduce)}


class _ShapeOnly:
    """DLPack-looking carrier so a kernel can be traced without device memory."""

    def __init__(self, shape, dtype):
        self.shape, self.dtype = tuple(shape), dtype

    def __dlpack__(self, stream=None):
        return "capsule"

    def __dlpack_device__(self):
        return (2, 0)

    def data_ptr(self):
        return 0


# ---------------------------------------------------------------------------------------------
# CPU legs
# ---------------------------------------------------------------------------------------------
def scale_of(unit: str) -> float:
    return 1e9 if unit == "GB/s" else 1e12


def reference_runtime_available() -> bool:
    return (ROOT / "oracle" / "_ref" / "baybridge" / "__init__.py").exists() and (ROOT / "oracle" / "ref_runtime.py").exists()


def run_reference_runtime(workload: Workload, size: int, steps: int, warmup: int, timeout: float = 240.0) -> dict:
    """Upstream's own CPU reference runtime, unmodified, in a subprocess (``oracle/ref_runtime.py``)."""
    command = [sys.executable, str(ROOT / "oracle" / "ref_runtime.py"), "--workload", workload.name, "--size", str(size),
               "--steps", str(steps), "--warmup", str(warmup)]
    try:
        done = subprocess.run(command, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, timeout=timeout, cwd=str(ROOT))
        if done.returncode:
            tail = (done.stderr or done.stdout).strip().splitlines()
            return {"error": tail[-1][:200] if tail else f"exit status {done.returncode}"}
        return json.loads(done.stdout.strip().splitlines()[-1])
    except (subprocess.TimeoutExpired, ValueError, IndexError, OSError) as error:
        return {"error": f"{type(error).__name__}: {error}"[:200]}


def full_size_work(workload: Workload) -> float:
    fresh = type(workload)()
    return fresh.work(fresh.extent)


def reference_leg(workload: Workload, size: int, steps: int, warmup: int) -> dict | None:
    if not reference_runtime_available() or not size:
        return None
    result = run_reference_runtime(workload, size, steps, warmup)
    if "error" in result:
        return {"kind": "reference", "unavailable": result["error"]}
    seconds = sorted(result["seconds"])[len(result["seconds"]) // 2]
    return {"value": result["work_per_step"] / seconds / scale_of(workload.unit), "unit": workload.unit, "cores": 1,
            "of_host_cores": os.cpu_count(), "kind": "reference",
            "sample": f"upstream CPU reference runtime (interpreted Python, unmodified, subprocess): {result['sample']}",
            "seconds_per_sample": seconds, "runs": len(result["seconds"]),
            "linear_extrapolation_to_full_size_s": seconds * full_size_work(workload) / result["work_per_step"]}


def port_leg(workload: Workload, budget_s: float = 3.0) -> dict:
    run, work, sample, cores = workload.port_sample()
    run()  # warm-up
    durations = []
    started = time.perf_counter()
    while len(durations) < 2 or (time.perf_counter() - started < budget_s and len(durations) < 30):
        t0 = time.perf_counter()
        run()
        durations.append(time.perf_counter() - t0)
    median = sorted(durations)[len(durations) // 2]
    return {"value": work / median / scale_of(workload.unit), "unit": workload.unit, "cores": cores, "kind": "port",
            "sample": sample, "seconds_per_sample": median, "runs": len(durations)}


def cpu_baseline(workload: Workload) -> dict:
    """Upstream's CPU runtime at its reduced size (one run) with the numpy port beside it; the port alone when the copy
    of upstream is absent."""
    port = port_leg(workload)
    reference = reference_leg(workload, workload.reference_size, 1, 0)
    if reference is not None and "value" in reference:
        reference["port"] = port
        return reference
    if reference is not None:
        port["reference_unavailable"] = reference["unavailable"]
    return port


def reference_arm(args, names: list[str]) -> None:
    """``--impl reference``: K steps of upstream's CPU runtime per workload, each step a bounded sample."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    records = {}
    use_reference = reference_runtime_available()
    for index, name in enumerate(names):
        workload = WORKLOADS[name]()
        if args.small:
            workload.shrink()
        steps = max(1, min(args.steps, 20 if index == 0 else 3))
        warmup = min(args.warmup, 5 if index == 0 else 1)
        result = (run_reference_runtime(workload, workload.reference_arm_size, steps, warmup)
                  if use_reference and workload.reference_arm_size else {"error": "oracle/_ref is absent"})
        if "error" not in result:
            seconds = sum(result["seconds"]) / len(result["seconds"])
            work, kind, cores = result["work_per_step"], "reference", 1
            sample = f"upstream CPU reference runtime (interpreted Python, unmodified, subprocess): {result['sample']} per step"
        else:
            run, work, sample, cores = workload.port_sample()
            for _ in range(warmup):
                run()
            started = time.perf_counter()
            for _ in range(steps):
                run()
            seconds, kind = (time.perf_counter() - started) / steps, "port"
            sample += f" (upstream runtime not used: {result['error']})"
        value = work / seconds / scale_of(workload.unit)
        shard = workload.extent // (1 if args.scaling == "weak" else max(args.gpus, 1))
        records[name] = {
            "metric": workload.metric, "value": value, "unit": workload.unit, "steps": steps, "warmup": warmup,
            "ms_per_step": seconds * 1e3, "dtype": "f64 (CPU runtime arithmetic)", "config": {"workload": workload.describe(shard)},
            "cpu_baseline": {"value": value, "unit": workload.unit, "cores": cores, "kind": kind, "sample": sample},
            "e2e": {"value": value, "unit": workload.unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        }
    head = records[names[0]]
    line = {"impl": "reference", "metric": head["metric"], "value": head["value"], "unit": head["unit"], "n_gpus": args.gpus,
            "steps": head["steps"], "warmup": head["warmup"], "ms_per_step": head["ms_per_step"], "higher_is_better": True,
            "scaling": args.scaling, "vs_baseline": None, "dtype": head["dtype"], "data": "synthetic", "config": head["config"],
            "cpu_baseline": head["cpu_baseline"], "e2e": head["e2e"], "gpu_launches": 0}
    if len(names) > 1:
        line["workloads"] = {name: records[name] for name in names[1:]}
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------------
def copy_breakdown(ctx: Context, workload: Workload, pipeline_ms: float) -> dict:
    """Where the end-to-end time goes: the shard's host→device and device→host copies alone (one large copy per
    tensor), with every rank copying at once and with rank 0 copying alone while the others idle."""
    torch = ctx.torch
    device_side = {**workload.inputs, **workload.rep}
    inputs = [(workload.host[name], device_side[name]) for name in workload.input_names + tuple(workload.rep)]
    outputs = [(workload.host[name], workload.outputs[name]) for name in workload.output_names]
    h2d_bytes = sum(h.numel() * h.element_size() for h, _ in inputs)
    d2h_bytes = sum(h.numel() * h.element_size() for h, _ in outputs)
    side = torch.cuda.Stream()
    repeats = 3

    def timed(body, active: bool) -> float:
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ctx.barrier()
        begin.record()
        if active:
            for _ in range(repeats):
                body()
        end.record()
        ctx.barrier()
        return begin.elapsed_time(end) / repeats

    def copy_in():
        for host, device in inputs:
            device.copy_(host, non_blocking=True)

    def copy_out():
        for host, device in outputs:
            host.copy_(device, non_blocking=True)

    def both():
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            copy_out()
        copy_in()
        torch.cuda.current_stream().wait_stream(side)

    copy_in(), copy_out()
    h2d_all = ctx.per_rank(timed(copy_in, True))
    d2h_all = ctx.per_rank(timed(copy_out, True))
    both_all = ctx.per_rank(timed(both, True))
    record = {"h2d_bytes_per_rank": h2d_bytes, "d2h_bytes_per_rank": d2h_bytes,
              "h2d_alone_gbs_per_rank": [round(h2d_bytes / (ms * 1e-3) / 1e9, 2) for ms in h2d_all],
              "d2h_alone_gbs_per_rank": [round(d2h_bytes / (ms * 1e-3) / 1e9, 2) for ms in d2h_all],
              "both_directions_at_once_ms_per_rank": [round(ms, 3) for ms in both_all], "pipeline_ms": pipeline_ms,
              "note": "every rank copies at the same time; one cudaMemcpyAsync per tensor from pinned host memory"}
    if ctx.world > 1:
        solo_in = timed(copy_in, ctx.rank == 0)
        solo_out = timed(copy_out, ctx.rank == 0)
        record["rank0_copying_alone_gbs"] = {"h2d": round(h2d_bytes / (solo_in * 1e-3) / 1e9, 2),
                                             "d2h": round(d2h_bytes / (solo_out * 1e-3) / 1e9, 2)}
    try:
        record["host_cpus_visible_to_rank0"] = len(os.sched_getaffinity(0))
    except AttributeError:
        pass
    if ctx.dist is not None:
        placements = [None] * ctx.world
        ctx.dist.all_gather_object(placements, ctx.placement)
        record["host_placement_per_rank"] = placements
    else:
        record["host_placement_per_rank"] = [ctx.placement]
    return record


def measure(ctx: Context, workload: Workload, *, steps: int, warmup: int, headline: bool) -> dict:
    torch, args, world = ctx.torch, ctx.args, ctx.world
    workload.prepare(ctx)
    scale = scale_of(workload.unit)
    total_work = workload.work(workload.local) * world
    for _ in range(warmup):
        workload.step()
    ctx.barrier()
    workload.launches = 0
    with ClockSampler(ctx.local_rank) as sampler:
        kernel_ms = ctx.time_ms(workload.step, steps, workload.flush)
        launches = workload.launches
        deadline = time.perf_counter() + 0.25  # keep the device busy so NVML has samples under this load when K is small
        while time.perf_counter() < deadline:
            for _ in range(10):
                workload.step()
            torch.cuda.synchronize()
    clocks = sampler.summary()
    per_rank = workload.work(workload.local) / (kernel_ms * 1e-3) / scale
    record: dict = {"metric": workload.metric, "value": per_rank * world, "unit": workload.unit, "ms_per_step": kernel_ms,
                    "steps": steps, "warmup": warmup, "dtype": workload.dtype, "gpu_launches": launches}
    resident_gb = workload.bytes_resident(workload.local) / 1e9
    if workload.flush:
        l2 = "256 MB L2 flush write before every timed step, outside the event pairs"
    elif workload.l2_resident:
        l2 = f"working set {resident_gb * 1e3:.2f} MB is L2-resident by design (launch-latency bound); no flush"
    elif len(workload.rotation) > 1:
        l2 = (f"working set {resident_gb:.2f} GB per GPU: steps rotate over {len(workload.rotation)} copies of every tensor "
              f"({resident_gb * len(workload.rotation):.2f} GB touched between two uses of a copy), no flush")
    else:
        l2 = f"working set {resident_gb:.2f} GB per GPU > 126 MB L2, no flush"
    record["config"] = {"workload": workload.describe(workload.local), "l2": l2}
    if world > 1:
        record["config"].update(shard=f"{workload.local} of {workload.total} {workload.axis_name} per rank",
                                whole_problem=workload.describe(workload.total).replace(" per GPU", " in total"))
    if workload.bound == "hbm":
        peak, peak_unit, peak_name = float(ctx.peaks["hbm_gbs"]), "GB/s", "hbm_gbs"
    else:
        peak, peak_unit, peak_name = float(ctx.peaks["bf16_tflops"]), "TFLOP/s", "bf16_tflops burst"
    capture = ctx.traffic.get((workload.name, workload.size_key())) if world == 1 else None
    roofline = {"bound": workload.bound, "achieved": per_rank, "peak": peak, "unit": peak_unit, "frac": per_rank / peak,
                "peak_source": f"{ctx.peak_source} ({peak_name})", "kernel_ms": kernel_ms,
                "traffic": (capture["dram_bytes_read"] + capture["dram_bytes_write"]) if capture else None}
    if capture:
        roofline["traffic_source"] = f"profiles/traffic.json: {capture['kernel']}, captured {capture['date']} at commit {capture['commit']}"
    if workload.bound == "tensor":
        roofline["frac_of_sustained_peak"] = per_rank / float(ctx.peaks.get("bf16_tflops_sustained", peak))
        roofline["algorithmic_flops"] = workload.work(workload.local)
    else:
        roofline["algorithmic_bytes"] = workload.work(workload.local)
    if workload.name == "indexed_add":
        roofline["note"] = "launch-latency bound (786 KB, L2-resident): no roofline is claimed for this configuration"
    record.update(roofline=roofline, clocks=clocks)
    if args.kernel_only:
        return record

    # ---- parity of the (gathered) output, and the two gather forms -------------------------------------------
    gather_steps = max(1, min(steps, 10))
    workload.step_in_place()  # the copy that is gathered and checked holds this run's result
    if world == 1:
        torch.cuda.synchronize()
        record["parity"] = workload.check(workload.outputs)
    else:
        dist = ctx.dist
        full = {name: torch.empty((workload.total,) + tuple(out.shape[1:]), device="cuda", dtype=out.dtype)
                for name, out in workload.outputs.items()}

        def gather() -> None:
            for name in workload.output_names:
                dist.all_gather_into_tensor(full[name], workload.outputs[name])

        def kernel_then_gather() -> None:
            workload.step_in_place()
            gather()

        flush_collective = not workload.l2_resident  # steps with a collective: an L2 flush write before each

        for _ in range(2):
            kernel_then_gather()
        with_gather_ms = ctx.time_ms(kernel_then_gather, gather_steps, flush_collective)
        gather_ms = ctx.time_ms(gather, gather_steps, flush_collective)
        output_bytes = sum(t.numel() * t.element_size() for t in full.values())
        parity = workload.check(full) if ctx.rank == 0 else None
        record["value_with_gather"] = total_work / (with_gather_ms * 1e-3) / scale
        record["allgather"] = {"collective": "ncclAllGather (torch.distributed.all_gather_into_tensor) of the output shards",
                               "kernel_plus_allgather_ms": with_gather_ms, "allgather_alone_ms": gather_ms,
                               "output_bytes_total": output_bytes,
                               "bus_gbs": output_bytes * (world - 1) / world / (gather_ms * 1e-3) / 1e9}
        fused_error, fused_step, fused_full = None, None, {}
        try:  # an extra form: a box without symmetric-memory support must not lose the line
            run, fused_barrier, fused_full = workload.fused(ctx)

            def fused_step() -> None:
                run()
                fused_barrier()

            for _ in range(3):
                fused_step()
        except Exception as error:  # noqa: BLE001
            fused_error = f"{type(error).__name__}: {error}"[:200]
        if ctx.everyone(fused_error is None):
            ctx.barrier()
            fused_ms = ctx.time_ms(fused_step, gather_steps, flush_collective)
            same = all(torch.equal(fused_full[name], full[name]) for name in workload.output_names)
            record["value_fused"] = total_work / (fused_ms * 1e-3) / scale
            record["allgather"].update(fused_kernel_and_gather_ms=fused_ms,
                                       fused_speedup_vs_kernel_plus_allgather=with_gather_ms / fused_ms,
                                       fused_equals_nccl_gather_bitwise=ctx.everyone(same))
            if ctx.rank == 0:
                fused_parity = workload.check(fused_full)
                parity["fused_form_ok"] = fused_parity["ok"]
                parity["ok"] = bool(parity["ok"] and fused_parity["ok"])
        else:
            record["allgather"]["fused_unavailable"] = fused_error or "another rank could not set it up"
        record["parity"] = parity
        del full, fused_full
    if isinstance(workload, Gemm):
        library_ms = workload.library_ms(ctx)
        record["library"] = {"what": "torch.matmul (cuBLAS) on the same operands with the same timing; a comparison, never the kernel",
                             "library_ms": library_ms, "library_tflops": workload.work(workload.local) / (library_ms * 1e-3) / 1e12,
                             "kernel_speed_over_library": library_ms / kernel_ms}

    # ---- end to end: pinned host inputs → device, kernel through the public host pipeline, result → host -------
    pipeline = workload.make_pipeline(ctx)
    for _ in range(2):
        pipeline.run()
    ctx.barrier()
    started = time.perf_counter()
    for _ in range(args.e2e_steps):
        pipeline.run()
    e2e_seconds = ctx.slowest((time.perf_counter() - started) / args.e2e_steps)
    record["e2e"] = {"value": total_work / e2e_seconds / scale, "unit": workload.unit,
                     "h2d_bytes_per_step": pipeline.h2d_bytes * world, "d2h_bytes_per_step": pipeline.d2h_bytes * world,
                     "ms_per_step": e2e_seconds * 1e3, "chunks": pipeline.chunks,
                     "through": "baybridge_b200.host_pipeline.HostPipeline (copy-in / kernel / copy-out overlapped per chunk)"}
    if headline:
        record["e2e"]["breakdown"] = copy_breakdown(ctx, workload, e2e_seconds * 1e3)
    if hasattr(workload, "extras") and world == 1:
        record.update(workload.extras(ctx))
    return record


def release(ctx: Context, workload: Workload) -> None:
    for field in ("inputs", "rep", "outputs", "tensors", "handles", "host", "artifact", "sample_inputs", "_b_host", "rotation", "rotation_keep"):
        if hasattr(workload, field):
            delattr(workload, field)
    ctx.torch.cuda.empty_cache()


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=20)
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--workload", default="all", choices=["all", *sorted(WORKLOADS)])
    parser.add_argument("--scaling", default="strong", choices=["strong", "weak"])
    parser.add_argument("--impl", default="b200", choices=["b200", "reference"])
    parser.add_argument("--no-cpu-baseline", action="store_true")
    parser.add_argument("--e2e-steps", type=int, default=3)
    parser.add_argument("--small", action="store_true",
                        help="reduced problem (still larger than L2) for profiler captures; never a bench value")
    parser.add_argument("--kernel-only", action="store_true", help="time the kernel alone (profiler captures)")
    args = parser.parse_args()
    names = list(CONFIGS) if args.workload == "all" else [args.workload]
    if args.impl == "reference":
        reference_arm(args, names)
        return

    from baybridge_b200.backend import native

    ctx = Context(args)
    warmup, steps = max(args.warmup, 3), max(args.steps, 1)
    records: dict[str, dict] = {}
    for index, name in enumerate(names):
        workload = WORKLOADS[name]()
        if args.small:
            workload.shrink()
        try:
            records[name] = measure(ctx, workload, steps=steps, warmup=warmup, headline=index == 0)
        except Exception as error:  # noqa: BLE001
            if index == 0:
                raise
            records[name] = {"metric": workload.metric, "error": f"{type(error).__name__}: {error}"[:300]}
        if ctx.rank == 0 and ctx.world == 1 and not args.no_cpu_baseline and not args.kernel_only and "error" not in records[name]:
            records[name]["cpu_baseline"] = cpu_baseline(workload)
        release(ctx, workload)
        del workload

    if ctx.rank == 0:
        head = records[names[0]]
        line = {"metric": head.pop("metric"), "value": head.pop("value"), "unit": head.pop("unit"), "n_gpus": ctx.world,
                "steps": head.pop("steps"), "warmup": head.pop("warmup"), "ms_per_step": head.pop("ms_per_step"),
                "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None, "dtype": head.pop("dtype"),
                "data": "synthetic (seeded; every rank derives the same global arrays and keeps its shard)"}
        line.update(head)
        if len(names) > 1:
            line["workloads"] = {name: records[name] for name in names[1:]}
            line["gpu_launches_all_workloads"] = sum(r.get("gpu_launches", 0) for r in records.values())
        info = native.DeviceInfo()
        if native.library().bb200_device_info_get(ctx.local_rank, ctypes.byref(info)) == 0:
            line["device"] = {"name": info.name.decode(), "sm_count": info.sm_count}
        print(json.dumps(line), flush=True)
    if ctx.dist is not None:
        ctx.dist.barrier()
        ctx.dist.destroy_process_group()


if __name__ == "__main__":
    main()
