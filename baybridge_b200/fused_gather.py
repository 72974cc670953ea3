"""Elementwise kernel fused with the all-gather of its output: peer stores instead of a collective.

The multi-GPU form of the hot path is "every rank runs the kernel on its shard, then the output shards are
all-gathered" (``sharding.py``; upstream itself is single-device).  With NCCL that is two steps: the kernel
writes its shard to local HBM and the collective then reads it again and pushes it to the peers.  Here the
kernel does both: a rank's kernel stores every result vector into the gathered output buffer of *every* rank —
its own through a local pointer, the others' through peer-mapped pointers over NVLink — at
``rank * shard + i``.  The shard never makes the extra round trip through local HBM, the NVLink transfer
overlaps the computation vector by vector, and the only collective left is a barrier that tells every rank the
peers' stores have landed.

Only ordinary stores to peer memory are used (no multicast, no remote loads, no TMA on peer memory).  The
gathered buffers come from ``torch.distributed._symmetric_memory`` (plumbing: allocation, handle exchange, the
barrier); the kernel is the generated elementwise kernel in its fan-out form
(``backend/elementwise.py: render(..., fanout=N)``).
"""
from __future__ import annotations

import ctypes
from typing import Any, Sequence

from .backend import native
from .backend.elementwise import MAX_FANOUT, STORAGE_BYTES, THREADS, UNROLL, compile_cubin, render
from .backend.matcher import ElementwisePlan, match
from .driver import _normalize_kernel, trace
from .errors import BackendNotImplementedError
from .host_values import normalize_runtime_argument


class FusedGatherGemm:
    """The BF16 GEMM with the output all-gather fused into its epilogue (``bb200_gemm_bf16_gather``).

    Every rank multiplies its own row block ``A_r [m, k]`` by the replicated ``B``; the epilogue stores each tile of
    ``C_r`` into the full ``C [world·m, n]`` of every rank (peer stores over NVLink) at row ``rank·m``.
    ``FusedGatherGemm.over_group(kernel, sample_args)`` allocates the full ``C`` in symmetric memory; ``run(a, b)``
    launches; ``barrier()`` makes all ranks' tiles visible."""

    def __init__(self, kernel: Any, sample_args: Sequence[Any], *, destinations: Sequence[int], shard_index: int):
        definition = _normalize_kernel(kernel)
        self.ir = trace(definition, tuple(normalize_runtime_argument(arg) for arg in sample_args))
        plan = match(self.ir)
        if plan.kind != "gemm":
            raise BackendNotImplementedError("FusedGatherGemm needs a kernel that lowers to the BF16 GEMM")
        if not 1 <= len(destinations) <= MAX_FANOUT:
            raise ValueError("1..8 destination buffers are needed")
        self.plan = plan
        self.row_offset = int(shard_index) * plan.m
        self._table = (ctypes.c_void_p * len(destinations))(*[int(pointer) for pointer in destinations])
        self._count = len(destinations)

    @classmethod
    def over_group(cls, kernel: Any, sample_args: Sequence[Any], *, group=None):
        import torch
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symmetric

        group = group or dist.group.WORLD
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        if world > MAX_FANOUT:
            raise BackendNotImplementedError(f"FusedGatherGemm fans out to at most {MAX_FANOUT} ranks")
        probe = cls(kernel, sample_args, destinations=[1], shard_index=0)  # trace + match only
        plan = probe.plan
        dtype = torch.bfloat16 if plan.c_dtype == "bf16" else torch.float32
        device = torch.device("cuda", torch.cuda.current_device())
        full = symmetric.empty((world * plan.m, plan.n), dtype=dtype, device=device)
        handle = symmetric.rendezvous(full, group)
        fused = cls(kernel, sample_args, destinations=[int(pointer) for pointer in handle.buffer_ptrs], shard_index=rank)
        fused._handle = handle
        return fused, full

    def barrier(self) -> None:
        handle = getattr(self, "_handle", None)
        if handle is not None:
            handle.barrier()

    def run(self, a: Any, b: Any, *, stream: Any = None) -> None:
        plan = self.plan
        native.require_device()
        pointers = []
        for value in (a, b):
            if not hasattr(value, "data_ptr"):
                value = normalize_runtime_argument(value)
            pointers.append(ctypes.c_void_p(int(value.data_ptr() or getattr(value, "raw_address", 0))))
        native.call("bb200_gemm_bf16_gather", pointers[0], pointers[1], self._table, self._count, self.row_offset, plan.m, plan.n, plan.k,
                    int(plan.transpose_a), int(plan.transpose_b), native.DTYPE_CODES[plan.c_dtype], native.stream_handle(stream))


class FusedGatherRmsNorm:
    """RMSNorm with the output all-gather fused into the kernel (``bb200_rmsnorm_gather``): every rank normalises its
    own rows and stores each output vector into the full ``[world·rows, hidden]`` output of every rank."""

    def __init__(self, kernel: Any, sample_args: Sequence[Any], *, destinations: Sequence[int], shard_index: int):
        definition = _normalize_kernel(kernel)
        self.ir = trace(definition, tuple(normalize_runtime_argument(arg) for arg in sample_args))
        plan = match(self.ir)
        if plan.kind != "rmsnorm":
            raise BackendNotImplementedError("FusedGatherRmsNorm needs a kernel that lowers to RMSNorm")
        if not 1 <= len(destinations) <= MAX_FANOUT:
            raise ValueError("1..8 destination buffers are needed")
        self.plan = plan
        self.row_offset = int(shard_index) * plan.rows
        self._table = (ctypes.c_void_p * len(destinations))(*[int(pointer) for pointer in destinations])
        self._count = len(destinations)

    @classmethod
    def over_group(cls, kernel: Any, sample_args: Sequence[Any], *, group=None):
        import torch
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symmetric

        group = group or dist.group.WORLD
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        if world > MAX_FANOUT:
            raise BackendNotImplementedError(f"FusedGatherRmsNorm fans out to at most {MAX_FANOUT} ranks")
        plan = cls(kernel, sample_args, destinations=[1], shard_index=0).plan  # trace + match only
        dtype = {"bf16": torch.bfloat16, "f16": torch.float16, "f32": torch.float32}[plan.dtype]
        full = symmetric.empty((world * plan.rows, plan.hidden), dtype=dtype, device=torch.device("cuda", torch.cuda.current_device()))
        handle = symmetric.rendezvous(full, group)
        fused = cls(kernel, sample_args, destinations=[int(pointer) for pointer in handle.buffer_ptrs], shard_index=rank)
        fused._handle = handle
        return fused, full

    def barrier(self) -> None:
        handle = getattr(self, "_handle", None)
        if handle is not None:
            handle.barrier()

    def run(self, x: Any, gamma: Any, *, stream: Any = None) -> None:
        plan = self.plan
        native.require_device()
        pointers = []
        for value in (x, gamma):
            if not hasattr(value, "data_ptr"):
                value = normalize_runtime_argument(value)
            pointers.append(ctypes.c_void_p(int(value.data_ptr() or getattr(value, "raw_address", 0))))
        native.call("bb200_rmsnorm_gather", native.DTYPE_CODES[plan.dtype], pointers[0], pointers[1], self._table, self._count,
                    self.row_offset, plan.rows, plan.hidden, 1 if plan.gamma_is_full else 0, plan.epsilon, native.stream_handle(stream))


class FusedGatherLayerNorm:
    """LayerNorm (with its fused residual add) whose two outputs are all-gathered by the kernel itself
    (``bb200_layernorm_gather``).  ``over_group`` returns ``(fused, (out_full, out_resid_full))``."""

    def __init__(self, kernel: Any, sample_args: Sequence[Any], *, out_destinations: Sequence[int],
                 out_resid_destinations: Sequence[int], shard_index: int):
        definition = _normalize_kernel(kernel)
        self.ir = trace(definition, tuple(normalize_runtime_argument(arg) for arg in sample_args))
        plan = match(self.ir)
        if plan.kind != "layernorm":
            raise BackendNotImplementedError("FusedGatherLayerNorm needs a kernel that lowers to LayerNorm")
        if not 1 <= len(out_destinations) <= MAX_FANOUT or len(out_destinations) != len(out_resid_destinations):
            raise ValueError("1..8 destination buffers are needed, as many for out_resid as for out")
        self.plan = plan
        self.row_offset = int(shard_index) * plan.rows
        self._out_table = (ctypes.c_void_p * len(out_destinations))(*[int(pointer) for pointer in out_destinations])
        self._resid_table = (ctypes.c_void_p * len(out_resid_destinations))(*[int(pointer) for pointer in out_resid_destinations])
        self._count = len(out_destinations)

    @classmethod
    def over_group(cls, kernel: Any, sample_args: Sequence[Any], *, group=None):
        import torch
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symmetric

        group = group or dist.group.WORLD
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        if world > MAX_FANOUT:
            raise BackendNotImplementedError(f"FusedGatherLayerNorm fans out to at most {MAX_FANOUT} ranks")
        plan = cls(kernel, sample_args, out_destinations=[1], out_resid_destinations=[1], shard_index=0).plan  # trace + match only
        dtype = {"bf16": torch.bfloat16, "f16": torch.float16, "f32": torch.float32}[plan.dtype]
        device = torch.device("cuda", torch.cuda.current_device())
        out_full = symmetric.empty((world * plan.rows, plan.hidden), dtype=dtype, device=device)
        resid_full = symmetric.empty((world * plan.rows, plan.hidden), dtype=dtype, device=device)
        out_handle = symmetric.rendezvous(out_full, group)
        resid_handle = symmetric.rendezvous(resid_full, group)
        fused = cls(kernel, sample_args, out_destinations=[int(pointer) for pointer in out_handle.buffer_ptrs],
                    out_resid_destinations=[int(pointer) for pointer in resid_handle.buffer_ptrs], shard_index=rank)
        fused._handle = out_handle
        fused._resid_handle = resid_handle
        return fused, (out_full, resid_full)

    def barrier(self) -> None:
        handle = getattr(self, "_handle", None)
        if handle is not None:
            handle.barrier()  # follows every store of the launch on the stream, so it orders both tensors

    def run(self, x: Any, residual: Any, weight: Any, bias: Any, *, stream: Any = None) -> None:
        plan = self.plan
        native.require_device()
        pointers = []
        for value in (x, residual, weight, bias):
            if not hasattr(value, "data_ptr"):
                value = normalize_runtime_argument(value)
            pointers.append(ctypes.c_void_p(int(value.data_ptr() or getattr(value, "raw_address", 0))))
        native.call("bb200_layernorm_gather", native.DTYPE_CODES[plan.dtype], *pointers, self._out_table, self._resid_table, self._count,
                    self.row_offset, plan.rows, plan.hidden, 1 if plan.weight_is_full else 0, 1 if plan.bias_is_full else 0,
                    plan.epsilon, native.stream_handle(stream))


class FusedGatherAttention:
    """Attention forward with the all-gather of ``out`` and ``lse`` fused into the kernel's epilogue
    (``bb200_attention_fwd_gather``): every rank attends over its own sequences and stores each finished output
    row and log-sum-exp into the full ``[world·batch, seq, heads, head_dim]`` / ``[world·batch, heads, 1, seq]``
    tensors of every rank.  ``over_group`` returns ``(fused, (out_full, lse_full))``."""

    def __init__(self, kernel: Any, sample_args: Sequence[Any], *, out_destinations: Sequence[int],
                 lse_destinations: Sequence[int], shard_index: int):
        definition = _normalize_kernel(kernel)
        self.ir = trace(definition, tuple(normalize_runtime_argument(arg) for arg in sample_args))
        plan = match(self.ir)
        if plan.kind != "attention":
            raise BackendNotImplementedError("FusedGatherAttention needs a kernel that lowers to the attention forward")
        if plan.head_dim not in (64, 128):
            raise BackendNotImplementedError("FusedGatherAttention supports head_dim 64 and 128")
        if not 1 <= len(out_destinations) <= MAX_FANOUT or len(out_destinations) != len(lse_destinations):
            raise ValueError("1..8 destination buffers are needed, as many for lse as for out")
        self.plan = plan
        self.batch_offset = int(shard_index) * plan.batch
        self._out_table = (ctypes.c_void_p * len(out_destinations))(*[int(pointer) for pointer in out_destinations])
        self._lse_table = (ctypes.c_void_p * len(lse_destinations))(*[int(pointer) for pointer in lse_destinations])
        self._count = len(out_destinations)

    @classmethod
    def over_group(cls, kernel: Any, sample_args: Sequence[Any], *, group=None):
        import torch
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symmetric

        group = group or dist.group.WORLD
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        if world > MAX_FANOUT:
            raise BackendNotImplementedError(f"FusedGatherAttention fans out to at most {MAX_FANOUT} ranks")
        plan = cls(kernel, sample_args, out_destinations=[1], lse_destinations=[1], shard_index=0).plan  # trace + match only
        device = torch.device("cuda", torch.cuda.current_device())
        out_full = symmetric.empty((world * plan.batch, plan.seq, plan.heads, plan.head_dim), dtype=torch.bfloat16, device=device)
        lse_full = symmetric.empty((world * plan.batch, plan.heads, 1, plan.seq), dtype=torch.float32, device=device)
        out_handle = symmetric.rendezvous(out_full, group)
        lse_handle = symmetric.rendezvous(lse_full, group)
        fused = cls(kernel, sample_args, out_destinations=[int(pointer) for pointer in out_handle.buffer_ptrs],
                    lse_destinations=[int(pointer) for pointer in lse_handle.buffer_ptrs], shard_index=rank)
        fused._handle = out_handle
        fused._lse_handle = lse_handle
        return fused, (out_full, lse_full)

    def barrier(self) -> None:
        handle = getattr(self, "_handle", None)
        if handle is not None:
            handle.barrier()  # one barrier orders both tensors: it follows every store of the launch on the stream

    def run(self, q: Any, k: Any, v: Any, *, stream: Any = None) -> None:
        plan = self.plan
        native.require_device()
        pointers = []
        for value in (q, k, v):
            if not hasattr(value, "data_ptr"):
                value = normalize_runtime_argument(value)
            pointers.append(ctypes.c_void_p(int(value.data_ptr() or getattr(value, "raw_address", 0))))
        native.call("bb200_attention_fwd_gather", pointers[0], pointers[1], pointers[2], self._out_table, self._lse_table,
                    self._count, self.batch_offset, plan.batch, plan.seq, plan.heads, plan.kv_heads, plan.head_dim,
                    int(plan.causal), native.stream_handle(stream))


class _DestinationTable(ctypes.Structure):
    _fields_ = [("p", ctypes.c_void_p * MAX_FANOUT)]


class FusedGather:
    """``fused = FusedGather(kernel, sample_args, destinations={position: [ptr, ...]}, shard_index=r)``.

    ``kernel`` is a ``@kernel`` / ``@jit`` object whose body is a flat elementwise map; ``sample_args`` describe ONE
    rank's shard (device tensors or shape carriers, scalars as numbers).  For every stored tensor argument
    ``destinations`` gives the base pointers of the gathered buffers to write (``len == fan-out``, each holding
    ``fan-out * shard`` elements... or more); the shard lands at element offset ``shard_index * shard_numel``.
    ``run(*args, stream=)`` takes the same arguments as the ordinary artifact; stored tensor arguments are ignored
    (their results go to the destinations).  Use ``FusedGather.over_group`` to get destinations from symmetric memory.
    """

    def __init__(self, kernel: Any, sample_args: Sequence[Any], *, destinations: dict[int, Sequence[int]], shard_index: int,
                 device: int = 0):
        definition = _normalize_kernel(kernel)
        self.ir = trace(definition, tuple(normalize_runtime_argument(arg) for arg in sample_args))
        plan = match(self.ir)
        if not isinstance(plan, ElementwisePlan) or plan.mode != "flat":
            raise BackendNotImplementedError("FusedGather needs a kernel that lowers to a flat elementwise map")
        self.plan = plan
        self.stored = [position for position, _ in plan.stores]
        fanouts = {len(destinations.get(position, ())) for position in self.stored}
        if len(fanouts) != 1 or not 1 <= next(iter(fanouts)) <= MAX_FANOUT:
            raise ValueError("every stored tensor needs the same number (1..8) of destination pointers")
        self.fanout = next(iter(fanouts))
        self.shard_offset = int(shard_index) * plan.extent
        rendered = render(plan, self.ir, fanout=self.fanout)
        self.rendered = rendered
        self.device = device
        self._cubin = compile_cubin(rendered.source)
        self._function = None
        arguments = self.ir.arguments
        self._tables = {}
        aligned = True
        for position in self.stored:
            table = _DestinationTable()
            element = STORAGE_BYTES[arguments[position].spec.dtype]
            for slot, pointer in enumerate(destinations[position]):
                table.p[slot] = int(pointer)
                aligned &= (int(pointer) + self.shard_offset * element) % 16 == 0
            self._tables[position] = table
        self._destinations_aligned = aligned
        tile = THREADS * rendered.vec * UNROLL
        self._grid = native.U3(max(1, -(-plan.extent // tile)), 1, 1)
        self._block = native.U3(THREADS, 1, 1)
        ctype_of = {"double": ctypes.c_double, "int32_t": ctypes.c_int32, "int64_t": ctypes.c_int64}
        self._scalar_ctypes = [ctype_of[name] for name in rendered.scalar_ctypes]

    # -- construction over a process group ---------------------------------------------------------------
    @classmethod
    def over_group(cls, kernel: Any, sample_args: Sequence[Any], *, group=None):
        """One gathered buffer per stored tensor in symmetric memory (``world * shard`` elements on every rank);
        returns ``(fused, gathered)`` with ``gathered[position]`` this rank's full buffer as a torch tensor."""
        import torch
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symmetric

        group = group or dist.group.WORLD
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        if world > MAX_FANOUT:
            raise BackendNotImplementedError(f"FusedGather fans out to at most {MAX_FANOUT} ranks")
        definition = _normalize_kernel(kernel)
        ir = trace(definition, tuple(normalize_runtime_argument(arg) for arg in sample_args))
        plan = match(ir)
        if not isinstance(plan, ElementwisePlan) or plan.mode != "flat":
            raise BackendNotImplementedError("FusedGather needs a kernel that lowers to a flat elementwise map")
        device = torch.device("cuda", torch.cuda.current_device())
        names = {"f32": torch.float32, "bf16": torch.bfloat16, "f16": torch.float16, "i32": torch.int32, "i1": torch.bool}
        gathered, handles, destinations = {}, {}, {}
        for position, _ in plan.stores:
            spec = ir.arguments[position].spec
            buffer = symmetric.empty(world * plan.extent, dtype=names[spec.dtype], device=device)
            handle = symmetric.rendezvous(buffer, group)
            gathered[position], handles[position] = buffer, handle
            destinations[position] = [int(pointer) for pointer in handle.buffer_ptrs]
        fused = cls(kernel, sample_args, destinations=destinations, shard_index=rank, device=device.index or 0)
        fused._handles = handles
        return fused, gathered

    def barrier(self) -> None:
        """After ``run``: every rank's stores into every gathered buffer are complete and visible (enqueued on the
        current stream; nothing is read back on the host)."""
        for handle in getattr(self, "_handles", {}).values():
            handle.barrier()
            break  # one barrier orders all earlier stores of the stream

    # -- launch ----------------------------------------------------------------------------------------
    def run(self, *args: Any, stream: Any = None) -> None:
        arguments = self.ir.arguments
        if len(args) != len(arguments):
            raise TypeError(f"{self.ir.name} expects {len(arguments)} arguments, got {len(args)}")
        native.require_device()
        if self._function is None:
            image = self._cubin.read_bytes()
            module, function = ctypes.c_void_p(), ctypes.c_void_p()
            native.call("bb200_init", self.device)
            native.call("bb200_module_load", image, len(image), ctypes.byref(module))
            native.call("bb200_get_function", module, self.rendered.entry.encode(), ctypes.byref(function))
            self._module, self._function = module, function
        values: list[Any] = []
        aligned = self._destinations_aligned
        for position in self.rendered.tensor_order:
            if position in self._tables:
                values.append(self._tables[position])
                continue
            value = args[position]
            if not hasattr(value, "data_ptr"):  # anything that is not already a device tensor or handle
                value = normalize_runtime_argument(value)
            pointer = int(value.data_ptr() or getattr(value, "raw_address", 0))
            if not pointer:
                raise TypeError(f"argument {position} does not expose a device pointer")
            if position not in self.rendered.relaxed:
                aligned &= pointer % 16 == 0
            values.append(ctypes.c_void_p(pointer))
        for position, ctype in zip(self.rendered.scalar_order, self._scalar_ctypes):
            value = args[position]
            values.append(ctype(getattr(value, "value", value)))
        values += [ctypes.c_size_t(self.plan.extent), ctypes.c_size_t(self.shard_offset), ctypes.c_int(1 if aligned else 0)]
        params = (ctypes.c_void_p * len(values))(*[ctypes.cast(ctypes.byref(value), ctypes.c_void_p) for value in values])
        native.call("bb200_launch", self._function, self._grid, self._block, native.U3(1, 1, 1), 0, native.stream_handle(stream), params)
