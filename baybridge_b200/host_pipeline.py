"""Run a b200 kernel over HOST-resident tensors with the PCIe copies overlapped with the kernel.

Upstream's executable backends stage host tensors synchronously: copy everything in, launch, wait,
copy everything out (``ptx_exec.py:118-176``).  On a B200 the kernels of this path finish in a
fraction of a millisecond while the copies take tens of milliseconds, and PCIe is full duplex, so
the end-to-end time of a host-to-host call is set by how well the two copy directions overlap.

``HostPipeline`` splits the work along the outer (shard) axis — the same axis ``sharding.py`` uses
across GPUs — into chunks and runs three streams: host→device copy of chunk *i+1*, kernel of chunk
*i*, device→host copy of chunk *i−1*.  Replicated operands (a GEMM's B, a norm's weight) are copied
once.  Every chunk runs the ordinary compiled artifact for the chunk's shape; nothing about the
kernels changes.  ``torch`` supplies pinned memory, device buffers, streams and events.
"""
from __future__ import annotations

from typing import Any, Callable, Sequence

from .backend.b200 import B200Backend
from .backend.matcher import match
from .driver import compile as _compile
from .driver import trace
from .sharding import ShardSpec, shard_bounds, shard_spec


def _ramped(rows: int, chunks: int) -> list[tuple[int, int]]:
    """``chunks`` equal parts of ``range(rows)``, the first cut into 1/8, 1/8, 1/4, 1/2 of itself and the last into the
    mirror image — when the parts are long enough to be cut into pieces that keep 16-byte alignment for every dtype."""
    bounds = [shard_bounds(rows, chunks, index) for index in range(chunks)]
    first, last = bounds[0][1] - bounds[0][0], bounds[-1][1] - bounds[-1][0]
    if chunks < 4 or first % 128 or last % 128 or first < 1024 or last < 1024:
        return bounds
    head = [first // 8, first // 8, first // 4, first // 2]
    tail = [last // 2, last // 4, last // 8, last // 8]
    pieces = head + [stop - start for start, stop in bounds[1:-1]] + tail
    out, start = [], 0
    for size in pieces:
        out.append((start, start + size))
        start += size
    assert start == rows
    return out


class HostPipeline:
    """``pipeline = HostPipeline(kernel_for, host_args, chunks=8); pipeline.run()``.

    ``kernel_for(rows)`` returns the ``@kernel``/``@jit`` object to compile for a chunk with ``rows``
    entries along the shard axis (kernels whose launch grid depends on the size need this; pass
    ``lambda rows: kernel`` otherwise).  ``host_args`` are the kernel's arguments in order: pinned (or
    pageable) CPU ``torch`` tensors for tensor arguments, Python numbers for scalars.  Outputs are
    written back into the given host tensors.  With ``ramp`` (the default) the first and the last of the ``chunks``
    equal chunks are cut into pieces of 1/8, 1/8, 1/4 and 1/2 of a chunk (mirrored at the end): nothing overlaps the
    first host→device copy and the last device→host copy, so they should be short.
    """

    def __init__(self, kernel_for: Callable[[int], Any], host_args: Sequence[Any], *, chunks: int = 8, device: int | None = None,
                 cache_dir: str | None = None, ramp: bool = True):
        import torch

        self.torch = torch
        self.device = torch.device("cuda", torch.cuda.current_device() if device is None else device)
        self.host_args = list(host_args)
        self.kernel_for = kernel_for
        self.cache_dir = cache_dir
        tensor_positions = [i for i, value in enumerate(self.host_args) if isinstance(value, torch.Tensor)]
        if not tensor_positions:
            raise ValueError("HostPipeline needs at least one tensor argument")
        # plan and shard axes come from the full-size trace
        full_rows = None
        carriers = [_Carrier(value) if isinstance(value, torch.Tensor) else value for value in self.host_args]
        probe_definition = _definition(kernel_for(self.host_args[tensor_positions[0]].shape[0]))
        ir = trace(probe_definition, tuple(_normalize(c) for c in carriers))
        self.spec: ShardSpec = shard_spec(match(ir), ir)
        full_rows = self.spec.extent
        self.rows = full_rows
        self.outputs = set(self.spec.outputs)
        self.reads = set(self.spec.reads)
        if any(axis != 0 for _, axis in self.spec.sharded):
            # a shard axis that is not the leading one (A of a GEMM stored [k, m]) is not contiguous in host memory:
            # one pass over whole tensors, every argument held at its full shape
            self.chunks, self.sharded = 1, set()
        else:
            self.chunks = max(1, min(int(chunks), full_rows))
            self.sharded = {position for position, _ in self.spec.sharded}
        self.bounds = _ramped(full_rows, self.chunks) if ramp else [shard_bounds(full_rows, self.chunks, index) for index in range(self.chunks)]
        self.chunks = len(self.bounds)
        longest = max(stop - start for start, stop in self.bounds)
        backend = B200Backend(device=self.device.index or 0, synchronize=False)
        # device storage: two slots per sharded argument, one full copy per other argument
        self.slots: list[dict[int, Any]] = [{}, {}]
        self.replicated: dict[int, Any] = {}
        for position in tensor_positions:
            host = self.host_args[position]
            if position in self.sharded:
                for slot in self.slots:
                    slot[position] = torch.empty((longest,) + tuple(host.shape[1:]), device=self.device, dtype=host.dtype)
            else:
                self.replicated[position] = torch.empty_like(host, device=self.device)
        # one artifact per distinct chunk length
        self.artifacts: dict[int, Any] = {}
        for start, stop in self.bounds:
            rows = stop - start
            if rows not in self.artifacts:
                sample = [self._device_view(0, position, rows) if isinstance(value, torch.Tensor) else value
                          for position, value in enumerate(self.host_args)]
                self.artifacts[rows] = _compile(kernel_for(rows), *sample, backend=backend, cache_dir=cache_dir)
        self.copy_in, self.compute, self.copy_out = (torch.cuda.Stream(device=self.device) for _ in range(3))
        self.h2d_bytes = sum(self.host_args[p].numel() * self.host_args[p].element_size()
                             for p in tensor_positions if p in self.reads)
        self.d2h_bytes = sum(self.host_args[p].numel() * self.host_args[p].element_size() for p in self.outputs)

    def _device_view(self, slot: int, position: int, rows: int):
        if position in self.sharded:
            return self.slots[slot][position][:rows]
        return self.replicated[position]

    def run(self) -> None:
        """One host-to-host pass; returns after the last device→host copy has completed."""
        torch = self.torch
        caller = torch.cuda.current_stream(self.device)
        for stream in (self.copy_in, self.compute, self.copy_out):
            stream.wait_stream(caller)
        with torch.cuda.stream(self.copy_in):
            for position, buffer in self.replicated.items():
                if position in self.reads:
                    buffer.copy_(self.host_args[position], non_blocking=True)
        kernel_done: list[Any] = []
        drained: list[Any] = []
        for index, (start, stop) in enumerate(self.bounds):
            rows, slot = stop - start, index & 1
            with torch.cuda.stream(self.copy_in):
                if index >= 2:
                    self.copy_in.wait_event(kernel_done[index - 2])  # the slot's inputs are free again
                for position in self.sharded & self.reads:
                    self.slots[slot][position][:rows].copy_(self.host_args[position][start:stop], non_blocking=True)
                loaded = torch.cuda.Event()
                loaded.record(self.copy_in)
            with torch.cuda.stream(self.compute):
                self.compute.wait_event(loaded)
                if index >= 2:
                    self.compute.wait_event(drained[index - 2])  # the slot's outputs have left the device
                arguments = [self._device_view(slot, position, rows) if isinstance(value, torch.Tensor) else value
                             for position, value in enumerate(self.host_args)]
                self.artifacts[rows](*arguments, stream=self.compute.cuda_stream)
                done = torch.cuda.Event()
                done.record(self.compute)
                kernel_done.append(done)
            with torch.cuda.stream(self.copy_out):
                self.copy_out.wait_event(done)
                for position in self.outputs:
                    if position in self.sharded:
                        self.host_args[position][start:stop].copy_(self.slots[slot][position][:rows], non_blocking=True)
                out = torch.cuda.Event()
                out.record(self.copy_out)
                drained.append(out)
        with torch.cuda.stream(self.copy_out):
            for position in self.outputs:
                if position not in self.sharded:
                    self.host_args[position].copy_(self.replicated[position], non_blocking=True)
        self.copy_out.synchronize()
        caller.wait_stream(self.copy_out)


class _Carrier:
    """Shape/dtype carrier so a kernel can be traced for host tensors without touching the device."""

    def __init__(self, tensor: Any):
        self.shape, self.dtype = tuple(tensor.shape), str(tensor.dtype)

    def __dlpack__(self, stream: Any = None):
        return "capsule"

    def __dlpack_device__(self):
        return (2, 0)

    def data_ptr(self) -> int:
        return 0


def _normalize(value: Any) -> Any:
    from .host_values import normalize_runtime_argument

    return normalize_runtime_argument(value)


def _definition(kernel: Any):
    from .driver import _normalize_kernel

    return _normalize_kernel(kernel)
