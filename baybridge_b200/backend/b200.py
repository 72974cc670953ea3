"""``B200Backend`` — the backend object ``compile(..., backend="b200")`` resolves to.

It implements the duck-typed backend contract of upstream ``backend.py:26-29``
and ``compiler.py:646-689``: ``name``, ``artifact_extension``, ``lower(ir,
target) -> LoweredModule``, ``build_launcher(ir, target, lowered_module,
lowered_path) -> launcher(*args, stream=None)``, ``available(target)`` and
``supports(ir, target)``.  The launcher follows upstream's executable backend
(``ptx_exec.py:87-176``): positional arguments in IR argument order, host
``RuntimeTensor`` arguments staged through device buffers that are cached per
argument slot and released on error, ``TensorHandle`` / DLPack arguments used
in place through their device pointer, synchronous completion by default.

Every matched plan runs a hand-written sm_100a kernel through the C ABI of
``libbb200.so``; when the library or a device is missing the launcher raises —
there is no CPU path.
"""
from __future__ import annotations

import ctypes
import json
import threading
import warnings
from dataclasses import asdict
from pathlib import Path
from typing import Any, Callable

import numpy as np

from ..errors import BackendNotImplementedError
from ..host_values import DLPACK_CUDA, RuntimeScalar, RuntimeTensor, TensorHandle, from_dlpack
from ..portable_ir import row_major_stride
from ..scalar_types import DEVICE_NUMPY, byte_width, normalize_dtype_name
from . import native
from .elementwise import THREADS, UNROLL, compile_cubin, debug_bounds_enabled, render
from . import reduction as reduction_lowering
from .matcher import (AttentionPlan, ElementwisePlan, GemmPlan, LayerNormPlan, ReductionBundlePlan, ReductionPlan, RmsNormPlan,
                      adopt, match)

_thread_state = threading.local()

#: kernels launched through this module since import (bench.py reports it as ``gpu_launches``)
LAUNCH_COUNTER = {"launches": 0}


def _lowered_module_type():
    from ..driver import LoweredModule

    return LoweredModule


def _bind_device(device_id: int) -> None:
    """Make ``device_id``'s primary context current on this thread (once per thread/device)."""
    if getattr(_thread_state, "device", None) != device_id:
        native.call("bb200_init", device_id)
        _thread_state.device = device_id


class _StagedSlot:
    """Device copy of one host tensor argument, reused while shape/dtype stay the same."""

    def __init__(self, nbytes: int, signature: tuple):
        self.signature = signature
        self.nbytes = nbytes
        self.pointer = ctypes.c_void_p()
        native.call("bb200_mem_alloc", ctypes.byref(self.pointer), max(nbytes, 16))

    def release(self) -> None:
        if self.pointer:
            native.library().bb200_mem_free(self.pointer)
            self.pointer = ctypes.c_void_p()


class B200Backend:
    name = "b200"
    artifact_extension = ".b200.json"

    def __init__(self, *, device: int = 0, synchronize: bool = True, overlap_launches: bool = True):
        self.device = device
        self.synchronize = synchronize
        # flat elementwise kernels are launched with programmatic stream serialisation (``bb200_launch_dependent``):
        # stream order is kept by the kernel's own ``griddepcontrol.wait``; False takes the plain launch
        self.overlap_launches = overlap_launches

    # -- contract: capability probes ---------------------------------------------------------------
    def available(self, target: Any = None) -> bool:
        if target is not None and getattr(target, "arch", "") not in ("sm_100a", "sm_100"):
            return False
        return native.device_available()

    def supports(self, ir: Any, target: Any = None) -> bool:
        try:
            match(ir)
        except BackendNotImplementedError:
            return False
        return True

    def supports_auto_selection(self, ir: Any, target: Any = None, sample_args: tuple = ()) -> bool:
        return self.available(target) and self.supports(ir, target)

    # -- contract: lowering ------------------------------------------------------------------------
    def lower(self, ir: Any, target: Any):
        arch = getattr(target, "arch", None)
        if arch not in ("sm_100a", "sm_100"):
            raise BackendNotImplementedError(f"b200 lowers for NvidiaTarget('sm_100a') only (got {arch!r})")
        ir = adopt(ir)
        plan = match(ir)
        record: dict[str, Any] = {"backend": self.name, "kernel": ir.name, "plan": plan.kind, "target": arch}
        if isinstance(plan, ElementwisePlan):
            rendered = render(plan, ir, debug_bounds=plan.mode == "literal" and debug_bounds_enabled())
            record.update(
                debug_bounds=rendered.debug_bounds,
                mode=rendered.mode, compute=rendered.compute, vector_elements=rendered.vec, extent=plan.extent,
                entry=rendered.entry, tensor_order=list(rendered.tensor_order), scalar_order=list(rendered.scalar_order),
                scalar_ctypes=list(rendered.scalar_ctypes), source=rendered.source,
                gathers=list(rendered.relaxed),  # operands only read element by element: they need no 16-byte alignment
            )
        elif isinstance(plan, ReductionPlan):
            record.update(self._reduction_record(plan, ir))
        elif isinstance(plan, ReductionBundlePlan):
            record.update(entry="bb200_reduce_bundle", parts=[self._reduction_record(part, ir) for part in plan.parts])
        else:
            record.update(asdict(plan))
            record["entry"] = {"gemm": "bb200_gemm_bf16", "rmsnorm": "bb200_rmsnorm", "layernorm": "bb200_layernorm",
                               "attention": "bb200_attention_fwd"}[plan.kind]
        text = json.dumps(record, indent=1, sort_keys=True) + "\n"
        return _lowered_module_type()(backend_name=self.name, entry_point=record["entry"], dialect="b200.plan", text=text)

    @staticmethod
    def _reduction_record(plan: ReductionPlan, ir: Any) -> dict[str, Any]:
        rendered = reduction_lowering.render(plan, ir)
        return dict(
            form=plan.form, op=plan.op, outer=plan.outer, inner=plan.inner, compute=rendered.compute,
            compute_bytes=rendered.compute_bytes, vector_elements=rendered.vec, entry=f"bb200_reduce_{plan.form}",
            tensor_order=list(rendered.tensor_order), scalar_order=list(rendered.scalar_order),
            scalar_ctypes=list(rendered.scalar_ctypes), source=rendered.source,
        )

    # -- contract: launcher ------------------------------------------------------------------------
    def build_launcher(self, ir: Any, target: Any, lowered_module: Any, lowered_path: Path | None = None) -> Callable[..., None]:
        del lowered_path
        ir = adopt(ir)
        plan = match(ir)
        record = json.loads(lowered_module.text)
        if isinstance(plan, ElementwisePlan) and plan.mode == "literal" and bool(record.get("debug_bounds")) != debug_bounds_enabled():
            record = json.loads(self.lower(ir, target).text)  # a cached lowering from the other build flavour
        state: dict[str, Any] = {"slots": {}}
        runner = {
            "elementwise": self._elementwise_runner, "reduction": self._reduction_runner,
            "reduction_bundle": self._reduction_bundle_runner, "gemm": self._gemm_runner,
            "rmsnorm": self._rmsnorm_runner, "layernorm": self._layernorm_runner, "attention": self._attention_runner,
        }[plan.kind](ir, plan, record, state)
        arguments = ir.arguments
        # what a device tensor handle must look like per argument, computed once
        expected = [(tuple(a.spec.shape), a.spec.dtype, row_major_stride(a.spec.shape)) if a.kind == "tensor" else None for a in arguments]
        tensor_positions = [position for position, a in enumerate(arguments) if a.kind == "tensor"]
        all_tensors = len(tensor_positions) == len(arguments)
        # kernels that can record a code in the device status word: the mbarrier pipelines (bounded waits) and the
        # bounds-checking debug build of thread-by-thread elementwise kernels
        waits_on_device = plan.kind in ("gemm", "attention") or bool(record.get("debug_bounds"))
        checked: dict[tuple[int, int], Any] = {}  # (argument position, id of handle) -> handle already validated there

        def launcher(*args: Any, **kwargs: Any) -> None:
            stream = kwargs.pop("stream", None)
            if kwargs:
                raise TypeError("b200 launcher only supports positional arguments and an optional stream=")
            if len(args) != len(arguments):
                raise TypeError(f"{ir.name} expects {len(arguments)} arguments, got {len(args)}")
            native.require_device()
            synchronize = self.synchronize and not native.recording()  # a recording stream must not be synchronised
            if all_tensors and not synchronize:
                # fast path: every argument is a contiguous CUDA tensor handle of the expected shape and dtype on one
                # device; anything else takes the general path below, which also produces the error messages
                pointers = {}
                device_id = None
                for position in tensor_positions:
                    value = args[position]
                    known = checked.get((position, id(value)))
                    if known is not value:
                        # a handle is immutable: its shape, dtype and strides are compared once per argument position
                        shape, dtype, stride = expected[position]
                        if (type(value) is not TensorHandle or value.device_type != DLPACK_CUDA or tuple(value.shape) != shape
                                or normalize_dtype_name(value.dtype) != dtype or (value.stride is not None and tuple(value.stride) != stride)):
                            break
                        if len(checked) >= 256:
                            checked.clear()
                        checked[(position, id(value))] = value  # keeps the handle alive, so its id cannot be reused
                    if device_id is not None and value.device_id != device_id:
                        break
                    device_id = value.device_id
                    pointer = value.data_ptr() or value.raw_address
                    if not pointer:
                        break
                    pointers[position] = int(pointer)
                else:
                    _bind_device(int(device_id))
                    runner(pointers, {}, native.stream_handle(stream))
                    LAUNCH_COUNTER["launches"] += 1
                    return
            staged: list[tuple[RuntimeTensor, _StagedSlot, Any]] = []
            stream_handle = native.stream_handle(stream)
            try:
                pointers: dict[int, int] = {}
                scalars: dict[int, Any] = {}
                device_id = self._device_of(args)
                _bind_device(device_id)
                for position, (argument, value) in enumerate(zip(arguments, args)):
                    if argument.kind == "tensor":
                        pointers[position] = self._tensor_pointer(position, argument, value, stream, stream_handle, state, staged)
                    else:
                        scalars[position] = self._scalar_value(argument, value)
                runner(pointers, scalars, stream_handle)
                LAUNCH_COUNTER["launches"] += 1
                if staged or synchronize:
                    native.call("bb200_stream_synchronize", stream_handle)
                    if waits_on_device:
                        # a bounded in-kernel wait that gave up leaves partial output: surface it like a native launch
                        # that returned non-zero (upstream hipcc_exec.py:181-182)
                        status = native.take_device_status(stream_handle)
                        if status:
                            raise RuntimeError(f"launch_{ir.name} returned device status {status}: a bounded device-side wait "
                                               f"gave up ({native.ERROR_NAMES[-6]}); the output is incomplete")
                for tensor, slot, foreign in staged:
                    image = np.empty(tensor.numel, dtype=DEVICE_NUMPY[tensor.dtype])
                    native.call("bb200_memcpy_d2h", image.ctypes.data_as(ctypes.c_void_p), slot.pointer, slot.nbytes, stream_handle)
                    native.call("bb200_stream_synchronize", stream_handle)
                    tensor.absorb_device_image(image)
                    if foreign is not None:
                        foreign._storage[:] = tensor.as_numpy().reshape(-1).tolist()
            except Exception:
                for slot in state.pop("slots", {}).values():
                    slot.release()
                state["slots"] = {}
                raise

        def release() -> None:
            """Free the staged device copies and unload the modules this launcher holds (it reloads them on the next call)."""
            holders = [state] + [value for key, value in state.items() if key.startswith("part") and isinstance(value, dict)]
            for holder in holders:
                for slot in holder.get("slots", {}).values():
                    slot.release()
                holder["slots"] = {}
                for module in holder.pop("modules", {}).values():
                    native.library().bb200_module_unload(module)
                holder.get("functions", {}).clear()

        launcher.plan = plan  # type: ignore[attr-defined]
        launcher.release = release  # type: ignore[attr-defined]
        return launcher

    # -- argument marshalling ------------------------------------------------------------------------
    def _device_of(self, args: tuple[Any, ...]) -> int:
        # duck-typed so handles created by an upstream checkout's runtime module count too
        devices = {int(value.device_id) for value in args
                   if getattr(value, "device_type", None) == DLPACK_CUDA and hasattr(value, "device_id")}
        if len(devices) > 1:
            raise BackendNotImplementedError(f"b200: tensor arguments live on different devices {sorted(devices)}")
        return devices.pop() if devices else self.device

    def _tensor_pointer(self, position, argument, value, stream, stream_handle, state, staged) -> int:
        spec = argument.spec
        foreign = None
        if not isinstance(value, (RuntimeTensor, TensorHandle)) and hasattr(value, "_storage") and hasattr(value, "tolist"):
            # a host tensor of an upstream checkout (list storage): stage a copy, write results back into its list
            foreign, value = value, RuntimeTensor.from_data(value.tolist(), dtype=value.dtype)
        if not isinstance(value, (RuntimeTensor, TensorHandle)) and hasattr(value, "__dlpack__") and hasattr(value, "__dlpack_device__"):
            value = from_dlpack(value, stream=stream)
        if isinstance(value, TensorHandle):
            if int(value.device_type) != DLPACK_CUDA:
                raise BackendNotImplementedError(f"b200 currently requires CUDA TensorHandle inputs for tensor argument '{argument.name}'")
            if tuple(value.shape) != tuple(spec.shape) or normalize_dtype_name(value.dtype) != spec.dtype:
                raise TypeError(
                    f"b200 tensor argument '{argument.name}' expects {spec.dtype}{list(spec.shape)}, got {value.dtype}{list(value.shape)}"
                )
            if value.stride is not None and tuple(value.stride) != row_major_stride(value.shape):
                raise BackendNotImplementedError(
                    f"b200 currently requires contiguous CUDA TensorHandle inputs for tensor argument '{argument.name}'"
                )
            pointer = value.data_ptr() or value.raw_address
            if not pointer:
                raise TypeError(f"b200 tensor handle for argument '{argument.name}' does not expose a usable data_ptr()")
            return int(pointer)
        if isinstance(value, RuntimeTensor):
            if native.recording():
                raise BackendNotImplementedError(
                    f"b200: host tensor argument '{argument.name}' cannot be staged while a launch graph records; pass device tensors")
            if tuple(value.shape) != tuple(spec.shape) or value.dtype != spec.dtype:
                raise TypeError(
                    f"b200 tensor argument '{argument.name}' expects {spec.dtype}{list(spec.shape)}, got {value.dtype}{list(value.shape)}"
                )
            if not state.get("warned_staging"):
                warnings.warn(
                    f"b200 is staging RuntimeTensor argument '{argument.name}' through host memory; pass CUDA TensorHandle "
                    "values (or DLPack-capable device tensors) to avoid host-copy dominated timings",
                    RuntimeWarning, stacklevel=4,
                )
                state["warned_staging"] = True
            image = value.device_image()
            signature = (value.shape, value.dtype)
            slot_key = (position, getattr(_thread_state, "device", self.device))  # device memory belongs to one device
            slot = state["slots"].get(slot_key)
            if slot is None or slot.signature != signature:
                if slot is not None:
                    slot.release()
                slot = state["slots"][slot_key] = _StagedSlot(image.nbytes, signature)
            native.call("bb200_memcpy_h2d", slot.pointer, image.ctypes.data_as(ctypes.c_void_p), image.nbytes, stream_handle)
            native.call("bb200_stream_synchronize", stream_handle)  # `image` is pageable and about to go out of scope
            staged.append((value, slot, foreign))
            return int(slot.pointer.value)
        raise TypeError(
            "b200 currently expects RuntimeTensor values, CUDA TensorHandle values, or CUDA DLPack-capable tensor objects "
            f"for tensor argument '{argument.name}', got {type(value).__name__}"
        )

    @staticmethod
    def _scalar_value(argument, value: Any) -> Any:
        if isinstance(value, RuntimeScalar):
            if normalize_dtype_name(value.dtype) != argument.spec.dtype:
                raise TypeError(f"b200 scalar argument '{argument.name}' expects dtype {argument.spec.dtype}, got {value.dtype}")
            return value.value
        if not isinstance(value, (bool, int, float)):
            raise TypeError(f"b200 scalar argument '{argument.name}' expects a number, got {type(value).__name__}")
        return value

    # -- per-plan runners ----------------------------------------------------------------------------
    def _elementwise_runner(self, ir, plan: ElementwisePlan, record: dict[str, Any], state: dict[str, Any]):
        cubin_path = compile_cubin(record["source"])  # nvcc runs here, at compile() time, GPU or not
        tensor_order, scalar_order = record["tensor_order"], record["scalar_order"]
        ctype_of = {"double": ctypes.c_double, "int32_t": ctypes.c_int32, "int64_t": ctypes.c_int64}
        scalar_ctypes = [ctype_of[name] for name in record["scalar_ctypes"]]
        flat = record["mode"] == "flat"
        extent = int(record["extent"])
        gathers = set(record.get("gathers", ()))
        if flat:
            tile = THREADS * int(record["vector_elements"]) * UNROLL
            grid = native.U3(max(1, -(-extent // tile)), 1, 1)
            block = native.U3(THREADS, 1, 1)
        else:
            grid, block = native.U3(*ir.launch.grid), native.U3(*ir.launch.block)
        cluster = native.U3(1, 1, 1)
        entry = record["entry"].encode()

        def run(pointers: dict[int, int], scalars: dict[int, Any], stream_handle) -> None:
            # a module belongs to the context it was loaded in: one per device this launcher has run on
            device_id = getattr(_thread_state, "device", self.device)
            function = functions.get(device_id)
            if function is None:
                image = cubin_path.read_bytes()
                module = ctypes.c_void_p()
                native.call("bb200_module_load", image, len(image), ctypes.byref(module))
                function = ctypes.c_void_p()
                native.call("bb200_get_function", module, entry, ctypes.byref(function))
                state.setdefault("modules", {})[device_id] = module
                functions[device_id] = function
            for slot, position in zip(tensor_slots, tensor_order):
                slot.value = pointers[position]
            for slot, position in zip(scalar_slots, scalar_order):
                slot.value = scalars[position]
            if flat:
                misaligned = 0
                for position in aligned_positions:
                    misaligned |= pointers[position]
                vector_flag.value = 0 if misaligned & 15 else 1
            if debug_bounds:
                native.call("bb200_device_status_address", ctypes.byref(status_slot))  # the current device's word
            # the flat kernels wait (griddepcontrol.wait) for the kernel before them before they touch memory, so their
            # CTAs may be placed while that kernel drains; a recording stream takes the plain launch
            overlapped = flat and self.overlap_launches and not native.recording()
            native.call_resolved(launch_dependent if overlapped else launch_plain, "bb200_launch_dependent" if overlapped else "bb200_launch",
                                 function, grid, block, cluster, 0, stream_handle, params)

        functions: dict[int, Any] = state.setdefault("functions", {})
        launch_plain, launch_dependent = native.entry_point("bb200_launch"), native.entry_point("bb200_launch_dependent")
        # the parameter block is built once; a call only rewrites the values (launchers are not thread-safe, like upstream's)
        tensor_slots = [ctypes.c_void_p() for _ in tensor_order]
        scalar_slots = [ctype() for ctype in scalar_ctypes]
        vector_flag = ctypes.c_int(0)
        aligned_positions = [position for position in tensor_order if position not in gathers]
        debug_bounds = bool(record.get("debug_bounds"))
        status_slot = ctypes.c_void_p()
        slots: list[Any] = tensor_slots + scalar_slots + ([ctypes.c_size_t(extent), vector_flag] if flat else []) + ([status_slot] if debug_bounds else [])
        params = (ctypes.c_void_p * len(slots))(*[ctypes.cast(ctypes.byref(slot), ctypes.c_void_p) for slot in slots])
        state["params"] = (slots, params)  # keep the ctypes objects alive with the launcher
        return run

    def _reduction_bundle_runner(self, ir, plan: ReductionBundlePlan, record: dict[str, Any], state: dict[str, Any]):
        """The folds of a bundle are independent of each other: one after the other on the caller's stream."""
        runners = [self._reduction_runner(ir, part, part_record, state.setdefault(f"part{index}", {"slots": {}}))
                   for index, (part, part_record) in enumerate(zip(plan.parts, record["parts"]))]

        def run(pointers: dict[int, int], scalars: dict[int, Any], stream_handle) -> None:
            for runner in runners:
                runner(pointers, scalars, stream_handle)

        return run

    def _reduction_runner(self, ir, plan: ReductionPlan, record: dict[str, Any], state: dict[str, Any]):
        cubin_path = compile_cubin(record["source"])
        tensor_order, scalar_order = record["tensor_order"], record["scalar_order"]
        ctype_of = {"double": ctypes.c_double, "int32_t": ctypes.c_int32, "int64_t": ctypes.c_int64}
        scalar_ctypes = [ctype_of[name] for name in record["scalar_ctypes"]]
        compute_ctype = {"double": ctypes.c_double, "float": ctypes.c_float, "long long": ctypes.c_longlong}[record["compute"]]
        compute_bytes, vec = int(record["compute_bytes"]), int(record["vector_elements"])
        threads = reduction_lowering.THREADS
        outer, inner, total = plan.outer, plan.inner, plan.outer * plan.inner
        one = native.U3(1, 1, 1)
        # launch geometry is fixed by the plan
        if plan.form == "all":
            chunks = max(1, min(148 * 8, -(-total // (threads * vec * 2))))
            chunk_len = -(-(-(-total // chunks)) // vec) * vec
            chunks = -(-total // chunk_len)
            scratch_bytes = chunks * compute_bytes if chunks > 1 else 0
        elif plan.form == "cols":
            slabs = max(1, min(outer, 256, (148 * 1024) // max(inner, 1)))
            # vectorised form (16-byte column groups): enough row slabs for ~8 CTAs per SM, at least 8 rows each
            partial_vec = 16 // compute_bytes
            vector_shape = inner % vec == 0 and inner % partial_vec == 0
            vec_threads = reduction_lowering.COLS_VEC_THREADS
            vec_blocks = -(-(inner // max(vec, 1)) // vec_threads) if vector_shape else 1
            vec_slabs = max(1, min(-(-(148 * 8) // vec_blocks), outer // 8, 1024))
            scratch_bytes = max(slabs, vec_slabs if vector_shape else 0) * inner * compute_bytes if max(slabs, vec_slabs) > 1 else 0
        else:
            scratch_bytes = 0

        def function(name: str):
            # modules and functions are per context, hence per device; so is the scratch buffer below
            device_id = getattr(_thread_state, "device", self.device)
            functions = state.setdefault("functions", {})
            if (device_id, name) not in functions:
                modules = state.setdefault("modules", {})
                if device_id not in modules:
                    image = cubin_path.read_bytes()
                    module = ctypes.c_void_p()
                    native.call("bb200_module_load", image, len(image), ctypes.byref(module))
                    modules[device_id] = module
                handle = ctypes.c_void_p()
                native.call("bb200_get_function", modules[device_id], name.encode(), ctypes.byref(handle))
                functions[(device_id, name)] = handle
            return functions[(device_id, name)]

        def launch(name: str, grid, block, values: list[Any], stream_handle) -> None:
            params = (ctypes.c_void_p * len(values))(*[ctypes.cast(ctypes.byref(v), ctypes.c_void_p) for v in values])
            native.call("bb200_launch", function(name), grid, block, one, 0, stream_handle, params)

        def run(pointers: dict[int, int], scalars: dict[int, Any], stream_handle) -> None:
            inputs: list[Any] = [ctypes.c_void_p(pointers[position]) for position in tensor_order]
            inputs += [ctype(scalars[position]) for position, ctype in zip(scalar_order, scalar_ctypes)]
            dst = [ctypes.c_void_p(pointers[plan.dst]), ctypes.c_size_t(plan.dst_offset)]
            init = compute_ctype(plan.init)
            aligned = ctypes.c_int(1 if all(pointers[position] % 16 == 0 for position in tensor_order) else 0)
            scratch = None
            if scratch_bytes:
                scratch_key = ("scratch", getattr(_thread_state, "device", self.device))
                slot = state["slots"].get(scratch_key)
                if slot is None or slot.nbytes < scratch_bytes:
                    if slot is not None:
                        slot.release()
                    slot = state["slots"][scratch_key] = _StagedSlot(scratch_bytes, ("scratch",))
                scratch = ctypes.c_void_p(slot.pointer.value)
            block = native.U3(threads, 1, 1)
            if plan.form == "rows":
                launch("bb200_reduce_rows", native.U3(outer, 1, 1), block,
                       inputs + dst + [ctypes.c_size_t(outer), ctypes.c_size_t(inner), ctypes.c_size_t(total), init, aligned], stream_handle)
            elif plan.form == "all":
                if chunks == 1:
                    launch("bb200_reduce_rows", native.U3(1, 1, 1), block,
                           inputs + dst + [ctypes.c_size_t(1), ctypes.c_size_t(total), ctypes.c_size_t(total), init, aligned], stream_handle)
                else:
                    launch("bb200_reduce_rows_partial", native.U3(chunks, 1, 1), block,
                           inputs + [scratch, ctypes.c_size_t(chunks), ctypes.c_size_t(chunk_len), ctypes.c_size_t(total), aligned],
                           stream_handle)
                    launch("bb200_reduce_partials_rows", native.U3(1, 1, 1), block, [scratch] + dst + [ctypes.c_size_t(chunks), init],
                           stream_handle)
            elif vector_shape and aligned.value:
                vec_block = native.U3(vec_threads, 1, 1)
                if vec_slabs == 1:
                    launch("bb200_reduce_cols_vec", native.U3(vec_blocks, 1, 1), vec_block,
                           inputs + dst + [ctypes.c_size_t(outer), ctypes.c_size_t(inner), init], stream_handle)
                else:
                    launch("bb200_reduce_cols_vec_partial", native.U3(vec_blocks, vec_slabs, 1), vec_block,
                           inputs + [scratch, ctypes.c_size_t(outer), ctypes.c_size_t(inner)], stream_handle)
                    # the fold over the slabs is a short serial walk per thread: one warp per CTA spreads it over more SMs
                    launch("bb200_reduce_partials_cols_vec", native.U3(-(-(inner // partial_vec) // 32), 1, 1), native.U3(32, 1, 1),
                           [scratch] + dst + [ctypes.c_size_t(vec_slabs), ctypes.c_size_t(inner), init], stream_handle)
            else:
                columns = native.U3(-(-inner // threads), slabs, 1)
                if slabs == 1:
                    launch("bb200_reduce_cols", columns, block, inputs + dst + [ctypes.c_size_t(outer), ctypes.c_size_t(inner), init],
                           stream_handle)
                else:
                    launch("bb200_reduce_cols_partial", columns, block, inputs + [scratch, ctypes.c_size_t(outer), ctypes.c_size_t(inner)],
                           stream_handle)
                    launch("bb200_reduce_partials_cols", native.U3(-(-inner // threads), 1, 1), block,
                           [scratch] + dst + [ctypes.c_size_t(slabs), ctypes.c_size_t(inner), init], stream_handle)

        return run

    def _rmsnorm_runner(self, ir, plan: RmsNormPlan, record, state):
        code = native.DTYPE_CODES[plan.dtype]

        def run(pointers, scalars, stream_handle) -> None:
            native.call("bb200_rmsnorm", code, pointers[plan.x], pointers[plan.gamma], pointers[plan.out], plan.rows,
                        plan.hidden, 1 if plan.gamma_is_full else 0, plan.epsilon, stream_handle)

        return run

    def _layernorm_runner(self, ir, plan: LayerNormPlan, record, state):
        code = native.DTYPE_CODES[plan.dtype]

        def run(pointers, scalars, stream_handle) -> None:
            native.call("bb200_layernorm", code, pointers[plan.x], pointers[plan.residual], pointers[plan.weight],
                        pointers[plan.bias], pointers[plan.out], pointers[plan.out_resid], plan.rows, plan.hidden,
                        1 if plan.weight_is_full else 0, 1 if plan.bias_is_full else 0, plan.epsilon, stream_handle)

        return run

    def _gemm_runner(self, ir, plan: GemmPlan, record, state):
        c_code = native.DTYPE_CODES[plan.c_dtype]

        def run(pointers, scalars, stream_handle) -> None:
            native.call("bb200_gemm_bf16", pointers[plan.a], pointers[plan.b], pointers[plan.c], plan.m, plan.n, plan.k,
                        int(plan.transpose_a), int(plan.transpose_b), c_code, stream_handle)

        return run

    def _attention_runner(self, ir, plan: AttentionPlan, record, state):
        def run(pointers, scalars, stream_handle) -> None:
            native.call("bb200_attention_fwd", pointers[plan.q], pointers[plan.k], pointers[plan.v], pointers[plan.out],
                        pointers[plan.lse], plan.batch, plan.seq, plan.heads, plan.kv_heads, plan.head_dim,
                        int(plan.causal), stream_handle)

        return run


def install_into_upstream(module: Any = None) -> None:
    """Register ``"b200"`` inside an importable upstream ``baybridge`` package.

    Upstream resolves backend names with a hard-coded chain (``compiler.py:127-162``); this wraps
    that resolver so ``baybridge.compile(kernel, ..., backend="b200", target=NvidiaTarget("sm_100a"))``
    returns an artifact that launches through this backend.  Idempotent.
    """
    if module is None:
        import importlib

        module = importlib.import_module("baybridge")
    compiler = module.compiler if hasattr(module, "compiler") else __import__("baybridge.compiler", fromlist=["compiler"])
    original = compiler._resolve_backend
    if getattr(original, "_bb200_installed", False):
        return

    def resolve(backend):
        if backend == "b200":
            return "b200", B200Backend()
        return original(backend)

    resolve._bb200_installed = True  # type: ignore[attr-defined]
    compiler._resolve_backend = resolve
