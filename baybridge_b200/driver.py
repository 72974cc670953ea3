"""``compile()``: trace → resolve backend → lower → cache → build launcher.

Follows the control flow of upstream ``compiler.py:624-701`` (and the launch
wrapper re-trace of ``:373-402``) with these deliberate differences:

* the backend registry is a real table (``register_backend``) instead of an
  if-chain (``compiler.py:127-162``); ``"b200"`` and ``"portable"`` are
  registered, any object with ``name`` + ``lower`` is accepted as-is;
* the default target is ``NvidiaTarget("sm_100a")`` and the default backend is
  ``b200``;
* an artifact whose backend has no launcher raises when called: there is no
  CPU runtime to fall back to.

The cache key is the same sha256 over ``{backend_name, ir, mode, target}``
(``compiler.py:522-533``) so keys computed here equal upstream's for the same
kernel; manifests live at ``<cache>/<backend>/<arch>/<key>.json``.
"""
from __future__ import annotations

import hashlib
import inspect
import json
import os
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Callable

from .errors import BackendNotImplementedError, CompilationError
from .host_values import TensorHandle, infer_runtime_spec, normalize_runtime_argument
from .portable_ir import PortableKernelIR, ScalarSpec, TensorSpec
from .targets import B200, AMDTarget, NvidiaTarget
from .trace import IRBuilder, ScalarValue, TensorValue, tracing

CACHE_ENV = "BAYBRIDGE_CACHE_DIR"
DEFAULT_BACKEND = "b200"


@dataclass(frozen=True)
class LoweredModule:
    backend_name: str
    entry_point: str
    dialect: str
    text: str

    def to_dict(self) -> dict[str, Any]:
        return {"backend_name": self.backend_name, "entry_point": self.entry_point, "dialect": self.dialect, "text": self.text}


@dataclass(frozen=True)
class GenerateLineInfo:
    """Accepted compile option (``compile[GenerateLineInfo()](...)``); b200 kernels always carry line info."""

    enabled: bool = True


# ---------------------------------------------------------------------------------------------
# backend registry
# ---------------------------------------------------------------------------------------------
_REGISTRY: dict[str, Callable[[], Any]] = {}


def register_backend(name: str, factory: Callable[[], Any]) -> None:
    """Make ``compile(..., backend=name)`` resolve to ``factory()``; ``None`` factories are IR-only."""
    _REGISTRY[name] = factory


def registered_backends() -> tuple[str, ...]:
    return tuple(sorted(_REGISTRY))


def resolve_backend(backend: Any) -> tuple[str, Any]:
    if backend is None:
        backend = DEFAULT_BACKEND
    if not isinstance(backend, str):
        return backend.name, backend
    if backend not in _REGISTRY:
        raise CompilationError(f"unknown backend '{backend}'")
    return backend, _REGISTRY[backend]()


def _b200_factory():
    from .backend import B200Backend

    return B200Backend()


register_backend("portable", lambda: None)
register_backend("b200", _b200_factory)


# ---------------------------------------------------------------------------------------------
# tracing
# ---------------------------------------------------------------------------------------------
def _normalize_kernel(kernel: Any):
    from .dsl import KernelDefinition
    from .portable_ir import LaunchConfig

    if isinstance(kernel, KernelDefinition):
        return kernel
    if callable(kernel):
        return KernelDefinition(fn=kernel, kind="kernel", launch=LaunchConfig())
    raise CompilationError("compile expects a @kernel/@jit function or a callable")


def _bind_leaf(builder: IRBuilder, bindings: list[dict[str, Any]], parameter: str, leaf: str, spec, path=()):
    bindings.append({"name": leaf, "parameter": parameter, "path": list(path)})
    return builder.bind_argument(leaf, spec)


def _proxy_for(parameter: str, value: Any, builder: IRBuilder, bindings: list[dict[str, Any]], path: tuple = ()) -> Any:
    """Sample argument → trace proxy.  Containers of tensors are walked; each leaf becomes one IR argument."""
    if isinstance(value, (TensorValue, ScalarValue)):
        return value
    dtype, shape = infer_runtime_spec(value)
    if dtype != "python_object":
        spec = ScalarSpec(dtype) if shape is None else TensorSpec(shape=shape, dtype=dtype)
        suffix = "".join("_" + str(item).replace("-", "_") for item in path)
        return _bind_leaf(builder, bindings, parameter, parameter + suffix, spec, path)
    if isinstance(value, (list, tuple)):
        walked = [_proxy_for(parameter, item, builder, bindings, path + (i,)) for i, item in enumerate(value)]
        return walked if isinstance(value, list) else tuple(walked)
    if isinstance(value, dict):
        return {key: _proxy_for(parameter, item, builder, bindings, path + (key,)) for key, item in value.items()}
    return value


def trace(definition, sample_args: tuple[Any, ...] = (), sample_kwargs: dict[str, Any] | None = None) -> PortableKernelIR:
    """Run the kernel body once on proxies and return its IR."""
    from .dsl import TraceKernelLaunch

    signature = inspect.signature(definition.fn)
    supplied = signature.bind_partial(*sample_args, **(sample_kwargs or {})).arguments
    builder = IRBuilder(kernel_name=definition.__name__, launch=definition.launch)
    bindings: list[dict[str, Any]] = []
    positional: list[Any] = []
    keyword: dict[str, Any] = {}
    for name, parameter in signature.parameters.items():
        annotation = parameter.annotation
        if isinstance(annotation, (TensorSpec, ScalarSpec)):
            proxy = _bind_leaf(builder, bindings, name, name, annotation)
        elif name in supplied:
            proxy = _proxy_for(name, supplied[name], builder, bindings)
        elif parameter.default is not inspect.Parameter.empty:
            proxy = parameter.default
        else:
            raise CompilationError(
                f"parameter '{name}' must be annotated with baybridge.TensorSpec(...) or baybridge.ScalarSpec(...), "
                "or compile(...) must be given sample arguments"
            )
        if parameter.kind is inspect.Parameter.KEYWORD_ONLY:
            keyword[name] = proxy
        else:
            positional.append(proxy)
    builder.metadata["trace_bindings"] = bindings
    with tracing(builder):
        try:
            definition.fn(*positional, **keyword)
        except TraceKernelLaunch as launched:
            return _trace_launched(definition, builder, launched)
    builder.metadata["frontend"] = definition.kind
    return builder.finalize()


def _trace_launched(wrapper, wrapper_builder: IRBuilder, launched) -> PortableKernelIR:
    """A @jit wrapper that launches one kernel collapses to that kernel's IR with the wrapper's arguments."""
    builder = IRBuilder(kernel_name=launched.definition.__name__, launch=launched.launch)
    rebound = {argument.name: builder.bind_argument(argument.name, argument.spec) for argument in wrapper_builder.arguments}

    def rehydrate(value: Any) -> Any:
        if isinstance(value, (TensorValue, ScalarValue)):
            if value.name not in rebound:
                kind = "tensor" if isinstance(value, TensorValue) else "scalar"
                raise CompilationError(
                    f"launched kernel captured {kind} '{value.name}' that is not a wrapper argument; "
                    "this trace path is not implemented yet"
                )
            return rebound[value.name]
        if isinstance(value, (list, tuple)):
            return type(value)(rehydrate(item) for item in value)
        if isinstance(value, dict):
            return {key: rehydrate(item) for key, item in value.items()}
        return value

    with tracing(builder):
        launched.definition.fn(*rehydrate(launched.args), **rehydrate(launched.kwargs))
    builder.metadata.update(
        frontend=launched.definition.kind,
        compiled_from="launch_wrapper",
        trace_bindings=list(wrapper_builder.metadata.get("trace_bindings", [])),
        wrapped_by=wrapper.__name__,
        wrapper_frontend=wrapper.kind,
    )
    return builder.finalize()


# ---------------------------------------------------------------------------------------------
# artifacts and the cache
# ---------------------------------------------------------------------------------------------
@dataclass(frozen=True)
class CompiledKernel:
    ir: PortableKernelIR | None
    target: NvidiaTarget | AMDTarget
    backend_name: str
    cache_key: str
    artifact_path: Path
    lowered_path: Path | None
    lowered_module: LoweredModule | None
    debug_bundle_dir: Path | None
    from_cache: bool
    runtime_callable: Callable[..., Any] | None = None

    def __call__(self, *args: Any, **kwargs: Any) -> Any:
        if self.runtime_callable is None:
            raise BackendNotImplementedError(
                f"backend '{self.backend_name}' produced IR only; compile with backend='b200' to get a launchable artifact "
                "(baybridge_b200 has no CPU runtime)"
            )
        stream = kwargs.get("stream") if kwargs else None
        for arg in args:
            if type(arg) is not TensorHandle:
                break
        else:
            # the hot call: device tensor handles only (plus stream=) need no normalisation
            if not kwargs or (len(kwargs) == 1 and "stream" in kwargs):
                return self.runtime_callable(*args, **kwargs)
        args = tuple(normalize_runtime_argument(arg, stream=stream) for arg in args)
        kwargs = {
            name: value if name == "stream" else normalize_runtime_argument(value, stream=stream)
            for name, value in kwargs.items()
        }
        return self.runtime_callable(*args, **kwargs)

    def to_dict(self) -> dict[str, Any]:
        return {
            "backend_name": self.backend_name,
            "cache_key": self.cache_key,
            "target": self.target.to_dict(),
            "ir": self.ir.to_dict() if self.ir else None,
            "lowered_module": self.lowered_module.to_dict() if self.lowered_module else None,
            "debug_bundle_dir": str(self.debug_bundle_dir) if self.debug_bundle_dir else None,
        }


def cache_key_for(ir: PortableKernelIR, target, backend_name: str) -> str:
    payload = {"backend_name": backend_name, "ir": ir.to_dict(), "mode": "traced", "target": target.to_dict()}
    return hashlib.sha256(json.dumps(payload, sort_keys=True).encode("utf-8")).hexdigest()


def default_cache_dir() -> Path:
    configured = os.environ.get(CACHE_ENV)
    return Path(configured).expanduser() if configured else Path.home() / ".cache" / "baybridge"


def _bind_user_arguments(definition, backend_launcher: Callable[..., Any], bindings: list[dict[str, Any]]):
    """User-signature call → IR-argument-order call (leaf extraction by recorded path), forwarding ``stream=``."""
    signature = inspect.signature(definition.fn)

    def pluck(value: Any, path: list[Any]) -> Any:
        for step in path:
            if isinstance(value, dict):
                value = value[step]
            elif isinstance(step, str) and hasattr(value, step):
                value = getattr(value, step)
            else:
                value = value[step]
        return value

    parameters = list(signature.parameters.values())
    positional = [p.name for p in parameters if p.kind in (p.POSITIONAL_ONLY, p.POSITIONAL_OR_KEYWORD)]
    # the common call — every parameter given positionally, each binding a whole parameter — needs no signature binding
    direct = (len(positional) == len(parameters) and "stream" not in signature.parameters
              and all(not binding["path"] and binding["parameter"] in positional for binding in bindings))
    order = [positional.index(binding["parameter"]) for binding in bindings] if direct else []

    def launcher(*args: Any, **kwargs: Any) -> Any:
        if direct and len(args) == len(positional) and (not kwargs or (len(kwargs) == 1 and "stream" in kwargs)):
            stream = kwargs.get("stream") if kwargs else None
            leaves = [args[index] for index in order]
            for leaf in leaves:
                if type(leaf) is not TensorHandle:
                    leaves = [normalize_runtime_argument(value, stream=stream) for value in leaves]
                    break
            return backend_launcher(*leaves) if stream is None else backend_launcher(*leaves, stream=stream)
        stream = None if "stream" in signature.parameters else kwargs.pop("stream", None)
        bound = signature.bind_partial(*args, **kwargs).arguments
        if stream is None and "stream" in bound:
            stream = bound["stream"]
        leaves = [
            normalize_runtime_argument(pluck(bound[binding["parameter"]], binding["path"]), stream=stream)
            for binding in bindings
        ]
        return backend_launcher(*leaves) if stream is None else backend_launcher(*leaves, stream=stream)

    return launcher


def _compile(kernel: Any, *sample_args: Any, target=None, backend: Any = None,
             cache_dir: str | os.PathLike[str] | None = None, use_cache: bool = True) -> CompiledKernel:
    definition = _normalize_kernel(kernel)
    target = target or B200
    cache_root = Path(cache_dir).expanduser() if cache_dir else default_cache_dir()
    samples = tuple(normalize_runtime_argument(arg) for arg in sample_args)
    ir = trace(definition, samples)
    backend_name, backend_object = resolve_backend(backend)
    key = cache_key_for(ir, target, backend_name)
    lowered = backend_object.lower(ir, target) if backend_object is not None else None

    root = cache_root / backend_name / target.arch
    manifest_path = root / f"{key}.json"
    extension = getattr(backend_object, "artifact_extension", ".mlir")
    lowered_path = None if backend_name == "portable" else root / f"{key}{extension}"
    from_cache = use_cache and manifest_path.exists()
    if not from_cache:
        root.mkdir(parents=True, exist_ok=True)
        manifest = {
            "backend_name": backend_name,
            "cache_key": key,
            "target": target.to_dict(),
            "ir": ir.to_dict(),
            "lowered_module": lowered.to_dict() if lowered else None,
        }
        manifest_path.write_text(json.dumps(manifest, indent=2, sort_keys=True) + "\n", encoding="utf-8")
        if lowered is not None and lowered_path is not None:
            lowered_path.write_text(lowered.text, encoding="utf-8")

    bundle = None
    launcher = None
    if lowered is not None and lowered_path is not None:
        if hasattr(backend_object, "emit_bundle"):
            bundle = backend_object.emit_bundle(ir, target, lowered, lowered_path)
        if hasattr(backend_object, "build_launcher"):
            launcher = backend_object.build_launcher(ir, target, lowered, lowered_path)
            bindings = ir.metadata.get("trace_bindings")
            if isinstance(bindings, list) and bindings:
                launcher = _bind_user_arguments(definition, launcher, bindings)
    return CompiledKernel(
        ir=ir, target=target, backend_name=backend_name, cache_key=key, artifact_path=manifest_path,
        lowered_path=lowered_path, lowered_module=lowered, debug_bundle_dir=bundle, from_cache=from_cache,
        runtime_callable=launcher,
    )


class _CompileDispatcher:
    """``compile(...)`` and ``compile[options](...)`` (options are validated, then ignored)."""

    def __call__(self, *args: Any, **kwargs: Any) -> CompiledKernel:
        return _compile(*args, **kwargs)

    def __getitem__(self, options: Any) -> Callable[..., CompiledKernel]:
        for option in options if isinstance(options, tuple) else (options,):
            if not isinstance(option, GenerateLineInfo):
                raise CompilationError(f"unsupported compile option '{type(option).__name__}'")
        return _compile


compile = _CompileDispatcher()


# ---------------------------------------------------------------------------------------------
# eager launches
# ---------------------------------------------------------------------------------------------
_EAGER: dict[tuple, CompiledKernel] = {}


def run_on_device(definition, args: tuple[Any, ...], kwargs: dict[str, Any], stream: Any | None = None) -> None:
    """``kernel(...).launch(...)`` / ``jit_fn(...)`` outside a trace: compile for b200 once per signature, then launch."""
    signature = tuple(infer_runtime_spec(value) for value in args) + tuple(
        (name, infer_runtime_spec(value)) for name, value in sorted(kwargs.items())
    )
    key = (definition.fn, definition.kind, definition.launch, signature)
    artifact = _EAGER.get(key)
    if artifact is None:
        bound = inspect.signature(definition.fn).bind_partial(*args, **kwargs)
        artifact = _EAGER[key] = _compile(definition, *bound.args, backend="b200")
        if bound.kwargs:
            raise CompilationError("eager launches accept keyword-only tensor arguments only through compile(...)")
    if stream is None:
        artifact(*args, **kwargs)
    else:
        artifact(*args, stream=stream, **kwargs)
