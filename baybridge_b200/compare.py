"""Compile one kernel on several backends, optionally execute it, and print a JSON summary.

    python -m baybridge_b200.compare <module-or-path.py> <kernel symbol> [--sample-factory NAME]
        [--backends b200,portable] [--execute] [--repeat N] [--include-env] [--cache-dir DIR] [--target sm_100a]

Output keys follow upstream's ``tools/compare_backends.py:255-397`` (``backend``, ``status``,
``resolved_backend``, ``target``, ``lowered_path``, ``dialect``, ``execute_status``, ``timings_ms``, ``cold_ms``,
``warm_median_ms``, ``warm_timings_ms``: first run = cold, median of the rest = warm, host clock around
``artifact(*args)``) so rows from either tool sit side by side; ``b200`` is the executable backend here.
The sample factory returns the sample/run arguments (a sequence, or ``{"run_args": [...], "result_indices": [...]}``)
and may accept ``backend_name=`` / ``target=`` keywords.
"""
from __future__ import annotations

import argparse
import importlib
import importlib.util
import inspect
import json
import platform
import statistics
import sys
import time
from pathlib import Path
from typing import Any

EXECUTABLE_BACKENDS = frozenset({"b200"})


def _load_module(reference: str):
    path = Path(reference)
    if path.suffix == ".py" and path.exists():
        spec = importlib.util.spec_from_file_location(path.stem, path)
        module = importlib.util.module_from_spec(spec)
        sys.modules[path.stem] = module
        spec.loader.exec_module(module)
        return module
    return importlib.import_module(reference)


def _call_factory(factory, **context: Any) -> Any:
    accepted = inspect.signature(factory).parameters
    return factory(**{name: value for name, value in context.items() if name in accepted})


def _payload(factory, **context: Any) -> dict[str, Any]:
    produced = _call_factory(factory, **context)
    if isinstance(produced, dict):
        return {"run_args": tuple(produced["run_args"]), "result_indices": produced.get("result_indices")}
    return {"run_args": tuple(produced), "result_indices": None}


def summarize_timings_ms(timings: list[float]) -> dict[str, Any]:
    if not timings:
        return {"cold_ms": 0.0, "warm_median_ms": 0.0, "warm_timings_ms": []}
    warm = timings[1:] if len(timings) > 1 else list(timings)
    return {"cold_ms": float(timings[0]), "warm_timings_ms": warm, "warm_median_ms": float(statistics.median(warm))}


def _summarize(value: Any) -> Any:
    if hasattr(value, "shape") and hasattr(value, "dtype"):
        summary = {"type": type(value).__name__, "shape": tuple(int(d) for d in value.shape), "dtype": str(value.dtype)}
        if hasattr(value, "float") and hasattr(value, "sum"):  # device tensor: a checksum instead of every element
            summary["sum"] = float(value.float().sum().item())
        elif hasattr(value, "tolist"):
            summary["value"] = value.tolist()
        return summary
    return value


def _synchronizer(run_args):
    for value in run_args:
        if type(value).__module__.startswith("torch") and getattr(value, "is_cuda", False):
            import torch

            return torch.cuda.synchronize
    return None


def environment(target: str | None, backends: tuple[str, ...]) -> dict[str, Any]:
    import baybridge_b200
    from baybridge_b200.backend import native

    info: dict[str, Any] = {
        "python": platform.python_version(), "platform": platform.platform(), "package": baybridge_b200.__version__,
        "target": target, "backends": list(backends), "device_available": native.device_available(),
    }
    try:
        import ctypes

        record = native.DeviceInfo()
        if native.library().bb200_device_info_get(0, ctypes.byref(record)) == 0:
            info["device"] = {"name": record.name.decode(), "sm_count": record.sm_count, "cc": f"{record.cc_major}.{record.cc_minor}"}
    except Exception:  # no driver: the fields above already say so
        pass
    return info


def main(argv: list[str] | None = None) -> int:
    parser = argparse.ArgumentParser(description="Compile a kernel across backends and print a JSON summary.")
    parser.add_argument("module")
    parser.add_argument("symbol")
    parser.add_argument("--sample-factory", default=None)
    parser.add_argument("--backends", default="b200,portable")
    parser.add_argument("--execute", action="store_true")
    parser.add_argument("--repeat", type=int, default=1)
    parser.add_argument("--include-env", action="store_true")
    parser.add_argument("--cache-dir", default=None)
    parser.add_argument("--target", default="sm_100a")
    args = parser.parse_args(argv)
    if args.repeat < 1:
        raise SystemExit("--repeat must be >= 1")
    import baybridge_b200 as cute

    module = _load_module(args.module)
    kernel = getattr(module, args.symbol)
    factory = getattr(module, args.sample_factory) if args.sample_factory else None
    target = cute.NvidiaTarget(sm=args.target) if args.target else None
    names = tuple(item.strip() for item in args.backends.split(",") if item.strip())
    results: list[dict[str, Any]] = []
    for name in names:
        samples = _payload(factory, backend_name=name, target=target)["run_args"] if factory else ()
        try:
            artifact = cute.compile(kernel, *samples, target=target, backend=name, cache_dir=args.cache_dir)
        except Exception as exc:
            results.append({"backend": name, "status": "error", "error_type": type(exc).__name__, "error": str(exc)})
            continue
        entry: dict[str, Any] = {
            "backend": name, "status": "ok", "resolved_backend": artifact.backend_name, "target": artifact.target.arch,
            "lowered_path": str(artifact.lowered_path) if artifact.lowered_path else None, "debug_bundle_dir": None,
            "dialect": artifact.lowered_module.dialect if artifact.lowered_module else None, "from_cache": artifact.from_cache,
        }
        results.append(entry)
        if not args.execute:
            continue
        if factory is None:
            entry["execute_status"] = "skipped_no_sample_factory"
            continue
        if artifact.backend_name not in EXECUTABLE_BACKENDS:
            entry["execute_status"] = "skipped_non_exec_backend"
            continue
        try:
            payload = _payload(factory, backend_name=artifact.backend_name, target=target)
            run_args = payload["run_args"]
            synchronize = _synchronizer(run_args)
            timings: list[float] = []
            for _ in range(args.repeat):
                if synchronize:
                    synchronize()
                started = time.perf_counter()
                artifact(*run_args)
                if synchronize:
                    synchronize()
                timings.append((time.perf_counter() - started) * 1000.0)
            indices = payload["result_indices"]
            if indices is None:
                indices = tuple(i for i, value in enumerate(run_args) if hasattr(value, "shape"))
            entry.update(execute_status="ok", timings_ms=timings, **summarize_timings_ms(timings))
            entry["result_summaries"] = {str(i): _summarize(run_args[i]) for i in indices}
        except Exception as exc:
            entry.update(execute_status="error", execute_error_type=type(exc).__name__, execute_error=str(exc))
    payload_out: Any = {"environment": environment(args.target, names), "results": results} if args.include_env else results
    json.dump(payload_out, sys.stdout, indent=2, sort_keys=True, default=str)
    sys.stdout.write("\n")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
