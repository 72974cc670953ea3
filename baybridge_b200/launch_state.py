"""Process-wide launch state shared by the argument marshalling and the launchers (no imports, so either may use it)."""
from __future__ import annotations

_recording = False


def recording() -> bool:
    """True while a launch graph records: launchers must not synchronise, and DLPack exporters must not be asked to
    order themselves against the recording stream (that would record a wait on work outside the graph)."""
    return _recording


def set_recording(value: bool) -> None:
    global _recording
    _recording = bool(value)
