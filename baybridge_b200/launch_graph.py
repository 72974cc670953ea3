"""Launch graphs: record a fixed sequence of compiled-kernel launches once, replay it with one driver call.

A launch through ``artifact(*handles, stream=...)`` costs about 10 µs of host time (argument checks, one
``cuLaunchKernelEx``), which is all there is to a kernel as small as the 256×256 indexed add.  A loop of such
launches is host-bound; recorded into a CUDA graph, the whole loop is submitted by a single ``cuGraphLaunch`` and the
GPU runs the kernels back to back.  Upstream has nothing comparable (its launchers run and synchronise one kernel at
a time, ``src/baybridge/backends/ptx_exec.py:160-171``).

    graph = LaunchGraph()
    with graph.record() as stream:            # `stream` is the recording stream
        for _ in range(100):
            artifact(a, b, c, stream=stream)  # recorded, not executed
    graph.replay()                             # on the default stream, or replay(stream=...)
    graph.close()

While a graph records, launchers do not synchronise (the default upstream-style synchronise after every launch
would invalidate the recording) and refuse host tensors that would have to be staged.  Pointers and shapes are
baked into the graph: replay reads and writes the same device buffers the recording named.
"""
from __future__ import annotations

import contextlib
import ctypes
from typing import Any, Iterator

from .backend import native


class LaunchGraph:
    def __init__(self) -> None:
        self._graph = ctypes.c_void_p(0)
        self._stream = ctypes.c_void_p(0)

    @contextlib.contextmanager
    def record(self) -> Iterator[int]:
        """Record every launch made on the yielded stream handle (an ``int``) until the block ends."""
        native.require_device()
        if self._graph:
            raise RuntimeError("this LaunchGraph already holds a recording; close() it or make a new one")
        if native.recording():
            raise RuntimeError("another LaunchGraph is recording on this thread")
        if not self._stream:
            native.call("bb200_stream_create", ctypes.byref(self._stream))
        native.call("bb200_graph_capture_begin", self._stream)
        native.set_recording(True)
        try:
            yield int(self._stream.value)
        except BaseException:
            native.set_recording(False)
            discarded = ctypes.c_void_p(0)
            try:  # leave the stream usable: end the recording and drop whatever it holds
                native.call("bb200_graph_capture_end", self._stream, ctypes.byref(discarded))
                if discarded:
                    native.call("bb200_graph_destroy", discarded)
            except Exception:  # noqa: BLE001 - the original error is the one to report
                pass
            raise
        native.set_recording(False)
        native.call("bb200_graph_capture_end", self._stream, ctypes.byref(self._graph))

    def replay(self, *, stream: Any = None) -> None:
        """Submit the recorded launches on ``stream`` (default stream when omitted); asynchronous."""
        if not self._graph:
            raise RuntimeError("nothing has been recorded")
        native.call("bb200_graph_launch", self._graph, native.stream_handle(stream))

    def close(self) -> None:
        if self._graph:
            native.call("bb200_graph_destroy", self._graph)
            self._graph = ctypes.c_void_p(0)
        if self._stream:
            native.call("bb200_stream_destroy", self._stream)
            self._stream = ctypes.c_void_p(0)

    def __del__(self) -> None:  # best effort; close() is the supported way
        try:
            self.close()
        except Exception:  # noqa: BLE001
            pass
