"""Captured launch sequences (CUDA graphs) over the C ABI.

A loop of short kernels pays the host's launch latency once per kernel; recorded once and
replayed, the whole sequence costs one call::

    stream = graph.Stream()
    ops.softmax(x, y, stream=stream.handle)          # every operator once, outside the capture
    with graph.capture(stream) as g:
        for i in range(100):
            ops.softmax(xs[i % 4], ys[i % 4], stream=stream.handle)
    g.launch(stream)                                  # 100 kernels, one call
    stream.synchronize()

Only launches and asynchronous copies on the capturing stream (or on streams joined to it by
events) are recorded; anything that synchronises raises from the library.
"""
from __future__ import annotations

import ctypes
from contextlib import contextmanager

from compiler_b200.runtime import abi


class Stream:
    """A non-blocking stream owned by this object (``handle`` is the raw ``cudaStream_t``)."""

    def __init__(self):
        out = ctypes.c_void_p()
        abi.check(abi.lib().b200_stream_create(ctypes.byref(out)))
        self._ptr = out
        self.handle = out.value

    def synchronize(self):
        abi.check(abi.lib().b200_stream_sync(self._ptr))

    def close(self):
        if self._ptr is not None:
            abi.lib().b200_stream_destroy(self._ptr)
            self._ptr, self.handle = None, None

    def __del__(self):
        try:
            self.close()
        except Exception:  # noqa: BLE001 - interpreter shutdown
            pass


class Graph:
    """An instantiated graph: ``launch(stream)`` replays the recorded sequence."""

    def __init__(self):
        self._exec = None

    def launch(self, stream: Stream) -> None:
        if self._exec is None:
            raise RuntimeError("the capture has not finished")
        abi.check(abi.lib().b200_graph_launch(self._exec, stream._ptr))

    def close(self):
        if self._exec is not None:
            abi.lib().b200_graph_destroy(self._exec)
            self._exec = None

    def __del__(self):
        try:
            self.close()
        except Exception:  # noqa: BLE001
            pass


@contextmanager
def capture(stream: Stream):
    """Record what the block enqueues on ``stream``; yields the :class:`Graph` that is ready
    when the block ends.  If the block raises, the capture is closed and discarded."""
    lib = abi.lib()
    abi.check(lib.b200_graph_begin_capture(stream._ptr))
    graph = Graph()
    try:
        yield graph
    except BaseException:
        out = ctypes.c_void_p()
        if lib.b200_graph_end_capture(stream._ptr, ctypes.byref(out)) == abi.OK and out.value:
            lib.b200_graph_destroy(out)
        raise
    out = ctypes.c_void_p()
    abi.check(lib.b200_graph_end_capture(stream._ptr, ctypes.byref(out)))
    graph._exec = out
