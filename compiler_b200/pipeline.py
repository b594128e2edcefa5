"""Host-to-host execution of row-wise operators with the copies overlapped.

A caller that holds its data in (pinned) host memory pays three serial costs per call:
host->device copy, kernel, device->host copy.  Rows are independent, so the rows are cut into
chunks: while chunk i's result travels back over PCIe, chunk i+1's kernel runs and chunk
i+2's input travels in.  PCIe is full duplex, so the two copy directions overlap and the
end-to-end time approaches max(H2D, D2H) + one chunk instead of their sum.

Two schedules.  Default: whole chunks (copy, kernel, copy) round-robin over ``streams``
streams; a stream's next inbound copy waits for its previous outbound one, so the two
directions move in step.  ``staged=True``: one stream per STAGE -- every host->device copy on
the first, back to back; every kernel on the second, each after the event of its chunk's
copy; every device->host copy on the third, each after the event of its chunk's kernel.
Measured on a B200 (131 MB each way, 8 chunks): 3.12 ms in step, 3.28 ms staged -- with the
inbound direction never idle the outbound copies get the smaller share of the link and end
later; both directions at once with no kernel take 2.65 ms (49.5 GB/s each, against 55 / 57
one at a time), and every further chunk costs about 27 us of hand-overs between the copy
engines and the SMs (16 chunks: 3.6 ms, 64: 4.8 ms).

``direct=True`` drops both staging copies: page-locked host memory is addressable from the
device, so ONE launch reads its input rows straight from the caller's buffer and stores its
results straight into the caller's buffer, and only what it loads crosses PCIe inbound -- a
masked softmax row loads its kept columns and nothing else, half the tensor on average.
Measured: 2.90 ms (the SMs write host memory at 51.7 GB/s alone, the copy engine at 56.9, and
the read requests of the loads share the outbound direction with the stores).  Mixing the two
-- direct loads with the copy engine taking the results out chunk by chunk -- measured worse
than either (3.22-3.65 ms for 2 to 32 chunks): the copy engine's stores slow down beside the
SMs' read requests by more than the saved inbound bytes give back.
The device buffers, streams and events are created once and reused.
"""
from __future__ import annotations

import ctypes

import numpy as np

from compiler_b200 import ops, shard
from compiler_b200.device import B200Buffer, PinnedArray
from compiler_b200.runtime import abi


class RowPipeline:
    """Pipelined ``host rows -> operator -> host rows`` for one [rows, cols] shape."""

    def __init__(self, device, rows: int, cols: int, dtype, chunks: int = 8, streams: int = 3,
                 staged: bool = False, direct: bool = False):
        self.device = device
        self.direct = bool(direct)
        self.staged = bool(staged) and not self.direct
        self.rows, self.cols = int(rows), int(cols)
        self.dtype = abi.dtype_name(dtype)
        self.itemsize = abi.DTYPE_SIZES[self.dtype]
        self.chunks = shard.row_chunks(self.rows, 1 if self.direct else chunks)
        lib = abi.lib()
        self._streams = []
        for _ in range(3 if self.staged else max(1, min(streams, len(self.chunks)))):
            handle = ctypes.c_void_p()
            abi.check(lib.b200_stream_create(ctypes.byref(handle)))
            self._streams.append(handle)
        self._events = []            # staged: (copied in, computed) per chunk
        for _ in range(2 * len(self.chunks) if self.staged else 0):
            handle = ctypes.c_void_p()
            abi.check(lib.b200_event_create(ctypes.byref(handle)))
            self._events.append(handle)
        self.x = self.y = None
        if not self.direct:
            self.x = device.alloc((self.rows, self.cols), self.dtype)
            self.y = device.alloc((self.rows, self.cols), self.dtype)

    def _view(self, buffer: B200Buffer, lo: int, hi: int) -> B200Buffer:
        offset = lo * self.cols * self.itemsize
        return B200Buffer(buffer.ptr + offset, self.dtype, (hi - lo, self.cols),
                          (hi - lo) * self.cols * self.itemsize, owner=False, base=buffer)

    def run(self, launch, host_in: PinnedArray, host_out: PinnedArray) -> np.ndarray:
        """``launch(x_chunk, y_chunk, first_row, stream)`` enqueues the operator for one chunk.
        Returns ``host_out.array`` after every chunk has landed."""
        lib = abi.lib()
        row_bytes = self.cols * self.itemsize
        if self.staged:
            inbound, compute, outbound = self._streams
            for i, (lo, hi) in enumerate(self.chunks):
                copied, computed = self._events[2 * i], self._events[2 * i + 1]
                nbytes = (hi - lo) * row_bytes
                abi.check(lib.b200_memcpy_h2d(self.x.ptr + lo * row_bytes,
                                              host_in.ptr + lo * row_bytes, nbytes, inbound))
                abi.check(lib.b200_event_record(copied, inbound))
                abi.check(lib.b200_stream_wait_event(compute, copied))
                launch(self._view(self.x, lo, hi), self._view(self.y, lo, hi), lo, compute.value)
                abi.check(lib.b200_event_record(computed, compute))
                abi.check(lib.b200_stream_wait_event(outbound, computed))
                abi.check(lib.b200_memcpy_d2h(host_out.ptr + lo * row_bytes,
                                              self.y.ptr + lo * row_bytes, nbytes, outbound))
            # the outbound stream ends after everything it waited for
            abi.check(lib.b200_stream_sync(outbound))
            return host_out.array
        if self.direct:
            nbytes = self.rows * row_bytes
            shape = (self.rows, self.cols)
            launch(B200Buffer(host_in.ptr, self.dtype, shape, nbytes, owner=False),
                   B200Buffer(host_out.ptr, self.dtype, shape, nbytes, owner=False), 0,
                   self._streams[0].value)
            abi.check(lib.b200_stream_sync(self._streams[0]))
            return host_out.array
        for i, (lo, hi) in enumerate(self.chunks):
            stream = self._streams[i % len(self._streams)]
            nbytes = (hi - lo) * row_bytes
            abi.check(lib.b200_memcpy_h2d(self.x.ptr + lo * row_bytes,
                                          host_in.ptr + lo * row_bytes, nbytes, stream))
            launch(self._view(self.x, lo, hi), self._view(self.y, lo, hi), lo, stream.value)
            abi.check(lib.b200_memcpy_d2h(host_out.ptr + lo * row_bytes,
                                          self.y.ptr + lo * row_bytes, nbytes, stream))
        for stream in self._streams:
            abi.check(lib.b200_stream_sync(stream))
        return host_out.array

    def close(self):
        lib = abi.lib()
        for stream in self._streams:
            lib.b200_stream_destroy(stream)
        self._streams = []
        for event in self._events:
            lib.b200_event_destroy(event)
        self._events = []
        if self.x is not None:
            self.device.release({"x": self.x, "y": self.y})
            self.x = self.y = None


def masked_softmax_host(pipeline: RowPipeline, host_in: PinnedArray, host_out: PinnedArray,
                        row_offset: int = 0) -> np.ndarray:
    """Masked row softmax from pinned host rows to pinned host rows."""
    def launch(x, y, first_row, stream):
        ops.softmax(x, y, causal_mod=True, row_offset=row_offset + first_row, stream=stream)
    return pipeline.run(launch, host_in, host_out)
