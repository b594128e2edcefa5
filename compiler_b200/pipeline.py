"""Host-to-host execution of row-wise operators with the copies overlapped.

A caller that holds its data in (pinned) host memory pays three serial costs per call:
host->device copy, kernel, device->host copy.  Rows are independent, so the rows are cut into
chunks and the chunks are spread over a few streams: while chunk i's result travels back over
PCIe, chunk i+1's kernel runs and chunk i+2's input travels in.  PCIe is full duplex, so the
two copy directions overlap and the end-to-end time approaches max(H2D, D2H) instead of their
sum.  The device buffers and streams are created once and reused.
"""
from __future__ import annotations

import ctypes

import numpy as np

from compiler_b200 import ops, shard
from compiler_b200.device import B200Buffer, PinnedArray
from compiler_b200.runtime import abi


class RowPipeline:
    """Pipelined ``host rows -> operator -> host rows`` for one [rows, cols] shape."""

    def __init__(self, device, rows: int, cols: int, dtype, chunks: int = 8, streams: int = 3):
        self.device = device
        self.rows, self.cols = int(rows), int(cols)
        self.dtype = abi.dtype_name(dtype)
        self.itemsize = abi.DTYPE_SIZES[self.dtype]
        self.chunks = shard.row_chunks(self.rows, chunks)
        lib = abi.lib()
        self._streams = []
        for _ in range(max(1, min(streams, len(self.chunks)))):
            handle = ctypes.c_void_p()
            abi.check(lib.b200_stream_create(ctypes.byref(handle)))
            self._streams.append(handle)
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
        self.device.release({"x": self.x, "y": self.y})


def masked_softmax_host(pipeline: RowPipeline, host_in: PinnedArray, host_out: PinnedArray,
                        row_offset: int = 0) -> np.ndarray:
    """Masked row softmax from pinned host rows to pinned host rows."""
    def launch(x, y, first_row, stream):
        ops.softmax(x, y, causal_mod=True, row_offset=row_offset + first_row, stream=stream)
    return pipeline.run(launch, host_in, host_out)
