"""ctypes binding of ``libb200ops.so`` (the C ABI declared in ``include/b200ops.h``).

The library is the only execution path: if it cannot be built or loaded the
import of :func:`lib` raises -- there is no CPU or Triton fallback behind it
(the reference states the same rule for compiler devices: "unsupported =>
explicit error", ops/harness/compiler_api/AGENT_GUIDE.md:255-256).
"""
from __future__ import annotations

import ctypes
import threading
from ctypes import (POINTER, Structure, c_char, c_char_p, c_double, c_float, c_int, c_int32,
                    c_int64, c_size_t, c_uint32, c_void_p)

import numpy as np

ABI_VERSION = 1

# enum b200_status (a100c/runtime/a100rt.h:49-55 numbering for 0..6)
OK, USAGE, REJECTED, RESOURCE, REPEAT_MISMATCH, SYNC, TIMEOUT, UNSUPPORTED = 0, 2, 3, 4, 5, 6, 7, 8

# enum b200_dtype (a100c/runtime/a100rt.h:58-72 numbering)
DTYPE_CODES = {
    "bool": 1, "int8": 2, "uint8": 3, "int16": 4, "uint16": 5, "int32": 6, "uint32": 7,
    "int64": 8, "uint64": 9, "float16": 10, "bfloat16": 11, "float32": 12, "float64": 13,
}
DTYPE_SIZES = {
    "bool": 1, "int8": 1, "uint8": 1, "int16": 2, "uint16": 2, "int32": 4, "uint32": 4,
    "int64": 8, "uint64": 8, "float16": 2, "bfloat16": 2, "float32": 4, "float64": 8,
}

ACT_NONE, ACT_GELU_ERF, ACT_GELU_TANH, ACT_LEAKY_RELU, ACT_SWIGLU = 0, 1, 2, 3, 4
MASK_NONE, MASK_CAUSAL_MOD = 0, 1
EW_GELU_ERF, EW_ADD_GELU_ERF, EW_GEGLU_TANH, EW_BIAS_SCALE_CLAMP_GELU = 1, 2, 3, 4


class Tensor(Structure):
    """``struct b200_tensor``."""
    _fields_ = [("data", c_void_p), ("shape", c_int64 * 4), ("stride", c_int64 * 4),
                ("dtype", c_uint32), ("ndim", c_uint32)]


class DeviceProps(Structure):
    """``struct b200_device_props``."""
    _fields_ = [("name", c_char * 64), ("cc_major", c_int32), ("cc_minor", c_int32),
                ("sm_count", c_int32), ("l2_bytes", c_int32), ("hbm_bytes", c_int64),
                ("smem_per_block_optin", c_int32), ("clock_khz", c_int32)]


assert ctypes.sizeof(Tensor) == 80, "b200_tensor layout pin (include/b200ops.h)"
assert ctypes.sizeof(DeviceProps) == 96, "b200_device_props layout pin"


class B200Error(RuntimeError):
    """A non-OK status from the library."""

    def __init__(self, status: int, text: str, detail: str):
        super().__init__(f"b200 status {status} ({text}): {detail}")
        self.status = status
        self.detail = detail


# Every exported symbol with its prototype.  tests/test_abi.py checks this
# table against the header.
_PTR = c_void_p
_T = POINTER(Tensor)
PROTOTYPES = {
    "b200_abi_version": (c_int, []),
    "b200_status_string": (c_char_p, [c_int]),
    "b200_last_error": (c_char_p, []),
    "b200_device_query": (c_int, [c_int, POINTER(DeviceProps)]),
    "b200_set_device": (c_int, [c_int]),
    "b200_last_device_status": (c_int, [_PTR]),
    "b200_malloc": (c_int, [POINTER(_PTR), c_size_t]),
    "b200_free": (c_int, [_PTR]),
    "b200_malloc_host": (c_int, [POINTER(_PTR), c_size_t]),
    "b200_free_host": (c_int, [_PTR]),
    "b200_memcpy_h2d": (c_int, [_PTR, _PTR, c_size_t, _PTR]),
    "b200_memcpy_d2h": (c_int, [_PTR, _PTR, c_size_t, _PTR]),
    "b200_memcpy_d2d": (c_int, [_PTR, _PTR, c_size_t, _PTR]),
    "b200_memset": (c_int, [_PTR, c_int, c_size_t, _PTR]),
    "b200_stream_create": (c_int, [POINTER(_PTR)]),
    "b200_stream_destroy": (c_int, [_PTR]),
    "b200_stream_sync": (c_int, [_PTR]),
    "b200_device_sync": (c_int, []),
    "b200_event_create": (c_int, [POINTER(_PTR)]),
    "b200_event_destroy": (c_int, [_PTR]),
    "b200_event_record": (c_int, [_PTR, _PTR]),
    "b200_event_elapsed_ms": (c_int, [_PTR, _PTR, POINTER(c_float)]),
    "b200_rmsnorm_fwd": (c_int, [_T, _T, _T, _T, c_float, _PTR]),
    "b200_rmsnorm_fwd_ex": (c_int, [_T, _T, _T, _T, c_float, c_float, _PTR]),
    "b200_softmax_fwd": (c_int, [_T, _T, c_int, c_int64, _PTR]),
    "b200_softmax_variant": (c_int, [_T, _T, _T, c_int, _PTR]),
    "b200_repeat_log_softmax": (c_int, [_T, _T, c_int, _PTR]),
    "b200_elementwise": (c_int, [c_int, _T, _T, _T, c_float, c_float, c_float, _PTR]),
    "b200_gemm_bias_act": (c_int, [_T, _T, _T, _T, _T, c_int, _PTR]),
    "b200_linear_bias_act": (c_int, [_T, _T, _T, _T, c_int, _PTR]),
    "b200_gemm_scatter_rows": (c_int, [_T, _T, _T, POINTER(_PTR), c_int, c_int, c_int64, _PTR]),
    "b200_reduce_slices_broadcast": (c_int, [_PTR, c_uint32, c_uint32, c_int, c_int64, c_int64,
                                             c_int64, POINTER(_PTR), _PTR]),
    "b200_multimem_allreduce": (c_int, [_PTR, c_uint32, _PTR, c_uint32, c_int64, c_int64, c_int,
                                        c_int, POINTER(_PTR), c_uint32, c_int, _PTR]),
    "b200_signal_pad_bytes": (c_size_t, []),
    "b200_peer_allreduce": (c_int, [POINTER(_PTR), c_uint32, POINTER(_PTR), c_uint32, c_int64,
                                    c_int64, c_int, c_int, POINTER(_PTR), c_uint32, c_int, _PTR]),
    "b200_gemm_progress": (c_int, [_T, _T, _T, c_int64, _PTR, POINTER(c_uint32), c_int,
                                   POINTER(c_int), _PTR]),
    "b200_peer_allreduce_blocks": (c_int, [POINTER(_PTR), c_uint32, POINTER(_PTR), c_uint32,
                                           c_int64, c_int64, _PTR, POINTER(c_uint32), c_int,
                                           c_int, POINTER(_PTR), c_uint32, c_int, _PTR]),
    "b200_multimem_allreduce_blocks": (c_int, [_PTR, c_uint32, _PTR, c_uint32, c_int64, c_int64,
                                               _PTR, POINTER(c_uint32), c_int, c_int,
                                               POINTER(_PTR), c_uint32, c_int, _PTR]),
    "b200_progress_words": (c_int, []),
    "b200_attn_fwd": (c_int, [_T, _T, _T, _T, _T, c_float, c_int, _PTR]),
    "b200_attn_fwd_modes": (c_int, [_T, _T, _T, _T, _T, c_float, c_int, c_float, _T, c_int, c_int,
                                    _T, c_int, c_int64, _PTR]),
    "b200_stream_wait_event": (c_int, [_PTR, _PTR]),
    "b200_graph_begin_capture": (c_int, [_PTR]),
    "b200_graph_end_capture": (c_int, [_PTR, POINTER(c_void_p)]),
    "b200_graph_launch": (c_int, [_PTR, _PTR]),
    "b200_graph_destroy": (c_int, [_PTR]),
    "b200_wait_selftest": (c_int, [POINTER(c_uint32), _PTR]),
    "b200_attn_window_fwd": (c_int, [_T, _T, _T, _T, _T, _T, _T, c_float, c_int, _PTR]),
    "b200_attn_decode": (c_int, [_T, _T, _T, _T, c_float, _PTR]),
    "b200_linear_log_softmax": (c_int, [_T, _T, _T, _PTR]),
    "b200_gemm_groupnorm_rowmin": (c_int, [_T, _T, _T, _T, _T, _T, c_int, c_float, _PTR]),
    "b200_dequantize_cols": (c_int, [_T, _T, _T, _PTR]),
    "b200_rms_matmul": (c_int, [_T, _T, _T, _T, c_float, _T, _T, _PTR]),
    "b200_swiglu_fwd": (c_int, [_T, _T, _T, _PTR]),
    "b200_allclose_f32": (c_int, [_PTR, _PTR, c_int64, c_double, c_double, c_int,
                                  POINTER(c_int64), POINTER(c_double), _PTR]),
    "b200_allclose_f32_static": (c_int, [_PTR, _PTR, c_int64, c_double, c_double, c_int,
                                         POINTER(c_int64), POINTER(c_double), _PTR]),
    "b200_bitwise_equal": (c_int, [_PTR, _PTR, c_size_t, POINTER(c_int), _PTR]),
}

_lock = threading.Lock()
_lib = None


class _Recorder:
    """Stands in for the library while a launch is being recorded: every entry point called
    through it runs as usual and is logged with its (ctypes) arguments."""

    def __init__(self, real):
        self._real = real
        self.calls = []

    def __getattr__(self, name):
        fn = getattr(self._real, name)

        def call(*args):
            self.calls.append((fn, args))
            return fn(*args)
        return call


_recorder = None


class recording:  # noqa: N801 - used as ``with abi.recording() as plan:``
    """Log the library calls made inside the block.  ``plan.calls`` can be replayed with
    :func:`replay` as long as the buffers the calls point at are alive and unmoved: the
    descriptors are kept by the log, the device memory they name is not.  One recording at a
    time, on the thread that launches."""

    def __enter__(self):
        global _recorder
        if _recorder is not None:
            raise RuntimeError("a launch recording is already open")
        _recorder = _Recorder(lib())
        return _recorder

    def __exit__(self, *exc):
        global _recorder
        _recorder = None
        return False


def replay(calls) -> None:
    """Issue recorded library calls again, checking every status."""
    for fn, args in calls:
        check(fn(*args))


def lib() -> ctypes.CDLL:
    """Build (if stale) and load the library; raises when that is impossible."""
    global _lib
    if _recorder is not None:
        return _recorder
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        from compiler_b200 import build as _build
        path = _build.LIB_PATH
        if not _build.is_current():
            try:
                path = _build.build()
            except Exception as exc:  # noqa: BLE001
                if not path.is_file():
                    raise RuntimeError(
                        "libb200ops.so is missing and cannot be built here "
                        f"({exc}); there is no fallback execution path") from exc
        handle = ctypes.CDLL(str(path))
        for name, (restype, argtypes) in PROTOTYPES.items():
            fn = getattr(handle, name)  # AttributeError => the library is not this ABI
            fn.restype = restype
            fn.argtypes = argtypes
        if handle.b200_abi_version() != ABI_VERSION:
            raise RuntimeError("libb200ops.so ABI version mismatch")
        _lib = handle
    return _lib


def check(status: int) -> None:
    """Raise :class:`B200Error` for a non-OK status."""
    if status != OK:
        handle = lib()
        raise B200Error(status, handle.b200_status_string(status).decode(),
                        handle.b200_last_error().decode(errors="replace"))


def dtype_name(dtype) -> str:
    """Plain type name of a numpy dtype / torch dtype / str ("torch.float16" -> "float16")."""
    if isinstance(dtype, str):
        return dtype.rsplit(".", 1)[-1]
    try:
        return np.dtype(dtype).name
    except TypeError:
        return str(dtype).rsplit(".", 1)[-1]


def make_tensor(ptr: int, shape, dtype, strides=None) -> Tensor:
    """Descriptor for a device buffer; ``strides`` in elements (default: contiguous)."""
    shape = tuple(int(v) for v in shape)
    if len(shape) > 4:
        raise ValueError("b200_tensor holds at most 4 dimensions")
    if strides is None:
        strides, running = [], 1
        for extent in reversed(shape):
            strides.append(running)
            running *= max(extent, 1)
        strides = tuple(reversed(strides))
    name = dtype_name(dtype)
    if name not in DTYPE_CODES:
        raise ValueError(f"no b200 dtype code for {dtype!r}")
    tensor = Tensor()
    tensor.data = int(ptr) if ptr else None
    tensor.ndim = len(shape)
    tensor.dtype = DTYPE_CODES[name]
    for i, (extent, stride) in enumerate(zip(shape, strides)):
        tensor.shape[i] = extent
        tensor.stride[i] = int(stride)
    return tensor
