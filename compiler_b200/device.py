"""``B200Device``: the ops-harness ``Device`` protocol on top of the C ABI.

Implements the surface of ``ops/harness/opslib/device.py:79-117`` (``alloc`` /
``upload`` / ``download`` / ``pointer`` / ``synchronize`` / ``compare`` /
``launch``) plus the optional hooks the harness probes for (``upload_aliased``
``device.py:397-406``, ``timer`` and ``release`` ``benchmark/run.py:126-168``,
``properties`` ``devices/cuda.py:329-345``).  Memory handling mirrors the
reference CUDA device (``devices/cuda.py:170-262``): raw device allocations,
pinned staging, bf16 uploaded by round-to-nearest-even from float32 hosts and
widened back on download, uint16 hosts treated as bit patterns.

``launch`` never runs Triton: the kernel object is resolved to a native
operator by :mod:`compiler_b200.registry`, and anything unregistered raises
``UnsupportedLaunch``.  The module is torch-free; it needs only numpy and
``libb200ops.so``.
"""
from __future__ import annotations

import ctypes

import numpy as np

from compiler_b200.runtime import abi


class _TypeName(str):
    """dtype marker whose ``str()`` is the plain type name (``"bfloat16"``)."""
    __slots__ = ()

    @property
    def name(self):
        return str(self)


_TYPE_NAMES: dict[str, _TypeName] = {}


def type_name(name) -> _TypeName:
    key = abi.dtype_name(name)
    marker = _TYPE_NAMES.get(key)
    if marker is None:
        marker = _TYPE_NAMES[key] = _TypeName(key)
    return marker


def storage_dtype(name) -> np.dtype:
    """numpy dtype that backs one element on the host (bf16 -> uint16 bits)."""
    key = abi.dtype_name(name)
    return np.dtype("uint16") if key == "bfloat16" else np.dtype(key)


def to_bf16_bits(array: np.ndarray) -> np.ndarray:
    """float32 -> bf16 bit patterns, round to nearest even, NaN kept quiet.

    Same rounding as ``_bf16_host`` (ops/harness/opslib/case.py:214-220)."""
    values = np.ascontiguousarray(array, dtype=np.float32)
    bits = values.view(np.uint32)
    rounded = (bits + np.uint32(0x7FFF) + ((bits >> np.uint32(16)) & np.uint32(1)))
    rounded = np.where(np.isnan(values), bits | np.uint32(0x00400000), rounded)
    return (rounded >> np.uint32(16)).astype(np.uint16)


def from_bf16_bits(bits: np.ndarray) -> np.ndarray:
    """bf16 bit patterns -> float32 (exact)."""
    return (np.ascontiguousarray(bits).astype(np.uint32) << np.uint32(16)).view(np.float32)


class B200Buffer:
    """A raw device allocation (``Buffer`` of ops/harness/opslib/device.py:38-54)."""

    def __init__(self, ptr, dtype, shape, nbytes, host_dtype=None, owner=True, base=None):
        self.ptr = int(ptr)
        self._dtype = type_name(dtype)
        self._shape = tuple(int(v) for v in shape)
        self.nbytes = int(nbytes)
        self.host_dtype = host_dtype
        self._owner = owner
        self._base = base  # keeps the owning allocation alive for views

    def data_ptr(self):
        return self.ptr

    @property
    def dtype(self):
        return self._dtype

    @property
    def shape(self):
        return self._shape

    def free(self):
        if self.ptr and self._owner:
            try:
                abi.lib().b200_free(self.ptr)
            finally:
                self.ptr = 0
        self._base = None

    def __del__(self):  # interpreter teardown may race the CUDA context
        try:
            self.free()
        except Exception:  # noqa: BLE001
            pass


class PinnedArray:
    """A numpy array over page-locked host memory (fast, truly asynchronous copies)."""

    def __init__(self, shape, dtype):
        self.array = None
        dtype = np.dtype(dtype)
        count = int(np.prod(shape, dtype=np.int64)) if len(tuple(shape)) else 1
        self.nbytes = max(1, count * dtype.itemsize)
        out = ctypes.c_void_p()
        abi.check(abi.lib().b200_malloc_host(ctypes.byref(out), self.nbytes))
        self.ptr = out.value
        raw = (ctypes.c_char * self.nbytes).from_address(self.ptr)
        self.array = np.frombuffer(raw, dtype=dtype, count=count).reshape(shape)

    def free(self):
        if getattr(self, "ptr", None):
            self.array = None
            try:
                abi.lib().b200_free_host(self.ptr)
            finally:
                self.ptr = None

    def __del__(self):
        try:
            self.free()
        except Exception:  # noqa: BLE001
            pass


class EventTimer:
    """``with device.timer() as t: launch()`` -> ``t.seconds`` from CUDA events on
    the device's stream (CudaEventTimer, ops/harness/opslib/devices/cuda.py:138-167).
    One timer serves any number of ``with`` blocks; its events live until it is closed
    or collected."""

    def __init__(self, stream=0):
        self._stream = stream
        self._seconds = None
        lib = abi.lib()
        start, stop = ctypes.c_void_p(), ctypes.c_void_p()
        abi.check(lib.b200_event_create(ctypes.byref(start)))
        abi.check(lib.b200_event_create(ctypes.byref(stop)))
        self._start, self._stop = start, stop

    def __enter__(self):
        abi.check(abi.lib().b200_event_record(self._start, self._stream))
        return self

    def __exit__(self, *exc):
        lib = abi.lib()
        abi.check(lib.b200_event_record(self._stop, self._stream))
        ms = ctypes.c_float()
        abi.check(lib.b200_event_elapsed_ms(self._start, self._stop, ctypes.byref(ms)))
        self._seconds = ms.value * 1e-3
        return False

    @property
    def seconds(self):
        if self._seconds is None:
            raise RuntimeError("timer read before its context exited")
        return self._seconds

    def close(self):
        if self._start is not None:
            lib = abi.lib()
            lib.b200_event_destroy(self._start)
            lib.b200_event_destroy(self._stop)
            self._start = self._stop = None

    def __del__(self):
        try:
            self.close()
        except Exception:  # noqa: BLE001 - interpreter shutdown
            pass


def _KEEP(*_objects):  # noqa: N802 - a no-op plan step that only holds references
    return abi.OK


class B200Device:
    """Compiler device for one B200 (``make_device("compiler_b200.device:make_device")``)."""

    name = "b200-native"
    PLAN_LIMIT = 512  # bound launches remembered per device

    def __init__(self, device_id: int = 0, registry=None):
        from compiler_b200 import registry as _registry
        self.device_id = int(device_id)
        self._lib = abi.lib()
        abi.check(self._lib.b200_set_device(self.device_id))
        self.registry = registry if registry is not None else _registry.default_registry()
        self.stream = 0  # launches and copies share the default stream: ordered
        self._pinned = None
        self.launch_count = 0
        self._plans = {}
        self._workspaces = {}

    # ------------------------------------------------------------ lifecycle
    def alloc(self, shape, dtype):
        target = type_name(dtype)
        shape = tuple(int(v) for v in shape)
        count = int(np.prod(shape, dtype=np.int64)) if shape else 1
        nbytes = max(1, count * storage_dtype(target).itemsize)
        out = ctypes.c_void_p()
        abi.check(self._lib.b200_malloc(ctypes.byref(out), nbytes))
        return B200Buffer(out.value, target, shape, nbytes)

    def workspace(self, key, specs):
        """Scratch buffers an operator needs besides its arguments, allocated once per
        ``key`` and kept with the device (``specs`` = ((shape, dtype), ...)).  Launches on one
        device share the device's stream, so they can share the buffers."""
        found = self._workspaces.get(key)
        if found is None:
            if len(self._workspaces) >= 16:  # shapes change: drop the old scratch
                for buffers in self._workspaces.values():
                    for buffer in buffers:
                        buffer.free()
                self._workspaces.clear()
                self._plans.clear()  # recorded launches may point at the freed scratch
            found = self._workspaces[key] = tuple(self.alloc(shape, dtype)
                                                  for shape, dtype in specs)
        return found

    def release(self, buffers):
        """Free staged buffers now (benchmarks call this per entry)."""
        for buffer in buffers.values():
            if isinstance(buffer, B200Buffer):
                buffer.free()

    def pinned_empty(self, shape, dtype) -> PinnedArray:
        return PinnedArray(shape, dtype)

    def _staging(self, nbytes) -> PinnedArray:
        if self._pinned is None or self._pinned.nbytes < nbytes:
            if self._pinned is not None:
                self._pinned.free()
            self._pinned = PinnedArray((nbytes,), np.uint8)
        return self._pinned

    # ------------------------------------------------------------ transfers
    @staticmethod
    def _payload(array, target_name):
        """Host bytes to copy for ``array`` stored as ``target_name`` on the device."""
        storage = storage_dtype(target_name)
        if target_name == "bfloat16":
            if array.dtype == np.uint16:
                return array
            if array.dtype == np.float32:
                return to_bf16_bits(array)
            raise TypeError("bfloat16 upload needs float32 or uint16 host data, "
                            f"got {array.dtype}")
        return array if array.dtype == storage else array.astype(storage)

    def upload(self, array, dtype=None, *, pinned: PinnedArray | None = None):
        """Host array -> new device buffer.  ``pinned``: the array already lives in
        page-locked memory (``pinned_empty``), so it is copied without staging."""
        array = np.ascontiguousarray(array)
        target_name = abi.dtype_name(array.dtype if dtype is None else dtype)
        payload = self._payload(array, target_name)
        buffer = self.alloc(array.shape, target_name)
        buffer.host_dtype = array.dtype
        nbytes = payload.nbytes
        if nbytes:
            if pinned is not None and payload is array:
                src = array.ctypes.data
            else:
                staging = self._staging(nbytes)
                ctypes.memmove(staging.ptr, payload.ctypes.data, nbytes)
                src = staging.ptr
            abi.check(self._lib.b200_memcpy_h2d(buffer.ptr, src, nbytes, self.stream))
            abi.check(self._lib.b200_stream_sync(self.stream))
        return buffer

    def copy_in(self, buffer, array, *, sync=False):
        """Host array (ideally from ``pinned_empty``) -> an EXISTING device buffer of the
        same storage type; asynchronous on the device stream unless ``sync``."""
        array = np.ascontiguousarray(array)
        if array.nbytes != buffer.nbytes:
            raise ValueError(f"copy_in: {array.nbytes} host bytes into a {buffer.nbytes}-byte buffer")
        abi.check(self._lib.b200_memcpy_h2d(buffer.ptr, array.ctypes.data, array.nbytes,
                                            self.stream))
        if sync:
            abi.check(self._lib.b200_stream_sync(self.stream))

    def copy_out(self, buffer, out: PinnedArray, *, sync=True):
        """Device buffer -> page-locked host array, raw storage bytes (no bf16 widening)."""
        if out.nbytes < buffer.nbytes:
            raise ValueError("copy_out: destination is smaller than the buffer")
        abi.check(self._lib.b200_memcpy_d2h(out.ptr, buffer.ptr, buffer.nbytes, self.stream))
        if sync:
            abi.check(self._lib.b200_stream_sync(self.stream))
        return out.array

    def upload_aliased(self, group: dict, pointer_types: dict):
        """Upload host arrays that share one storage as ONE device allocation and
        return per-name views at the same byte offsets (device.py:397-406)."""
        names = list(group)
        arrays = [group[n] for n in names]
        targets = {abi.dtype_name(pointer_types.get(n) or arrays[i].dtype)
                   for i, n in enumerate(names)}
        if len(targets) != 1 or len({a.dtype for a in arrays}) != 1:
            raise TypeError("aliased host buffers must share one dtype")
        target = targets.pop()
        host_itemsize = arrays[0].dtype.itemsize
        dev_itemsize = storage_dtype(target).itemsize
        for a in arrays:
            if not a.flags.c_contiguous:
                raise TypeError("aliased host views must be C-contiguous")
        lo = min(a.ctypes.data for a in arrays)
        hi = max(a.ctypes.data + a.nbytes for a in arrays)
        span = hi - lo
        if span % host_itemsize:
            raise TypeError("aliased storage is not element-aligned")
        raw = (ctypes.c_char * span).from_address(lo)
        flat = np.frombuffer(raw, dtype=arrays[0].dtype, count=span // host_itemsize)
        base = self.upload(flat, target)
        out = {}
        for name, a in zip(names, arrays):
            offset = (a.ctypes.data - lo) // host_itemsize * dev_itemsize
            view = B200Buffer(base.ptr + offset, target, a.shape,
                              a.size * dev_itemsize, host_dtype=a.dtype, owner=False, base=base)
            out[name] = view
        return out

    def download(self, buffer, *, out: PinnedArray | None = None):
        name = abi.dtype_name(buffer.dtype)
        storage = storage_dtype(name)
        count = int(np.prod(buffer.shape, dtype=np.int64)) if buffer.shape else 1
        if out is not None:
            host = out.array.reshape(-1).view(storage)[:count].reshape(buffer.shape)
        else:
            host = np.empty(buffer.shape, dtype=storage)
        if count:
            abi.check(self._lib.b200_memcpy_d2h(host.ctypes.data, buffer.ptr,
                                                count * storage.itemsize, self.stream))
            abi.check(self._lib.b200_stream_sync(self.stream))
        if name != "bfloat16" or buffer.host_dtype == np.dtype("uint16"):
            return host
        return from_bf16_bits(host)

    # ------------------------------------------------------------ execution
    def pointer(self, buffer):
        return buffer.data_ptr()

    def synchronize(self):
        """Block until the device is idle, then read the device status word: a kernel whose
        bounded wait expired returns normally with an unfinished result, so the one hook the
        harness protocol and the measuring lane call must be the one that raises for it."""
        abi.check(self._lib.b200_stream_sync(self.stream))
        abi.check(self._lib.b200_device_sync())
        abi.check(self._lib.b200_last_device_status(self.stream))

    def timer(self):
        return EventTimer(self.stream)

    def launch(self, kernel, grid, positional, keywords):
        """Resolve ``kernel`` to its native operator and enqueue it.  No Triton, no
        host arithmetic; an unknown kernel raises ``UnsupportedLaunch``."""
        key = (None if self.registry.reads_device(kernel)
               else self._plan_key(kernel, grid, positional, keywords))
        plan = self._plans.get(key) if key is not None else None
        if plan is not None:
            abi.replay(plan)
        elif key is None:
            self.registry.launch(self, kernel, grid, positional, keywords)
        else:
            with abi.recording() as recorded:
                self.registry.launch(self, kernel, grid, positional, keywords)
            if len(self._plans) >= self.PLAN_LIMIT:
                self._plans.clear()
            # the plan keeps the kernel object alive, so its id cannot name another kernel
            self._plans[key] = recorded.calls + [(_KEEP, (kernel,))]
        self.launch_count += 1

    @staticmethod
    def _plan_key(kernel, grid, positional, keywords):
        """What a bound launch depends on: the kernel object, the grid, and per argument the
        device address, shape and dtype of a buffer or the value of a scalar.  Binding the
        same key again would rebuild the same library calls, so they are recorded once and
        replayed (a repeated launch then costs a few microseconds of host time instead of the
        whole binding path -- benchmarks time launches back to back).  ``None`` = not
        cacheable (a callable grid, an argument that does not hash)."""
        if callable(grid):
            return None
        parts = [id(kernel), tuple(grid)]
        try:
            for value in list(positional) + sorted(keywords.items()):
                name = None
                if isinstance(value, tuple):
                    name, value = value
                if isinstance(value, B200Buffer):
                    value = ("buffer", value.ptr, value.shape, str(value.dtype))
                elif hasattr(value, "data_ptr"):
                    return None  # foreign device arrays: strides are not part of the key
                parts.append((name, value))
            key = tuple(parts)
            hash(key)
        except TypeError:
            return None
        return key

    def check_status(self):
        """Drain the stream and raise if a kernel's bounded wait expired."""
        abi.check(self._lib.b200_last_device_status(self.stream))

    def compare(self, buffer, expected, policy):
        """On-device allclose for float32 buffers (devices/cuda.py:287-327); other
        dtypes return ``None`` so the caller compares on the host."""
        if not isinstance(buffer, B200Buffer):
            return None
        reference = np.ascontiguousarray(expected)
        if reference.dtype != np.float32 or abi.dtype_name(buffer.dtype) != "float32":
            return None
        if policy.get("comparator", "allclose") != "allclose":
            return None
        count = int(reference.size)
        if count == 0:
            return True, 0.0
        desired = self.upload(reference)
        try:
            bad = ctypes.c_int64()
            err = ctypes.c_double()
            abi.check(self._lib.b200_allclose_f32(
                buffer.ptr, desired.ptr, count, float(policy["rtol"]), float(policy["atol"]),
                1 if policy.get("equal_nan", False) else 0, ctypes.byref(bad), ctypes.byref(err),
                self.stream))
        finally:
            desired.free()
        return bad.value == 0, float(err.value)

    def properties(self):
        props = abi.DeviceProps()
        abi.check(self._lib.b200_device_query(self.device_id, ctypes.byref(props)))
        return {
            "name": props.name.decode(errors="replace"),
            "llc_bytes": int(props.l2_bytes),
            "sm_count": int(props.sm_count),
            "hbm_bytes": int(props.hbm_bytes),
            "compute_capability": f"{props.cc_major}.{props.cc_minor}",
            "device": f"cuda:{self.device_id}",
        }


def make_device(device_id: int | None = None) -> B200Device:
    """Factory for ``run_cases.py --device compiler_b200.device:make_device``."""
    import os
    if device_id is None:
        device_id = int(os.environ.get("B200OPS_DEVICE", "0"))
    return B200Device(device_id)

