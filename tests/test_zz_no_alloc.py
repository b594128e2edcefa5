"""The allocation-free comparison entry point, ``b200_allclose_f32_static``.

Some users of this library cannot allocate device memory at the moment they need a
comparison: their own allocator owns the whole device (a cudaMalloc would fail or fragment
the pool), or they are in a loop where the device-wide stall of cudaMalloc / cudaFree is not
acceptable.  For them the library offers a variant whose scratch is an array inside the
library image.  This test calls it through the C ABI and requires the very same verdict and
error metric as the allocating entry point AND as numpy (the count of elements numpy's
isclose rejects and the largest |a - b|, computed on the host) -- twice in a row with
different data, because the scratch array keeps the previous call's contents and a stale
slot must never leak into the next result -- and checks that a size beyond the built-in
array is refused.  The file sorts last so a run
that stops at the first failure has already run everything else.
"""
import ctypes

import numpy as np
import pytest

from compiler_b200.runtime import abi

pytestmark = pytest.mark.gpu


def _same(a, b):
    """(bad count, max error) pairs agree; a NaN error (a lone NaN in the data) equals itself."""
    return a[0] == b[0] and (a[1] == b[1] or (np.isnan(a[1]) and np.isnan(b[1])))


def _numpy_expected(got, ref, rtol, atol, equal_nan):
    """What the device must report: how many elements np.isclose rejects (float32 arithmetic,
    as the kernel's) and the largest |got - ref| over elements that are not equal (NaN when a
    lone NaN takes part, as the reference's int64-ordered maximum gives)."""
    close = np.isclose(got, ref, rtol=np.float32(rtol), atol=np.float32(atol),
                       equal_nan=equal_nan)
    both_nan = np.isnan(got) & np.isnan(ref)
    differs = ~((got == ref) | (both_nan if equal_nan else False))
    delta = np.abs(got.astype(np.float64) - ref.astype(np.float64))[differs]
    if delta.size == 0:
        worst = 0.0
    elif np.isnan(delta).any():
        worst = float("nan")
    else:
        worst = float(delta.max())
    return int((~close).sum()), worst


def _both(device, got, ref, rtol, atol, equal_nan):
    lib = abi.lib()
    d_got, d_ref = device.upload(got), device.upload(ref)
    out = []
    for fn in (lib.b200_allclose_f32, lib.b200_allclose_f32_static):
        bad, err = ctypes.c_int64(-1), ctypes.c_double(-1.0)
        status = fn(d_got.ptr, d_ref.ptr, got.size, rtol, atol, 1 if equal_nan else 0,
                    ctypes.byref(bad), ctypes.byref(err), device.stream)
        assert status == abi.OK, lib.b200_last_error()
        out.append((bad.value, err.value))
    return out


def test_static_scratch_variant_matches_the_allocating_one(device):
    rng = np.random.default_rng(42)
    # call 1: many blocks, several violations, a NaN pair and a lone NaN
    n1 = 3_000_017
    ref = rng.standard_normal(n1).astype(np.float32)
    got = ref.copy()
    idx = rng.choice(n1, 500, replace=False)
    got[idx] += rng.standard_normal(500).astype(np.float32)
    ref[7] = got[7] = np.nan
    got[11] = np.nan
    first = _both(device, got, ref, 1e-3, 1e-3, True)
    assert _same(first[0], first[1])
    assert _same(first[1], _numpy_expected(got, ref, 1e-3, 1e-3, True))
    assert first[1][0] > 400 and np.isnan(first[1][1])
    # call 2, right after: fewer blocks and clean data -- leftovers of call 1 in the
    # scratch array must not show up
    n2 = 70_001
    ref2 = rng.standard_normal(n2).astype(np.float32)
    got2 = ref2 + np.float32(1e-6)
    second = _both(device, got2, ref2, 1e-3, 1e-3, False)
    assert _same(second[0], second[1])
    assert _same(second[1], _numpy_expected(got2, ref2, 1e-3, 1e-3, False))
    assert second[1][0] == 0 and 0 < second[1][1] < 1e-5
    # and once more with the first data: same answer as before
    third = _both(device, got, ref, 1e-3, 1e-3, True)
    assert _same(third[1], first[1])
    # a comparison with violations but no NaN: exact count and exact largest difference
    got3 = ref2.copy()
    hit = rng.choice(n2, 97, replace=False)
    got3[hit] += (rng.uniform(0.5, 2.0, 97) * rng.choice([-1, 1], 97)).astype(np.float32)
    fourth = _both(device, got3, ref2, 1e-3, 1e-3, False)
    expected = _numpy_expected(got3, ref2, 1e-3, 1e-3, False)
    assert fourth[0] == fourth[1] == expected and expected[0] == 97


def test_static_scratch_variant_rejects_sizes_beyond_its_array(device):
    lib = abi.lib()
    buf = device.alloc((16,), "float32")
    bad, err = ctypes.c_int64(), ctypes.c_double()
    too_many = (8192 - 1) * 16384 + 1
    status = lib.b200_allclose_f32_static(buf.ptr, buf.ptr, too_many, 1e-3, 1e-3, 0,
                                          ctypes.byref(bad), ctypes.byref(err), device.stream)
    assert status == abi.REJECTED
    assert b"built-in scratch array" in lib.b200_last_error()
    assert lib.b200_allclose_f32_static(buf.ptr, buf.ptr, 0, 1e-3, 1e-3, 0, ctypes.byref(bad),
                                        ctypes.byref(err), device.stream) == abi.OK
