"""The C-ABI library loads and exports exactly what ``include/b200ops.h`` declares,
and descriptor validation answers with status codes before any device work."""
import ctypes
import re
from pathlib import Path

import numpy as np
import pytest

from compiler_b200 import build
from compiler_b200.runtime import abi

ROOT = Path(__file__).resolve().parent.parent
HEADER = (ROOT / "include" / "b200ops.h").read_text()


def declared_functions():
    body = re.sub(r"/\*.*?\*/", "", HEADER, flags=re.S)
    return sorted(set(re.findall(r"\b(b200_[a-z0-9_]+)\s*\(", body)))


def test_library_builds_and_loads():
    path = build.build()
    assert path.is_file()
    lib = abi.lib()
    assert lib.b200_abi_version() == abi.ABI_VERSION


def test_every_declared_symbol_is_exported_and_bound():
    lib = abi.lib()
    names = declared_functions()
    assert len(names) >= 25
    for name in names:
        assert hasattr(lib, name), f"{name} declared in b200ops.h but not exported"
    assert sorted(abi.PROTOTYPES) == names, "ctypes prototype table and header disagree"


def test_struct_layout_pins():
    assert ctypes.sizeof(abi.Tensor) == 80
    assert abi.Tensor.shape.offset == 8 and abi.Tensor.stride.offset == 40
    assert abi.Tensor.dtype.offset == 72 and abi.Tensor.ndim.offset == 76
    assert ctypes.sizeof(abi.DeviceProps) == 96


def test_dtype_codes_follow_a100rt_numbering():
    # a100c/runtime/a100rt.h:58-72
    assert abi.DTYPE_CODES["float16"] == 10
    assert abi.DTYPE_CODES["bfloat16"] == 11
    assert abi.DTYPE_CODES["float32"] == 12
    for name, code in abi.DTYPE_CODES.items():
        assert re.search(rf"B200_DTYPE_{name.upper()} = {code}\b", HEADER), name


def test_status_strings():
    lib = abi.lib()
    seen = set()
    for code in (0, 2, 3, 4, 5, 6, 7, 8):
        text = lib.b200_status_string(code).decode()
        assert text and text != "unknown status"
        seen.add(text)
    assert len(seen) == 8
    assert lib.b200_status_string(99).decode() == "unknown status"


def _t(shape, dtype="float32", ptr=0x1000, strides=None):
    return abi.make_tensor(ptr, shape, dtype, strides)


def test_rejections_never_reach_the_device():
    """Validation precedes every CUDA call, so these run without a GPU."""
    lib = abi.lib()
    x, w, y = _t((4, 8)), _t((8,)), _t((4, 8))
    # null descriptor -> USAGE
    assert lib.b200_rmsnorm_fwd(None, ctypes.byref(w), ctypes.byref(y), None, 1e-6, None) == abi.USAGE
    # weight length mismatch -> REJECTED with a message
    w_bad = _t((7,))
    assert lib.b200_rmsnorm_fwd(ctypes.byref(x), ctypes.byref(w_bad), ctypes.byref(y), None,
                                1e-6, None) == abi.REJECTED
    assert b"w has 7" in lib.b200_last_error()
    # dtype mismatch
    y16 = _t((4, 8), "float16")
    assert lib.b200_rmsnorm_fwd(ctypes.byref(x), ctypes.byref(w), ctypes.byref(y16), None, 1e-6,
                                None) == abi.REJECTED
    # integer tensors are not norm inputs
    xi = _t((4, 8), "int32")
    assert lib.b200_softmax_fwd(ctypes.byref(xi), ctypes.byref(xi), 0, 0, None) == abi.REJECTED
    # bad enum values -> USAGE
    assert lib.b200_softmax_fwd(ctypes.byref(x), ctypes.byref(y), 7, 0, None) == abi.USAGE
    a, b, c = _t((4, 8), "bfloat16"), _t((8, 16), "bfloat16"), _t((4, 16), "bfloat16")
    assert lib.b200_gemm_bias_act(ctypes.byref(a), ctypes.byref(b), None, None, ctypes.byref(c),
                                  42, None) == abi.USAGE
    # SWIGLU without the second operand
    assert lib.b200_gemm_bias_act(ctypes.byref(a), ctypes.byref(b), None, None, ctypes.byref(c),
                                  abi.ACT_SWIGLU, None) == abi.USAGE
    # inner dimensions disagree
    b_bad = _t((9, 16), "bfloat16")
    assert lib.b200_gemm_bias_act(ctypes.byref(a), ctypes.byref(b_bad), None, None,
                                  ctypes.byref(c), 0, None) == abi.REJECTED
    # null data pointer with a non-empty shape
    a_null = _t((4, 8), "bfloat16", ptr=0)
    assert lib.b200_gemm_bias_act(ctypes.byref(a_null), ctypes.byref(b), None, None,
                                  ctypes.byref(c), 0, None) == abi.REJECTED
    # attention: K/V length must equal N_CTX, lse must be f32
    q = _t((1, 2, 16, 64), "bfloat16")
    k_bad = _t((1, 2, 8, 64), "bfloat16")
    assert lib.b200_attn_fwd(ctypes.byref(q), ctypes.byref(k_bad), ctypes.byref(q),
                             ctypes.byref(q), None, 0.125, 1, None) == abi.REJECTED
    lse_bad = _t((1, 2, 16), "float16")
    assert lib.b200_attn_fwd(ctypes.byref(q), ctypes.byref(q), ctypes.byref(q), ctypes.byref(q),
                             ctypes.byref(lse_bad), 0.125, 1, None) == abi.REJECTED
    # wrong rank
    x3 = _t((2, 4, 8))
    assert lib.b200_swiglu_fwd(ctypes.byref(x3), ctypes.byref(x3), ctypes.byref(x3), None) == abi.REJECTED


def test_empty_inputs_are_ok_without_a_device():
    lib = abi.lib()
    x, y, w = _t((0, 8), ptr=0), _t((0, 8), ptr=0), _t((8,))
    assert lib.b200_rmsnorm_fwd(ctypes.byref(x), ctypes.byref(w), ctypes.byref(y), None, 1e-6,
                                None) == abi.OK
    assert lib.b200_softmax_fwd(ctypes.byref(x), ctypes.byref(y), 0, 0, None) == abi.OK


def test_check_raises_with_detail():
    lib = abi.lib()
    x = _t((4, 8))
    with pytest.raises(abi.B200Error) as err:
        abi.check(lib.b200_softmax_fwd(ctypes.byref(x), ctypes.byref(_t((4, 9))), 0, 0, None))
    assert err.value.status == abi.REJECTED and "shape" in err.value.detail


def test_make_tensor_strides_and_limits():
    t = abi.make_tensor(0x10, (2, 3, 4), np.float16)
    assert list(t.stride)[:3] == [12, 4, 1] and t.dtype == 10 and t.ndim == 3
    with pytest.raises(ValueError):
        abi.make_tensor(0x10, (1, 1, 1, 1, 1), "float32")
    with pytest.raises(ValueError):
        abi.make_tensor(0x10, (1,), "complex64")
