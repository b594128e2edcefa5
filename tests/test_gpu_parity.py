"""GPU parity: the CUDA kernels, called through the C ABI, against the CPU oracle.

Three layers, as the reference tests its devices (ops/harness/tests/
test_cuda_device.py:185-211 runs its whole perf lane through the device):
  1. every golden fixture (the reference's own cases and expected outputs) through
     ``B200Device`` + ``stage_case`` + ``launch`` with the case's own tolerance;
  2. seeded ragged sweeps per operator (1, tile-1, tile, tile+1, primes) with
     poisoned outputs so an unwritten element fails;
  3. the full-size configurations through size-independent properties plus
     oracle checks on sampled rows / heads.
Tolerances: fp32 RMSNorm rtol 1e-5; fp16 1e-2; bf16 2e-2 (ops/harness/opslib/case.py:153-157).
"""
import os
import zlib

import numpy as np
import pytest

import golden_cases
from compiler_b200 import harness, kernels, ops
from compiler_b200.runtime import abi
from oracle import oracle

pytestmark = pytest.mark.gpu

TOL = {"float32": (1e-5, 1e-6), "float16": (1e-2, 1e-2), "bfloat16": (2e-2, 2e-2)}
POISON = -7.0


def _seed(*parts):
    return zlib.crc32(repr(parts).encode())


def _host(rng_values, dtype):
    return oracle.to_storage(np.asarray(rng_values, dtype=np.float32), dtype)


def _up(device, array, dtype):
    return device.upload(array, dtype)


def _poisoned(device, shape, dtype):
    host = oracle.to_storage(np.full(shape, POISON, dtype=np.float32), dtype)
    return device.upload(host, dtype)


# ------------------------------------------------------------------ 1. golden
@pytest.mark.parametrize("tag", golden_cases.tags())
def test_golden_case_through_device(device, tag):
    case, meta = golden_cases.load(tag)
    actual = harness.run_case(case, device)
    device.check_status()
    for name in case["outputs"]:
        policy = case["comparison"][name]
        oracle.compare(actual[name], case["expected"][name], policy["rtol"], policy["atol"],
                       equal_nan=policy.get("equal_nan", True), name=f"{tag}:{name}")


# ------------------------------------------------------------------ 2. sweeps
RMS_SHAPES = [(1, 1), (3, 5), (7, 67), (5, 128), (33, 1000), (64, 4096), (9, 4100), (130, 2048),
              (3, 16384), (2, 40000)]


@pytest.mark.parametrize("dtype", ["float32", "float16", "bfloat16"])
@pytest.mark.parametrize("shape", RMS_SHAPES)
def test_rmsnorm_sweep(device, shape, dtype):
    rng = np.random.default_rng(_seed(shape, dtype))
    x = _host(rng.standard_normal(shape), dtype)
    w = _host(rng.uniform(0.5, 1.5, shape[1]), dtype)
    dx, dw = _up(device, x, dtype), _up(device, w, dtype)
    dy, dr = _poisoned(device, shape, dtype), _poisoned(device, (shape[0],), dtype)
    ops.rmsnorm(dx, dw, dy, dr, eps=1e-6)
    y_ref, r_ref = oracle.rmsnorm_ref(x, w, 1e-6)
    rtol, atol = TOL[dtype]
    oracle.compare(device.download(dy).astype(np.float64), y_ref, rtol, atol, name="Y")
    oracle.compare(device.download(dr).astype(np.float64), r_ref, rtol, atol, name="r")


# many rows of 512 or 1024 threads' width: the persistent form with the next row in flight
@pytest.mark.parametrize("dtype", ["float32", "float16", "bfloat16"])
@pytest.mark.parametrize("shape", [(700, 16384), (333, 21840), (301, 32768), (650, 8200)])
def test_rmsnorm_many_wide_rows(device, shape, dtype):
    if dtype == "float32":
        shape = (shape[0], shape[1] // 2)
    rng = np.random.default_rng(_seed(shape, dtype, "many wide rms"))
    x = _host(rng.standard_normal(shape), dtype)
    w = _host(rng.uniform(0.5, 1.5, shape[1]), dtype)
    dx, dw = _up(device, x, dtype), _up(device, w, dtype)
    dy, dr = _poisoned(device, shape, dtype), _poisoned(device, (shape[0],), dtype)
    ops.rmsnorm(dx, dw, dy, dr, eps=1e-6)
    y_ref, r_ref = oracle.rmsnorm_ref(x, w, 1e-6)
    rtol, atol = TOL[dtype]
    oracle.compare(device.download(dy).astype(np.float64), y_ref, rtol, atol, name="Y")
    oracle.compare(device.download(dr).astype(np.float64), r_ref, rtol, atol, name="r")
    # the zero-centred weight (gamma + 1) takes the same kernel
    ops.rmsnorm(dx, dw, dy, dr, eps=1e-6, gamma_offset=1.0)
    y_ref, _ = oracle.rmsnorm_ref(x, np.asarray(w, np.float64) + 1.0, 1e-6)
    oracle.compare(device.download(dy).astype(np.float64), y_ref, rtol, atol, name="Y (gamma + 1)")


def test_rmsnorm_strided_rows_and_guard(device):
    """Row pitch wider than the row: the gap must stay untouched (masked tails)."""
    rng = np.random.default_rng(11)
    rows, cols, pitch = 37, 1000, 1024
    x = rng.standard_normal((rows, pitch)).astype(np.float32)
    w = rng.uniform(0.5, 1.5, cols).astype(np.float32)
    dx, dw = device.upload(x), device.upload(w)
    dy = device.upload(np.full((rows, pitch), POISON, np.float32))
    ops.rmsnorm(registry_view(dx, (rows, cols), (pitch, 1)), dw,
                registry_view(dy, (rows, cols), (pitch, 1)), None, eps=1e-6)
    y = device.download(dy)
    y_ref, _ = oracle.rmsnorm_ref(x[:, :cols], w, 1e-6)
    oracle.compare(y[:, :cols].astype(np.float64), y_ref, 1e-5, 1e-6)
    assert (y[:, cols:] == POISON).all()


def registry_view(buffer, shape, strides):
    from compiler_b200.registry import _View
    return _View(buffer, shape, strides)


SOFTMAX_SHAPES = [(1, 1), (4, 16), (4, 97), (3, 1000), (64, 1024), (10, 4000), (6, 4104),
                  (5, 8192), (2, 33000)]


@pytest.mark.parametrize("dtype", ["float32", "float16", "bfloat16"])
@pytest.mark.parametrize("masked", [False, True])
@pytest.mark.parametrize("shape", SOFTMAX_SHAPES)
def test_softmax_sweep(device, shape, dtype, masked):
    rng = np.random.default_rng(_seed(shape, dtype, masked))
    x = _host(rng.standard_normal(shape) * 2, dtype)
    dx, dy = _up(device, x, dtype), _poisoned(device, shape, dtype)
    offset = 3 if masked else 0
    ops.softmax(dx, dy, causal_mod=masked, row_offset=offset)
    y = device.download(dy)
    ref = oracle.masked_softmax_ref(x, offset) if masked else oracle.softmax_ref(x)
    rtol, atol = (2e-3, 1e-6) if dtype == "float32" else TOL[dtype]
    oracle.compare(y.astype(np.float64), ref, rtol, atol)
    if masked:  # masked positions are written as exact zeros
        assert (y[ref == 0] == 0).all()


# masked rows in bulk: many rows of 32 .. 512 vectors, odd row counts, row offsets that put the
# wrap-around of the mask inside the launch
MASKED_BULK_CASES = [((64, 256), 0), ((65, 4000), 3999), ((777, 1000), 123), ((3000, 4096), 5),
                     ((6001, 512), 509), ((14000, 264), 7)]


@pytest.mark.parametrize("dtype", ["float32", "float16", "bfloat16"])
@pytest.mark.parametrize("case", MASKED_BULK_CASES)
def test_masked_softmax_many_rows(device, case, dtype):
    shape, offset = case
    if dtype == "float32" and shape[1] > 2048:
        shape = (shape[0], shape[1] // 2)   # 512 four-element vectors at most
    rng = np.random.default_rng(_seed(shape, dtype, True))
    x = _host(rng.standard_normal(shape) * 2, dtype)
    dx, dy = _up(device, x, dtype), _poisoned(device, shape, dtype)
    ops.softmax(dx, dy, causal_mod=True, row_offset=offset)
    y = device.download(dy)
    ref = oracle.masked_softmax_ref(x, offset)
    rtol, atol = (2e-3, 1e-6) if dtype == "float32" else TOL[dtype]
    oracle.compare(y.astype(np.float64), ref, rtol, atol)
    assert (y[ref == 0] == 0).all() and np.isfinite(y).all()


# many rows of 512 or 1024 threads' width (more rows than resident CTAs): the pipelined form
# with the CTA as the row group; 16-bit widths, halved for float32 (four-element vectors)
MANY_WIDE_ROWS = [((700, 16384), 0), ((333, 21840), 21000), ((301, 32768), 5), ((420, 9000), 8000),
                  ((650, 8200), 3)]


@pytest.mark.parametrize("masked", [False, True])
@pytest.mark.parametrize("dtype", ["float32", "float16", "bfloat16"])
@pytest.mark.parametrize("case", MANY_WIDE_ROWS)
def test_softmax_many_wide_rows(device, case, dtype, masked):
    shape, offset = case
    if dtype == "float32":
        shape = (shape[0], shape[1] // 2)
    rng = np.random.default_rng(_seed(shape, dtype, masked, "many wide"))
    x = _host(rng.standard_normal(shape) * 2, dtype)
    dx, dy = _up(device, x, dtype), _poisoned(device, shape, dtype)
    ops.softmax(dx, dy, causal_mod=masked, row_offset=offset if masked else 0)
    y = device.download(dy)
    ref = oracle.masked_softmax_ref(x, offset) if masked else oracle.softmax_ref(x)
    rtol, atol = (2e-3, 1e-6) if dtype == "float32" else TOL[dtype]
    oracle.compare(y.astype(np.float64), ref, rtol, atol)
    assert np.isfinite(y).all()
    if masked:
        assert (y[ref == 0] == 0).all()
    np.testing.assert_allclose(y.astype(np.float64).sum(axis=1), 1.0, atol=2e-2)


# rows wider than one CTA keeps in registers (32768 16-bit / 16384 32-bit elements): a cluster
# of 2, 4 or 8 CTAs per row with the partial results merged through distributed shared memory;
# widths that are not a whole number of CTAs, a width beyond eight CTAs (looping kernel)
WIDE_ROWS = [(3, 33000), (2, 40000), (5, 65536), (2, 131072 + 8), (3, 262144), (1, 262144 + 512)]


@pytest.mark.parametrize("dtype", ["float32", "float16", "bfloat16"])
@pytest.mark.parametrize("shape", WIDE_ROWS)
def test_wide_rows_cluster_softmax_and_rmsnorm(device, shape, dtype):
    rows, cols = shape
    if dtype == "float32":
        cols //= 2
    rng = np.random.default_rng(_seed(shape, dtype, "wide"))
    x = _host(rng.standard_normal((rows, cols)) * 2, dtype)
    dx = _up(device, x, dtype)
    for masked, offset in ((False, 0), (True, cols - 2)):
        dy = _poisoned(device, (rows, cols), dtype)
        ops.softmax(dx, dy, causal_mod=masked, row_offset=offset)
        y = device.download(dy)
        ref = oracle.masked_softmax_ref(x, offset) if masked else oracle.softmax_ref(x)
        rtol, atol = (2e-3, 1e-7) if dtype == "float32" else TOL[dtype]
        oracle.compare(y.astype(np.float64), ref, rtol, atol, name=f"softmax masked={masked}")
        if masked:
            assert (y[ref == 0] == 0).all()
    w = _host(rng.uniform(0.5, 1.5, cols), dtype)
    dw = _up(device, w, dtype)
    dyr, dr = _poisoned(device, (rows, cols), dtype), _poisoned(device, (rows,), dtype)
    ops.rmsnorm(dx, dw, dyr, dr, eps=1e-6)
    y_ref, r_ref = oracle.rmsnorm_ref(x, w, 1e-6)
    rtol, atol = (1e-5, 1e-6) if dtype == "float32" else TOL[dtype]
    oracle.compare(device.download(dyr).astype(np.float64), y_ref, rtol, atol, name="rmsnorm y")
    oracle.compare(device.download(dr).astype(np.float64), r_ref, rtol, atol, name="rmsnorm r")


GEMM_SHAPES = [(128, 256, 64), (256, 512, 256), (1, 8, 8), (129, 264, 72), (257, 520, 200),
               (100, 40, 24), (384, 1024, 1000), (130, 96, 8)]


@pytest.mark.parametrize("dtype", ["bfloat16", "float16"])
@pytest.mark.parametrize("act", ["none", "gelu_tanh", "gelu_erf", "leaky_relu"])
@pytest.mark.parametrize("shape", GEMM_SHAPES)
def test_gemm_sweep(device, shape, dtype, act):
    m, n, k = shape
    rng = np.random.default_rng(_seed(shape, dtype, act))
    a = _host(rng.standard_normal((m, k)) / np.sqrt(k), dtype)
    b = _host(rng.standard_normal((k, n)), dtype)
    bias = _host(rng.normal(0, 0.1, n), dtype)
    da, db, dbias = _up(device, a, dtype), _up(device, b, dtype), _up(device, bias, dtype)
    dc = _poisoned(device, (m, n), dtype)
    code = {"none": abi.ACT_NONE, "gelu_tanh": abi.ACT_GELU_TANH, "gelu_erf": abi.ACT_GELU_ERF,
            "leaky_relu": abi.ACT_LEAKY_RELU}[act]
    use_bias = act != "none"
    ops.gemm(da, db, dc, bias=dbias if use_bias else None, act=code)
    device.check_status()
    ref = oracle.linear_act_ref(a, b, bias if use_bias else None, act)
    oracle.compare(device.download(dc).astype(np.float64), ref, *TOL[dtype], name=f"C{shape}")


# The weight given as [N, K] (a linear layer's layout): small and ragged shapes on the one-CTA
# kernel, shapes with a wave of 256 x 256 tiles on the CTA-pair kernel, fp32 and unaligned rows
# on the CUDA-core kernel; cross-checked against the oracle on w.T.
LINEAR_SHAPES = [(128, 256, 64), (129, 264, 72), (100, 40, 24), (384, 1024, 1000),
                 (3328, 3072, 192), (3300, 3096, 200), (2050, 4872, 8), (2048, 5000, 520),
                 (130, 96, 12)]


@pytest.mark.parametrize("dtype,act", [("bfloat16", "gelu_erf"), ("float16", "none"),
                                        ("bfloat16", "leaky_relu"), ("float32", "gelu_tanh")])
@pytest.mark.parametrize("shape", LINEAR_SHAPES)
def test_linear_weight_rows_of_k(device, shape, dtype, act):
    m, n, k = shape
    if dtype == "float32" and m * n * k > 1 << 28:
        pytest.skip("the CUDA-core path is for correctness, not for this size")
    rng = np.random.default_rng(_seed(shape, dtype, act, "linear"))
    x = _host(rng.standard_normal((m, k)) / np.sqrt(k), dtype)
    w = _host(rng.standard_normal((n, k)), dtype)
    bias = _host(rng.normal(0, 0.1, n), dtype)
    dx, dw, dbias = _up(device, x, dtype), _up(device, w, dtype), _up(device, bias, dtype)
    dy = _poisoned(device, (m, n), dtype)
    code = {"none": abi.ACT_NONE, "gelu_tanh": abi.ACT_GELU_TANH, "gelu_erf": abi.ACT_GELU_ERF,
            "leaky_relu": abi.ACT_LEAKY_RELU}[act]
    use_bias = act != "none"
    ops.linear(dx, dw, dy, bias=dbias if use_bias else None, act=code)
    device.check_status()
    ref = oracle.linear_act_ref(x, np.ascontiguousarray(w.T), bias if use_bias else None, act)
    rtol, atol = (2e-3, 2e-3) if dtype == "float32" else TOL[dtype]
    oracle.compare(device.download(dy).astype(np.float64), ref, rtol, atol, name=f"Y{shape}")


def test_strided_matmul_with_transposed_b_through_the_device(device):
    """matmul_kernel's general strides (ops/suite/perf/matmul_triton2.py:27-30): B handed over
    as the transpose in memory of a [K, N] matrix (stride_bk = 1, stride_bn = K)."""
    case, _ = golden_cases.load("matmul_triton2__32x32x32__bfloat16")
    m, n, k = 200, 264, 136
    rng = np.random.default_rng(77)
    a = _host(rng.standard_normal((m, k)) / np.sqrt(k), "bfloat16")
    bt = _host(rng.standard_normal((n, k)), "bfloat16")          # B^T, contiguous
    args = dict(case["args"])
    args.update({"a_ptr": a, "b_ptr": bt, "c_ptr": np.full((m, n), POISON, np.float32),
                 "M": m, "N": n, "K": k, "stride_am": k, "stride_ak": 1, "stride_bk": 1,
                 "stride_bn": k, "stride_cm": n, "stride_cn": 1})
    grown = dict(case, args=args, grid=lambda meta: (-(-m // meta["BLOCK_M"]),
                                                     -(-n // meta["BLOCK_N"])))
    out = harness.run_case(grown, device)["c_ptr"]
    leaky = bool({**case["args"], **case["meta"]}.get("LEAKY", False))
    ref = oracle.linear_act_ref(a, np.ascontiguousarray(bt.T), None,
                                "leaky_relu" if leaky else "none")
    oracle.compare(out.astype(np.float64), ref, *TOL["bfloat16"], name="c_ptr")


# Shapes with at least one 256 x 256 tile per pair of SMs take the CTA-pair kernel: whole
# tiles, a ragged edge in both directions, a last row block whose second CTA is all padding,
# and K shorter / longer than the six-stage ring.
PAIR_SHAPES = [(3328, 3072, 192), (3300, 3096, 200), (3072 + 100, 3328, 64), (2048, 5000, 520),
               (2050, 4872, 8),
               # more tiles than SM pairs with a short last wave: its tiles are cut along K
               # (4 and 2 slices; whole and ragged K, a ragged last row block)
               (4096, 4864, 4096), (4096, 4096, 2048), (4000, 4870, 4200)]


@pytest.mark.parametrize("dtype,act", [("bfloat16", "gelu_tanh"), ("float16", "none"),
                                        ("bfloat16", "leaky_relu")])
@pytest.mark.parametrize("shape", PAIR_SHAPES)
def test_gemm_pair_tiles(device, shape, dtype, act):
    m, n, k = shape
    rng = np.random.default_rng(_seed(shape, dtype, act))
    a = _host(rng.standard_normal((m, k)) / np.sqrt(k), dtype)
    b = _host(rng.standard_normal((k, n)), dtype)
    bias = _host(rng.normal(0, 0.1, n), dtype)
    da, db, dbias = _up(device, a, dtype), _up(device, b, dtype), _up(device, bias, dtype)
    dc = _poisoned(device, (m, n), dtype)
    code = {"none": abi.ACT_NONE, "gelu_tanh": abi.ACT_GELU_TANH,
            "leaky_relu": abi.ACT_LEAKY_RELU}[act]
    use_bias = act != "none"
    ops.gemm(da, db, dc, bias=dbias if use_bias else None, act=code)
    device.check_status()
    ref = oracle.linear_act_ref(a, b, bias if use_bias else None, act)
    oracle.compare(device.download(dc).astype(np.float64), ref, *TOL[dtype], name=f"C{shape}")


@pytest.mark.parametrize("shape", [(128, 128, 64), (200, 264, 136), (256, 1024, 512)])
def test_gemm_f32_bias_and_f32_output(device, shape):
    m, n, k = shape
    rng = np.random.default_rng(5)
    a = _host(rng.standard_normal((m, k)) / np.sqrt(k), "bfloat16")
    b = _host(rng.standard_normal((k, n)), "bfloat16")
    bias = rng.normal(0, 0.1, n).astype(np.float32)
    da, db = _up(device, a, "bfloat16"), _up(device, b, "bfloat16")
    dbias = device.upload(bias)
    dc = device.upload(np.full((m, n), POISON, np.float32))
    ops.gemm(da, db, dc, bias=dbias, act=abi.ACT_GELU_TANH)
    device.check_status()
    ref = oracle.linear_act_ref(a, b, bias, "gelu_tanh")
    oracle.compare(device.download(dc).astype(np.float64), ref, 2e-3, 2e-3)


# the shapes from the fourth on have enough 256-row tiles for the CTA-pair form of the dual
# GEMM (whole tiles, ragged last row and column blocks, the MLP's up-projection at 8 ranks)
@pytest.mark.parametrize("shape", [(128, 128, 64), (130, 200, 72), (256, 384, 512),
                                   (3328, 1536, 192), (2050, 2440, 72), (4096, 1792, 136),
                                   (4090, 1784, 72), (4096, 1792, 4096)])
def test_gemm_swiglu_dual(device, shape):
    m, n, k = shape
    rng = np.random.default_rng(6)
    x = _host(rng.standard_normal((m, k)), "bfloat16")
    wg = _host(rng.normal(0, 0.05, (k, n)), "bfloat16")
    wu = _host(rng.normal(0, 0.05, (k, n)), "bfloat16")
    dx, dg, du = (_up(device, t, "bfloat16") for t in (x, wg, wu))
    dh = _poisoned(device, (m, n), "bfloat16")
    ops.gemm(dx, dg, dh, b2=du, act=abi.ACT_SWIGLU)
    device.check_status()
    ref = oracle.swiglu_ref(oracle.matmul_ref(x, wg), oracle.matmul_ref(x, wu))
    oracle.compare(device.download(dh).astype(np.float64), ref, 2e-2, 2e-2)


def test_gemm_fp32_operands_take_the_ieee_path(device):
    rng = np.random.default_rng(7)
    a = rng.standard_normal((33, 47)).astype(np.float32)
    b = rng.standard_normal((47, 29)).astype(np.float32)
    da, db = device.upload(a), device.upload(b)
    dc = device.upload(np.full((33, 29), POISON, np.float32))
    ops.gemm(da, db, dc)
    oracle.compare(device.download(dc).astype(np.float64), oracle.matmul_ref(a, b), 1e-5, 1e-5)


ATTN_SHAPES = [(1, 2, 256, 128), (2, 1, 384, 64), (1, 2, 200, 128), (1, 1, 128, 128),
               (1, 1, 640, 128), (1, 3, 77, 64), (3, 70, 512, 128), (1, 2, 1100, 64)]


@pytest.mark.parametrize("variant", ["pair", "single-tmem", "single-smem"])
@pytest.mark.parametrize("dtype", ["bfloat16", "float16"])
@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("shape", ATTN_SHAPES)
def test_attention_sweep(device, shape, dtype, causal, variant):
    z, h, n, d = shape
    rng = np.random.default_rng(_seed(shape, dtype, causal))
    q, k, v = (_host(rng.standard_normal(shape), dtype) for _ in range(3))
    dq, dk, dv = (_up(device, t, dtype) for t in (q, k, v))
    do = _poisoned(device, shape, dtype)
    dl = device.upload(np.full((z, h, n), POISON, np.float32))
    scale = 1.0 / np.sqrt(d)
    kernel, _, p_location = variant.partition("-")
    os.environ["B200OPS_ATTN_KERNEL"] = kernel
    os.environ["B200OPS_ATTN_P"] = p_location or "tmem"
    try:
        ops.attention(dq, dk, dv, do, lse=dl, scale=scale, causal=causal)
        device.check_status()
    finally:
        os.environ.pop("B200OPS_ATTN_P", None)
        os.environ.pop("B200OPS_ATTN_KERNEL", None)
    out_ref, lse_ref = oracle.attention_ref(q, k, v, scale, causal)
    oracle.compare(device.download(do).astype(np.float64), out_ref, *TOL[dtype], name="out")
    oracle.compare(device.download(dl).astype(np.float64), lse_ref, 1e-3, 1e-3, name="lse")


@pytest.mark.parametrize("variant", ["pair", "single"])
@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("shape", [(2, 8, 2, 300, 64), (1, 6, 3, 512, 128), (2, 4, 1, 129, 128)])
def test_attention_grouped_kv_heads(device, shape, causal, variant):
    """Fewer K / V heads than query heads (the head mapping of ops/suite/dev/gqa.py:27-32) on
    the tensor-core kernels."""
    z, hq, hkv, n, d = shape
    rng = np.random.default_rng(_seed(shape, causal))
    q = _host(rng.standard_normal((z, hq, n, d)), "bfloat16")
    k, v = (_host(rng.standard_normal((z, hkv, n, d)), "bfloat16") for _ in range(2))
    dq, dk, dv = (_up(device, t, "bfloat16") for t in (q, k, v))
    do = _poisoned(device, (z, hq, n, d), "bfloat16")
    dl = device.upload(np.full((z, hq, n), POISON, np.float32))
    scale = 1.0 / np.sqrt(d)
    os.environ["B200OPS_ATTN_KERNEL"] = variant
    try:
        ops.attention(dq, dk, dv, do, lse=dl, scale=scale, causal=causal)
        device.check_status()
    finally:
        os.environ.pop("B200OPS_ATTN_KERNEL", None)
    out_ref, lse_ref = oracle.gqa_attention_ref(q, k, v, scale, causal)
    oracle.compare(device.download(do).astype(np.float64), out_ref, *TOL["bfloat16"], name="out")
    oracle.compare(device.download(dl).astype(np.float64), lse_ref, 1e-3, 1e-3, name="lse")
    from compiler_b200.runtime.abi import B200Error
    with pytest.raises(B200Error):  # 3 K/V heads do not divide 8 query heads
        bad = device.alloc((z, 3, n, d), "bfloat16") if hq % 3 else device.alloc((z, 5, n, d), "bfloat16")
        ops.attention(dq, bad, bad, do, scale=scale, causal=causal)


@pytest.mark.parametrize("variant", ["pair", "single"])
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("shape", [(2, 4, 2, 300, 517, 64), (1, 2, 2, 129, 64, 128),
                                   (1, 3, 1, 640, 1000, 128), (1, 2, 1, 100, 1200, 128)])
def test_attention_other_key_length(device, shape, causal, variant):
    """N_K keys for N query rows, the causal mask aligned to the last key (row i sees keys
    <= i + N_K - N), the log-sum-exp written through strides."""
    from compiler_b200.runtime.abi import B200Error
    z, hq, hkv, n, nk, d = shape
    rng = np.random.default_rng(_seed(shape, causal))
    q = _host(rng.standard_normal((z, hq, n, d)), "bfloat16")
    k, v = (_host(rng.standard_normal((z, hkv, nk, d)), "bfloat16") for _ in range(2))
    dq, dk, dv = (_up(device, t, "bfloat16") for t in (q, k, v))
    do = _poisoned(device, (z, hq, n, d), "bfloat16")
    pad = 7  # lse rows are n + pad apart
    dl = device.upload(np.full((z, hq, n + pad), POISON, np.float32))

    class Strided:
        shape, dtype = (z, hq, n), dl.dtype

        def data_ptr(self):
            return dl.data_ptr()

        def stride(self):
            return (hq * (n + pad), n + pad, 1)

    scale = 1.0 / np.sqrt(d)
    os.environ["B200OPS_ATTN_KERNEL"] = variant
    try:
        if causal and nk < n:
            with pytest.raises(B200Error):  # rows without any visible key
                ops.attention(dq, dk, dv, do, scale=scale, causal=True)
            return
        ops.attention(dq, dk, dv, do, lse=Strided(), scale=scale, causal=causal)
        device.check_status()
    finally:
        os.environ.pop("B200OPS_ATTN_KERNEL", None)
    out_ref, lse_ref = oracle.gqa_attention_ref(q, k, v, scale, causal)
    oracle.compare(device.download(do).astype(np.float64), out_ref, *TOL["bfloat16"], name="out")
    got_lse = device.download(dl)
    oracle.compare(got_lse[..., :n].astype(np.float64), lse_ref, 1e-3, 1e-3, name="lse")
    assert np.all(got_lse[..., n:] == POISON)  # the padding between rows is untouched


@pytest.mark.parametrize("shape", [(2, 17, 40, 16), (1, 33, 33, 80)])
def test_attention_other_key_length_cuda_core(device, shape):
    """The same mask rule on the CUDA-core kernel (fp32)."""
    z, n, nk, d = shape
    rng = np.random.default_rng(_seed(shape))
    q = rng.standard_normal((z, 2, n, d)).astype(np.float32)
    k, v = (rng.standard_normal((z, 2, nk, d)).astype(np.float32) for _ in range(2))
    dq, dk, dv = (device.upload(t) for t in (q, k, v))
    do = device.upload(np.full((z, 2, n, d), POISON, np.float32))
    for causal in (False, True):
        ops.attention(dq, dk, dv, do, scale=0.25, causal=causal)
        out_ref, _ = oracle.attention_ref(q, k, v, 0.25, causal)
        oracle.compare(device.download(do).astype(np.float64), out_ref, 1e-4, 1e-5)


def test_varlen_attention_through_the_launch_surface(device):
    """flash_varlen_fwd_kernel's dense case at tensor-core sizes: packed sequences, query and
    key lengths that differ, two query heads per K / V head, lse laid out [h, total_q]."""
    from compiler_b200.registry import _VARLEN
    case, _ = golden_cases.load("flash_varlen_fwd_kernel__2x17x19x4x2x16__bfloat16")
    h, hk, d = 4, 2, 64
    q_len, k_len = [300, 129, 64], [500, 200, 130]
    cu_q = np.concatenate(([0], np.cumsum(q_len))).astype(np.int32)
    cu_k = np.concatenate(([0], np.cumsum(k_len))).astype(np.int32)
    total_q, total_k = int(cu_q[-1]), int(cu_k[-1])
    rng = np.random.default_rng(77)
    q = _host(rng.normal(0, 0.5, (total_q, h, d)), "bfloat16")
    k = _host(rng.normal(0, 0.5, (total_k, hk, d)), "bfloat16")
    v = _host(rng.normal(0, 0.5, (total_k, hk, d)), "bfloat16")
    scale = 1.0 / np.sqrt(d)
    args = dict(case["args"])
    args.update({"q_ptr": q.reshape(-1), "k_ptr": k.reshape(-1), "v_ptr": v.reshape(-1),
                 "o_ptr": np.zeros(total_q * h * d, np.float32),
                 "softmax_lse_ptr": np.zeros(h * total_q, np.float32),
                 "q_row_stride": h * d, "o_row_stride": h * d, "k_row_stride": hk * d,
                 "v_row_stride": hk * d, "q_head_stride": d, "k_head_stride": d,
                 "v_head_stride": d, "o_head_stride": d, "cu_seqlens_q_ptr": cu_q,
                 "cu_seqlens_k_ptr": cu_k, "b": 3, "bk": 3, "seqlen_q": max(q_len),
                 "seqlen_k": max(k_len), "total_q": total_q})
    case = dict(case, args=args, grid=(19, 3, h),
                meta={**case["meta"], "h": h, "hk": hk, "h_hk_ratio": h // hk, "d": d,
                      "d_rounded": d, "scale_softmax": float(scale)})
    assert tuple(golden_cases.kernel_parameters(case["kernel"])) == _VARLEN
    before = len(device._plans)
    got = harness.run_case(case, device)
    device.check_status()
    assert len(device._plans) == before  # sequence bounds are read back: never replayed
    out_ref, lse_ref = oracle.varlen_attention_ref(q, k, v, cu_q, cu_k, scale)
    oracle.compare(got["o_ptr"].reshape(total_q, h, d).astype(np.float64), out_ref,
                   *TOL["bfloat16"], name="o")
    oracle.compare(got["softmax_lse_ptr"].reshape(h, total_q).astype(np.float64), lse_ref,
                   1e-3, 1e-3, name="lse")


ATTENTION_MODES = [
    dict(softcap=0.5), dict(softcap=0.05, causal=True), dict(window=(7, 0)), dict(window=(3, 5)),
    dict(window=(0, 0), causal=True), dict(alibi="heads"), dict(alibi="batch", causal=True),
    dict(alibi="heads", softcap=0.3, window=(9, 2)), dict(window=(64, 64), causal=True, softcap=1.0),
]


@pytest.mark.parametrize("dtype", ["float32", "float16", "bfloat16"])
@pytest.mark.parametrize("shape", [(2, 4, 2, 33, 47, 16), (1, 6, 6, 70, 70, 64), (2, 2, 1, 40, 12, 32),
                                   (1, 2, 2, 12, 300, 128)])
@pytest.mark.parametrize("modes", ATTENTION_MODES, ids=lambda m: "-".join(f"{k}" for k in m))
def test_attention_modes(device, modes, shape, dtype):
    """The soft-cap, ALiBi and local-window modes of flash_varlen_fwd_kernel
    (ops/suite/dev/flash_varlen_fwd_kernel.py:121-146) against the restatement of the kernel's
    lines: other key lengths (also fewer keys than rows: rows without a key give zeros and
    lse = +inf), grouped K / V heads, slopes per head and per batch and head."""
    z, hq, hkv, n, nk, d = shape
    modes = dict(modes)
    rng = np.random.default_rng(_seed(shape, dtype, sorted(modes)))
    q = _host(rng.standard_normal((z, hq, n, d)), dtype)
    k, v = (_host(rng.standard_normal((z, hkv, nk, d)), dtype) for _ in range(2))
    slopes = None
    if "alibi" in modes:
        per = modes.pop("alibi")
        slopes = (2.0 ** -np.arange(1, hq + 1, dtype=np.float32) if per == "heads"
                  else rng.uniform(0.01, 0.5, (z, hq)).astype(np.float32))
    dq, dk, dv = (_up(device, t, dtype) for t in (q, k, v))
    do = _poisoned(device, (z, hq, n, d), dtype)
    dl = device.upload(np.full((z, hq, n), POISON, np.float32))
    scale = 1.0 / np.sqrt(d)
    ops.attention(dq, dk, dv, do, lse=dl, scale=scale, causal=modes.get("causal", False),
                  softcap=modes.get("softcap", 0.0), window=modes.get("window"),
                  alibi_slopes=device.upload(slopes) if slopes is not None else None)
    device.check_status()
    out_ref, lse_ref = oracle.attention_modes_ref(
        q, k, v, scale, causal=modes.get("causal", False), softcap=modes.get("softcap", 0.0),
        alibi_slopes=slopes, window=modes.get("window"))
    rtol, atol = (1e-4, 1e-5) if dtype == "float32" else TOL[dtype]
    oracle.compare(device.download(do).astype(np.float64), out_ref, rtol, atol, name="out")
    got_lse = device.download(dl).astype(np.float64)
    empty = np.isinf(lse_ref)
    assert np.array_equal(np.isposinf(got_lse), empty)
    oracle.compare(got_lse[~empty], lse_ref[~empty], 1e-3, 1e-3, name="lse")


def test_varlen_attention_modes_through_the_launch_surface(device):
    """The varlen kernel's flags through the launch surface: key lengths from seqused_k,
    soft-cap, a local window, ALiBi slopes per (batch, head) -- one case with all of them."""
    case, _ = golden_cases.load("flash_varlen_fwd_kernel__2x17x19x4x2x16__float32")
    h, hk, d = 4, 2, 16
    q_len, k_cache, k_used = [17, 9, 30], [19, 25, 30], [19, 20, 11]
    cu_q = np.concatenate(([0], np.cumsum(q_len))).astype(np.int32)
    cu_k = np.concatenate(([0], np.cumsum(k_cache))).astype(np.int32)
    total_q, total_k = int(cu_q[-1]), int(cu_k[-1])
    rng = np.random.default_rng(78)
    q = rng.normal(0, 0.7, (total_q, h, d)).astype(np.float32)
    k = rng.normal(0, 0.7, (total_k, hk, d)).astype(np.float32)
    v = rng.normal(0, 0.7, (total_k, hk, d)).astype(np.float32)
    slopes = rng.uniform(0.05, 0.4, (3, h)).astype(np.float32)
    scale, softcap, window = 1.0 / np.sqrt(d), 0.4, (6, 3)
    args = dict(case["args"])
    args.update({"q_ptr": q.reshape(-1), "k_ptr": k.reshape(-1), "v_ptr": v.reshape(-1),
                 "o_ptr": np.zeros(total_q * h * d, np.float32),
                 "softmax_lse_ptr": np.zeros(h * total_q, np.float32),
                 "q_row_stride": h * d, "o_row_stride": h * d, "k_row_stride": hk * d,
                 "v_row_stride": hk * d, "q_head_stride": d, "k_head_stride": d,
                 "v_head_stride": d, "o_head_stride": d, "cu_seqlens_q_ptr": cu_q,
                 "cu_seqlens_k_ptr": cu_k, "seqused_k_ptr": np.asarray(k_used, np.int32),
                 "alibi_slopes_ptr": slopes.reshape(-1), "b": 3, "bk": 3,
                 "seqlen_q": max(q_len), "seqlen_k": max(k_cache), "total_q": total_q})
    meta = {**case["meta"], "h": h, "hk": hk, "h_hk_ratio": h // hk, "d": d, "d_rounded": d,
            "scale_softmax": float(scale), "is_cu_seqlens_q": True, "is_cu_seqlens_k": True,
            "is_seqused_k": True, "is_softcap": True, "softcap": softcap, "is_local": True,
            "window_size_left": window[0], "window_size_right": window[1], "is_alibi": True,
            "alibi_slopes_batch_stride": h}
    case = dict(case, args=args, grid=(30, 3, h), meta=meta)
    got = harness.run_case(case, device)
    device.check_status()
    out = got["o_ptr"].reshape(total_q, h, d).astype(np.float64)
    lse = got["softmax_lse_ptr"].reshape(h, total_q).astype(np.float64)
    for b in range(3):
        qs, ks = slice(cu_q[b], cu_q[b + 1]), slice(cu_k[b], cu_k[b] + k_used[b])
        ref_o, ref_l = oracle.attention_modes_ref(
            q[qs].transpose(1, 0, 2)[None], k[ks].transpose(1, 0, 2)[None],
            v[ks].transpose(1, 0, 2)[None], scale, softcap=softcap, alibi_slopes=slopes[b],
            window=window)
        oracle.compare(out[qs].transpose(1, 0, 2), ref_o[0], 1e-4, 1e-5, name=f"o[{b}]")
        empty = np.isinf(ref_l[0])
        assert np.array_equal(np.isposinf(lse[:, qs]), empty)
        oracle.compare(lse[:, qs][~empty], ref_l[0][~empty], 1e-3, 1e-3, name=f"lse[{b}]")


def test_varlen_attention_paged_through_the_launch_surface(device):
    """is_paged through the launch surface: fixed query length, key lengths from seqused_k, the
    keys of every batch scattered over a page cache by its row of the page table."""
    case, _ = golden_cases.load("flash_varlen_fwd_kernel__2x17x19x4x2x16__float32")
    h, hk, d, block = 4, 2, 16, 8
    batches, q_len, k_used = 3, 11, [19, 8, 30]
    pages_per_batch = 4
    num_pages = batches * pages_per_batch + 2
    rng = np.random.default_rng(79)
    q = rng.normal(0, 0.7, (batches, q_len, h, d)).astype(np.float32)
    kcache = rng.normal(0, 0.7, (num_pages, block, hk, d)).astype(np.float32)
    vcache = rng.normal(0, 0.7, (num_pages, block, hk, d)).astype(np.float32)
    table = rng.permutation(num_pages)[:batches * pages_per_batch].astype(np.int32)
    table = table.reshape(batches, pages_per_batch)
    scale = 1.0 / np.sqrt(d)
    args = dict(case["args"])
    args.update({"q_ptr": q.reshape(-1), "k_ptr": kcache.reshape(-1), "v_ptr": vcache.reshape(-1),
                 "o_ptr": np.zeros(q.size, np.float32),
                 "softmax_lse_ptr": np.zeros(h * batches * q_len, np.float32),
                 "q_row_stride": h * d, "o_row_stride": h * d, "k_row_stride": hk * d,
                 "v_row_stride": hk * d, "q_head_stride": d, "k_head_stride": d,
                 "v_head_stride": d, "o_head_stride": d, "q_batch_stride": q_len * h * d,
                 "o_batch_stride": q_len * h * d, "k_batch_stride": 0, "v_batch_stride": 0,
                 "seqused_k_ptr": np.asarray(k_used, np.int32), "page_table_ptr": table.reshape(-1),
                 "k_page_stride": block * hk * d, "b": batches, "bk": batches,
                 "seqlen_q": q_len, "seqlen_k": pages_per_batch * block,
                 "total_q": batches * q_len})
    meta = {**case["meta"], "h": h, "hk": hk, "h_hk_ratio": h // hk, "d": d, "d_rounded": d,
            "scale_softmax": float(scale), "is_cu_seqlens_q": False, "is_cu_seqlens_k": False,
            "is_seqused_k": True, "is_paged": True, "block_size": block,
            "page_table_batch_stride": pages_per_batch, "is_causal": True}
    case = dict(case, args=args, grid=(q_len, batches, h), meta=meta)
    got = harness.run_case(case, device)
    device.check_status()
    out = got["o_ptr"].reshape(batches, q_len, h, d).astype(np.float64)
    lse = got["softmax_lse_ptr"].reshape(h, batches, q_len).astype(np.float64)
    for b in range(batches):
        j = np.arange(k_used[b])
        kb = kcache[table[b, j // block], j % block].transpose(1, 0, 2)[None]
        vb = vcache[table[b, j // block], j % block].transpose(1, 0, 2)[None]
        ref_o, ref_l = oracle.attention_modes_ref(q[b].transpose(1, 0, 2)[None], kb, vb, scale,
                                                  causal=True)
        empty = np.isinf(ref_l[0])
        oracle.compare(out[b].transpose(1, 0, 2), ref_o[0], 1e-4, 1e-5, name=f"o[{b}]")
        assert np.array_equal(np.isposinf(lse[:, b]), empty)
        oracle.compare(lse[:, b][~empty], ref_l[0][~empty], 1e-3, 1e-3, name=f"lse[{b}]")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("block_size", [1, 4, 16])
def test_attention_paged_kv(device, block_size, dtype):
    """Paged K / V (ops/suite/dev/flash_varlen_fwd_kernel.py:91-108): the keys of a batch are
    scattered over the pages of a cache in the order its page table gives; the result must be
    that of attention over the gathered keys (here with a causal mask and a soft-cap on top)."""
    z, hq, hkv, n, nk, d = 2, 4, 2, 21, 37, 16
    pages_per_batch = -(-nk // block_size)
    num_pages = 2 * pages_per_batch + 3
    rng = np.random.default_rng(_seed(block_size, dtype, "paged"))
    kcache = _host(rng.standard_normal((num_pages, block_size, hkv, d)), dtype)
    vcache = _host(rng.standard_normal((num_pages, block_size, hkv, d)), dtype)
    table = rng.permutation(num_pages)[:z * pages_per_batch].reshape(z, pages_per_batch)
    table = table.astype(np.int32)
    q = _host(rng.standard_normal((z, hq, n, d)), dtype)
    # what the page table means: key j of batch b = row j % block of page table[b, j // block]
    j = np.arange(nk)
    k = np.stack([kcache[table[b, j // block_size], j % block_size] for b in range(z)])
    v = np.stack([vcache[table[b, j // block_size], j % block_size] for b in range(z)])
    k, v = k.transpose(0, 2, 1, 3), v.transpose(0, 2, 1, 3)          # [Z, H_KV, N_K, D]
    dq, dkc, dvc = _up(device, q, dtype), _up(device, kcache, dtype), _up(device, vcache, dtype)
    dt = device.upload(table)
    do = _poisoned(device, (z, hq, n, d), dtype)
    dl = device.upload(np.full((z, hq, n), POISON, np.float32))
    row, page = hkv * d, block_size * hkv * d
    kview = registry_view(dkc, (z, hkv, nk, d), (0, d, row, 1))
    vview = registry_view(dvc, (z, hkv, nk, d), (0, d, row, 1))
    scale = 1.0 / np.sqrt(d)
    ops.attention(dq, kview, vview, do, lse=dl, scale=scale, causal=True, softcap=0.7,
                  page_table=dt, block_size=block_size, page_stride=page)
    device.check_status()
    out_ref, lse_ref = oracle.attention_modes_ref(q, k, v, scale, causal=True, softcap=0.7)
    rtol, atol = (1e-4, 1e-5) if dtype == "float32" else TOL[dtype]
    oracle.compare(device.download(do).astype(np.float64), out_ref, rtol, atol, name="out")
    oracle.compare(device.download(dl).astype(np.float64), lse_ref, 1e-3, 1e-3, name="lse")


@pytest.mark.parametrize("shape", [(1, 1, 8, 16), (2, 2, 16, 32), (1, 2, 100, 80)])
def test_attention_cuda_core_path(device, shape):
    z, h, n, d = shape
    rng = np.random.default_rng(8)
    q, k, v = (rng.standard_normal(shape).astype(np.float32) for _ in range(3))
    dq, dk, dv = (device.upload(t) for t in (q, k, v))
    do = device.upload(np.full(shape, POISON, np.float32))
    dl = device.upload(np.full((z, h, n), POISON, np.float32))
    ops.attention(dq, dk, dv, do, lse=dl, scale=0.25, causal=True)
    out_ref, lse_ref = oracle.attention_ref(q, k, v, 0.25, True)
    oracle.compare(device.download(do).astype(np.float64), out_ref, 1e-4, 1e-5)
    oracle.compare(device.download(dl).astype(np.float64), lse_ref, 1e-4, 1e-5)


@pytest.mark.parametrize("out_dtype", ["same", "float32"])
@pytest.mark.parametrize("dtype", ["bfloat16", "float16", "float32"])
@pytest.mark.parametrize("shape", [(1, 1, 64), (100, 24, 1000), (300, 64, 4096), (129, 200, 512),
                                   (4096, 256, 256), (257, 33, 72), (64, 24, 33)])
def test_linear_log_softmax_sweep(device, shape, dtype, out_dtype):
    """y = log_softmax(x @ w.T): the tensor-core GEMM with w as a K-major operand and the
    reduction in its epilogue; fp32 and unaligned rows on the CUDA-core kernel."""
    m, n, k = shape
    rng = np.random.default_rng(_seed(shape, dtype))
    x = _host(rng.standard_normal((m, k)), dtype)
    w = _host(rng.standard_normal((n, k)) / np.sqrt(k) * 3, dtype)
    dx, dw = _up(device, x, dtype), _up(device, w, dtype)
    ydt = dtype if out_dtype == "same" else "float32"
    dy = _poisoned(device, (m, n), ydt)
    ops.linear_log_softmax(dx, dw, dy)
    device.check_status()
    ref = oracle.log_softmax_linear_ref(x, w)
    rtol, atol = (2e-3, 2e-3) if dtype == "float32" else ((2e-2, 2e-2) if ydt != "float32" else (5e-3, 5e-3))
    oracle.compare(device.download(dy).astype(np.float64), ref, rtol, atol, name="y")


@pytest.mark.parametrize("dtype", ["bfloat16", "float16", "float32"])
@pytest.mark.parametrize("shape", [(1, 8, 64), (300, 136, 512), (1024, 1000, 4096), (129, 72, 100)])
def test_rms_matmul_sweep(device, shape, dtype):
    """out = rinv(x) * ((x * g) @ w): row factor applied in the GEMM epilogue."""
    m, n, k = shape
    rng = np.random.default_rng(_seed(shape, dtype))
    x = _host(rng.standard_normal((m, k)) * 0.5, dtype)
    g = _host(rng.standard_normal(k) * 0.2 + 1.0, dtype)
    w = _host(rng.standard_normal((k, n)) * 0.5, dtype)
    dx, dg, dw = (_up(device, t, dtype) for t in (x, g, w))
    do = _poisoned(device, (m, n), dtype)
    sw, sr = device.alloc((k, n), dtype), device.alloc((m,), "float32")
    ops.rms_matmul(dx, dg, dw, do, sw, sr, eps=1e-5)
    device.check_status()
    ref = oracle.rms_matmul_ref(x, g, w, 1e-5)
    # 16-bit: the products g*w are rounded once before the dot product (the reference rounds
    # x*g instead: the same error size); K such errors of about 2^-9 * 0.25 add up in a row
    rtol, atol = (1e-4, 5e-5 * np.sqrt(k)) if dtype == "float32" else (2e-2, 5e-3 * np.sqrt(k))
    oracle.compare(device.download(do).astype(np.float64), ref, rtol, atol, name="out")
    rinv_ref = 1.0 / np.sqrt((x.astype(np.float64) ** 2).mean(axis=1) + 1e-5)
    oracle.compare(device.download(sr).astype(np.float64), rinv_ref, 1e-5, 1e-6, name="rinv")


@pytest.mark.parametrize("dtype", ["bfloat16", "float16", "float32"])
@pytest.mark.parametrize("shape", [(1, 1), (33, 33), (64, 4096), (257, 1000), (1024, 11008),
                                   (1027, 8192), (3, 16)])
def test_dequantize_sweep(device, shape, dtype):
    k, n = shape
    rng = np.random.default_rng(_seed(shape, dtype))
    b = rng.integers(-127, 128, (k, n)).astype(np.int8)
    scale = _host(rng.random(n), dtype)
    db, ds = device.upload(b), _up(device, scale, dtype)
    do = _poisoned(device, (k, n), dtype)
    ops.dequantize_cols(db, ds, do)
    ref = oracle.dequantize_ref(b, scale)
    rtol = 1e-6 if dtype == "float32" else (1e-3 if dtype == "float16" else 8e-3)
    oracle.compare(device.download(do).astype(np.float64), ref, rtol, 1e-6, name="out")


@pytest.mark.parametrize("dtype", ["bfloat16", "float16", "float32"])
@pytest.mark.parametrize("shape", [(64, 128, 128, 32), (37, 192, 96, 32), (300, 512, 256, 64),
                                   (129, 320, 72, 16), (1000, 1024, 512, 8), (5, 64, 40, 32)])
def test_gemm_groupnorm_rowmin_sweep(device, shape, dtype):
    """GEMM + bias + group norm over column groups + row minimum, nothing but mins written.
    Operands on a 1/16 grid as in the reference's case, so the products are exact in 16 bits."""
    m, n, k, gs = shape
    if dtype == "float32" and gs != 32:
        pytest.skip("the CUDA-core path takes groups of 32")
    rng = np.random.default_rng(_seed(shape, dtype))
    x = _host(rng.integers(-16, 16, (m, k)) / 16, dtype)
    w = _host(rng.integers(-16, 16, (k, n)) / 16, dtype)
    bias = _host(rng.integers(-8, 9, n) / 16, dtype)
    gamma = _host(rng.integers(8, 24, n) / 16, dtype)
    beta = _host(rng.integers(-8, 9, n) / 16, dtype)
    x[0, :] = 0  # a row whose groups have (almost) no variance
    dx, dw, db, dg, dbt = (_up(device, t, dtype) for t in (x, w, bias, gamma, beta))
    start = np.full(m, np.inf, np.float32)
    start[m // 2] = -100.0  # an existing minimum must survive
    dm = device.upload(start)
    ops.gemm_groupnorm_rowmin(dx, dw, dg, dbt, dm, bias=db, group_size=gs, eps=1e-5)
    device.check_status()
    ref = oracle.gemm_groupnorm_rowmin_ref(x, w, bias, gamma, beta, gs, 1e-5)
    ref[m // 2] = min(ref[m // 2], -100.0)
    oracle.compare(device.download(dm).astype(np.float64), ref, 5e-3, 5e-3, name="mins")


def test_linear_log_softmax_rejections(device):
    from compiler_b200.runtime.abi import B200Error
    x = _up(device, _host(np.zeros((8, 64)), "bfloat16"), "bfloat16")
    with pytest.raises(B200Error):  # more outputs than one column block
        ops.linear_log_softmax(x, device.alloc((257, 64), "bfloat16"), device.alloc((8, 257), "bfloat16"))
    with pytest.raises(B200Error):  # K mismatch
        ops.linear_log_softmax(x, device.alloc((24, 32), "bfloat16"), device.alloc((8, 24), "bfloat16"))


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
@pytest.mark.parametrize("shape", [(2, 17, 2, 4, 7, 9, 9), (1, 300, 2, 2, 64, 64, 128),
                                   (2, 129, 1, 4, 32, 48, 0), (1, 1, 1, 1, 5, 3, 4)])
@pytest.mark.parametrize("extras", ["gate+sink", "plain"])
def test_attention_window_sweep(device, shape, dtype, extras):
    b, t, h, hq, kd, vd, window = shape
    rng = np.random.default_rng(_seed(shape, dtype, extras))
    q = _host(rng.normal(0, 0.5, (b, t, hq, kd)), dtype)
    k = _host(rng.normal(0, 0.5, (b, t, h, kd)), dtype)
    v = _host(rng.normal(0, 0.5, (b, t, h, vd)), dtype)
    use = extras == "gate+sink"
    gate = _host(np.cumsum(-np.abs(rng.normal(0, 0.1, (b, t, hq))), axis=1), dtype) if use else None
    sink = _host(rng.normal(0, 0.5, hq), dtype) if use else None
    dq, dk, dv = (_up(device, x, dtype) for x in (q, k, v))
    do = _poisoned(device, (b, t, hq, vd), dtype)
    dl = device.upload(np.full((b, t, hq), POISON, np.float32))
    scale = 1.0 / np.sqrt(kd)
    ops.attention_window(dq, dk, dv, do, g_cumsum=_up(device, gate, dtype) if use else None,
                         sink_bias=_up(device, sink, dtype) if use else None, lse=dl, scale=scale,
                         window=window)
    out_ref, lse_ref = oracle.window_attention_ref(q, k, v, gate, sink, scale, window)
    rtol, atol = (1e-4, 1e-5) if dtype == "float32" else TOL[dtype]
    oracle.compare(device.download(do).astype(np.float64), out_ref, rtol, atol, name="o")
    oracle.compare(device.download(dl).astype(np.float64), lse_ref, 1e-4, 1e-4, name="lse")


DECODE_SHAPES = [  # (query rows B, group, N_CTX, head_dim)
    (1, 1, 1, 16), (3, 1, 7, 32), (4, 1, 255, 64), (4, 1, 256, 128), (2, 1, 1000, 128),
    (5, 1, 4097, 64), (1, 1, 32768, 128),      # one row: its keys are split over a cluster
    (8, 4, 513, 128), (6, 2, 2048, 64),        # grouped-query layout
    (3, 1, 300, 24), (2, 2, 77, 80),           # head sizes of the one-CTA-per-row kernel
]


@pytest.mark.parametrize("dtype", ["bfloat16", "float16", "float32"])
@pytest.mark.parametrize("shape", DECODE_SHAPES)
def test_attention_decode_sweep(device, shape, dtype):
    rows, group, n, d = shape
    rng = np.random.default_rng(_seed(shape, dtype))
    q = _host(rng.standard_normal((rows, d)), dtype)
    k = _host(rng.standard_normal((rows // group, n, d)), dtype)
    v = _host(rng.standard_normal((rows // group, n, d)), dtype)
    dq, dk, dv = (_up(device, t, dtype) for t in (q, k, v))
    do = _poisoned(device, (rows, d), dtype)
    scale = 1.0 / np.sqrt(d)
    ops.attention_decode(dq, dk, dv, do, scale=scale)
    ref = oracle.flash_decode_ref(q, k, v, scale, group)
    rtol, atol = (1e-4, 1e-5) if dtype == "float32" else TOL[dtype]
    oracle.compare(device.download(do).astype(np.float64), ref, rtol, atol, name="out")


def test_attention_decode_strided_cache_and_rejections(device):
    """K / V as slices of a longer cache (row pitch > head size), an unaligned pitch (generic
    kernel), and descriptors the entry point refuses before anything is launched."""
    from compiler_b200.runtime.abi import B200Error
    rng = np.random.default_rng(41)
    rows, n, d, pitch = 4, 600, 64, 96
    q = _host(rng.standard_normal((rows, d)), "bfloat16")
    cache_k = _host(rng.standard_normal((rows, n, pitch)), "bfloat16")
    cache_v = _host(rng.standard_normal((rows, n, pitch)), "bfloat16")
    dq, dk, dv = (_up(device, t, "bfloat16") for t in (q, cache_k, cache_v))
    do = _poisoned(device, (rows, d), "bfloat16")
    scale = 0.125

    class Slice:  # the first d columns of every cache row
        def __init__(self, buffer, offset=0):
            self.buffer, self.shape, self.dtype, self.offset = buffer, (rows, n, d), buffer.dtype, offset

        def data_ptr(self):
            return self.buffer.data_ptr() + 2 * self.offset

        def stride(self):
            return (n * pitch, pitch, 1)

    ops.attention_decode(dq, Slice(dk), Slice(dv), do, scale=scale)
    ref = oracle.flash_decode_ref(q, cache_k[..., :d], cache_v[..., :d], scale)
    oracle.compare(device.download(do).astype(np.float64), ref, *TOL["bfloat16"])
    # columns [3, 3 + d): rows start 6 bytes off a 16-byte boundary
    do2 = _poisoned(device, (rows, d), "bfloat16")
    ops.attention_decode(dq, Slice(dk, 3), Slice(dv, 3), do2, scale=scale)
    ref = oracle.flash_decode_ref(q, cache_k[..., 3:3 + d], cache_v[..., 3:3 + d], scale)
    oracle.compare(device.download(do2).astype(np.float64), ref, *TOL["bfloat16"])
    with pytest.raises(B200Error):   # 3 query rows cannot share 2 K/V heads
        ops.attention_decode(_up(device, q[:3], "bfloat16"),
                             _up(device, cache_k[:2, :, :d].copy(), "bfloat16"),
                             _up(device, cache_v[:2, :, :d].copy(), "bfloat16"),
                             _poisoned(device, (3, d), "bfloat16"), scale=scale)
    with pytest.raises(B200Error):   # softmax over no keys
        empty = device.alloc((rows, 0, d), "bfloat16")
        ops.attention_decode(dq, empty, empty, do, scale=scale)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("shape", [(4, 64), (8, 128), (5, 99), (64, 1024), (33, 14336),
                                   (1031, 4096)])
def test_swiglu_sweep(device, shape, dtype):
    rng = np.random.default_rng(9)
    x, y = (_host(rng.standard_normal(shape), dtype) for _ in range(2))
    dx, dy = _up(device, x, dtype), _up(device, y, dtype)
    dout = _poisoned(device, shape, dtype)
    ops.swiglu(dx, dy, dout)
    rtol, atol = (1e-4, 1e-5) if dtype == "float32" else TOL[dtype]
    oracle.compare(device.download(dout).astype(np.float64), oracle.swiglu_ref(x, y), rtol, atol)


VARIANT_SHAPES = [(4, 16), (4, 97), (3, 1000), (64, 1024), (10, 4000), (6, 4104), (5, 8192),
                  (2, 33000), (3, 70000)]


@pytest.mark.parametrize("dtype", ["float32", "float16", "bfloat16"])
@pytest.mark.parametrize("shape", VARIANT_SHAPES)
def test_softmax_mul_sweep(device, shape, dtype):
    rng = np.random.default_rng(_seed(shape, dtype, "mul"))
    x = _host(rng.standard_normal(shape) * 2, dtype)
    o = _host(rng.uniform(-2, 2, shape), dtype)
    dx, do, dy = _up(device, x, dtype), _up(device, o, dtype), _poisoned(device, shape, dtype)
    ops.softmax_variant(dx, dy, mul=do)
    rtol, atol = (2e-3, 1e-6) if dtype == "float32" else TOL[dtype]
    oracle.compare(device.download(dy).astype(np.float64), oracle.softmax_mul_ref(x, o), rtol, atol)


@pytest.mark.parametrize("dtype", ["float32", "float16", "bfloat16"])
@pytest.mark.parametrize("shape", VARIANT_SHAPES)
def test_softmax_log_sweep(device, shape, dtype):
    """softmax(log x): positive rows, rows with zeros (log 0 = -inf: weight 0), and the rows
    the reference turns into NaN as a whole: a negative entry, a NaN entry, an infinite entry,
    an all-zero row (ops/suite/perf/softmax_log.py:27-31)."""
    rows, cols = shape
    rng = np.random.default_rng(_seed(shape, dtype, "log"))
    x = rng.uniform(0.05, 4.0, shape).astype(np.float32)
    x[0, :: 3] = 0.0
    if rows > 1:
        x[1, cols // 2] = -1.0
    if rows > 2:
        x[2, cols - 1] = np.nan
    if rows > 3:
        x[3, 0] = np.inf
    if rows > 4:
        x[4, :] = 0.0
    x = _host(x, dtype)
    dx, dy = _up(device, x, dtype), _poisoned(device, shape, dtype)
    ops.softmax_variant(dx, dy, log_input=True)
    y = device.download(dy).astype(np.float64)
    ref = oracle.softmax_log_ref(x)
    rtol, atol = (2e-3, 1e-6) if dtype == "float32" else TOL[dtype]
    oracle.compare(y, ref, rtol, atol, equal_nan=True)
    for r in range(1, min(rows, 5)):
        assert np.isnan(y[r]).all(), f"row {r} must be NaN as a whole"
    assert not np.isnan(y[0]).any()


@pytest.mark.parametrize("dtype", ["float32", "float16", "bfloat16"])
@pytest.mark.parametrize("case", [((4, 16), 2, None), ((3, 100), 3, 299), ((5, 1000), 4, None),
                                  ((64, 1024), 4, None), ((7, 1024), 8, 8000), ((3, 513), 5, 2560),
                                  ((2, 4096), 1, None), ((2, 20000), 4, None)])
def test_repeat_log_softmax_sweep(device, case, dtype):
    shape, repeat, length = case
    rng = np.random.default_rng(_seed(case, dtype))
    x = _host(rng.standard_normal(shape) * 2, dtype)
    out_len = shape[1] * repeat if length is None else length
    dx, dy = _up(device, x, dtype), _poisoned(device, (shape[0], out_len), dtype)
    ops.repeat_log_softmax(dx, dy, repeat)
    ref = oracle.repeat_log_softmax_ref(x, repeat, out_len)
    rtol, atol = (1e-4, 1e-5) if dtype == "float32" else TOL[dtype]
    # the log-probabilities are of size log(length): the 16-bit tolerance is on their scale
    if dtype != "float32":
        atol = max(atol, 2 * rtol * np.log(out_len))
    oracle.compare(device.download(dy).astype(np.float64), ref, rtol, atol)


@pytest.mark.parametrize("dtype", ["float32", "float16", "bfloat16"])
@pytest.mark.parametrize("n", [1, 7, 8, 1000, 4099, 1 << 20, (1 << 20) + 13, 1_200_000,
                               12_000_000])
def test_elementwise_family_sweep(device, n, dtype):
    """The flat GELU family over lengths with and without a ragged end of the 16-byte vectors;
    the two largest lengths make the bias index of the epilogue operator wrap inside a thread's
    slots (1.2 M) and across the grid's passes (12 M)."""
    rng = np.random.default_rng(_seed(n, dtype))
    a = _host(rng.standard_normal(n) * 2, dtype)
    b = _host(rng.standard_normal(n), dtype)
    da, db = _up(device, a, dtype), _up(device, b, dtype)
    rtol, atol = (1e-4, 1e-5) if dtype == "float32" else TOL[dtype]

    def run(op, second=None, **params):
        dout = _poisoned(device, (n,), dtype)
        ops.elementwise(op, da, dout, b=second, **params)
        return device.download(dout).astype(np.float64)

    oracle.compare(run(abi.EW_GELU_ERF), oracle.gelu_erf(a.astype(np.float64)), rtol, atol)
    oracle.compare(run(abi.EW_ADD_GELU_ERF, db, p0=1.5), oracle.add_gelu_ref(a, b, 1.5), rtol, atol)
    oracle.compare(run(abi.EW_GEGLU_TANH, db), oracle.geglu_tanh_ref(a, b), rtol, atol)
    for n_cols in (1, 8, 24, 1000, 2400, 4096):
        if n % n_cols:
            continue
        bias = _host(rng.standard_normal(n_cols), dtype)
        dbias = _up(device, bias, dtype)
        ref = oracle.epilogue_ref(a, bias, n_cols, 0.75, -1.5, 2.0)
        oracle.compare(run(abi.EW_BIAS_SCALE_CLAMP_GELU, dbias, p0=0.75, p1=-1.5, p2=2.0), ref,
                       rtol, atol)


# ------------------------------------------------------------------ native handles
def test_native_handles_through_the_launch_surface(device):
    """The BASELINE configurations use handles the registry resolves like any kernel."""
    rng = np.random.default_rng(10)
    rows, cols = 16, 4000
    x = _host(rng.standard_normal((rows, cols)) * 2, "float16")
    case = {"kernel": kernels.masked_softmax_kernel,
            "args": {"x_ptr": x, "y_ptr": np.zeros_like(x), "n_cols": cols, "row_offset": 3990},
            "meta": {}, "grid": (rows,), "outputs": ("y_ptr",)}
    y = harness.run_case(case, device)["y_ptr"]
    oracle.compare(y.astype(np.float64), oracle.masked_softmax_ref(x, 3990), 1e-2, 1e-2)

    m, n, k = 96, 136, 72
    a = _host(rng.standard_normal((m, k)) / np.sqrt(k), "bfloat16")
    b = _host(rng.standard_normal((k, n)), "bfloat16")
    bias = _host(rng.normal(0, 0.1, n), "bfloat16")
    case = {"kernel": kernels.gemm_bias_act_kernel,
            "args": {"a_ptr": a, "b_ptr": b, "bias_ptr": bias, "c_ptr": np.zeros((m, n), np.float32),
                     "M": m, "N": n, "K": k},
            "meta": {"ACT": abi.ACT_GELU_TANH}, "grid": (1,), "outputs": ("c_ptr",),
            "pointer_dtypes": {name: "bfloat16" for name in ("a_ptr", "b_ptr", "bias_ptr", "c_ptr")}}
    c = harness.run_case(case, device)["c_ptr"]
    oracle.compare(c.astype(np.float64), oracle.linear_act_ref(a, b, bias, "gelu_tanh"), 2e-2, 2e-2)


def test_compiled_kernel_callable(device):
    """``make_compiler().compile_case(case)[grid](*args, **meta)`` launches the operator."""
    from compiler_b200.factory import make_compiler
    compiler = make_compiler()
    rng = np.random.default_rng(12)
    x = rng.standard_normal((8, 256)).astype(np.float32)
    case, _ = golden_cases.load("softmax__4x16__float32")
    artifact = compiler.compile_case(case).bind(device)
    again = compiler.compile_case(case)
    assert compiler.compile_count == 1 and compiler.cache_hits == 1 and again.cache_hit
    assert again.identity == artifact.identity and len(artifact.sha256) == 64
    dx, dy = device.upload(x), device.upload(np.zeros_like(x))
    artifact[(8,)](dx, dy, 256, BLOCK_N=1024)
    oracle.compare(device.download(dy).astype(np.float64), oracle.softmax_ref(x), 2e-3, 1e-6)


def test_unknown_kernel_is_a_located_refusal(device):
    from compiler_b200.registry import UnsupportedLaunch
    handle = golden_cases.make_handle("mystery_kernel", ["a_ptr", "n"])
    with pytest.raises(UnsupportedLaunch) as err:
        device.launch(handle, (1,), [device.alloc((4,), "float32"), 4], {})
    assert err.value.kernel_name == "mystery_kernel" and "no native" in err.value.message


# ------------------------------------------------------------------ repeat consistency
def test_repeat_launches_are_bitwise_identical(device):
    """The --repeats check of a100c/runtime/main.c:117-152 for the pipelined kernels."""
    import ctypes
    rng = np.random.default_rng(13)
    m, n, k = 512, 768, 1024
    a = _host(rng.standard_normal((m, k)) / np.sqrt(k), "bfloat16")
    b = _host(rng.standard_normal((k, n)), "bfloat16")
    da, db = _up(device, a, "bfloat16"), _up(device, b, "bfloat16")
    outs = [_poisoned(device, (m, n), "bfloat16") for _ in range(3)]
    for out in outs:
        ops.gemm(da, db, out, act=abi.ACT_GELU_TANH)
    shape = (1, 4, 512, 128)
    q, kk, v = (_host(rng.standard_normal(shape), "bfloat16") for _ in range(3))
    dq, dk, dv = (_up(device, t, "bfloat16") for t in (q, kk, v))
    attn = [_poisoned(device, shape, "bfloat16") for _ in range(3)]
    for out in attn:
        ops.attention(dq, dk, dv, out, causal=True)
    device.check_status()
    for group in (outs, attn):
        for other in group[1:]:
            equal = ctypes.c_int()
            status = abi.lib().b200_bitwise_equal(group[0].ptr, other.ptr, group[0].nbytes,
                                                  ctypes.byref(equal), 0)
            assert status == abi.OK and equal.value == 1


# ------------------------------------------------------------------ fused reduce-scatter path
@pytest.mark.parametrize("staged", ["bfloat16", "float16"])
@pytest.mark.parametrize("world", [1, 2, 4])
def test_scatter_gemm_and_reduce_emulated_ranks(device, world, staged):
    """The tensor-parallel all-reduce pieces on ONE GPU: every "rank" is a set of local
    buffers.  Rank r multiplies its K-shard and its GEMM epilogue scatters row blocks to the
    owners' staging slots (in the operands' type, or as float16: three more mantissa bits for
    the partials at the same traffic); each owner then sums its slots and broadcasts the rows
    to every rank's output.  All outputs must equal the unsharded product."""
    import ctypes
    lib = abi.lib()
    rows, n, k = 128, 264, 96 * world
    m = rows * world
    rng = np.random.default_rng(21)
    a = _host(rng.standard_normal((m, k)) / np.sqrt(k), "bfloat16")
    b = _host(rng.standard_normal((k, n)), "bfloat16")
    staging = [_poisoned(device, (world, rows, n), staged) for _ in range(world)]
    outputs = [_poisoned(device, (m, n), "bfloat16") for _ in range(world)]
    ptrs = ctypes.c_void_p * world
    staging_ptrs = ptrs(*[s.ptr for s in staging])
    output_ptrs = ptrs(*[o.ptr for o in outputs])
    ks = k // world
    for r in range(world):
        da = _up(device, np.ascontiguousarray(a[:, r * ks:(r + 1) * ks]), "bfloat16")
        db = _up(device, np.ascontiguousarray(b[r * ks:(r + 1) * ks]), "bfloat16")
        ta = abi.make_tensor(da.ptr, (m, ks), "bfloat16")
        tb = abi.make_tensor(db.ptr, (ks, n), "bfloat16")
        tc = abi.make_tensor(outputs[r].ptr, (m, n), staged)
        abi.check(lib.b200_gemm_scatter_rows(ctypes.byref(ta), ctypes.byref(tb), ctypes.byref(tc),
                                             staging_ptrs, world, r, rows, device.stream))
    for owner in range(world):
        abi.check(lib.b200_reduce_slices_broadcast(staging[owner].ptr, abi.DTYPE_CODES[staged],
                                                   abi.DTYPE_CODES["bfloat16"], world, rows, n,
                                                   owner * rows, output_ptrs, device.stream))
    device.check_status()
    ref = oracle.matmul_ref(a, b)
    for r in range(world):
        oracle.compare(device.download(outputs[r]).astype(np.float64), ref, 2e-2, 2e-2,
                       name=f"rank {r}")


@pytest.mark.parametrize("partial_dtype", ["float16", "bfloat16"])
@pytest.mark.parametrize("world", [2, 3, 4, 8])
def test_peer_load_allreduce_emulated_ranks(device, world, partial_dtype):
    """``b200_peer_allreduce`` on ONE GPU: every "rank" is a pair of local buffers and the
    launches run one after the other without the cross-rank barriers (no signal pads).  Rank r
    sums its share of every rank's partial in fp32, in rank order, and stores the rounded sums
    into every rank's output (even ranks on 3 CTAs, so each CTA walks many steps): after all
    ranks have run, every output holds the sum over the whole range -- bit for bit the fp32
    sum in rank order rounded once -- and nothing outside [offset, offset + count) is touched.  World sizes 2 / 3-4 / 8 take the three unrollings of
    the kernel (8 x 2, 4 x 4, 2 x 8 loads in flight)."""
    import ctypes
    lib = abi.lib()
    offset, count = 64, 8 * world * 40_001   # a ragged last step of every unrolling
    total = offset + count + 40
    rng = np.random.default_rng(77 + world)
    partials = [_host(rng.standard_normal(total) * 3, partial_dtype) for _ in range(world)]
    d_partials = [_up(device, p, partial_dtype) for p in partials]
    outputs = [_poisoned(device, (total,), "bfloat16") for _ in range(world)]
    ptrs = ctypes.c_void_p * world
    partial_ptrs, output_ptrs = ptrs(*[p.ptr for p in d_partials]), ptrs(*[o.ptr for o in outputs])
    for r in range(world):
        abi.check(lib.b200_peer_allreduce(partial_ptrs, abi.DTYPE_CODES[partial_dtype],
                                          output_ptrs, abi.DTYPE_CODES["bfloat16"], offset, count,
                                          r, world, None, 0, 0 if r % 2 else 3, device.stream))
    device.check_status()
    acc = np.zeros(count, np.float32)
    for p in partials:                              # fp32, rank order: what the kernel does
        acc = acc + np.asarray(p[offset:offset + count], np.float32)
    expect = oracle.to_storage(acc, "bfloat16")
    for r in range(world):
        got = np.asarray(device.download(outputs[r]), np.float32)
        assert np.array_equal(got[offset:offset + count], np.asarray(expect, np.float32)), r
        assert np.all(got[:offset] == POISON) and np.all(got[offset + count:] == POISON), r
    # a count the ranks cannot share in whole vectors never reaches the device
    assert lib.b200_peer_allreduce(partial_ptrs, abi.DTYPE_CODES[partial_dtype], output_ptrs,
                                   abi.DTYPE_CODES["bfloat16"], 0, 8 * world + 8, 0, world, None,
                                   0, 0, device.stream) == abi.REJECTED


@pytest.mark.parametrize("shape,rows_per_block", [((4096, 4096, 2048), 1024),   # split last wave
                                                   ((2048, 4096, 512), 512),     # whole tiles only
                                                   ((4096, 2048, 1024), 768)])   # ragged last block
def test_gemm_progress_feeds_the_allreduce_beside_it(device, shape, rows_per_block):
    """``b200_gemm_progress`` + ``b200_peer_allreduce_blocks`` on one GPU (a world of one rank:
    the "all-reduce" rounds the float16 partial into the bfloat16 result).  The all-reduce
    kernel is launched behind the GEMM as its programmatic dependent and takes every block of
    rows when the GEMM has counted it complete: the result must be the product, the counters
    must be back at zero, and a second pair of launches must give the same bits."""
    import ctypes
    lib = abi.lib()
    m, n, k = shape
    rng = np.random.default_rng(sum(shape))
    a = _host(rng.standard_normal((m, k)) / np.sqrt(k), "bfloat16")
    b = _host(rng.standard_normal((k, n)), "bfloat16")
    da, db = _up(device, a, "bfloat16"), _up(device, b, "bfloat16")
    partial = _poisoned(device, (m, n), "float16")
    out = _poisoned(device, (m, n), "bfloat16")
    words = lib.b200_progress_words()
    counters = device.upload(np.zeros(words, np.int32))
    ta = abi.make_tensor(da.ptr, (m, k), "bfloat16")
    tb = abi.make_tensor(db.ptr, (k, n), "bfloat16")
    tc = abi.make_tensor(partial.ptr, (m, n), "float16")
    partial_ptrs, out_ptrs = (ctypes.c_void_p * 1)(partial.ptr), (ctypes.c_void_p * 1)(out.ptr)
    results = []
    for _ in range(2):
        targets = (ctypes.c_uint32 * 16)()
        blocks = ctypes.c_int(0)
        abi.check(lib.b200_gemm_progress(ctypes.byref(ta), ctypes.byref(tb), ctypes.byref(tc),
                                         rows_per_block, counters.ptr, targets, 16,
                                         ctypes.byref(blocks), device.stream))
        assert blocks.value == -(-m // rows_per_block)
        # eight epilogue warps per tile of 256 x 256, more where the last wave is split
        tiles = [min(rows_per_block, m - g * rows_per_block) // 256 * (n // 256)
                 for g in range(blocks.value)]
        assert all(targets[g] >= 8 * tiles[g] for g in range(blocks.value))
        assert sum(targets[g] == 8 * tiles[g] for g in range(blocks.value)) >= blocks.value - 1
        abi.check(lib.b200_peer_allreduce_blocks(
            partial_ptrs, abi.DTYPE_CODES["float16"], out_ptrs, abi.DTYPE_CODES["bfloat16"],
            m * n, rows_per_block * n, counters.ptr, targets, 0, 1, None, 0, 0, device.stream))
        device.check_status()
        results.append(np.asarray(device.download(out), np.float32).copy())
        # the counters and the count of CTAs done with them; time stamps follow them
        assert not device.download(counters)[:17].any()
    assert np.array_equal(results[0], results[1])
    oracle.compare(results[0].astype(np.float64), oracle.matmul_ref(a, b), 2e-2, 2e-2)
    # a shape below one wave of tile pairs has no CTA-pair kernel to count
    small = abi.make_tensor(da.ptr, (256, k), "bfloat16")
    small_c = abi.make_tensor(partial.ptr, (256, n), "float16")
    targets, blocks = (ctypes.c_uint32 * 16)(), ctypes.c_int(0)
    assert lib.b200_gemm_progress(ctypes.byref(small), ctypes.byref(tb), ctypes.byref(small_c), 256,
                                  counters.ptr, targets, 16, ctypes.byref(blocks),
                                  device.stream) == abi.REJECTED


def test_scatter_gemm_rejections(device):
    import ctypes
    lib = abi.lib()
    buf = device.alloc((256, 64), "bfloat16")
    t = abi.make_tensor(buf.ptr, (256, 64), "bfloat16")
    tb = abi.make_tensor(buf.ptr, (64, 64), "bfloat16")
    tc = abi.make_tensor(buf.ptr, (256, 64), "bfloat16")
    ptrs = (ctypes.c_void_p * 2)(buf.ptr, buf.ptr)
    # rows per rank must be a multiple of the 128-row tile and cover M
    assert lib.b200_gemm_scatter_rows(ctypes.byref(t), ctypes.byref(tb), ctypes.byref(tc), ptrs, 2,
                                      0, 100, device.stream) == abi.REJECTED
    assert lib.b200_gemm_scatter_rows(ctypes.byref(t), ctypes.byref(tb), ctypes.byref(tc), ptrs, 9,
                                      0, 128, device.stream) == abi.REJECTED
    assert lib.b200_reduce_slices_broadcast(buf.ptr, abi.DTYPE_CODES["float32"],
                                            abi.DTYPE_CODES["bfloat16"], 2, 128, 64, 0,
                                            ptrs, device.stream) == abi.REJECTED
