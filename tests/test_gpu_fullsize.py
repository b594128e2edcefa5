"""The full-size configurations (the shapes the benchmark times), checked through
size-independent properties plus oracle comparisons on sampled rows / heads, since the
float64 oracle takes minutes on the whole tensors."""
import numpy as np
import pytest

from compiler_b200 import ops
from compiler_b200.runtime import abi
from oracle import oracle

pytestmark = pytest.mark.gpu


def test_rmsnorm_8192x4096_fp32(device):
    rng = np.random.default_rng(30)
    x = rng.standard_normal((8192, 4096), dtype=np.float32)
    w = rng.uniform(0.5, 1.5, 4096).astype(np.float32)
    dx, dw = device.upload(x), device.upload(w)
    dy, dr = device.alloc(x.shape, "float32"), device.alloc((8192,), "float32")
    ops.rmsnorm(dx, dw, dy, dr, eps=1e-6)
    y, r = device.download(dy), device.download(dr)
    y_ref, r_ref = oracle.rmsnorm_ref(x, w, 1e-6)          # ~1 s on the host
    oracle.compare(y.astype(np.float64), y_ref, 1e-5, 1e-6, name="Y")
    oracle.compare(r.astype(np.float64), r_ref, 1e-5, 1e-6, name="r")
    # property: mean((y/w)^2) == 1 - eps*inv^2 per row, independent of size
    ms = ((y.astype(np.float64) / w) ** 2).mean(axis=1)
    np.testing.assert_allclose(ms, 1.0 - 1e-6 * r.astype(np.float64) ** 2, rtol=1e-5)


def test_masked_softmax_16384x4000_fp16(device):
    rng = np.random.default_rng(31)
    rows, cols = 16384, 4000
    x = (rng.standard_normal((rows, cols), dtype=np.float32) * 2).astype(np.float16)
    dx, dy = device.upload(x), device.alloc(x.shape, "float16")
    ops.softmax(dx, dy, causal_mod=True, row_offset=0)
    y = device.download(dy)
    # properties: rows sum to 1, masked part is exactly zero, row r keeps r % 4000 + 1 columns
    sums = y.astype(np.float64).sum(axis=1)
    np.testing.assert_allclose(sums, 1.0, atol=4e-3)
    keep = np.arange(rows) % cols + 1
    mask = np.arange(cols)[None, :] < keep[:, None]
    assert not y[~mask].any()
    assert (y[mask] >= 0).all()
    # oracle on a spread of rows, including the shortest and longest
    sample = np.array([0, 1, 7, 3999, 4000, 4001, 8191, 12345, 16383])
    ref = oracle.masked_softmax_ref(x[sample[0]:sample[0] + 1], 0)
    for r in sample:
        ref = oracle.masked_softmax_ref(x[r:r + 1], r)
        oracle.compare(y[r:r + 1].astype(np.float64), ref, 1e-2, 1e-2, name=f"row{r}")


@pytest.mark.parametrize("shape", [(8192, 8192, 8192), (4097, 11008, 4096)])
def test_gemm_bias_gelu_fullsize(device, shape):
    m, n, k = shape
    rng = np.random.default_rng(32)
    a = oracle.bf16_round(rng.standard_normal((m, k), dtype=np.float32) / np.sqrt(k))
    b = oracle.bf16_round(rng.standard_normal((k, n), dtype=np.float32) / np.sqrt(k))
    bias = oracle.bf16_round(rng.normal(0, 0.1, n).astype(np.float32))
    da, db, dbias = (device.upload(t, "bfloat16") for t in (a, b, bias))
    dc = device.alloc((m, n), "bfloat16")
    ops.gemm(da, db, dc, bias=dbias, act=abi.ACT_GELU_TANH)
    device.check_status()
    c = device.download(dc)
    assert np.isfinite(c).all()
    rows = np.array([0, 1, 127, 128, m // 2 + 3, m - 129, m - 2, m - 1])
    ref = oracle.linear_act_ref(a[rows], b, bias, "gelu_tanh")
    oracle.compare(c[rows].astype(np.float64), ref, 2e-2, 2e-2, name="rows")
    cols = np.array([0, 255, 256, n // 2 + 1, n - 257, n - 1])
    ref_c = oracle.linear_act_ref(a, b[:, cols], bias[cols], "gelu_tanh")
    oracle.compare(c[:, cols].astype(np.float64), ref_c, 2e-2, 2e-2, name="cols")


def test_attention_fullsize_heads(device):
    """The BASELINE tensor itself, [8,32,4096,128] causal bf16 (1 GiB on the device): the
    kernel's work order depends on the number of (batch, head) pairs (balanced pairs of query
    blocks dealt head by head over the SMs, in waves of a few heads), so heads are checked
    where that order changes -- the first and last head, both sides of wave boundaries and of
    the point where the CTAs wrap around -- against the float64 oracle per head; every head
    goes through the cheap properties; and one head is launched again on its own, which must
    give the same numbers whatever work order surrounded it."""
    z, h, n, d = 8, 32, 4096, 128
    rng = np.random.default_rng(33)
    q, k, v = (oracle.bf16_round(rng.standard_normal((z, h, n, d), dtype=np.float32))
               for _ in range(3))
    dq, dk, dv = (device.upload(t, "bfloat16") for t in (q, k, v))
    do = device.alloc((z, h, n, d), "bfloat16")
    dl = device.alloc((z, h, n), "float32")
    scale = 1.0 / np.sqrt(d)
    ops.attention(dq, dk, dv, do, lse=dl, scale=scale, causal=True)
    device.check_status()
    out, lse = device.download(do), device.download(dl)
    assert np.isfinite(out).all() and np.isfinite(lse).all()
    for flat in (0, 3, 4, 37, 127, 128, 255):
        zi, hi = divmod(flat, h)
        out_ref, lse_ref = oracle.attention_head_ref(q[zi, hi], k[zi, hi], v[zi, hi], scale, True)
        oracle.compare(out[zi, hi].astype(np.float64), out_ref, 2e-2, 2e-2, name=f"out[{zi},{hi}]")
        oracle.compare(lse[zi, hi].astype(np.float64), lse_ref, 1e-3, 1e-3, name=f"lse[{zi},{hi}]")
    # row 0 attends only to key 0: out == v[0], lse == scale * q0.k0 -- all 256 heads
    np.testing.assert_allclose(out[:, :, 0, :], v[:, :, 0, :], rtol=1e-2, atol=1e-2)
    s00 = scale * np.einsum("zhd,zhd->zh", q[:, :, 0, :].astype(np.float64),
                            k[:, :, 0, :].astype(np.float64))
    np.testing.assert_allclose(lse[:, :, 0], s00, rtol=1e-4, atol=1e-4)
    # row 1 of every head: two keys, closed form
    s1 = scale * np.einsum("zhd,zhkd->zhk", q[:, :, 1, :].astype(np.float64),
                           k[:, :, :2, :].astype(np.float64))
    np.testing.assert_allclose(lse[:, :, 1], np.log(np.exp(s1).sum(-1)), rtol=1e-4, atol=1e-4)
    # one head on its own ([1,1,4096,128]) gives what it gave inside the 256-head launch
    zi, hi = 5, 17
    d1 = [device.upload(np.ascontiguousarray(t[zi:zi + 1, hi:hi + 1]), "bfloat16")
          for t in (q, k, v)]
    o1, l1 = device.alloc((1, 1, n, d), "bfloat16"), device.alloc((1, 1, n), "float32")
    ops.attention(*d1, o1, lse=l1, scale=scale, causal=True)
    device.check_status()
    np.testing.assert_allclose(device.download(l1)[0, 0], lse[zi, hi], rtol=0, atol=1e-5)
    np.testing.assert_allclose(device.download(o1)[0, 0], out[zi, hi], rtol=2 ** -7, atol=1e-6)
    # batch shards (what each of 8 GPUs would run): slab 3 alone equals slab 3 of the whole
    d3 = [device.upload(np.ascontiguousarray(t[3:4]), "bfloat16") for t in (q, k, v)]
    o3, l3 = device.alloc((1, h, n, d), "bfloat16"), device.alloc((1, h, n), "float32")
    ops.attention(*d3, o3, lse=l3, scale=scale, causal=True)
    device.check_status()
    np.testing.assert_allclose(device.download(l3)[0], lse[3], rtol=0, atol=1e-5)
    np.testing.assert_allclose(device.download(o3)[0], out[3], rtol=2 ** -7, atol=1e-6)


def test_row_shards_equal_the_unsharded_result(device):
    """The BASELINE row operators split 8 ways (what each GPU of a box runs): a block of rows
    launched on its own, with its global row offset, gives the rows of the unsharded launch."""
    rng = np.random.default_rng(34)
    rows, cols, parts = 16384, 4000, 8
    x = (rng.standard_normal((rows, cols), dtype=np.float32) * 2).astype(np.float16)
    dx, dy = device.upload(x), device.alloc(x.shape, "float16")
    ops.softmax(dx, dy, causal_mod=True, row_offset=0)
    whole = device.download(dy)
    block = rows // parts
    for part in (0, 1, 5, 7):
        lo = part * block
        sx, sy = device.upload(x[lo:lo + block]), device.alloc((block, cols), "float16")
        ops.softmax(sx, sy, causal_mod=True, row_offset=lo)
        got = device.download(sy)
        np.testing.assert_allclose(got.astype(np.float32), whole[lo:lo + block].astype(np.float32),
                                   rtol=0, atol=2e-3)
        for r in (0, block // 2, block - 1):
            oracle.compare(got[r:r + 1].astype(np.float64),
                           oracle.masked_softmax_ref(x[lo + r:lo + r + 1], lo + r), 1e-2, 1e-2,
                           name=f"shard {part} row {r}")
    xr = rng.standard_normal((8192, 4096), dtype=np.float32)
    w = rng.uniform(0.5, 1.5, 4096).astype(np.float32)
    dxr, dw = device.upload(xr), device.upload(w)
    dyr, dr = device.alloc(xr.shape, "float32"), device.alloc((8192,), "float32")
    ops.rmsnorm(dxr, dw, dyr, dr, eps=1e-6)
    whole_y, whole_r = device.download(dyr), device.download(dr)
    for part in (0, 6):
        lo = part * 1024
        sx = device.upload(xr[lo:lo + 1024])
        sy, sr = device.alloc((1024, 4096), "float32"), device.alloc((1024,), "float32")
        ops.rmsnorm(sx, dw, sy, sr, eps=1e-6)
        np.testing.assert_allclose(device.download(sy), whole_y[lo:lo + 1024], rtol=1e-6)
        np.testing.assert_allclose(device.download(sr), whole_r[lo:lo + 1024], rtol=1e-6)
