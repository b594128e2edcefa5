"""Pins the CPU oracle against outputs of the reference's own ``ref`` functions.

The fixtures hold, for every declared shape and dtype of the hot-path operator
files, the inputs and the ``expected`` arrays the reference computed.  The oracle
must reproduce them to float64 round-off (the only difference allowed is the
final cast to the output storage type, which the fixtures already applied).
"""
import numpy as np
import pytest

import golden_cases
from oracle import oracle


def _cast_like(value, like, dtype):
    """Apply the reference's final ``astype(output dtype)`` and bf16 host rounding."""
    out = np.asarray(value).astype(like.dtype)
    return out


def _assert_same(actual, expected, dtype):
    # ref() rounds once to the host array dtype; bf16 hosts are float32, so the
    # reference's expected values are float32-rounded float64 results.
    np.testing.assert_allclose(actual.astype(np.float64), expected.astype(np.float64),
                               rtol=1e-6 if expected.dtype == np.float32 else 2e-3, atol=1e-7
                               if expected.dtype == np.float32 else 1e-3)


@pytest.mark.parametrize("tag", golden_cases.tags("fast_rms_layernorm"))
def test_rmsnorm(tag):
    case, meta = golden_cases.load(tag)
    a = case["args"]
    y, r = oracle.rmsnorm_ref(a["X"], a["W"], a["eps"])
    _assert_same(_cast_like(y, case["expected"]["Y"], meta["dtype"]), case["expected"]["Y"], meta["dtype"])
    _assert_same(_cast_like(r, case["expected"]["r"], meta["dtype"]), case["expected"]["r"], meta["dtype"])


@pytest.mark.parametrize("tag", golden_cases.tags("hidden__rms_norm_loop_kernel"))
def test_rmsnorm_loop_variant(tag):
    # this dev-lane file's ref computes in the ARRAY dtype (no float64 widening,
    # ops/suite/dev/hidden__rms_norm_loop_kernel.py ref), so its fp16/bf16 expected values
    # carry storage-precision arithmetic: cross-check with the case's own tolerance
    case, meta = golden_cases.load(tag)
    a = case["args"]
    rows, n = case["grid"][0], a["N"]
    y, r = oracle.rmsnorm_ref(a["in_ptr"].reshape(rows, n), a["w_ptr"][:n], a["eps"])
    for name, value in (("out_ptr", y.reshape(-1)), ("INV_RMS", r)):
        policy = case["comparison"][name]
        oracle.compare(value.astype(case["expected"][name].dtype), case["expected"][name],
                       policy["rtol"], policy["atol"], name=name)


@pytest.mark.parametrize("tag", golden_cases.tags("softmax"))
def test_softmax(tag):
    case, meta = golden_cases.load(tag)
    y = oracle.softmax_ref(case["args"]["x_ptr"])
    _assert_same(y.astype(case["expected"]["y_ptr"].dtype), case["expected"]["y_ptr"], meta["dtype"])


@pytest.mark.parametrize("tag", golden_cases.tags("softmax_kernel_inner"))
def test_softmax_inner(tag):
    case, meta = golden_cases.load(tag)
    a = case["args"]
    y = oracle.softmax_ref(a["input_ptr"].reshape(a["M"], a["N"]))
    _assert_same(y.reshape(-1).astype(case["expected"]["output_ptr"].dtype),
                 case["expected"]["output_ptr"], meta["dtype"])


@pytest.mark.parametrize("tag", golden_cases.tags("softmax_multi_block_forward_kernel"))
def test_softmax_multi_block(tag):
    # this operator file's ref works in float32 (softmax_multi_block_forward_kernel.py:93-98)
    case, meta = golden_cases.load(tag)
    y = oracle.softmax_ref(case["args"]["X_ptr"])
    _assert_same(y.astype(case["expected"]["Y_ptr"].dtype), case["expected"]["Y_ptr"],
                 meta["dtype"])


@pytest.mark.parametrize("tag", golden_cases.tags("matmul"))
def test_matmul(tag):
    case, meta = golden_cases.load(tag)
    y = oracle.matmul_ref(case["args"]["a_ptr"], case["args"]["b_ptr"])
    _assert_same(y.astype(case["expected"]["y_ptr"].dtype), case["expected"]["y_ptr"], meta["dtype"])


@pytest.mark.parametrize("tag", golden_cases.tags("matmul_triton2"))
def test_matmul_leaky(tag):
    case, meta = golden_cases.load(tag)
    a = case["args"]
    act = "leaky_relu" if case["meta"].get("LEAKY") else "none"
    y = oracle.linear_act_ref(a["a_ptr"], a["b_ptr"], None, act)
    _assert_same(y.astype(case["expected"]["c_ptr"].dtype), case["expected"]["c_ptr"], meta["dtype"])


@pytest.mark.parametrize("tag", golden_cases.tags("triton_linear_activation"))
def test_linear_act(tag):
    case, meta = golden_cases.load(tag)
    a = case["args"]
    y = oracle.linear_act_ref(a["x_ptr"], a["w_ptr"], a["b_ptr"], "gelu_erf")
    _assert_same(y.astype(case["expected"]["y_ptr"].dtype), case["expected"]["y_ptr"], meta["dtype"])


@pytest.mark.parametrize("tag", golden_cases.tags("attn_fwd_causal") + golden_cases.tags("context_attn_fwd"))
def test_attention(tag):
    case, meta = golden_cases.load(tag)
    a = case["args"]
    out, lse = oracle.attention_ref(a["q_ptr"], a["k_ptr"], a["v_ptr"], a["scale"],
                                    causal=bool(case["meta"]["CAUSAL"]))
    _assert_same(out.astype(case["expected"]["out_ptr"].dtype), case["expected"]["out_ptr"], meta["dtype"])
    assert np.isfinite(lse).all()


@pytest.mark.parametrize("tag", golden_cases.tags("gqa"))
def test_gqa(tag):
    case, meta = golden_cases.load(tag)
    a = case["args"]
    out, _ = oracle.gqa_attention_ref(a["Q"], a["K"], a["V"], a["scale"], causal=False)
    expected = case["expected"]["Out"]
    _assert_same(out.astype(expected.dtype), expected, meta["dtype"])


@pytest.mark.parametrize("tag", golden_cases.tags("fused_gemm_gn_min_kernel"))
def test_gemm_groupnorm_rowmin(tag):
    case, meta = golden_cases.load(tag)
    a = case["args"]
    m, n, k = int(a["M"]), int(a["N"]), int(a["K"])
    mins = oracle.gemm_groupnorm_rowmin_ref(
        np.asarray(a["X_ptr"]).reshape(m, k), np.asarray(a["W_ptr"]).reshape(k, n), a["B_ptr"],
        a["Gamma_ptr"], a["Beta_ptr"], int(case["meta"]["GROUP_SIZE"]), a["eps"])
    expected = case["expected"]["Mins_ptr"]
    _assert_same(mins.astype(expected.dtype), expected, meta["dtype"])


@pytest.mark.parametrize("tag", golden_cases.tags("dequantize_matmul"))
def test_dequantize(tag):
    case, meta = golden_cases.load(tag)
    out = oracle.dequantize_ref(case["args"]["b_ptr"], case["args"]["b_scale_ptr"])
    expected = case["expected"]["fpb_ptr"]
    _assert_same(out.astype(expected.dtype), expected, meta["dtype"])


@pytest.mark.parametrize("tag", golden_cases.tags("rms_matmul_rbe"))
def test_rms_matmul(tag):
    case, meta = golden_cases.load(tag)
    a = case["args"]
    out = oracle.rms_matmul_ref(a["x_ptr"], a["rms_w_ptr"], a["w_ptr"], a["EPS"])
    expected = case["expected"]["out_ptr"]
    _assert_same(out.astype(expected.dtype), expected, meta["dtype"])


@pytest.mark.parametrize("tag", golden_cases.tags("parallel_attn_fwd_kernel"))
def test_window_attention(tag):
    case, meta = golden_cases.load(tag)
    a, m = case["args"], case["meta"]
    b, t, h, hq, kd, vd = m["B"], int(a["T"]), m["H"], m["HQ"], m["K"], m["V"]
    out, lse = oracle.window_attention_ref(
        np.asarray(a["q"]).reshape(b, t, hq, kd), np.asarray(a["k"]).reshape(b, t, h, kd),
        np.asarray(a["v"]).reshape(b, t, h, vd), np.asarray(a["g_cumsum"]).reshape(b, t, hq),
        a["sink_bias"], a["scale"], m["W"])
    tol = 1e-4 if meta["dtype"] == "float32" else 2e-2
    np.testing.assert_allclose(out.reshape(-1), np.asarray(case["expected"]["o"], dtype=np.float64),
                               rtol=tol, atol=tol)
    np.testing.assert_allclose(lse.reshape(-1), np.asarray(case["expected"]["lse"], dtype=np.float64),
                               rtol=tol, atol=tol)


@pytest.mark.parametrize("tag", golden_cases.tags("log_softmax_linear"))
def test_log_softmax_linear(tag):
    case, meta = golden_cases.load(tag)
    y = oracle.log_softmax_linear_ref(case["args"]["x_ptr"], case["args"]["w_ptr"])
    expected = case["expected"]["y_ptr"]
    _assert_same(y.astype(expected.dtype), expected, meta["dtype"])


@pytest.mark.parametrize("tag", golden_cases.tags("flash_varlen_fwd_kernel"))
def test_flash_varlen(tag):
    case, meta = golden_cases.load(tag)
    a, m = case["args"], case["meta"]
    h, hk, d = m["h"], m["hk"], m["d"]
    cu_q, cu_k = a["cu_seqlens_q_ptr"], a["cu_seqlens_k_ptr"]
    total_q, total_k = int(cu_q[-1]), int(cu_k[-1])
    q = np.asarray(a["q_ptr"])[:total_q * h * d].reshape(total_q, h, d)
    k = np.asarray(a["k_ptr"])[:total_k * hk * d].reshape(total_k, hk, d)
    v = np.asarray(a["v_ptr"])[:total_k * hk * d].reshape(total_k, hk, d)
    out, lse = oracle.varlen_attention_ref(q, k, v, cu_q, cu_k, m["scale_softmax"])
    want_o = np.asarray(case["expected"]["o_ptr"])[:total_q * h * d].reshape(total_q, h, d)
    want_l = np.asarray(case["expected"]["softmax_lse_ptr"])[:h * total_q].reshape(h, total_q)
    # the reference's ref computes in float32: agree to its rounding, not bit for bit
    np.testing.assert_allclose(out, want_o.astype(np.float64), rtol=2e-2 if meta["dtype"] != "float32" else 1e-5, atol=1e-2 if meta["dtype"] != "float32" else 1e-5)
    np.testing.assert_allclose(lse, want_l.astype(np.float64), rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize("tag", golden_cases.tags("flash_decode"))
def test_flash_decode(tag):
    case, meta = golden_cases.load(tag)
    a = case["args"]
    z_h, d = a["Q"].shape[0] * a["Q"].shape[1], a["Q"].shape[2]
    out = oracle.flash_decode_ref(a["Q"].reshape(z_h, d), a["K"].reshape(z_h, -1, d),
                                  a["V"].reshape(z_h, -1, d), a["scale"])
    expected = case["expected"]["Out"]
    _assert_same(out.reshape(expected.shape).astype(expected.dtype), expected, meta["dtype"])


@pytest.mark.parametrize("tag", golden_cases.tags("swiglu_fwd"))
def test_swiglu(tag):
    case, meta = golden_cases.load(tag)
    y = oracle.swiglu_ref(case["args"]["X"], case["args"]["Y"])
    _assert_same(y.astype(case["expected"]["OUT"].dtype), case["expected"]["OUT"], meta["dtype"])


def test_bf16_round_matches_reference_rule():
    x = np.array([1.0, 1.00390625, 1.01171875, -3.1415927, np.nan, np.inf, 65504.0, 1e-40],
                 dtype=np.float32)
    r = oracle.bf16_round(x)
    assert (r.view(np.uint32) & 0xFFFF == 0).all()
    assert r[0] == 1.0 and np.isnan(r[4]) and np.isinf(r[5])
    # ties to even: 1.00390625 = 1 + 2^-8 is exactly half way between 1 and 1 + 2^-7
    assert r[1] == 1.0
    assert r[2] == np.float32(1.015625)


def test_masked_softmax_composition():
    rng = np.random.default_rng(3)
    x = rng.standard_normal((9, 7)) * 2
    y = oracle.masked_softmax_ref(x, row_offset=5)
    for r in range(9):
        keep = (r + 5) % 7 + 1
        np.testing.assert_allclose(y[r, :keep], oracle.softmax_ref(x[r:r + 1, :keep])[0], rtol=1e-12)
        assert (y[r, keep:] == 0).all()


def test_lse_definition():
    rng = np.random.default_rng(4)
    q, k, v = (rng.standard_normal((12, 8)) for _ in range(3))
    out, lse = oracle.attention_head_ref(q, k, v, 0.3, causal=True)
    s = np.where(np.tril(np.ones((12, 12), bool)), (q @ k.T) * 0.3, -np.inf)
    np.testing.assert_allclose(lse, np.log(np.exp(s).sum(-1)), rtol=1e-12)


# ------------------------------------------------------------------ sibling operators
def _check(case, name, value):
    """The oracle against a fixture, with the fixture's own policy (some of these files'
    refs compute in the storage dtype, so exact float64 agreement is not defined)."""
    policy = case["comparison"][name]
    expected = case["expected"][name]
    oracle.compare(np.asarray(value).astype(expected.dtype), expected, policy["rtol"],
                   policy["atol"], name=name)


@pytest.mark.parametrize("tag", golden_cases.tags("softmax_mul"))
def test_softmax_mul(tag):
    case, _ = golden_cases.load(tag)
    _check(case, "y_ptr", oracle.softmax_mul_ref(case["args"]["x_ptr"], case["args"]["o_ptr"]))


@pytest.mark.parametrize("tag", golden_cases.tags("softmax_log"))
def test_softmax_log(tag):
    case, _ = golden_cases.load(tag)
    _check(case, "y_ptr", oracle.softmax_log_ref(case["args"]["x_ptr"]))


@pytest.mark.parametrize("tag", golden_cases.tags("fused_repeat_interleave_log_softmax"))
def test_repeat_log_softmax(tag):
    case, _ = golden_cases.load(tag)
    a = case["args"]
    _check(case, "y_ptr", oracle.repeat_log_softmax_ref(a["x_ptr"], a["R"], a["L"]))


@pytest.mark.parametrize("tag", golden_cases.tags("gelu"))
def test_gelu(tag):
    case, _ = golden_cases.load(tag)
    _check(case, "y_ptr", oracle.gelu_erf(case["args"]["x_ptr"].astype(np.float64)))


@pytest.mark.parametrize("tag", golden_cases.tags("add_gelu"))
def test_add_gelu(tag):
    case, _ = golden_cases.load(tag)
    _check(case, "y_ptr", oracle.add_gelu_ref(case["args"]["x_ptr"], case["args"]["o_ptr"]))


@pytest.mark.parametrize("tag", golden_cases.tags("geglu_tanh_triton"))
def test_geglu_tanh(tag):
    case, _ = golden_cases.load(tag)
    _check(case, "c_ptr", oracle.geglu_tanh_ref(case["args"]["a_ptr"], case["args"]["b_ptr"]))


@pytest.mark.parametrize("tag", golden_cases.tags("epilogue_kernel"))
def test_epilogue(tag):
    case, _ = golden_cases.load(tag)
    a = case["args"]
    _check(case, "out_ptr", oracle.epilogue_ref(a["out_ptr"], a["bias_ptr"], a["n_cols"], a["scale"],
                                                a["ht_min"], a["ht_max"]))


@pytest.mark.parametrize("tag", golden_cases.tags("rmsnorm_fwd_loop_kernel"))
def test_rmsnorm_zero_centred_gamma(tag):
    case, _ = golden_cases.load(tag)
    a = case["args"]
    rows, n = case["grid"][0], a["N"]
    offset = 1.0 if case["meta"].get("zero_centered_gamma") else 0.0
    y, r = oracle.rmsnorm_ref(a["in_ptr"].reshape(rows, n), a["weight_ptr"][:n].astype(np.float64) + offset,
                              a["eps"])
    _check(case, "out_ptr", y.reshape(-1))
    _check(case, "rsigma_ptr", r)


@pytest.mark.parametrize("tag", golden_cases.tags("swiglu_triton") + golden_cases.tags("matmul_triton_autotune")
                         + golden_cases.tags("attention_forward_triton") + golden_cases.tags("attention_kernel"))
def test_twins(tag):
    case, _ = golden_cases.load(tag)
    a = case["args"]
    if tag.startswith("swiglu"):
        _check(case, "OUT", oracle.swiglu_ref(a["X"], a["Y"]))
    elif tag.startswith("matmul"):
        act = "leaky_relu" if case["meta"].get("LEAKY") else "none"
        _check(case, "c_ptr", oracle.linear_act_ref(a["a_ptr"], a["b_ptr"], None, act))
    else:
        out, _ = oracle.attention_ref(a["q_ptr"], a["k_ptr"], a["v_ptr"], a["scale"],
                                      causal=bool(case["meta"]["CAUSAL"]))
        _check(case, "out_ptr", out)


def test_attention_modes_restatement_properties():
    """The restatement of flash_varlen_fwd_kernel's soft-cap / ALiBi / local-window lines has no
    reference ``ref`` to be pinned to (ops/suite/dev/flash_varlen_fwd_kernel.py:370-373 raises
    for them), so it is held to what must be true of it: with every mode off it is the dense /
    causal oracle that IS pinned; a window that covers everything changes nothing; a zero
    slope changes nothing; a tiny soft-cap makes all kept keys equal (uniform weights); rows
    without a key give zeros and lse = +inf."""
    rng = np.random.default_rng(5)
    q = rng.standard_normal((2, 4, 9, 8))
    k, v = rng.standard_normal((2, 2, 13, 8)), rng.standard_normal((2, 2, 13, 8))
    scale = 0.35
    for causal in (False, True):
        base_o, base_l = oracle.gqa_attention_ref(q, k, v, scale, causal)
        o, l = oracle.attention_modes_ref(q, k, v, scale, causal=causal)
        assert np.allclose(o, base_o) and np.allclose(l, base_l)
        o, l = oracle.attention_modes_ref(q, k, v, scale, causal=causal,
                                          alibi_slopes=np.zeros(4))
        assert np.allclose(o, base_o) and np.allclose(l, base_l)
    o, l = oracle.attention_modes_ref(q, k, v, scale, window=(100, 100))
    base_o, base_l = oracle.gqa_attention_ref(q, k, v, scale, False)
    assert np.allclose(o, base_o) and np.allclose(l, base_l)
    # causal = a window with nothing to the right and everything to the left
    o, l = oracle.attention_modes_ref(q, k, v, scale, window=(100, 0))
    base_o, base_l = oracle.gqa_attention_ref(q, k, v, scale, True)
    assert np.allclose(o, base_o) and np.allclose(l, base_l)
    # soft-cap -> 0: every kept score is ~0, the weights are uniform over the window
    o, _ = oracle.attention_modes_ref(q, k, v, scale, softcap=1e-9, window=(2, 1))
    rows, shift = np.arange(9), 13 - 9
    for i in rows:
        lo, hi = max(0, i + shift - 2), min(12, i + shift + 1)
        assert np.allclose(o[0, 0, i], v[0, 0, lo:hi + 1].mean(axis=0), atol=1e-6)
    # ALiBi, non-causal: the bias is -slope * |j - N_K + N - i| on the scaled score
    o, l = oracle.attention_modes_ref(q[:, :1], k[:, :1], v[:, :1], scale, alibi_slopes=[0.25])
    s = (q[0, 0] @ k[0, 0].T) * scale - 0.25 * np.abs(np.arange(13)[None, :] - 13 + 9
                                                     - np.arange(9)[:, None])
    assert np.allclose(l[0, 0], np.log(np.exp(s).sum(axis=1)))
    # more rows than keys, causal: the first rows see nothing
    o, l = oracle.attention_modes_ref(q[:, :, :, :], k[:, :, :3], v[:, :, :3], scale, causal=True,
                                      softcap=0.5)
    assert np.isposinf(l[:, :, :6]).all() and not o[:, :, :6].any() and np.isfinite(l[:, :, 6:]).all()
