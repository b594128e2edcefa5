"""CPU oracle: numpy restatement of the reference's ``ref`` functions.

TEST INFRASTRUCTURE ONLY.  Nothing in ``compiler_b200/`` imports this module;
it is the checker for ``tests/``, ``__graft_entry__.smoke()`` and the
``cpu_baseline`` / ``--impl reference`` legs of ``bench.py``.

Every function restates the float64 numpy oracle of one reference operator file
(paths relative to the reference tree) and says which lines it follows.  Parity
is PINNED: ``tests/test_oracle_golden.py`` checks each function against golden
inputs/outputs produced by importing the reference's own operator modules
(``tests/golden/make_golden.py``; fixtures in ``tests/golden/*.npz``), for every
declared shape and dtype of those files.

Inputs are expected in their host representation -- float32 values already
rounded to bf16 for bf16 cases (ops/harness/opslib/case.py:223-232) -- and all
arithmetic is float64, as in the reference.
"""
from __future__ import annotations

import math

import numpy as np

try:  # scipy-backed erf, as ops/harness/opslib/mathref.py:42-52 prefers
    from scipy.special import erf as _erf
except Exception:  # noqa: BLE001 - same fallback as mathref.py:30-39
    _erf = np.vectorize(math.erf, otypes=[np.float64])


# ----------------------------------------------------------------- rounding
def bf16_round(array) -> np.ndarray:
    """float32 values rounded to bfloat16, round-to-nearest-even, NaN kept quiet.

    Follows ``_bf16_host`` (ops/harness/opslib/case.py:214-220)."""
    values = np.ascontiguousarray(array, dtype=np.float32)
    bits = values.view(np.uint32)
    rounded = (bits + np.uint32(0x7FFF) + ((bits >> 16) & np.uint32(1))) & np.uint32(0xFFFF0000)
    rounded = np.where(np.isnan(values), bits | np.uint32(0x00400000), rounded)
    return rounded.astype(np.uint32).view(np.float32)


def to_storage(array, dtype: str) -> np.ndarray:
    """Host representation of ``array`` in a case dtype (``_cast_float_array``,
    ops/harness/opslib/case.py:223-232): bf16 -> rounded float32, else astype."""
    if dtype == "bfloat16":
        return bf16_round(array)
    return np.ascontiguousarray(array, dtype=np.dtype(dtype))


# ----------------------------------------------------------------- operators
def rmsnorm_ref(x, w, eps):
    """``ref`` of ops/suite/perf/fast_rms_layernorm.py:52-61.

    Returns (Y, r) in float64: var = sum(x*x)/n_cols; inv = 1/sqrt(var+eps);
    Y = (x*inv)*w; r = inv per row."""
    x = np.asarray(x, dtype=np.float64)
    w = np.asarray(w, dtype=np.float64)
    n_cols = x.shape[1]
    var = (x * x).sum(axis=1, keepdims=True) / n_cols
    inv = 1.0 / np.sqrt(var + float(eps))
    return (x * inv) * w[None, :], inv.reshape(-1)


def softmax_ref(x):
    """``ref`` of ops/suite/perf/softmax.py:40-45: e = exp(x - rowmax); e / sum(e)."""
    x64 = np.asarray(x, dtype=np.float64)
    e = np.exp(x64 - x64.max(-1, keepdims=True))
    return e / e.sum(-1, keepdims=True)


def masked_softmax_ref(x, row_offset: int = 0):
    """softmax.ref (ops/suite/perf/softmax.py:40-45) applied to
    ``np.where(mask, x, -inf)`` with the mask of attn_fwd_causal.ref
    (ops/suite/perf/attn_fwd_causal.py:70-71): column c of global row g is kept
    iff c <= g % n_cols.  A composition of two reference oracles; the reference
    has no single file for it."""
    x64 = np.asarray(x, dtype=np.float64)
    rows, cols = x64.shape
    limit = (np.arange(rows, dtype=np.int64) + int(row_offset)) % cols
    mask = np.arange(cols, dtype=np.int64)[None, :] <= limit[:, None]
    return softmax_ref(np.where(mask, x64, -np.inf))


def matmul_ref(a, b):
    """``ref`` of ops/suite/perf/matmul.py:46-50: float64 a @ b."""
    return np.asarray(a, dtype=np.float64) @ np.asarray(b, dtype=np.float64)


def gelu_erf(z):
    """0.5 z (1 + erf(z/sqrt 2)) (ops/suite/perf/triton_linear_activation.py:62)."""
    return 0.5 * z * (1.0 + _erf(z * 0.7071067811865476))


def gelu_tanh(z):
    """0.5 z (1 + tanh(0.79788456 (z + 0.044715 z^3))) (ops/suite/perf/geglu_tanh_triton.py:44-49)."""
    return 0.5 * z * (1.0 + np.tanh(0.7978845608028654 * (z + 0.044715 * z * z * z)))


def leaky_relu(z, slope=0.01):
    """np.where(z >= 0, z, slope*z) (ops/suite/perf/matmul_triton2.py ref)."""
    return np.where(z >= 0, z, slope * z)


def linear_act_ref(x, w, bias=None, act: str = "gelu_erf"):
    """``ref`` of ops/suite/perf/triton_linear_activation.py:56-63 (x @ w + b, erf-GELU),
    with the activation selectable: "none", "gelu_erf", "gelu_tanh" (the formula of
    ops/suite/perf/geglu_tanh_triton.py:44-49), "leaky_relu"."""
    acc = matmul_ref(x, w)
    if bias is not None:
        acc = acc + np.asarray(bias, dtype=np.float64)[None, :]
    if act == "none":
        return acc
    if act == "gelu_erf":
        return gelu_erf(acc)
    if act == "gelu_tanh":
        return gelu_tanh(acc)
    if act == "leaky_relu":
        return leaky_relu(acc)
    raise ValueError(f"unknown activation {act!r}")


def attention_head_ref(q, k, v, scale, causal=True):
    """One (batch, head) slice of ``ref`` of ops/suite/perf/attn_fwd_causal.py:63-76,
    plus the log-sum-exp of ops/suite/dev/flash_varlen_fwd_kernel.py:412-418
    (rowmax + log(sum(exp(scores - rowmax))) over the scaled, masked scores).

    q: [N, D]; k, v: [N_K, D].  With N_K != N the causal mask is aligned to the last key:
    row i sees keys <= i + N_K - N (ops/suite/dev/flash_varlen_fwd_kernel.py:138).
    Returns (out [N, D], lse [N]) in float64.  Heads are
    independent, so evaluating the reference per slice gives the same numbers as
    its whole-tensor einsum while holding one [N, N] score matrix at a time."""
    q = np.asarray(q, dtype=np.float64)
    k = np.asarray(k, dtype=np.float64)
    v = np.asarray(v, dtype=np.float64)
    n, nk = q.shape[0], k.shape[0]
    scores = (q @ k.T) * float(scale)
    if causal:
        scores = np.where(np.tril(np.ones((n, nk), dtype=bool), nk - n), scores, -np.inf)
    row_max = scores.max(axis=-1, keepdims=True)
    p = np.exp(scores - row_max)
    denom = p.sum(axis=-1, keepdims=True)
    out = (p / denom) @ v
    lse = row_max[:, 0] + np.log(denom[:, 0])
    return out, lse


def attention_ref(q, k, v, scale, causal=True):
    """``ref`` of ops/suite/perf/attn_fwd_causal.py:63-76 over [Z,H,N,D], slice by slice."""
    q = np.asarray(q)
    z, h, n, d = q.shape
    out = np.empty((z, h, n, d), dtype=np.float64)
    lse = np.empty((z, h, n), dtype=np.float64)
    for zi in range(z):
        for hi in range(h):
            out[zi, hi], lse[zi, hi] = attention_head_ref(q[zi, hi], k[zi, hi], v[zi, hi], scale,
                                                          causal)
    return out, lse


def attention_modes_head_ref(q, k, v, scale, *, causal=False, softcap=0.0, alibi_slope=None,
                             window=None):
    """One (batch, head) slice with the further modes of flash_varlen_fwd_kernel, restated
    from the KERNEL's lines (its own ``ref``, ops/suite/dev/flash_varlen_fwd_kernel.py:370-418,
    covers dense attention only, so this part of the oracle is unpinned):

    raw S = q k^T; soft-cap S = 2 / (1 + exp(-2 S softcap)) - 1 (:121-124); ALiBi with
    slope / scale on the raw score -- causal: + (j - N_K + 1), otherwise - |j - N_K + N - i|
    (:76-81, :125-133); masks with col_lb = max(0, i + N_K - N - left),
    col_rb = min(N_K - 1, i + N_K - N + right): causal hides j > col_rb (right = 0), local
    hides j outside [col_lb, col_rb] (:137-146); softmax of scale * S (:149-160); a row without
    keys gives zeros and lse = +inf (:309-311).  q [N, D]; k, v [N_K, D]; float64 results."""
    q = np.asarray(q, dtype=np.float64)
    k = np.asarray(k, dtype=np.float64)
    v = np.asarray(v, dtype=np.float64)
    n, nk = q.shape[0], k.shape[0]
    s = q @ k.T
    if softcap:
        s = 2.0 / (1.0 + np.exp(-2.0 * (s * float(softcap)))) - 1.0
    rows = np.arange(n)[:, None]
    cols = np.arange(nk)[None, :]
    if alibi_slope is not None:
        slope = float(alibi_slope) / float(scale)
        if causal:
            s = s + slope * (cols - nk + 1)
        else:
            s = s - slope * np.abs(cols - nk + n - rows)
    left, right = window if window is not None else (0, 0)
    col_lb = np.maximum(0, rows + nk - n - left)
    col_rb = np.minimum(nk - 1, rows + nk - n + (right if window is not None else 0))
    hidden = np.zeros((n, nk), dtype=bool)
    if causal:
        hidden |= cols > col_rb
    if window is not None:
        hidden |= (cols > col_rb) | (cols < col_lb)
    s = np.where(hidden, -np.inf, s) * float(scale)
    row_max = s.max(axis=1, keepdims=True)
    safe_max = np.where(np.isinf(row_max), 0.0, row_max)
    p = np.exp(s - safe_max)
    denom = p.sum(axis=1, keepdims=True)
    empty = denom[:, 0] == 0
    out = (p / np.where(denom == 0, 1.0, denom)) @ v
    with np.errstate(divide="ignore"):
        lse = np.where(empty, np.inf, safe_max[:, 0] + np.log(denom[:, 0]))
    return out, lse


def attention_modes_ref(q, k, v, scale, *, causal=False, softcap=0.0, alibi_slopes=None,
                        window=None):
    """``attention_modes_head_ref`` over q [Z,H,N,D], k / v [Z,H_KV,N_K,D] (query head h reads
    K / V head h // (H // H_KV)); ``alibi_slopes`` [H] or [Z,H]."""
    q = np.asarray(q)
    z, h, n, d = q.shape
    group = h // np.asarray(k).shape[1]
    out = np.empty((z, h, n, d), dtype=np.float64)
    lse = np.empty((z, h, n), dtype=np.float64)
    slopes = None if alibi_slopes is None else np.broadcast_to(np.asarray(alibi_slopes), (z, h))
    for zi in range(z):
        for hi in range(h):
            out[zi, hi], lse[zi, hi] = attention_modes_head_ref(
                q[zi, hi], k[zi, hi // group], v[zi, hi // group], scale, causal=causal,
                softcap=softcap, alibi_slope=None if slopes is None else slopes[zi, hi],
                window=window)
    return out, lse


def gemm_groupnorm_rowmin_ref(x, w, bias, gamma, beta, group_size, eps):
    """Row minimum of GroupNorm(x @ w + bias) with groups of ``group_size`` columns (ref of
    ops/suite/dev/fused_gemm_gn_min_kernel.py:88-105), float64 [M]."""
    x = np.asarray(x, dtype=np.float64)
    w = np.asarray(w, dtype=np.float64)
    m, n = x.shape[0], w.shape[1]
    acc = x @ w + (0.0 if bias is None else np.asarray(bias, dtype=np.float64)[None, :])
    acc3 = acc.reshape(m, n // group_size, group_size)
    mean = acc3.mean(axis=2)
    rstd = 1.0 / np.sqrt(acc3.var(axis=2) + float(eps))
    out = ((acc3 - mean[:, :, None]) * rstd[:, :, None]
           * np.asarray(gamma, dtype=np.float64).reshape(n // group_size, group_size)[None]
           + np.asarray(beta, dtype=np.float64).reshape(n // group_size, group_size)[None])
    return out.min(axis=(1, 2))


def dequantize_ref(b, scale):
    """int8 b [K,N] times scale [N] (ref of ops/suite/perf/dequantize_matmul.py:49-52)."""
    return np.asarray(b, dtype=np.float64) * np.asarray(scale, dtype=np.float64)[None, :]


def rms_matmul_ref(x, g, w, eps):
    """rsqrt(mean(x^2) + eps) * ((x * g) @ w) (ref of ops/suite/dev/rms_matmul_rbe.py:70-80),
    float64; x [..., K], g [K], w [K, N]."""
    x = np.asarray(x, dtype=np.float64)
    acc = (x * np.asarray(g, dtype=np.float64)) @ np.asarray(w, dtype=np.float64)
    return acc / np.sqrt((x * x).sum(axis=-1, keepdims=True) / x.shape[-1] + float(eps))


def log_softmax_linear_ref(x, w):
    """log_softmax(x @ w.T) over the last axis (ref of
    ops/suite/perf/log_softmax_linear.py:45-51), float64."""
    z = np.asarray(x, dtype=np.float64) @ np.asarray(w, dtype=np.float64).T
    m = z.max(-1, keepdims=True)
    return z - m - np.log(np.exp(z - m).sum(-1, keepdims=True))


def gqa_attention_ref(q, k, v, scale, causal=False):
    """Attention with fewer K / V heads than query heads: query head h reads K / V head
    h // (H_Q // H_KV) (ref of ops/suite/dev/gqa.py:69-85).  q [Z,H_Q,N,D], k / v
    [Z,H_KV,N,D] -> (out, lse) like ``attention_ref``."""
    group = np.asarray(q).shape[1] // np.asarray(k).shape[1]
    return attention_ref(q, np.repeat(np.asarray(k), group, axis=1),
                         np.repeat(np.asarray(v), group, axis=1), scale, causal)


def window_attention_ref(q, k, v, gate, sink_bias, scale, window):
    """Causal sliding-window attention in base 2 with gate bias and sink (ref of
    ops/suite/dev/parallel_attn_fwd_kernel.py:142-166).  q [B,T,HQ,K], k [B,T,H,K],
    v [B,T,H,V], gate [B,T,HQ] or None, sink_bias [HQ] or None, window <= 0 = unlimited.
    Returns (o [B,T,HQ,V], lse [B,T,HQ]) in float64."""
    q = np.asarray(q, dtype=np.float64)
    k = np.asarray(k, dtype=np.float64)
    v = np.asarray(v, dtype=np.float64)
    B, T, HQ, _ = q.shape
    group = HQ // k.shape[2]
    out = np.zeros((B, T, HQ, v.shape[3]))
    lse = np.zeros((B, T, HQ))
    log2e = 1.4426950216
    for b in range(B):
        for hq in range(HQ):
            h = hq // group
            logits = (q[b, :, hq] @ k[b, :, h].T) * float(scale) * log2e
            if gate is not None:
                g = np.asarray(gate, dtype=np.float64)[b, :, hq]
                logits = logits + g[:, None] - g[None, :]
            for row in range(T):
                first = max(0, row - int(window) + 1) if window > 0 else 0
                valid = logits[row, first:row + 1]
                sink = float(np.asarray(sink_bias, dtype=np.float64)[hq]) if sink_bias is not None else -np.inf
                mx = max(float(valid.max()), sink)
                w = np.exp2(valid - mx)
                den = w.sum() + (np.exp2(sink - mx) if sink_bias is not None else 0.0)
                out[b, row, hq] = (w / den) @ v[b, first:row + 1, h]
                lse[b, row, hq] = mx + np.log2(den)
    return out, lse


def varlen_attention_ref(q, k, v, cu_q, cu_k, scale):
    """Dense attention over packed sequences (ref of
    ops/suite/dev/flash_varlen_fwd_kernel.py:370-418): q [total_q, H, D], k / v
    [total_k, H_K, D], sequence b owns rows cu[b]:cu[b+1]; query head h reads K / V head
    h // (H // H_K).  Returns (out [total_q, H, D], lse [H, total_q]) in float64."""
    q = np.asarray(q, dtype=np.float64)
    k = np.asarray(k, dtype=np.float64)
    v = np.asarray(v, dtype=np.float64)
    ratio = q.shape[1] // k.shape[1]
    out = np.zeros(q.shape)
    lse = np.zeros((q.shape[1], q.shape[0]))
    for b in range(len(cu_q) - 1):
        q0, q1, k0, k1 = int(cu_q[b]), int(cu_q[b + 1]), int(cu_k[b]), int(cu_k[b + 1])
        for h in range(q.shape[1]):
            s = (q[q0:q1, h] @ k[k0:k1, h // ratio].T) * float(scale)
            mx = s.max(axis=1, keepdims=True)
            w = np.exp(s - mx)
            den = w.sum(axis=1, keepdims=True)
            out[q0:q1, h] = (w / den) @ v[k0:k1, h // ratio]
            lse[h, q0:q1] = mx[:, 0] + np.log(den[:, 0])
    return out, lse


def flash_decode_ref(q, k, v, scale, group: int = 1):
    """One query row per (batch, head): out[b] = softmax(scale * K[b // group] q[b]) V[b // group]
    (ref of ops/suite/perf/flash_decode.py:57-70; ``group`` > 1 is the head mapping of
    ops/suite/dev/gqa.py:29).  q [B, D], k / v [B // group, N, D] -> [B, D] float64."""
    q = np.asarray(q, dtype=np.float64)
    k = np.asarray(k, dtype=np.float64)
    v = np.asarray(v, dtype=np.float64)
    out = np.zeros(q.shape)
    for b in range(q.shape[0]):
        s = (k[b // group] @ q[b]) * float(scale)
        s = s - s.max()
        p = np.exp(s)
        out[b] = (p / p.sum()) @ v[b // group]
    return out


def swiglu_ref(x, y):
    """``ref`` of ops/suite/perf/swiglu_fwd.py:43-47: x / (1 + exp(-x)) * y."""
    x = np.asarray(x, dtype=np.float64)
    y = np.asarray(y, dtype=np.float64)
    return x / (1.0 + np.exp(-x)) * y


def swiglu_mlp_ref(x, wg, wu, wd, h_dtype: str | None = None):
    """y = (silu(x @ Wg) * (x @ Wu)) @ Wd built from matmul.ref
    (ops/suite/perf/matmul.py:46-50) and swiglu_fwd.ref (ops/suite/perf/swiglu_fwd.py:43-47).
    The reference never performs this composition in one case and has no multi-device
    path; the unsharded float64 result pins the tensor-parallel one end to end.
    ``h_dtype``: optionally round the intermediate to its storage type first, to bound the
    error a 16-bit intermediate buffer is allowed to add."""
    h = swiglu_ref(matmul_ref(x, wg), matmul_ref(x, wu))
    if h_dtype is not None:
        h = to_storage(h.astype(np.float32), h_dtype).astype(np.float64)
    return matmul_ref(h, wd)


# ----------------------------------------------------------------- sibling operators
def softmax_mul_ref(x, o):
    """``ref`` of ops/suite/perf/softmax_mul.py: softmax(x) * o."""
    return softmax_ref(x) * np.asarray(o, dtype=np.float64)


def softmax_log_ref(x):
    """``ref`` of ops/suite/perf/softmax_log.py: softmax(log x) (NaN rows stay NaN)."""
    with np.errstate(divide="ignore", invalid="ignore"):
        return softmax_ref(np.log(np.asarray(x, dtype=np.float64)))


def repeat_log_softmax_ref(x, repeat, length=None):
    """``ref`` of ops/suite/perf/fused_repeat_interleave_log_softmax.py: log-softmax of
    np.repeat(x, R, axis=1) (the first ``length`` positions)."""
    rep = np.repeat(np.asarray(x, dtype=np.float64), int(repeat), axis=1)
    if length is not None:
        rep = rep[:, :int(length)]
    m = rep.max(axis=1, keepdims=True)
    return rep - (m + np.log(np.exp(rep - m).sum(axis=1, keepdims=True)))


def add_gelu_ref(x, o, alpha=1.5):
    """``ref`` of ops/suite/perf/add_gelu.py: gelu_erf(x + 1.5 o)."""
    return gelu_erf(np.asarray(x, dtype=np.float64) + alpha * np.asarray(o, dtype=np.float64))


def geglu_tanh_ref(a, b):
    """``ref`` of ops/suite/perf/geglu_tanh_triton.py:44-49: gelu_tanh(a) * b."""
    return gelu_tanh(np.asarray(a, dtype=np.float64)) * np.asarray(b, dtype=np.float64)


def epilogue_ref(x, bias, n_cols, scale, lo, hi):
    """``ref`` of ops/suite/dev/epilogue_kernel.py: gelu_erf(clip((x + bias) * scale, lo, hi))."""
    x = np.asarray(x, dtype=np.float64).reshape(-1, int(n_cols))
    y = (x + np.asarray(bias, dtype=np.float64)[None, :]) * float(scale)
    return gelu_erf(np.minimum(np.maximum(y, float(lo)), float(hi))).reshape(-1)


# ----------------------------------------------------------------- comparison
DTYPE_TOLERANCES = {  # ops/harness/opslib/case.py:153-157
    "float32": (1e-3, 1e-3),
    "float16": (1e-2, 1e-2),
    "bfloat16": (2e-2, 2e-2),
}


def compare(actual, expected, rtol, atol, equal_nan=True, name="output"):
    """``_allclose_pass`` of ops/harness/opslib/compare.py:107-140: the verdict is
    ``np.isclose(actual, expected)`` evaluated in the arrays' own dtypes; returns the
    informational max |a-b| (float64, over elements that are not exactly equal) and
    raises AssertionError listing the first violating flat indices."""
    actual = np.asarray(actual)
    expected = np.asarray(expected)
    if actual.shape != expected.shape:
        raise AssertionError(f"{name}: shape {actual.shape} != expected {expected.shape}")
    a = actual.reshape(-1)
    b = expected.reshape(-1)
    chunk = 16 * 1024 * 1024
    max_error = 0.0
    violations = []
    for start in range(0, a.size, chunk):
        ca, cb = a[start:start + chunk], b[start:start + chunk]
        close = np.isclose(ca, cb, rtol=rtol, atol=atol, equal_nan=equal_nan)
        if not close.all():
            violations.extend(int(i) + start for i in np.flatnonzero(~close)[:8])
        with np.errstate(invalid="ignore", over="ignore"):
            delta = np.abs(ca.astype(np.float64) - cb.astype(np.float64))
            equal = ca == cb
            if equal_nan:
                equal = equal | (np.isnan(ca) & np.isnan(cb))
            max_error = max(max_error, float(np.where(equal, 0.0, delta).max(initial=0.0)))
    if violations:
        first = violations[0]
        raise AssertionError(
            f"{name}: not close to tolerance rtol={rtol:g}, atol={atol:g}; first bad flat "
            f"indices {violations[:8]}, e.g. output={a[first]!r} vs reference={b[first]!r}; "
            f"max_abs_error={max_error:g}")
    return max_error
