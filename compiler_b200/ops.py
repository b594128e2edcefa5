"""Python entry points of the native operators.

Each function takes device arrays -- anything with ``data_ptr()``, ``shape`` and
``dtype`` (a :class:`compiler_b200.device.B200Buffer` or a CUDA ``torch.Tensor``;
a tensor's own strides are honoured) -- builds the ``b200_tensor`` descriptors
and calls the C ABI on ``stream`` (a raw ``cudaStream_t`` integer, 0 = the
default stream).  Nothing here computes: a rejected descriptor raises
:class:`compiler_b200.runtime.abi.B200Error`.
"""
from __future__ import annotations

import ctypes

from compiler_b200.runtime import abi


def _desc(array, shape=None, strides=None):
    if array is None:
        return None
    shape = tuple(array.shape) if shape is None else tuple(shape)
    if strides is None:
        stride_fn = getattr(array, "stride", None)
        if callable(stride_fn) and len(tuple(array.shape)) == len(shape):
            strides = tuple(int(s) for s in stride_fn())
    return abi.make_tensor(array.data_ptr(), shape, array.dtype, strides)


def _ref(tensor):
    return ctypes.byref(tensor) if tensor is not None else None


def rmsnorm(x, w, y, rinv=None, eps=1e-6, *, x_row_stride=None, y_row_stride=None,
            gamma_offset=0.0, stream=0):
    """y = x * rsqrt(mean(x^2) + eps) * w per row; rinv[row] = the inverse rms.

    Native form of rms_layernorm_forward_kernel
    (ops/suite/perf/fast_rms_layernorm.py:19-44)."""
    rows, cols = (int(v) for v in x.shape)
    xd = _desc(x, strides=None if x_row_stride is None else (int(x_row_stride), 1))
    yd = _desc(y, strides=None if y_row_stride is None else (int(y_row_stride), 1))
    wd = _desc(w, shape=(cols,), strides=(1,))
    rd = _desc(rinv, shape=(rows,), strides=(1,)) if rinv is not None else None
    abi.check(abi.lib().b200_rmsnorm_fwd_ex(_ref(xd), _ref(wd), _ref(yd), _ref(rd), float(eps),
                                            float(gamma_offset), stream))


def softmax(x, y, *, causal_mod=False, row_offset=0, stream=0):
    """Row softmax; with ``causal_mod`` columns > (row_offset+row) % n_cols are -inf.

    Native form of softmax_kernel (ops/suite/perf/softmax.py:20-31) with the mask
    expression of ops/suite/perf/attn_fwd_causal.py:46-47."""
    xd, yd = _desc(x), _desc(y)
    mask = abi.MASK_CAUSAL_MOD if causal_mod else abi.MASK_NONE
    abi.check(abi.lib().b200_softmax_fwd(_ref(xd), _ref(yd), mask, int(row_offset), stream))


def gemm(a, b, c, *, bias=None, act=abi.ACT_NONE, b2=None, stream=0):
    """c = act(a @ b + bias); with ``act=ACT_SWIGLU``: c = silu(a @ b) * (a @ b2).

    Native form of matmul_kernel (ops/suite/perf/matmul.py:20-38) and
    linear_act_kernel (ops/suite/perf/triton_linear_activation.py:27-49)."""
    ad, bd, cd = _desc(a), _desc(b), _desc(c)
    b2d = _desc(b2) if b2 is not None else None
    biasd = _desc(bias, shape=(int(b.shape[1]),), strides=(1,)) if bias is not None else None
    abi.check(abi.lib().b200_gemm_bias_act(_ref(ad), _ref(bd), _ref(b2d), _ref(biasd), _ref(cd),
                                           int(act), stream))


def gemm_progress(a, b, c, rows_per_block, counters, *, stream=0):
    """c = a @ b on the CTA-pair kernel with a progress counter per block of
    ``rows_per_block`` rows of c (``counters``: device int32 array of
    ``b200_progress_words()`` words, zero before the launch).  Returns the list of counts the
    blocks reach -- what ``peer_allreduce_blocks`` waits for.  No reference counterpart."""
    ad, bd, cd = _desc(a), _desc(b), _desc(c)
    targets = (ctypes.c_uint32 * 16)()
    blocks = ctypes.c_int(0)
    abi.check(abi.lib().b200_gemm_progress(_ref(ad), _ref(bd), _ref(cd), int(rows_per_block),
                                           counters.data_ptr(), targets, 16,
                                           ctypes.byref(blocks), stream))
    return [int(targets[i]) for i in range(blocks.value)]


def peer_allreduce_blocks(partials, outs, total, block_elems, counters, targets, rank, world,
                          *, in_dtype, out_dtype, signal_pads=None, epoch0=0, ctas=0, stream=0):
    """The all-reduce that runs beside ``gemm_progress`` (launch it directly behind it on the
    same stream).  ``partials`` / ``outs``: one device address per rank; ``counters`` /
    ``targets``: what ``gemm_progress`` took and returned (None / None: no producer to wait
    for).  ``signal_pads``: ctypes array of the ranks' flag arrays, or None for one rank."""
    pointers = ctypes.c_void_p * world
    target_array = (ctypes.c_uint32 * len(targets))(*targets) if targets is not None else None
    abi.check(abi.lib().b200_peer_allreduce_blocks(
        pointers(*[int(p) for p in partials]), abi.DTYPE_CODES[abi.dtype_name(in_dtype)],
        pointers(*[int(p) for p in outs]), abi.DTYPE_CODES[abi.dtype_name(out_dtype)],
        int(total), int(block_elems), counters.data_ptr() if counters is not None else None,
        target_array, int(rank), int(world), signal_pads, int(epoch0), int(ctas), stream))


def multimem_allreduce_blocks(in_multicast, out_multicast, total, block_elems, counters, targets,
                              rank, world, *, in_dtype, out_dtype, signal_pads=None, epoch0=0,
                              ctas=0, stream=0):
    """``peer_allreduce_blocks`` through the switch: multicast addresses of the partial and
    the result (in-switch fp32 sum, store to all ranks)."""
    target_array = (ctypes.c_uint32 * len(targets))(*targets) if targets is not None else None
    abi.check(abi.lib().b200_multimem_allreduce_blocks(
        int(in_multicast), abi.DTYPE_CODES[abi.dtype_name(in_dtype)], int(out_multicast),
        abi.DTYPE_CODES[abi.dtype_name(out_dtype)], int(total), int(block_elems),
        counters.data_ptr() if counters is not None else None, target_array, int(rank),
        int(world), signal_pads, int(epoch0), int(ctas), stream))


def linear(x, w, y, *, bias=None, act=abi.ACT_NONE, stream=0):
    """y = act(x @ w.T + bias) with the weight as [N, K] (a linear layer's layout; the
    transposed-B case of matmul_kernel's general strides, ops/suite/perf/matmul_triton2.py:27-30)."""
    xd, wd, yd = _desc(x), _desc(w), _desc(y)
    biasd = _desc(bias, shape=(int(w.shape[0]),), strides=(1,)) if bias is not None else None
    abi.check(abi.lib().b200_linear_bias_act(_ref(xd), _ref(wd), _ref(biasd), _ref(yd), int(act),
                                             stream))


def gemm_groupnorm_rowmin(x, w, gamma, beta, mins, *, bias=None, group_size=32, eps=1e-5,
                          stream=0):
    """mins[m] = min(mins[m], min over n of GroupNorm(x @ w + bias)[m, n]) with groups of
    ``group_size`` columns (fused_gemm_gn_min_kernel,
    ops/suite/dev/fused_gemm_gn_min_kernel.py:26-59)."""
    n = int(w.shape[1])
    xd, wd, md = _desc(x), _desc(w), _desc(mins)
    gd = _desc(gamma, shape=(n,), strides=(1,))
    bd = _desc(beta, shape=(n,), strides=(1,))
    biasd = _desc(bias, shape=(n,), strides=(1,)) if bias is not None else None
    abi.check(abi.lib().b200_gemm_groupnorm_rowmin(_ref(xd), _ref(wd), _ref(biasd), _ref(gd),
                                                   _ref(bd), _ref(md), int(group_size),
                                                   float(eps), stream))


def dequantize_cols(b, scale, out, *, stream=0):
    """out[k, n] = int8 b[k, n] * scale[n] (dequantize_kernel,
    ops/suite/perf/dequantize_matmul.py:27-40)."""
    bd, sd, od = _desc(b), _desc(scale), _desc(out)
    abi.check(abi.lib().b200_dequantize_cols(_ref(bd), _ref(sd), _ref(od), stream))


def rms_matmul(x, g, w, out, scratch_w, scratch_rinv, eps=1e-5, *, stream=0):
    """out = rsqrt(mean(x^2) + eps) * ((x * g) @ w); scratch_w [K,N] (x's type) and
    scratch_rinv (float32, >= M) are workspace the caller owns.

    Native form of rms_matmul_rbe_kernel (ops/suite/dev/rms_matmul_rbe.py:18-63)."""
    xd, gd, wd, od = _desc(x), _desc(g), _desc(w), _desc(out)
    sw, sr = _desc(scratch_w), _desc(scratch_rinv)
    abi.check(abi.lib().b200_rms_matmul(_ref(xd), _ref(gd), _ref(wd), _ref(od), float(eps),
                                        _ref(sw), _ref(sr), stream))


def linear_log_softmax(x, w, y, *, stream=0):
    """y = log_softmax(x @ w.T) per row; x [M,K], w [N,K], N <= 256.

    Native form of log_softmax_linear_kernel (ops/suite/perf/log_softmax_linear.py:19-35)."""
    xd, wd, yd = _desc(x), _desc(w), _desc(y)
    abi.check(abi.lib().b200_linear_log_softmax(_ref(xd), _ref(wd), _ref(yd), stream))


def attention(q, k, v, o, *, lse=None, scale=None, causal=True, softcap=0.0, alibi_slopes=None,
              window=None, page_table=None, block_size=0, page_stride=0, stream=0):
    """o = softmax(scale * q k^T (+ causal mask)) v over [Z,H,N,D]; lse = log-sum-exp.

    Native form of attn_fwd_causal_kernel (ops/suite/perf/attn_fwd_causal.py:19-57).
    ``softcap`` / ``alibi_slopes`` ([H] or [Z,H] float32) / ``window=(left, right)`` are the
    further modes of flash_varlen_fwd_kernel
    (ops/suite/dev/flash_varlen_fwd_kernel.py:121-146), ``page_table`` (int32 [Z, pages]) with
    ``block_size`` / ``page_stride`` its paged K / V (:91-108); all taken by the CUDA-core
    kernel."""
    if scale is None:
        scale = 1.0 / float(q.shape[-1]) ** 0.5
    qd, kd, vd, od = _desc(q), _desc(k), _desc(v), _desc(o)
    ld = _desc(lse) if lse is not None else None
    if not softcap and alibi_slopes is None and window is None and page_table is None:
        abi.check(abi.lib().b200_attn_fwd(_ref(qd), _ref(kd), _ref(vd), _ref(od), _ref(ld),
                                          float(scale), 1 if causal else 0, stream))
        return
    ad = _desc(alibi_slopes) if alibi_slopes is not None else None
    left, right = (int(window[0]), int(window[1])) if window is not None else (-1, -1)
    pd = _desc(page_table) if page_table is not None else None
    abi.check(abi.lib().b200_attn_fwd_modes(_ref(qd), _ref(kd), _ref(vd), _ref(od), _ref(ld),
                                            float(scale), 1 if causal else 0, float(softcap),
                                            _ref(ad), left, right, _ref(pd), int(block_size),
                                            int(page_stride), stream))


def attention_window(q, k, v, o, *, g_cumsum=None, sink_bias=None, lse=None, scale=None,
                     window=0, stream=0):
    """Causal sliding-window attention with gate bias and sink on token-major tensors
    (parallel_attn_fwd_kernel, ops/suite/dev/parallel_attn_fwd_kernel.py:142-166)."""
    if scale is None:
        scale = 1.0 / float(q.shape[-1]) ** 0.5
    qd, kd, vd, od = _desc(q), _desc(k), _desc(v), _desc(o)
    gd = _desc(g_cumsum) if g_cumsum is not None else None
    sd = _desc(sink_bias) if sink_bias is not None else None
    ld = _desc(lse) if lse is not None else None
    abi.check(abi.lib().b200_attn_window_fwd(_ref(qd), _ref(kd), _ref(vd), _ref(od), _ref(gd),
                                             _ref(sd), _ref(ld), float(scale), int(window),
                                             stream))


def attention_decode(q, k, v, out, *, scale=None, stream=0):
    """out[b] = softmax(scale * K[b // group] q[b]) V[b // group]; q/out [B, D], k/v
    [B // group, N, D].

    Native form of flash_decode_kernel (ops/suite/perf/flash_decode.py:21-49)."""
    if scale is None:
        scale = 1.0 / float(q.shape[-1]) ** 0.5
    qd, kd, vd, od = _desc(q), _desc(k), _desc(v), _desc(out)
    abi.check(abi.lib().b200_attn_decode(_ref(qd), _ref(kd), _ref(vd), _ref(od), float(scale),
                                         stream))


def swiglu(x, y, out, *, stream=0):
    """out = x * sigmoid(x) * y (swiglu_fwd_kernel, ops/suite/perf/swiglu_fwd.py:18-36)."""
    xd, yd, od = _desc(x), _desc(y), _desc(out)
    abi.check(abi.lib().b200_swiglu_fwd(_ref(xd), _ref(yd), _ref(od), stream))


def softmax_variant(x, y, *, mul=None, log_input=False, stream=0):
    """y = softmax(x) * mul (softmax_mul_kernel, ops/suite/perf/softmax_mul.py:21-32) or
    y = softmax(log x) (softmax_log_kernel, ops/suite/perf/softmax_log.py:20-40)."""
    xd, yd = _desc(x), _desc(y)
    md = _desc(mul) if mul is not None else None
    abi.check(abi.lib().b200_softmax_variant(_ref(xd), _ref(md), _ref(yd),
                                             1 if log_input else 0, stream))


def repeat_log_softmax(x, y, repeat, *, stream=0):
    """y[row, p] = x[row, p // repeat] - logsumexp (fused_repeat_interleave_log_softmax_kernel,
    ops/suite/perf/fused_repeat_interleave_log_softmax.py:19-31)."""
    xd, yd = _desc(x), _desc(y)
    abi.check(abi.lib().b200_repeat_log_softmax(_ref(xd), _ref(yd), int(repeat), stream))


def elementwise(op, a, out, *, b=None, p0=0.0, p1=0.0, p2=0.0, stream=0):
    """Flat GELU-family operators (``abi.EW_*``): gelu.py, add_gelu.py, geglu_tanh_triton.py and
    dev/epilogue_kernel.py of the reference's corpus."""
    ad, od = _desc(a), _desc(out)
    bd = _desc(b) if b is not None else None
    abi.check(abi.lib().b200_elementwise(int(op), _ref(ad), _ref(bd), _ref(od), float(p0),
                                         float(p1), float(p2), stream))


def device_status(stream=0) -> None:
    """Drain ``stream`` and raise if a kernel recorded an expired wait."""
    abi.check(abi.lib().b200_last_device_status(stream))
