"""Kernel handle -> native operator resolution for ``B200Device.launch``.

The harness hands ``launch`` the object in ``case["kernel"]`` -- a Triton
``JITFunction`` / ``Autotuner`` whose ``.fn`` chain ends in the Python function
(``_kernel_target``, ops/harness/opslib/device.py:213-222) -- plus the grid, the
positional values in signature order and the keyword metas.  The registry keys
an operator on the function's *name and parameter list* (what ``bind_arguments``
itself inspects, device.py:232-260), rebinds the values by name, checks the
structural preconditions the native kernel needs, and calls the C ABI.  It never
calls ``kernel[grid]``, never compiles, and raises :class:`UnsupportedLaunch`
(located: kernel name + the violated precondition) for anything else, the
counterpart of a100c's ``PipelineError`` (a100c/driver.py:79-87).
"""
from __future__ import annotations

import inspect

from compiler_b200 import ops
from compiler_b200.runtime import abi


class UnsupportedLaunch(RuntimeError):
    """A launch this backend has no native operator for (never a silent guess)."""

    def __init__(self, kernel_name: str, construct: str, message: str):
        super().__init__(f"{kernel_name}: {construct}: {message}")
        self.kernel_name = kernel_name
        self.construct = construct
        self.message = message


def kernel_target(kernel):
    target = kernel
    for _ in range(8):
        if inspect.isfunction(target):
            return target
        nested = getattr(target, "fn", None)
        if nested is None or nested is target:
            return target
        target = nested
    return target


def kernel_signature(kernel):
    """(function name, parameter names, names the autotuner supplies itself)."""
    target = kernel_target(kernel)
    name = getattr(target, "__name__", type(target).__name__)
    try:
        parameters = inspect.signature(target).parameters
    except (TypeError, ValueError):
        parameters = {}
    configs = getattr(kernel, "configs", None)
    autotuned = set((getattr(configs[0], "kwargs", {}) or {}).keys()) if configs else set()
    return name, parameters, autotuned


def bind_by_name(kernel, positional, keywords):
    """Inverse of ``bind_arguments``: positional values back to a name -> value map."""
    name, parameters, autotuned = kernel_signature(kernel)
    values = dict(keywords)
    it = iter(positional)
    for pname, parameter in parameters.items():
        if pname in values:
            continue  # supplied by keyword (constexpr metas usually are)
        if parameter.kind == inspect.Parameter.KEYWORD_ONLY or pname in autotuned:
            continue
        try:
            values[pname] = next(it)
        except StopIteration:
            if parameter.default is inspect.Parameter.empty:
                raise UnsupportedLaunch(name, "arguments",
                                        f"missing positional value for {pname!r}") from None
            values[pname] = parameter.default
    leftover = list(it)
    if leftover:
        raise UnsupportedLaunch(name, "arguments", f"{len(leftover)} surplus positional values")
    return values


def _require(cond, kernel_name, construct, message):
    if not cond:
        raise UnsupportedLaunch(kernel_name, construct, message)


def _is_buffer(value):
    return hasattr(value, "data_ptr") and hasattr(value, "shape")


def _count(buffer):
    n = 1
    for extent in buffer.shape:
        n *= int(extent)
    return n


def _grid_tuple(grid, meta=None):
    if callable(grid):
        grid = grid(meta or {})
    grid = tuple(int(v) for v in grid)
    return grid + (1,) * (3 - len(grid))


class _View:
    """A reshaped alias of a device buffer (same pointer, new logical shape)."""

    def __init__(self, buffer, shape, strides=None, offset=0):
        self._buffer = buffer
        self.shape = tuple(int(v) for v in shape)
        self._strides = strides
        self.dtype = buffer.dtype
        self._offset = int(offset)  # elements past the start of the buffer

    def data_ptr(self):
        return self._buffer.data_ptr() + self._offset * abi.DTYPE_SIZES[abi.dtype_name(self.dtype)]

    def stride(self):
        if self._strides is not None:
            return tuple(self._strides)
        out, running = [], 1
        for extent in reversed(self.shape):
            out.append(running)
            running *= max(extent, 1)
        return tuple(reversed(out))


# --------------------------------------------------------------------- adapters
def _rmsnorm(device, v, grid, name):
    """rms_layernorm_forward_kernel (ops/suite/perf/fast_rms_layernorm.py:20-27)."""
    rows = _grid_tuple(grid)[0]
    n_cols = int(v["n_cols"])
    _require(int(v.get("BLOCK_SIZE", n_cols)) >= n_cols, name, "BLOCK_SIZE",
             "the reference program covers a row with one block: BLOCK_SIZE >= n_cols")
    _require(int(v["W_row_stride"]) == 1 and int(v["r_row_stride"]) == 1, name, "strides",
             "W_row_stride and r_row_stride must be 1")
    xs, ys = int(v["X_row_stride"]), int(v["Y_row_stride"])
    _require(xs >= n_cols and ys >= n_cols, name, "strides", "row stride below n_cols")
    x = _View(v["X"], (rows, n_cols), (xs, 1))
    y = _View(v["Y"], (rows, n_cols), (ys, 1))
    ops.rmsnorm(x, _View(v["W"], (n_cols,)), y, _View(v["r"], (rows,)), float(v["eps"]),
                stream=device.stream)


def _rmsnorm_loop(device, v, grid, name):
    """rms_norm_loop_kernel (ops/suite/dev/hidden__rms_norm_loop_kernel.py:10-46) and
    rmsnorm_fwd_loop_kernel (ops/suite/dev/rmsnorm_fwd_loop_kernel.py:10-34)."""
    rows = _grid_tuple(grid)[0]
    n = int(v["N"])
    rinv = v.get("INV_RMS", v.get("rsigma_ptr"))
    w = v.get("w_ptr", v.get("weight_ptr"))
    ops.rmsnorm(_View(v["in_ptr"], (rows, n)), _View(w, (n,)), _View(v["out_ptr"], (rows, n)),
                _View(rinv, (rows,)), float(v["eps"]),
                gamma_offset=1.0 if v.get("zero_centered_gamma", False) else 0.0,
                stream=device.stream)


def _softmax(device, v, grid, name):
    """softmax_kernel (ops/suite/perf/softmax.py:21)."""
    rows = _grid_tuple(grid)[0]
    n_cols = int(v["n_cols"])
    ops.softmax(_View(v["x_ptr"], (rows, n_cols)), _View(v["y_ptr"], (rows, n_cols)),
                stream=device.stream)


def _softmax_inner(device, v, grid, name):
    """softmax_kernel_inner (ops/suite/dev/softmax_kernel_inner.py:12)."""
    m, n = int(v["M"]), int(v["N"])
    _require(_grid_tuple(grid)[0] == m, name, "grid", "expected one program per row")
    ops.softmax(_View(v["input_ptr"], (m, n)), _View(v["output_ptr"], (m, n)),
                stream=device.stream)


def _softmax_multi_block(device, v, grid, name):
    """_softmax_multi_block_forward_kernel
    (ops/suite/dev/softmax_multi_block_forward_kernel.py:12-48): every program walks rows
    program_id, program_id + num_programs, ... with an online max / sum over BLOCK_SIZE
    columns at a time -- the algorithm of the native persistent row kernel, which picks its
    own program count."""
    rows, cols = int(v["n_rows"]), int(v["n_cols"])
    _require(_grid_tuple(grid)[0] >= 1, name, "grid", "expected at least one program")
    _require(int(v["X_row_stride"]) == cols and int(v["Y_row_stride"]) == cols, name,
             "X_row_stride", "only contiguous rows (row stride == n_cols) have a native kernel")
    ops.softmax(_View(v["X_ptr"], (rows, cols)), _View(v["Y_ptr"], (rows, cols)),
                stream=device.stream)


def _masked_softmax(device, v, grid, name):
    """Native handle: row softmax with the causal-mod mask (kernels.masked_softmax_kernel)."""
    rows = _grid_tuple(grid)[0]
    n_cols = int(v["n_cols"])
    ops.softmax(_View(v["x_ptr"], (rows, n_cols)), _View(v["y_ptr"], (rows, n_cols)),
                causal_mod=True, row_offset=int(v.get("row_offset", 0)), stream=device.stream)


def _matmul_plain(device, v, grid, name):
    """matmul_kernel (ops/suite/perf/matmul.py:21): contiguous row-major A, B, Y."""
    m, n, k = int(v["M"]), int(v["N"]), int(v["K"])
    ops.gemm(_View(v["a_ptr"], (m, k)), _View(v["b_ptr"], (k, n)), _View(v["y_ptr"], (m, n)),
             stream=device.stream)


def _row_major(v, name, prefix_pairs):
    for rows_key, unit_key in prefix_pairs:
        _require(int(v[unit_key]) == 1, name, unit_key,
                 "only row-major operands (unit inner stride) have a native kernel")


def _b_operand(v, name, rows_key, cols_key, k, n):
    """The B operand of a strided matmul: row-major [K, N] (unit stride along N), or its
    transpose in memory -- unit stride along K, i.e. a [N, K] weight -- which the native GEMM
    takes as a K-major operand.  Returns (view, transposed)."""
    stride_k, stride_n = int(v[rows_key]), int(v[cols_key])
    if stride_n == 1:
        return (k, n), (stride_k, 1), False
    _require(stride_k == 1, name, cols_key,
             "B needs a unit stride along N (row-major [K,N]) or along K (a [N,K] weight)")
    return (n, k), (stride_n, 1), True


def _matmul_strided(device, v, grid, name):
    """matmul_kernel (ops/suite/perf/matmul_triton2.py:27-30, matmul_triton_autotune.py:28-31)."""
    m, n, k = int(v["M"]), int(v["N"]), int(v["K"])
    _row_major(v, name, (("stride_am", "stride_ak"), ("stride_cm", "stride_cn")))
    shape, strides, transposed = _b_operand(v, name, "stride_bk", "stride_bn", k, n)
    leaky = bool(v.get("LEAKY", False))
    if leaky:
        _require(abs(float(v.get("SLOPE", 0.01)) - 0.01) < 1e-12, name, "SLOPE",
                 "the native leaky-ReLU epilogue uses slope 0.01")
    (ops.linear if transposed else ops.gemm)(
        _View(v["a_ptr"], (m, k), (int(v["stride_am"]), 1)), _View(v["b_ptr"], shape, strides),
        _View(v["c_ptr"], (m, n), (int(v["stride_cm"]), 1)),
        act=abi.ACT_LEAKY_RELU if leaky else abi.ACT_NONE, stream=device.stream)


def _linear_act(device, v, grid, name):
    """linear_act_kernel (ops/suite/perf/triton_linear_activation.py:28-30): bias + erf-GELU."""
    m, n, k = int(v["M"]), int(v["N"]), int(v["K"])
    _row_major(v, name, (("stride_xm", "stride_xk"), ("stride_ym", "stride_yn")))
    shape, strides, transposed = _b_operand(v, name, "stride_wk", "stride_wn", k, n)
    (ops.linear if transposed else ops.gemm)(
        _View(v["x_ptr"], (m, k), (int(v["stride_xm"]), 1)), _View(v["w_ptr"], shape, strides),
        _View(v["y_ptr"], (m, n), (int(v["stride_ym"]), 1)),
        bias=_View(v["b_ptr"], (n,)), act=abi.ACT_GELU_ERF, stream=device.stream)


def _gemm_gn_min(device, v, grid, name):
    """fused_gemm_gn_min_kernel (ops/suite/dev/fused_gemm_gn_min_kernel.py:26): row-major
    X [M,K], W [K,N]."""
    m, n, k = int(v["M"]), int(v["N"]), int(v["K"])
    _require(int(v["stride_xk"]) == 1 and int(v["stride_wn"]) == 1, name, "strides",
             "only row-major X and W have a native kernel")
    ops.gemm_groupnorm_rowmin(
        _View(v["X_ptr"], (m, k), (int(v["stride_xm"]), 1)),
        _View(v["W_ptr"], (k, n), (int(v["stride_wk"]), 1)), _View(v["Gamma_ptr"], (n,)),
        _View(v["Beta_ptr"], (n,)), _View(v["Mins_ptr"], (m,)), bias=_View(v["B_ptr"], (n,)),
        group_size=int(v["GROUP_SIZE"]), eps=float(v["eps"]), stream=device.stream)


def _dequantize(device, v, grid, name):
    """dequantize_kernel (ops/suite/perf/dequantize_matmul.py:27-29)."""
    k, n = int(v["K"]), int(v["N"])
    _require(int(v["stride_bn"]) == 1 and int(v["stride_fpbn"]) == 1, name, "strides",
             "only unit column strides have a native kernel")
    ops.dequantize_cols(_View(v["b_ptr"], (k, n), (int(v["stride_bk"]), 1)),
                        _View(v["b_scale_ptr"], (n,)),
                        _View(v["fpb_ptr"], (k, n), (int(v["stride_fpbk"]), 1)),
                        stream=device.stream)


def _rms_matmul(device, v, grid, name):
    """rms_matmul_rbe_kernel (ops/suite/dev/rms_matmul_rbe.py:18-30): batches of [M,K] rows
    against one [K,N] weight.  (USE_FP8 / RBE_EPILOGUE are constexprs without code behind them
    in the reference's compile unit; anything but False is refused.)"""
    _require(not v.get("RBE_EPILOGUE", False) and not v.get("USE_FP8", False), name,
             "RBE_EPILOGUE", "only USE_FP8=False, RBE_EPILOGUE=False exist in the reference program")
    m, n, k = int(v["M"]), int(v["N"]), int(v["K"])
    batches = _grid_tuple(grid)[0]
    _require(int(v["stride_x_k"]) == 1 and int(v["stride_w_n"]) == 1 and
             int(v["stride_out_n"]) == 1 and int(v["stride_rms_w"]) == 1, name, "strides",
             "only unit inner strides have a native kernel")
    xm, om = int(v["stride_x_m"]), int(v["stride_out_m"])
    _require(batches == 1 or (int(v["stride_x_batch"]) == m * xm and
                              int(v["stride_out_batch"]) == m * om), name, "strides",
             "batches must follow each other without gaps")
    rows = batches * m
    scratch = device.workspace(("rms_matmul", k, n, rows, str(v["w_ptr"].dtype)),
                               (((k, n), v["w_ptr"].dtype), ((rows,), "float32")))
    ops.rms_matmul(_View(v["x_ptr"], (rows, k), (xm, 1)), _View(v["rms_w_ptr"], (k,)),
                   _View(v["w_ptr"], (k, n), (int(v["stride_w_k"]), 1)),
                   _View(v["out_ptr"], (rows, n), (om, 1)), scratch[0], scratch[1],
                   eps=float(v["EPS"]), stream=device.stream)


def _log_softmax_linear(device, v, grid, name):
    """log_softmax_linear_kernel (ops/suite/perf/log_softmax_linear.py:19): one program per row,
    contiguous x [rows, K], w [N, K], y [rows, N]."""
    rows = _grid_tuple(grid)[0]
    k, n = int(v["K"]), int(v["N"])
    _require(n <= 64, name, "N", "the reference program covers at most 64 outputs")
    ops.linear_log_softmax(_View(v["x_ptr"], (rows, k)), _View(v["w_ptr"], (n, k)),
                           _View(v["y_ptr"], (rows, n)), stream=device.stream)


def _gemm_bias_act(device, v, grid, name):
    """Native handle: C = act(A @ B + bias) with a selectable epilogue
    (kernels.gemm_bias_act_kernel)."""
    m, n, k = int(v["M"]), int(v["N"]), int(v["K"])
    bias = v.get("bias_ptr")
    ops.gemm(_View(v["a_ptr"], (m, k)), _View(v["b_ptr"], (k, n)), _View(v["c_ptr"], (m, n)),
             bias=_View(bias, (n,)) if _is_buffer(bias) else None, act=int(v["ACT"]),
             stream=device.stream)


def _attention(device, v, grid, name):
    """attn_fwd_causal_kernel (ops/suite/perf/attn_fwd_causal.py:20-28) and its twins."""
    z, h, n = int(v["Z"]), int(v["H"]), int(v["N_CTX"])
    d = int(v["HEAD_DIM"])
    _require(int(v["stride_qk"]) == 1 and int(v["stride_kk"]) == 1 and
             int(v["stride_vn"]) == 1 and int(v["stride_on"]) == 1, name, "strides",
             "the head dimension must have unit stride")
    g = _grid_tuple(grid)
    _require(g[0] == n and g[1] == z * h, name, "grid", "expected grid (N_CTX, Z*H)")

    def view(key, sz, sh, sm):
        return _View(v[key], (z, h, n, d), (int(v[sz]), int(v[sh]), int(v[sm]), 1))

    lse = v.get("lse_ptr")
    ops.attention(view("q_ptr", "stride_qz", "stride_qh", "stride_qm"),
                  view("k_ptr", "stride_kz", "stride_kh", "stride_kn"),
                  view("v_ptr", "stride_vz", "stride_vh", "stride_vk"),
                  view("out_ptr", "stride_oz", "stride_oh", "stride_om"),
                  lse=_View(lse, (z, h, n)) if _is_buffer(lse) else None,
                  scale=float(v["scale"]), causal=bool(v["CAUSAL"]), stream=device.stream)


def _gqa(device, v, grid, name):
    """gqa_kernel (ops/suite/dev/gqa.py:19-58): non-causal attention, GROUP query heads per
    K / V head; batch and head share one stride, so both are folded into the head axis."""
    n, d, group = int(v["N_CTX"]), int(v["HEAD_DIM"]), int(v["GROUP"])
    hq, hkv = int(v["H_Q"]), int(v["H_KV"])
    _require(hq == hkv * group, name, "GROUP", "H_Q must be H_KV * GROUP")
    _require(int(v["stride_qk"]) == 1 and int(v["stride_kk"]) == 1 and
             int(v["stride_vn"]) == 1 and int(v["stride_on"]) == 1, name, "strides",
             "the head dimension must have unit stride")
    rows = _grid_tuple(grid)[1]          # Z * H_Q
    _require(rows % hq == 0, name, "grid", "expected grid (cdiv(N_CTX, BLOCK_N), Z*H_Q)")
    kv_rows = rows // group

    def view(key, heads, sh, sm):
        return _View(v[key], (1, heads, n, d), (heads * int(v[sh]), int(v[sh]), int(v[sm]), 1))

    ops.attention(view("Q", rows, "stride_qh", "stride_qm"), view("K", kv_rows, "stride_kh", "stride_kn"),
                  view("V", kv_rows, "stride_vh", "stride_vk"), view("Out", rows, "stride_oh", "stride_om"),
                  scale=float(v["scale"]), causal=False, stream=device.stream)


def _parallel_attn(device, v, grid, name):
    """parallel_attn_fwd_kernel (ops/suite/dev/parallel_attn_fwd_kernel.py): contiguous
    token-major q [B,T,HQ,K], k [B,T,H,K], v [B,T,H,V], o, g_cumsum, lse."""
    _require(not v.get("IS_VARLEN", False), name, "IS_VARLEN",
             "packed variable-length input has no native kernel")
    b, t, h, hq = int(v["B"]), int(v["T"]), int(v["H"]), int(v["HQ"])
    kd, vd = int(v["K"]), int(v["V"])
    _require(h > 0 and hq == h * int(v["G"]), name, "G", "HQ must be H * G")
    ops.attention_window(
        _View(v["q"], (b, t, hq, kd)), _View(v["k"], (b, t, h, kd)), _View(v["v"], (b, t, h, vd)),
        _View(v["o"], (b, t, hq, vd)),
        g_cumsum=_View(v["g_cumsum"], (b, t, hq)) if v.get("USE_G", False) else None,
        sink_bias=_View(v["sink_bias"], (hq,)) if v.get("USE_SINK_BIAS", False) else None,
        lse=_View(v["lse"], (b, t, hq)), scale=float(v["scale"]),
        window=int(v["W"]) if v.get("USE_WINDOW", False) else 0, stream=device.stream)


def _flash_varlen(device, v, grid, name):
    """flash_varlen_fwd_kernel (ops/suite/dev/flash_varlen_fwd_kernel.py:21-335), the dense
    case its reference covers (:370-418) and the causal one (mask aligned to the last key,
    :138; key length >= query length): packed sequences addressed through cu_seqlens (or
    fixed lengths with batch strides), key lengths from seqused_k, query and key lengths that
    differ, h / hk query heads per K / V head, log-sum-exp laid out [h, total_q]; and the
    soft-cap, ALiBi, local-window and paged-K/V modes (:91-146, CUDA-core kernel).  One launch of the
    attention operator per sequence, on strided views of the packed buffers.  The sequence
    boundaries are read back from the device, so this launch is bound afresh every time."""
    for flag in ("is_dropout", "return_softmax", "seqlenq_ngroups_swapped"):
        _require(not v.get(flag, False), name, flag,
                 "dropout, the returned softmax and the swapped-groups layout have no native "
                 "operator")
    h, hk, d, batches = int(v["h"]), int(v["hk"]), int(v["d"]), int(v["b"])
    _require(hk > 0 and h % hk == 0, name, "hk", "h must be a multiple of hk")
    total_q = int(v["total_q"])
    bounds = {}
    for side in ("q", "k"):
        if v.get(f"is_cu_seqlens_{side}", False):
            bounds[side] = [int(x) for x in device.download(v[f"cu_seqlens_{side}_ptr"])]
            _require(len(bounds[side]) >= batches + 1, name, f"cu_seqlens_{side}_ptr",
                     "needs b + 1 entries")
    used_k = ([int(x) for x in device.download(v["seqused_k_ptr"])]
              if v.get("is_seqused_k", False) else None)
    modes = {}
    if v.get("is_softcap", False):
        modes["softcap"] = float(v["softcap"])
    if v.get("is_local", False):
        modes["window"] = (int(v["window_size_left"]), int(v["window_size_right"]))
    for batch in range(batches):
        span = {}
        for side, rows in (("q", "q"), ("k", "k"), ("v", "k"), ("o", "q")):
            if rows in bounds:
                start, stop = bounds[rows][batch], bounds[rows][batch + 1]
                span[side] = (start * int(v[f"{side}_row_stride"]), stop - start, start)
            else:
                length = int(v[f"seqlen_{rows}"])
                span[side] = (batch * int(v[f"{side}_batch_stride"]), length, batch * length)
        q_len, k_len = span["q"][1], span["k"][1]
        if used_k is not None:
            k_len = used_k[batch]                      # :49-52
        if q_len <= 0:
            continue
        _require(k_len > 0, name, "cu_seqlens_k_ptr", "a sequence without keys")

        paged = bool(v.get("is_paged", False))

        def view(side, heads, length):
            head, row = int(v[f"{side}_head_stride"]), int(v[f"{side}_row_stride"])
            # paged K / V start at the cache's base: the page table places the rows (:91-108)
            offset = 0 if paged and side in ("k", "v") else span[side][0]
            return _View(v[f"{side}_ptr"], (1, heads, length, d), (heads * head, head, row, 1),
                         offset=offset)

        if paged:
            block = int(v["block_size"])
            pages = -(-k_len // block)
            modes["page_table"] = _View(v["page_table_ptr"], (1, pages), (pages, 1),
                                        offset=batch * int(v["page_table_batch_stride"]))
            modes["block_size"], modes["page_stride"] = block, int(v["k_page_stride"])

        lse = _View(v["softmax_lse_ptr"], (1, h, q_len), (h * total_q, total_q, 1),
                    offset=span["q"][2])
        if v.get("is_alibi", False):                   # one slope per (batch, head), :76-78
            modes["alibi_slopes"] = _View(v["alibi_slopes_ptr"], (h,), (1,),
                                          offset=batch * int(v["alibi_slopes_batch_stride"]))
        ops.attention(view("q", h, q_len), view("k", hk, k_len), view("v", hk, k_len),
                      view("o", h, q_len), lse=lse, scale=float(v["scale_softmax"]),
                      causal=bool(v.get("is_causal", False)), stream=device.stream, **modes)


_flash_varlen.reads_device = True


def _flash_decode(device, v, grid, name):
    """flash_decode_kernel (ops/suite/perf/flash_decode.py:21-23): one query row per program."""
    rows = _grid_tuple(grid)[0]
    n, d = int(v["N_CTX"]), int(v["HEAD_DIM"])
    _require(int(v["stride_kk"]) == 1 and int(v["stride_vn"]) == 1, name, "strides",
             "the head dimension must have unit stride")
    _require(rows % int(v["H"]) == 0, name, "grid", "expected one program per (batch, head)")
    ops.attention_decode(
        _View(v["Q"], (rows, d), (int(v["stride_qh"]), 1)),
        _View(v["K"], (rows, n, d), (int(v["stride_kh"]), int(v["stride_kn"]), 1)),
        _View(v["V"], (rows, n, d), (int(v["stride_vh"]), int(v["stride_vk"]), 1)),
        _View(v["Out"], (rows, d), (int(v["stride_oh"]), 1)),
        scale=float(v["scale"]), stream=device.stream)


def _swiglu(device, v, grid, name):
    """swiglu_fwd_kernel (ops/suite/perf/swiglu_fwd.py:27-28, swiglu_triton.py:19-20)."""
    rows = _grid_tuple(grid, {"BLOCK_N": 32})[0]
    cols = int(v["ncols"])
    ops.swiglu(_View(v["X"], (rows, cols), (int(v["stride_x_row"]), 1)),
               _View(v["Y"], (rows, cols), (int(v["stride_y_row"]), 1)),
               _View(v["OUT"], (rows, cols), (int(v["stride_out_row"]), 1)),
               stream=device.stream)


def _softmax_mul(device, v, grid, name):
    """softmax_mul_kernel (ops/suite/perf/softmax_mul.py:21)."""
    rows, n_cols = _grid_tuple(grid)[0], int(v["n_cols"])
    ops.softmax_variant(_View(v["x_ptr"], (rows, n_cols)), _View(v["y_ptr"], (rows, n_cols)),
                        mul=_View(v["o_ptr"], (rows, n_cols)), stream=device.stream)


def _softmax_log(device, v, grid, name):
    """softmax_log_kernel (ops/suite/perf/softmax_log.py:20)."""
    rows, n_cols = _grid_tuple(grid)[0], int(v["n_cols"])
    ops.softmax_variant(_View(v["x_ptr"], (rows, n_cols)), _View(v["y_ptr"], (rows, n_cols)),
                        log_input=True, stream=device.stream)


def _repeat_log_softmax(device, v, grid, name):
    """fused_repeat_interleave_log_softmax_kernel
    (ops/suite/perf/fused_repeat_interleave_log_softmax.py:19-20)."""
    rows = _grid_tuple(grid)[0]
    cols, repeat, length = int(v["COLS"]), int(v["R"]), int(v["L"])
    _require(int(v.get("BE", length)) >= length, name, "BE",
             "the reference program covers a row with one block: BE >= L")
    ops.repeat_log_softmax(_View(v["x_ptr"], (rows, cols)), _View(v["y_ptr"], (rows, length)),
                           repeat, stream=device.stream)


def _gelu(device, v, grid, name):
    """gelu_kernel (ops/suite/perf/gelu.py:21)."""
    n = int(v["n_elements"])
    ops.elementwise(abi.EW_GELU_ERF, _View(v["x_ptr"], (n,)), _View(v["y_ptr"], (n,)),
                    stream=device.stream)


def _add_gelu(device, v, grid, name):
    """add_gelu_kernel (ops/suite/perf/add_gelu.py:21): the kernel body overrides its alpha
    argument with 1.5 (:26), and so does this adapter."""
    n = int(v["n_elements"])
    ops.elementwise(abi.EW_ADD_GELU_ERF, _View(v["x_ptr"], (n,)), _View(v["y_ptr"], (n,)),
                    b=_View(v["o_ptr"], (n,)), p0=1.5, stream=device.stream)


def _geglu_tanh(device, v, grid, name):
    """geglu_tanh_forward_kernel (ops/suite/perf/geglu_tanh_triton.py:19-20): rows of n_cols
    elements at pitch `stride`; only the dense layout (stride == n_cols) has a flat kernel."""
    rows, n_cols = _grid_tuple(grid)[0], int(v["n_cols"])
    _require(int(v["stride"]) == n_cols, name, "stride", "rows must be dense (stride == n_cols)")
    n = rows * n_cols
    ops.elementwise(abi.EW_GEGLU_TANH, _View(v["a_ptr"], (n,)), _View(v["c_ptr"], (n,)),
                    b=_View(v["b_ptr"], (n,)), stream=device.stream)


def _epilogue(device, v, grid, name):
    """epilogue_kernel (ops/suite/dev/epilogue_kernel.py:24): in place on out_ptr."""
    n, n_cols = int(v["n_elements"]), int(v["n_cols"])
    ops.elementwise(abi.EW_BIAS_SCALE_CLAMP_GELU, _View(v["out_ptr"], (n,)),
                    _View(v["out_ptr"], (n,)), b=_View(v["bias_ptr"], (n_cols,)),
                    p0=float(v["scale"]), p1=float(v["ht_min"]), p2=float(v["ht_max"]),
                    stream=device.stream)


def _swiglu_gemm(device, v, grid, name):
    """Native handle: H = silu(X @ Wg) * (X @ Wu) in one kernel (kernels.swiglu_gemm_kernel)."""
    m, n, k = int(v["M"]), int(v["N"]), int(v["K"])
    ops.gemm(_View(v["x_ptr"], (m, k)), _View(v["wg_ptr"], (k, n)), _View(v["h_ptr"], (m, n)),
             b2=_View(v["wu_ptr"], (k, n)), act=abi.ACT_SWIGLU, stream=device.stream)


class Registry:
    """(kernel name, parameter names) -> adapter."""

    def __init__(self):
        self._entries = {}

    def register(self, name, parameters, adapter):
        self._entries[(name, tuple(parameters))] = adapter

    def resolve(self, kernel):
        name, parameters, _ = kernel_signature(kernel)
        adapter = self._entries.get((name, tuple(parameters)))
        if adapter is None:
            raise UnsupportedLaunch(
                name, "kernel",
                f"no native sm_100a operator is registered for signature "
                f"({', '.join(parameters)}); nothing falls back to Triton or the host")
        return name, adapter

    def reads_device(self, kernel) -> bool:
        """True when binding this kernel's launch reads device memory back (its library calls
        then depend on more than the arguments, and must not be replayed)."""
        name, parameters, _ = kernel_signature(kernel)
        return bool(getattr(self._entries.get((name, tuple(parameters))), "reads_device", False))

    def supports(self, kernel) -> bool:
        name, parameters, _ = kernel_signature(kernel)
        return (name, tuple(parameters)) in self._entries

    def launch(self, device, kernel, grid, positional, keywords):
        name, adapter = self.resolve(kernel)
        values = bind_by_name(kernel, positional, keywords)
        adapter(device, values, grid, name)


_ATTN = ("q_ptr", "k_ptr", "v_ptr", "out_ptr", "Z", "H", "N_CTX", "scale",
         "stride_qz", "stride_qh", "stride_qm", "stride_qk",
         "stride_kz", "stride_kh", "stride_kn", "stride_kk",
         "stride_vz", "stride_vh", "stride_vk", "stride_vn",
         "stride_oz", "stride_oh", "stride_om", "stride_on",
         "HEAD_DIM", "BLOCK_N", "CAUSAL")
_MATMUL_STRIDED = ("a_ptr", "b_ptr", "c_ptr", "M", "N", "K", "stride_am", "stride_ak",
                   "stride_bk", "stride_bn", "stride_cm", "stride_cn", "LEAKY", "SLOPE",
                   "BLOCK_M", "BLOCK_N", "BLOCK_K")


_VARLEN = (
    "q_ptr", "k_ptr", "v_ptr", "o_ptr", "p_ptr", "softmax_lse_ptr", "q_row_stride",
    "k_row_stride", "v_row_stride", "q_head_stride", "k_head_stride", "v_head_stride",
    "o_row_stride", "o_head_stride", "q_batch_stride", "k_batch_stride",
    "v_batch_stride", "o_batch_stride", "is_cu_seqlens_q", "cu_seqlens_q_ptr",
    "is_cu_seqlens_k", "cu_seqlens_k_ptr", "is_seqused_k", "seqused_k_ptr", "b", "bk",
    "h", "hk", "h_hk_ratio", "seqlen_q", "seqlen_k", "seqlen_q_rounded",
    "seqlen_k_rounded", "d", "d_rounded", "is_softcap", "softcap", "scale_softmax",
    "scale_softmax_log2", "is_dropout", "p_dropout", "rp_dropout",
    "p_dropout_in_uint8_t", "philox_args", "return_softmax", "is_causal", "is_local",
    "window_size_left", "window_size_right", "seqlenq_ngroups_swapped", "is_paged",
    "is_alibi", "alibi_slopes_ptr", "alibi_slopes_batch_stride", "total_q",
    "page_table_ptr", "page_table_batch_stride", "block_size", "k_page_stride",
    "BLOCK_M", "BLOCK_N", "BLOCK_K", "KERNEL_NUM_WARPS", "PIPELINE_STAGES")


def default_registry() -> Registry:
    from compiler_b200 import kernels
    r = Registry()
    r.register("rms_layernorm_forward_kernel",
               ("Y", "Y_row_stride", "X", "X_row_stride", "W", "W_row_stride", "r",
                "r_row_stride", "n_cols", "eps", "BLOCK_SIZE"), _rmsnorm)
    r.register("rms_norm_loop_kernel",
               ("out_ptr", "INV_RMS", "in_ptr", "w_ptr", "N", "eps", "TILE_N"), _rmsnorm_loop)
    r.register("rmsnorm_fwd_loop_kernel",
               ("out_ptr", "rsigma_ptr", "in_ptr", "weight_ptr", "N", "eps",
                "zero_centered_gamma", "TILE_N"), _rmsnorm_loop)
    r.register("softmax_kernel", ("x_ptr", "y_ptr", "n_cols", "BLOCK_N"), _softmax)
    r.register("softmax_kernel_inner",
               ("output_ptr", "input_ptr", "M", "N", "TILE_N", "ONE_TILE_PER_CTA"),
               _softmax_inner)
    r.register("_softmax_multi_block_forward_kernel",
               ("Y_ptr", "Y_row_stride", "X_ptr", "X_row_stride", "n_rows", "n_cols",
                "BLOCK_SIZE"), _softmax_multi_block)
    r.register("matmul_kernel", ("a_ptr", "b_ptr", "y_ptr", "M", "N", "K"), _matmul_plain)
    r.register("matmul_kernel", _MATMUL_STRIDED, _matmul_strided)
    r.register("linear_act_kernel",
               ("x_ptr", "w_ptr", "b_ptr", "y_ptr", "M", "N", "K", "stride_xm", "stride_xk",
                "stride_wk", "stride_wn", "stride_ym", "stride_yn", "BLOCK_M", "BLOCK_N",
                "BLOCK_K"), _linear_act)
    for attn_name in ("attn_fwd_causal_kernel", "attention_forward_kernel", "attention_kernel",
                      "context_attn_fwd_kernel"):
        r.register(attn_name, _ATTN, _attention)
    r.register("fused_gemm_gn_min_kernel",
               ("X_ptr", "W_ptr", "B_ptr", "Gamma_ptr", "Beta_ptr", "Mins_ptr", "M", "N", "K",
                "stride_xm", "stride_xk", "stride_wn", "stride_wk", "eps", "BLOCK_M", "BLOCK_N",
                "BLOCK_K", "GROUP_SIZE", "GROUP_M"), _gemm_gn_min)
    r.register("dequantize_kernel",
               ("b_ptr", "b_scale_ptr", "fpb_ptr", "K", "N", "stride_bk", "stride_bn",
                "stride_fpbk", "stride_fpbn", "BLOCK_K", "BLOCK_N"), _dequantize)
    r.register("rms_matmul_rbe_kernel",
               ("x_ptr", "w_ptr", "rms_w_ptr", "out_ptr", "M", "N", "K", "stride_x_batch",
                "stride_x_m", "stride_x_k", "stride_w_k", "stride_w_n", "stride_rms_w",
                "stride_out_batch", "stride_out_m", "stride_out_n", "start_token_position",
                "USE_FP8", "RBE_EPILOGUE", "THETA", "EPS", "BLOCK_SIZE_M", "BLOCK_SIZE_N",
                "BLOCK_SIZE_K"), _rms_matmul)
    r.register("log_softmax_linear_kernel", ("x_ptr", "w_ptr", "y_ptr", "K", "N"),
               _log_softmax_linear)
    r.register("parallel_attn_fwd_kernel",
               ("q", "k", "v", "o", "g_cumsum", "sink_bias", "lse", "scale", "cu_seqlens",
                "chunk_indices", "T", "W", "B", "H", "HQ", "G", "K", "V", "BT", "BS", "BK", "BV",
                "USE_G", "USE_SINK_BIAS", "USE_WINDOW", "IS_VARLEN"), _parallel_attn)
    r.register("flash_varlen_fwd_kernel", _VARLEN, _flash_varlen)
    r.register("gqa_kernel",
               ("Q", "K", "V", "Out", "stride_qh", "stride_qm", "stride_qk", "stride_kh",
                "stride_kn", "stride_kk", "stride_vh", "stride_vk", "stride_vn", "stride_oh",
                "stride_om", "stride_on", "H_Q", "H_KV", "N_CTX", "scale", "GROUP", "HEAD_DIM",
                "BLOCK_N"), _gqa)
    r.register("flash_decode_kernel",
               ("Q", "K", "V", "Out", "stride_qh", "stride_kh", "stride_kn", "stride_kk",
                "stride_vh", "stride_vk", "stride_vn", "stride_oh", "H", "N_CTX", "scale",
                "HEAD_DIM", "BLOCK_N"), _flash_decode)
    r.register("swiglu_fwd_kernel",
               ("X", "Y", "OUT", "stride_x_row", "stride_y_row", "stride_out_row", "ncols",
                "BLOCK_N"), _swiglu)
    r.register("softmax_mul_kernel", ("x_ptr", "o_ptr", "y_ptr", "n_cols", "BLOCK_N"), _softmax_mul)
    r.register("softmax_log_kernel", ("x_ptr", "y_ptr", "n_cols", "BLOCK_N"), _softmax_log)
    r.register("fused_repeat_interleave_log_softmax_kernel",
               ("x_ptr", "y_ptr", "COLS", "R", "L", "BE"), _repeat_log_softmax)
    r.register("gelu_kernel", ("x_ptr", "y_ptr", "n_elements", "BLOCK_SIZE"), _gelu)
    r.register("add_gelu_kernel", ("x_ptr", "o_ptr", "y_ptr", "alpha", "n_elements", "BLOCK"),
               _add_gelu)
    r.register("geglu_tanh_forward_kernel",
               ("a_ptr", "b_ptr", "c_ptr", "stride", "n_cols", "BLOCK_SIZE"), _geglu_tanh)
    r.register("epilogue_kernel",
               ("out_ptr", "bias_ptr", "n_elements", "n_cols", "scale", "ht_min", "ht_max",
                "BLOCK_SIZE"), _epilogue)
    # native handles for the configurations no single reference kernel covers
    for handle, adapter in ((kernels.masked_softmax_kernel, _masked_softmax),
                            (kernels.gemm_bias_act_kernel, _gemm_bias_act),
                            (kernels.attn_fwd_lse_kernel, _attention),
                            (kernels.swiglu_gemm_kernel, _swiglu_gemm)):
        name, parameters, _ = kernel_signature(handle)
        r.register(name, tuple(parameters), adapter)
    return r
