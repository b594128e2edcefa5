"""Kernel handles for the configurations that no single reference kernel covers.

A handle plays the part of ``case["kernel"]`` in a harness case
(ops/harness/opslib/device.py:341-349): the harness only inspects the signature
of its ``.fn`` to bind arguments by name, and ``B200Device.launch`` resolves the
handle to a native operator through the registry.  The bodies are empty on
purpose -- a handle is a *name and a parameter list*, not an implementation.
"""
from __future__ import annotations


class NativeKernel:
    """``JITFunction``-shaped handle: ``.fn`` is the signature carrier."""

    def __init__(self, fn):
        self.fn = fn
        self.__name__ = fn.__name__
        self.__doc__ = fn.__doc__

    def __getitem__(self, grid):
        raise RuntimeError(
            f"{self.__name__} is a handle, not a launcher: stage the case on a B200Device "
            "or obtain a compiled kernel from compiler_b200.factory.make_compiler()")

    def __repr__(self):
        return f"<NativeKernel {self.__name__}>"


def _masked_softmax_kernel(x_ptr, y_ptr, n_cols, row_offset):
    """Row softmax over contiguous [rows, n_cols] where column c of global row
    (row_offset + program_id) is kept iff c <= (row_offset + program_id) % n_cols and is
    -inf otherwise: softmax_kernel (ops/suite/perf/softmax.py:20-31) composed with the mask
    expression of ops/suite/perf/attn_fwd_causal.py:46-47.  grid = (rows,)."""


def _gemm_bias_act_kernel(a_ptr, b_ptr, bias_ptr, c_ptr, M, N, K, ACT):
    """C[M,N] = act(A[M,K] @ B[K,N] + bias[N]), contiguous row-major, fp32 accumulation;
    ACT is a ``b200_act`` code (0 none, 1 erf-GELU, 2 tanh-GELU, 3 leaky-ReLU); bias_ptr may
    be None: linear_act_kernel (ops/suite/perf/triton_linear_activation.py:27-49) with the
    activation of ops/suite/perf/geglu_tanh_triton.py:32-36 selectable."""


def _attn_fwd_lse_kernel(q_ptr, k_ptr, v_ptr, out_ptr, lse_ptr, Z, H, N_CTX, scale,
                         stride_qz, stride_qh, stride_qm, stride_qk,
                         stride_kz, stride_kh, stride_kn, stride_kk,
                         stride_vz, stride_vh, stride_vk, stride_vn,
                         stride_oz, stride_oh, stride_om, stride_on,
                         HEAD_DIM, CAUSAL):
    """attn_fwd_causal_kernel (ops/suite/perf/attn_fwd_causal.py:19-57) with one more
    output: lse[Z,H,N_CTX] fp32 = log sum exp of the scaled masked scores
    (ops/suite/dev/flash_varlen_fwd_kernel.py:309).  grid = (N_CTX, Z*H)."""


def _swiglu_gemm_kernel(x_ptr, wg_ptr, wu_ptr, h_ptr, M, N, K):
    """H[M,N] = silu(X[M,K] @ Wg[K,N]) * (X @ Wu[K,N]): swiglu_fwd_kernel
    (ops/suite/perf/swiglu_fwd.py:27-36) fused behind the two matmuls that feed it."""


masked_softmax_kernel = NativeKernel(_masked_softmax_kernel)
gemm_bias_act_kernel = NativeKernel(_gemm_bias_act_kernel)
attn_fwd_lse_kernel = NativeKernel(_attn_fwd_lse_kernel)
swiglu_gemm_kernel = NativeKernel(_swiglu_gemm_kernel)
