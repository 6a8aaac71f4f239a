"""MXFP8 quantiser and block-scaled GEMM with the call surface of anima-trainer's
``mxfp8_gemm.py`` — same names, argument meaning and error behaviour — running on
the hand-written sm_100a kernels of ``libanima_b200.so`` instead of Triton.

Mirrored interface (anima-trainer ``src/anima_trainer/mxfp8_gemm.py``):
``MXFP8Block`` (:51), ``quantize_rowwise`` (:150), ``quantize_weight_for_lhs``
(:186), ``quantize_weight_for_dgrad`` (:201), ``dequantize_rowwise`` (:225),
``mxfp8_matmul`` (:315), ``MXFP8FrozenLinearTriton`` (:342, here
``MXFP8FrozenLinearB200``; the old name is kept as an alias) and
``mxfp8_frozen_linear_triton`` (:422).

Differences a caller can observe:
* ``MXFP8Block.scales`` is still the plain ``(..., K//32)`` e8m0 tensor, but the
  block may also carry the tensor-core ("tiled") copy of the scales so that the
  GEMM does not have to re-lay them out on every call.
* ``quantize_weight_for_dgrad`` returns ``data`` as a ``(N, K)`` *view* of a
  ``(K, N)`` buffer (strides ``(1, N)``): element for element the reference's
  tensor, already contiguous along the dgrad contraction axis.
* ``mxfp8_matmul`` needs ``B_stride_k == 1``; both reference call sites
  (:375-380, :409-414) satisfy it with the blocks produced here.
"""
from __future__ import annotations

from typing import NamedTuple

import torch

from . import ops
from ._lib import SCALES_PLAIN, SCALES_TILED

FP8_E4M3_MAX = 448.0


class MXFP8Block(NamedTuple):
    """MXFP8 tensor: ``data`` uint8 e4m3 codes (shape of the source), ``scales`` uint8
    e8m0 ``(..., K//32)``. ``tiled`` optionally caches the GEMM-layout scales."""

    data: torch.Tensor
    scales: torch.Tensor
    tiled: torch.Tensor | None = None


def _as_operand(codes_2d: torch.Tensor, blk_scales: torch.Tensor, tiled: torch.Tensor | None
                ) -> ops.MXOperand:
    if tiled is not None:
        return ops.MXOperand(codes_2d, tiled, SCALES_TILED)
    rows, k = codes_2d.shape
    return ops.mx_retile(ops.MXOperand(codes_2d, blk_scales.reshape(rows, k // 32), SCALES_PLAIN))


def quantize_rowwise(x: torch.Tensor) -> MXFP8Block:
    """Rowwise MXFP8 quantise of ``x[..., K]``; scales ``(..., K//32)``."""
    assert x.shape[-1] % 32 == 0, f"K={x.shape[-1]} must be %32"
    shape = x.shape
    K = shape[-1]
    x_2d = x.reshape(-1, K)
    if x_2d.dtype != torch.bfloat16:
        x_2d = x_2d.to(torch.bfloat16)
    row, _ = ops.mx_quantize(x_2d, rowwise=True, colwise=False, layout=SCALES_PLAIN)
    return MXFP8Block(data=row.codes.reshape(*shape), scales=row.scales.reshape(*shape[:-1], K // 32))


def quantize_weight_for_lhs(W: torch.Tensor) -> MXFP8Block:
    """``W (N, K)`` as the forward operand of ``y = x @ W.T``: rowwise quantisation of W."""
    assert W.shape[-1] % 32 == 0, f"K={W.shape[-1]} must be %32"
    row, _ = ops.mx_quantize(W.to(torch.bfloat16), rowwise=True, colwise=False, layout=SCALES_PLAIN)
    tiled = ops.mx_retile(row)
    return MXFP8Block(data=row.codes, scales=row.scales, tiled=tiled.scales)


def quantize_weight_for_dgrad(W: torch.Tensor) -> MXFP8Block:
    """``W (N, K)`` as the operand of ``grad_x = grad_y @ W``: blocks of 32 along N.
    ``data`` has shape ``(N, K)``; ``scales`` has shape ``(K, N//32)``."""
    N, K = W.shape
    assert N % 32 == 0, f"N={N} must be %32 for columnwise MXFP8 dgrad path"
    _, col = ops.mx_quantize(W.to(torch.bfloat16), rowwise=False, colwise=True, layout=SCALES_PLAIN)
    tiled = ops.mx_retile(col)
    return MXFP8Block(data=col.codes.t(), scales=col.scales, tiled=tiled.scales)


def dequantize_rowwise(blk: MXFP8Block, original_shape: tuple) -> torch.Tensor:
    """Inverse of :func:`quantize_rowwise`; returns bf16 of ``original_shape``."""
    K = original_shape[-1]
    codes = blk.data.reshape(-1, K).contiguous()
    op = ops.MXOperand(codes, blk.scales.reshape(codes.shape[0], K // 32).contiguous(), SCALES_PLAIN)
    return ops.mx_dequantize(op).reshape(original_shape)


def mxfp8_matmul(A: MXFP8Block, B_data: torch.Tensor, B_scales: torch.Tensor,
                 M: int, N: int, K: int, B_stride_k: int, B_stride_n: int,
                 *, B_tiled: torch.Tensor | None = None, bias: torch.Tensor | None = None) -> torch.Tensor:
    """``C[M,N] = A.data[M,K] @ B[K,N]`` in MXFP8, bf16 out. ``B_data`` is addressed as
    ``B[k, n] = base[k * B_stride_k + n * B_stride_n]`` with scales ``B_scales (N, K//32)``."""
    if B_stride_k != 1 or B_stride_n != K:
        raise NotImplementedError(
            "mxfp8_matmul: the B operand must be contiguous along the contraction axis "
            f"(B_stride_k == 1, B_stride_n == K); got ({B_stride_k}, {B_stride_n})")
    a_op = _as_operand(A.data.reshape(M, K), A.scales, A.tiled)
    b_codes = torch.as_strided(B_data, (N, K), (K, 1), B_data.storage_offset())
    b_op = _as_operand(b_codes, B_scales, B_tiled)
    return ops.mx_gemm(a_op, b_op, bias=bias)


class MXFP8FrozenLinearB200(torch.autograd.Function):
    """``y = x @ W.T (+ bias)`` for a frozen, pre-quantised W; forward and dgrad both run
    as MXFP8 tensor-core GEMMs. Signature of ``MXFP8FrozenLinearTriton.apply``; the saved
    activation is the quantised one, as in the reference (:384-385)."""

    @staticmethod
    def forward(ctx, x, W_fwd_data, W_fwd_scales, W_bwd_data, W_bwd_scales, bias=None,
                W_fwd_tiled=None, W_bwd_tiled=None):
        D_in = x.shape[-1]
        D_out = W_fwd_data.shape[0]
        x_2d = x.reshape(-1, D_in)
        M = x_2d.shape[0]
        x_row, _ = ops.mx_quantize(x_2d.to(torch.bfloat16), rowwise=True, layout=SCALES_TILED)
        w_op = _as_operand(W_fwd_data, W_fwd_scales, W_fwd_tiled)
        y = ops.mx_gemm(x_row, w_op, bias=bias.to(torch.bfloat16) if bias is not None else None)
        ctx.save_for_backward(x_row.codes, x_row.scales, W_bwd_data, W_bwd_scales)
        ctx.W_bwd_tiled = W_bwd_tiled
        ctx.D_in, ctx.D_out, ctx.M = D_in, D_out, M
        ctx.has_bias = bias is not None
        ctx.x_orig_shape = x.shape
        return y.reshape(*x.shape[:-1], D_out).to(x.dtype)

    @staticmethod
    def backward(ctx, grad_y):
        _, _, W_bwd_data, W_bwd_scales = ctx.saved_tensors
        gy_2d = grad_y.reshape(ctx.M, ctx.D_out)
        gy_row, _ = ops.mx_quantize(gy_2d.to(torch.bfloat16), rowwise=True, layout=SCALES_TILED)
        # W_bwd_data is the (D_out, D_in) view of a (D_in, D_out) buffer: K-major for dgrad.
        wT = W_bwd_data.t()
        if not wT.is_contiguous():
            raise NotImplementedError("W_bwd must come from quantize_weight_for_dgrad()")
        w_op = _as_operand(wT, W_bwd_scales, ctx.W_bwd_tiled)
        grad_x = ops.mx_gemm(gy_row, w_op).reshape(ctx.x_orig_shape).to(grad_y.dtype)
        grad_bias = grad_y.reshape(-1, ctx.D_out).sum(dim=0) if ctx.has_bias else None
        return grad_x, None, None, None, None, grad_bias, None, None


MXFP8FrozenLinearTriton = MXFP8FrozenLinearB200  # name used by anima-trainer call sites


def mxfp8_frozen_linear_triton(x: torch.Tensor, W_fwd: MXFP8Block, W_bwd: MXFP8Block,
                               bias: torch.Tensor | None = None) -> torch.Tensor:
    """Functional wrapper (anima-trainer ``mxfp8_gemm.py:422-431``)."""
    return MXFP8FrozenLinearB200.apply(x, W_fwd.data, W_fwd.scales, W_bwd.data, W_bwd.scales, bias,
                                       W_fwd.tiled, W_bwd.tiled)


mxfp8_frozen_linear = mxfp8_frozen_linear_triton
