"""Fused AdaLN and gated-residual autograd ops with the call surface of
anima-trainer's ``adaln_kernel.py`` (``FusedAdaLN`` :157, ``fused_adaln`` :258,
``FusedGatedAdd`` :332, ``fused_gated_add`` :422), backed by the sm_100a kernels
in ``csrc/adaln.cu``.

Shapes follow the reference: ``x``/``y`` are ``(B, T, H, W, D)``, modulation
tensors are ``(B, T, 1, 1, D)`` and broadcast over ``(H, W)``. Statistics and all
elementwise math are fp32; results are stored in bf16. Unlike the reference the
``(H, W)`` reductions (dscale, dshift, dgate) are deterministic.
"""
from __future__ import annotations

import torch

from . import ops

BF16 = torch.bfloat16

# When set, the AdaLN forward kernels also write the row-wise MXFP8 operand of their output (same pass, one
# more byte per element) and hand it to the quantised linears that consume the output through
# ``fp8_quant.adopt_row_operand``; those linears then launch no quantiser for it (the column-wise operand a
# trainable linear needs for its weight gradient is still made from y when asked for).
_EMIT_ROW_OPERAND = False


def emit_row_operand(enabled: bool = True) -> None:
    """Switch the quantise-in-the-producer forward on or off (off by default: it only pays when the consumers
    of the AdaLN output are this package's MXFP8 linears)."""
    global _EMIT_ROW_OPERAND
    _EMIT_ROW_OPERAND = bool(enabled)


def _emits(x: torch.Tensor, rows: int, d: int) -> bool:
    return _EMIT_ROW_OPERAND and x.dtype == BF16 and ops.can_emit_row_codes(rows, d)


def _flat(t: torch.Tensor, d: int) -> torch.Tensor:
    t = t.contiguous().view(-1, d)
    return t if t.dtype == BF16 else t.to(BF16)


def _need_bf16_stream(name: str, *tensors: torch.Tensor) -> None:
    """The kernels store bf16. The reference's ops keep the input dtype (``torch.empty_like(x_flat)``,
    adaln_kernel.py:185-187), so an fp32 residual stream would be rounded to bf16 at every sublayer here without
    notice; it is refused instead (modulation tensors of another dtype are cast, their gradients cast back)."""
    for t in tensors:
        if t.dtype != BF16:
            raise TypeError(f"{name}: activations must be bfloat16, got {t.dtype} (the fused kernels have no "
                            "fp32-stream form; use the block's unpatched forward for use_fp32)")


class FusedAdaLN(torch.autograd.Function):
    """``LayerNorm(x, no affine, eps) * (1 + scale) + shift``."""

    @staticmethod
    def forward(ctx, x, scale, shift, eps):
        assert x.is_cuda, "FusedAdaLN requires CUDA tensors"
        _need_bf16_stream("FusedAdaLN", x)
        B, T, H, W, D = x.shape
        x_flat, scale_flat, shift_flat = _flat(x, D), _flat(scale, D), _flat(shift, D)
        N, M, HW = x_flat.shape[0], scale_flat.shape[0], H * W
        assert N == M * HW, f"shape mismatch: N={N}, M={M}, HW={HW}"
        if _emits(x, N, D):
            from . import fp8_quant
            y, mean, rstd, y_row = ops.adaln_fwd(x_flat, scale_flat, shift_flat, eps, HW, quant=True)
            fp8_quant.adopt_row_operand(y, y_row)
        else:
            y, mean, rstd = ops.adaln_fwd(x_flat, scale_flat, shift_flat, eps, HW)
        ctx.save_for_backward(x_flat, scale_flat, mean, rstd)
        ctx.x_shape, ctx.scale_shape, ctx.HW = (B, T, H, W, D), scale.shape, HW
        ctx.dtypes = (x.dtype, scale.dtype, shift.dtype)
        return y.view(B, T, H, W, D).to(x.dtype)

    @staticmethod
    def backward(ctx, dy):
        x_flat, scale_flat, mean, rstd = ctx.saved_tensors
        B, T, H, W, D = ctx.x_shape
        dx, dscale, dshift = ops.adaln_bwd(_flat(dy, D), x_flat, scale_flat, mean, rstd, ctx.HW)
        xd, sd, bd = ctx.dtypes
        return (dx.view(B, T, H, W, D).to(xd), dscale.view(ctx.scale_shape).to(sd),
                dshift.view(ctx.scale_shape).to(bd), None)


def fused_adaln(x: torch.Tensor, scale: torch.Tensor, shift: torch.Tensor, eps: float) -> torch.Tensor:
    return FusedAdaLN.apply(x, scale, shift, eps)


class FusedGatedAdd(torch.autograd.Function):
    """``out = x + gate * y``; backward ``dx = dout``, ``dy = gate * dout``,
    ``dgate = sum_{h,w}(dout * y)``."""

    @staticmethod
    def forward(ctx, x, gate, y):
        assert x.is_cuda, "FusedGatedAdd requires CUDA tensors"
        assert x.shape == y.shape, f"x {x.shape} != y {y.shape}"
        _need_bf16_stream("FusedGatedAdd", x, y)
        B, T, H, W, D = x.shape
        x_flat, y_flat, gate_flat = _flat(x, D), _flat(y, D), _flat(gate, D)
        N, M, HW = x_flat.shape[0], gate_flat.shape[0], H * W
        assert N == M * HW, f"shape mismatch: N={N}, M={M}, HW={HW}"
        out = ops.gated_add_fwd(x_flat, gate_flat, y_flat, HW)
        ctx.save_for_backward(y_flat, gate_flat)
        ctx.shape, ctx.gate_shape, ctx.HW = (B, T, H, W, D), gate.shape, HW
        ctx.dtypes = (gate.dtype, y.dtype)
        return out.view(B, T, H, W, D).to(x.dtype)

    @staticmethod
    def backward(ctx, dout):
        y_flat, gate_flat = ctx.saved_tensors
        B, T, H, W, D = ctx.shape
        dy, dgate = ops.gated_add_bwd(_flat(dout, D), y_flat, gate_flat, ctx.HW)
        gd, yd = ctx.dtypes
        return dout, dgate.view(ctx.gate_shape).to(gd), dy.view(B, T, H, W, D).to(yd)


def fused_gated_add(x: torch.Tensor, gate: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
    return FusedGatedAdd.apply(x, gate, y)


class FusedGatedAddAdaLN(torch.autograd.Function):
    """``x_new = x + gate * sub`` followed by ``y = AdaLN(x_new; scale, shift)``: the residual update of one
    sublayer and the modulation of the next, from one read of x and sub. Returns ``(x_new, y)``, each
    bit-identical to ``FusedGatedAdd`` then ``FusedAdaLN``; backward is one kernel too (the AdaLN input
    gradient, its sum with the residual-stream gradient, and the gated-residual backward), again bit-identical
    to the separate kernels."""

    @staticmethod
    def forward(ctx, x, gate, sub, scale, shift, eps):
        assert x.is_cuda, "FusedGatedAddAdaLN requires CUDA tensors"
        assert x.shape == sub.shape, f"x {x.shape} != sub {sub.shape}"
        _need_bf16_stream("FusedGatedAddAdaLN", x, sub)
        B, T, H, W, D = x.shape
        x_flat, sub_flat = _flat(x, D), _flat(sub, D)
        gate_flat, scale_flat, shift_flat = _flat(gate, D), _flat(scale, D), _flat(shift, D)
        HW = H * W
        assert x_flat.shape[0] == gate_flat.shape[0] * HW == scale_flat.shape[0] * HW, "modulation shape mismatch"
        if _emits(x, x_flat.shape[0], D):
            from . import fp8_quant
            x_new, y, mean, rstd, y_row = ops.gated_add_adaln_fwd(x_flat, gate_flat, sub_flat, scale_flat, shift_flat,
                                                                  eps, HW, quant=True)
            fp8_quant.adopt_row_operand(y, y_row)
        else:
            x_new, y, mean, rstd = ops.gated_add_adaln_fwd(x_flat, gate_flat, sub_flat, scale_flat, shift_flat, eps, HW)
        ctx.save_for_backward(sub_flat, gate_flat, x_new, scale_flat, mean, rstd)
        ctx.shape, ctx.mod_shape, ctx.HW = (B, T, H, W, D), gate.shape, HW
        ctx.dtypes = (x.dtype, gate.dtype, sub.dtype, scale.dtype, shift.dtype)
        return x_new.view(B, T, H, W, D).to(x.dtype), y.view(B, T, H, W, D).to(x.dtype)

    @staticmethod
    def backward(ctx, d_xnew, d_y):
        sub_flat, gate_flat, x_new, scale_flat, mean, rstd = ctx.saved_tensors
        B, T, H, W, D = ctx.shape
        xd, gd, ud, sd, bd = ctx.dtypes
        if d_xnew is not None and d_y is not None:      # the usual case: one kernel for both backward ops
            dout, dsub, dscale, dshift, dgate = ops.gated_add_adaln_bwd(
                _flat(d_y, D), _flat(d_xnew, D), x_new, scale_flat, mean, rstd, sub_flat, gate_flat, ctx.HW)
        else:
            dout = None if d_xnew is None else _flat(d_xnew, D)
            dscale = dshift = None
            if d_y is not None:
                dout, dscale, dshift = ops.adaln_bwd(_flat(d_y, D), x_new, scale_flat, mean, rstd, ctx.HW)
            dsub, dgate = ops.gated_add_bwd(dout, sub_flat, gate_flat, ctx.HW)
        if dscale is not None:
            dscale, dshift = dscale.view(ctx.mod_shape).to(sd), dshift.view(ctx.mod_shape).to(bd)
        return (dout.view(B, T, H, W, D).to(xd), dgate.view(ctx.mod_shape).to(gd), dsub.view(B, T, H, W, D).to(ud),
                dscale, dshift, None)


def fused_gated_add_adaln(x, gate, sub, scale, shift, eps):
    return FusedGatedAddAdaLN.apply(x, gate, sub, scale, shift, eps)
