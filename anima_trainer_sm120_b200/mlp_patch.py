"""Fused LoKr MLP: ``layer2(gelu(layer1(x)))`` with the activation quantised inside its producer.

anima-trainer runs the block MLP as two independent LoKr linears with an eager GELU between them
(``lokr.py:65-67`` wraps ``mlp.layer1`` / ``mlp.layer2``; each call goes through
``lokr_patch._patched_forward`` :47-94 and ``FP8LoKrLinear`` ``fp8_quant.py:460-511``). Per MLP that
writes the activation ``gelu(h)`` [rows, 8192] to HBM and reads it back to quantise it, and in backward
writes ``grad_act * gelu'(h)`` and reads it back again. Here the two linears and the activation are ONE
autograd node:

forward   quantise x; merge+quantise W1; h = x W1^T (bf16, kept for backward);
          ``mx_quantize_gelu(h)`` emits the MXFP8 operands of gelu(h) straight from h;
          merge+quantise W2; y = gelu(h) W2^T.
backward  quantise grad_y; grad_act = grad_y W2 (bf16); dW2 = grad_y^T gelu(h) (fp32) -> dw1, dw2;
          ``mx_quantize_gelu(h, grad_act)`` emits the operands of grad_h; dx = grad_h W1;
          dW1 = grad_h^T x (fp32) -> dw1, dw2.

The arithmetic of each step is that of the unfused chain (the activation and its gradient are rounded
to bf16 before quantisation exactly where the eager kernels would round them, and the GELU values come
from a table of the eager kernel's own fp32 expressions), so the result equals
``lokr_linear_fused -> F.gelu -> lokr_linear_fused`` bit for bit.

``install`` patches ``GPT2FeedForward.forward``; a call falls through to the original forward unless
both layers carry an eligible LoKr adapter on the quantised path and the activation is the exact GELU.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from . import lokr_patch, ops
from .fp8_quant import _bias_bf16, _flat2d, _pack, _placeholder, _unpack, in_first_pass, quantize_activation

_PATCHED: dict[type, object] = {}


class LoKrMLPFused(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, W1, b1, w1a, w2a, alpha1: float, W2, b2, w1b, w2b, alpha2: float):
        first = in_first_pass()           # a checkpointed block's first pass keeps nothing for backward
        train = any(ctx.needs_input_grad[i] for i in (3, 4, 8, 9))
        both = not first
        x_row, x_col = quantize_activation(x, colwise=train and both)
        _, W1_row, W1_col = ops.lokr_merge_quantize(W1.detach(), w1a.detach(), w2a.detach(), alpha1, want_merged=False,
                                                    rowwise=True, colwise=both)
        h = ops.mx_gemm(x_row, W1_row, bias=_bias_bf16(b1))
        a_row, a_col = ops.mx_quantize_gelu(h, rowwise=True, colwise=train and both)
        _, W2_row, W2_col = ops.lokr_merge_quantize(W2.detach(), w1b.detach(), w2b.detach(), alpha2, want_merged=False,
                                                    rowwise=True, colwise=both)
        y = ops.mx_gemm(a_row, W2_row, bias=_bias_bf16(b2))
        if first:
            rows, (hid, k_in), n_out = h.shape[0], W1.shape, W2.shape[0]
            W1_col, W2_col = _placeholder(k_in, hid, x.device), _placeholder(hid, n_out, x.device)
            if train:
                x_col, a_col = _placeholder(k_in, rows, x.device), _placeholder(hid, rows, x.device)
        ctx.save_for_backward(h, w1a, w2a, w1b, w2b, *_pack(x_col), *_pack(a_col), *_pack(W1_col), *_pack(W2_col))
        ctx.alphas = (float(alpha1), float(alpha2))
        ctx.in_features = W1.shape[1]
        return y.reshape(*x.shape[:-1], W2.shape[0]).to(x.dtype)

    @staticmethod
    def backward(ctx, grad_y):
        saved = ctx.saved_tensors
        h, w1a, w2a, w1b, w2b = saved[:5]
        x_col, a_col, W1_col, W2_col = (_unpack(*saved[i:i + 2]) for i in (5, 7, 9, 11))
        alpha1, alpha2 = ctx.alphas
        train = x_col is not None
        g_row, g_col = ops.mx_quantize(_flat2d(grad_y), rowwise=True, colwise=train)
        grad_act = ops.mx_gemm(g_row, W2_col)
        g1a = g2a = g1b = g2b = None
        if train:
            d1, d2 = ops.lokr_kron_backward(ops.mx_gemm(g_col, a_col, out_dtype=torch.float32),
                                            w1b.detach(), w2b.detach(), alpha2)
            g1b, g2b = d1.to(w1b.dtype), d2.to(w2b.dtype)
        dh_row, dh_col = ops.mx_quantize_gelu(h, grad_act, rowwise=True, colwise=train)
        del grad_act
        grad_x = ops.mx_gemm(dh_row, W1_col).reshape(*grad_y.shape[:-1], ctx.in_features).to(grad_y.dtype)
        if train:
            d1, d2 = ops.lokr_kron_backward(ops.mx_gemm(dh_col, x_col, out_dtype=torch.float32),
                                            w1a.detach(), w2a.detach(), alpha1)
            g1a, g2a = d1.to(w1a.dtype), d2.to(w2a.dtype)
        return grad_x, None, None, g1a, g2a, None, None, None, g1b, g2b, None


def _adapter(linear: nn.Module):
    """The LoKr module that took over ``linear.forward`` (LyCORIS-style wrapping), if it can take the quantised path."""
    mod = getattr(getattr(linear, "forward", None), "__self__", None)
    if mod is None or not hasattr(mod, "lokr_w1") or not hasattr(mod, "lokr_w2"):
        return None
    if not (lokr_patch._FP8_ACTIVE and getattr(mod, "_fp8_ok", False)):
        return None
    if getattr(mod, "_tlokr_enabled", False) or mod.bypass_mode or mod.wd or (mod.module_dropout and mod.training):
        return None
    org = mod.org_module[0]
    if org.bias is not None and org.bias.requires_grad:
        return None
    return mod


def _tlokr_adapter(linear: nn.Module):
    mod = getattr(getattr(linear, "forward", None), "__self__", None)
    if mod is None or not getattr(mod, "_tlokr_enabled", False):
        return None
    if mod.module_dropout and mod.training:
        return None
    return mod


def _patched_forward(self, x: torch.Tensor) -> torch.Tensor:
    act = self.activation
    exact_gelu = isinstance(act, nn.GELU) and getattr(act, "approximate", "none") == "none"
    t1, t2 = _tlokr_adapter(self.layer1), _tlokr_adapter(self.layer2)
    if t1 is not None and t2 is not None and exact_gelu:
        from . import tlokr
        p1 = tlokr.single_node_plan(t1, x) if tlokr.DELTA_PRECISION == "mxfp8" else None
        if p1 is not None:
            # layer 2 sees a tensor of layer 1's output shape; only shape, dtype and device enter its plan
            hidden = tlokr._ActSpec((*x.shape[:-1], t1.org_module[0].out_features), x.dtype, x.device)
            p2 = tlokr.single_node_plan(t2, hidden)
            if p2 is not None:
                return tlokr._MXTLoKrMLP.apply(x.contiguous(), *p1, *p2)
    m1, m2 = _adapter(self.layer1), _adapter(self.layer2)
    if (m1 is None or m2 is None or not exact_gelu or not x.is_cuda
            or (x.numel() // x.shape[-1]) % lokr_patch.MX_ALIGN):
        return _PATCHED[type(self)](self, x)
    o1, o2 = m1.org_module[0], m2.org_module[0]
    return LoKrMLPFused.apply(x, o1.weight, o1.bias, m1.lokr_w1, m1.lokr_w2, lokr_patch._alpha(m1) * m1.scale,
                              o2.weight, o2.bias, m2.lokr_w1, m2.lokr_w2, lokr_patch._alpha(m2) * m2.scale)


def install(mlp_cls: type | None = None) -> None:
    """Patch ``mlp_cls.forward`` (default: the stand-in ``anima_dit.GPT2FeedForward``). Idempotent."""
    if mlp_cls is None:
        from .anima_dit import GPT2FeedForward as mlp_cls
    if mlp_cls in _PATCHED:
        return
    _PATCHED[mlp_cls] = mlp_cls.forward
    mlp_cls.forward = _patched_forward


def uninstall(mlp_cls: type | None = None) -> None:
    if mlp_cls is None:
        from .anima_dit import GPT2FeedForward as mlp_cls
    orig = _PATCHED.pop(mlp_cls, None)
    if orig is not None:
        mlp_cls.forward = orig
