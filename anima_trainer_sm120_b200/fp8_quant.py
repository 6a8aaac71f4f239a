"""Quantised linears with the call surface of anima-trainer's ``fp8_quant.py``, on the
sm_100a MXFP8 kernels (no Transformer Engine, no cuBLASLt).

Mirrored interface (anima-trainer ``src/anima_trainer/fp8_quant.py``):
``MXFP8FrozenLinear`` (:118) / ``mxfp8_frozen_linear`` (:180), ``MXFP8LoKrLinear`` (:190) /
``mxfp8_lokr_linear`` (:267), ``FP8LoKrLinear`` (:460) / ``fp8_lokr_linear`` (:514),
``FP8FrozenLinear`` (:519) / ``fp8_frozen_linear`` (:573), ``is_quantized`` (:276),
``quantize_frozen_linears`` (:313), ``collect_lokr_wrapped_linears`` (:408),
``quantize_tlokr_base_weights`` (:583).

What differs from the reference, by design of the B200 path:
* every GEMM — forward, dgrad AND wgrad — runs in MXFP8 on tcgen05. The reference keeps the
  MXFP8 backward in bf16 because cuBLAS lacks those layouts on sm_120 (:196-205) and uses TE
  block-FP8 for its production ``fp8`` mode; here ``FP8LoKrLinear`` is the same three-GEMM
  contract in MXFP8.
* a pre-quantised weight is a :class:`QuantWeight` (row-wise operand for forward, column-wise
  operand for dgrad, both made from one read of W) instead of a TE tensor object.
* :class:`LoKrLinearFused` goes further than the reference API: it takes W, w1, w2 directly,
  never materialises kron(w1, w2) in HBM, and returns the adapter gradients from the wgrad.
"""
from __future__ import annotations

import contextlib
import threading
import types
import weakref
from typing import Iterable, NamedTuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import ops
from ._lib import SCALES_TILED

BF16 = torch.bfloat16
MXFP8_BLOCK = 32


class QuantWeight(NamedTuple):
    """MXFP8 forms of a weight ``W [N, K]``: ``row`` quantised along K (forward operand),
    ``col`` quantised along N and stored ``[K, N]`` (dgrad operand)."""

    row: ops.MXOperand
    col: ops.MXOperand | None


def quantize_weight(W: torch.Tensor, *, with_dgrad: bool = True) -> QuantWeight:
    W = W.detach()
    if W.dtype != BF16:
        W = W.to(BF16)
    row, col = ops.mx_quantize(W.contiguous(), rowwise=True, colwise=with_dgrad, layout=SCALES_TILED)
    return QuantWeight(row, col)


def _flat2d(x: torch.Tensor) -> torch.Tensor:
    x2 = x.reshape(-1, x.shape[-1])
    return x2 if x2.dtype == BF16 else x2.to(BF16)


# Activation quantisation shared between consumers of one tensor (q / k / v projections read the same
# AdaLN output; the reference measured this sharing at 5.339 -> 5.085 ms per block,
# docs/claude/sm120-optimization-audit-2026-08.md:116-119), and between a producer that already made the
# operand (the AdaLN forward kernels can emit the row-wise codes of their output) and its consumers.
# An entry is keyed on the tensor whose storage holds the values (the base of a view; weak reference, so a
# freed tensor can never alias a new one at the same address), the extent viewed (address, element count,
# row length) and the in-place version counter: a contiguous reshape of the producer's output still hits.
# The two most recent tensors are kept.
class _MemoEntry:
    __slots__ = ("base", "addr", "numel", "k", "version", "row", "col")

    def __init__(self, x: torch.Tensor, row: ops.MXOperand, col: ops.MXOperand | None):
        self.base = weakref.ref(_storage_owner(x))
        self.addr, self.numel, self.k, self.version = x.data_ptr(), x.numel(), x.shape[-1], x._version
        self.row, self.col = row, col

    def holds(self, x: torch.Tensor) -> bool:
        return (self.base() is _storage_owner(x) and self.addr == x.data_ptr() and self.numel == x.numel()
                and self.k == x.shape[-1] and self.version == x._version)


def _storage_owner(x: torch.Tensor) -> torch.Tensor:
    # only a contiguous bf16 view reads its base's bytes in the order the operand was made from
    if x._base is not None and x.is_contiguous() and x.dtype == BF16:
        return x._base
    return x


_ACT_MEMO: list[_MemoEntry] = []
_ACT_MEMO_SLOTS = 2
act_memo_stats = {"hits": 0, "misses": 0, "adopted": 0}


def clear_activation_memo() -> None:
    _ACT_MEMO.clear()


def _memo_insert(entry: _MemoEntry) -> None:
    _ACT_MEMO[:] = [e for e in _ACT_MEMO if e.base() is not None and e.base() is not entry.base()][:_ACT_MEMO_SLOTS - 1]
    _ACT_MEMO.insert(0, entry)


def adopt_row_operand(x: torch.Tensor, row: ops.MXOperand) -> None:
    """Register ``row`` as the row-wise MXFP8 operand of the contiguous bf16 tensor ``x`` (made by x's producer),
    so the linears that consume x, or a contiguous reshape of it, skip their own quantiser launch."""
    if x.dtype != BF16 or not x.is_contiguous() or row.codes.shape[1] != x.shape[-1]:
        raise ValueError("adopt_row_operand: x must be contiguous bfloat16 with the operand's row length")
    act_memo_stats["adopted"] += 1
    _memo_insert(_MemoEntry(x, row, None))


def quantize_activation(x: torch.Tensor, *, colwise: bool) -> tuple[ops.MXOperand, ops.MXOperand | None]:
    """Row-wise (and, if asked, column-wise) MXFP8 operands of ``x`` flattened to 2-D, memoised per tensor."""
    for i, e in enumerate(_ACT_MEMO):
        if e.holds(x):
            if i:
                _ACT_MEMO.insert(0, _ACT_MEMO.pop(i))
            act_memo_stats["hits"] += 1
            if colwise and e.col is None:     # the row-wise form is there already: add the other one
                e.col = ops.mx_quantize(_flat2d(x), rowwise=False, colwise=True)[1]
            return e.row, (e.col if colwise else None)
    act_memo_stats["misses"] += 1
    row, col = ops.mx_quantize(_flat2d(x), rowwise=True, colwise=colwise)
    _memo_insert(_MemoEntry(x, row, col))
    return row, col


# Activation checkpointing (non-reentrant) runs every block twice: a first pass whose saved tensors
# are discarded, and a recomputation just before the block's backward. Inside ``first_pass()`` the
# quantised linears therefore skip the operands that only backward reads (column-wise forms) and
# hand ``save_for_backward`` uninitialised buffers of the same shapes, which the checkpoint drops.
_pass = threading.local()


@contextlib.contextmanager
def first_pass():
    """Mark a forward whose saved tensors will be thrown away and recomputed (a checkpointed block)."""
    prev = getattr(_pass, "first", False)
    _pass.first = True
    try:
        yield
    finally:
        _pass.first = prev


def in_first_pass() -> bool:
    return getattr(_pass, "first", False)


def _placeholder(rows: int, k: int, device) -> ops.MXOperand:
    """An operand-shaped pair of uninitialised buffers (no kernel runs)."""
    return ops.MXOperand(torch.empty((rows, k), dtype=torch.uint8, device=device),
                         torch.empty(ops.scales_bytes(rows, k, SCALES_TILED), dtype=torch.uint8, device=device),
                         SCALES_TILED)


def _pack(op: ops.MXOperand | None) -> tuple:
    return (None, None) if op is None else (op.codes, op.scales)


def _unpack(codes, scales) -> ops.MXOperand | None:
    return None if codes is None else ops.MXOperand(codes, scales, SCALES_TILED)


def _bias_bf16(bias):
    return None if bias is None else bias.detach().to(BF16).contiguous()


class MXFP8FrozenLinear(torch.autograd.Function):
    """``y = x @ W.T (+ bias)`` for a frozen, pre-quantised W (reference signature
    ``apply(x, W_mx, W_bf16, bias)``). Forward: quantise x, MXFP8 GEMM. Backward: MXFP8 dgrad
    against the column-wise operand when ``W_mx`` carries one, else the reference's bf16
    ``grad_y @ W_bf16`` (:171)."""

    @staticmethod
    def forward(ctx, x, W_mx: QuantWeight, W_bf16, bias=None):
        x_row, _ = quantize_activation(x, colwise=False)
        ctx.W_mx, ctx.W_bf16, ctx.has_bias = W_mx, W_bf16, bias is not None
        n_out = W_bf16.shape[0]
        if x.dtype == BF16:
            # allocated in its final shape (not a view of a 2-D result), so a following op may update it in place
            y = torch.empty(*x.shape[:-1], n_out, dtype=BF16, device=x.device)
            ops.mx_gemm(x_row, W_mx.row, bias=_bias_bf16(bias), out=y.view(-1, n_out))
            return y
        y = ops.mx_gemm(x_row, W_mx.row, bias=_bias_bf16(bias))
        return y.reshape(*x.shape[:-1], n_out).to(x.dtype)

    @staticmethod
    def backward(ctx, grad_y):
        gy2 = _flat2d(grad_y)
        if ctx.W_mx.col is not None:
            g_row, _ = ops.mx_quantize(gy2, rowwise=True)
            gx2 = ops.mx_gemm(g_row, ctx.W_mx.col)
        else:
            gx2 = gy2 @ ctx.W_bf16.to(BF16)
        grad_x = gx2.reshape(*grad_y.shape[:-1], ctx.W_bf16.shape[1]).to(grad_y.dtype)
        grad_bias = grad_y.reshape(-1, grad_y.shape[-1]).sum(dim=0) if ctx.has_bias else None
        return grad_x, None, None, grad_bias


def mxfp8_frozen_linear(x, W_mx, W_bf16, bias=None):
    return MXFP8FrozenLinear.apply(x, W_mx, W_bf16, bias)


# T-LoKr's frozen base projection has the same contract (reference :519-580).
FP8FrozenLinear = MXFP8FrozenLinear


def fp8_frozen_linear(x, weight_q, weight_bf16, bias):
    return MXFP8FrozenLinear.apply(x, weight_q, weight_bf16, bias)


class MXFP8LoKrLinear(torch.autograd.Function):
    """``y = x @ merged_W.T (+ bias)`` with merged_W quantised just in time (reference
    signature ``apply(x, merged_W, bias)``, :224-264 / :480-511): forward, dgrad and wgrad are
    MXFP8 GEMMs; x and merged_W are each read once to produce both of their operand forms."""

    @staticmethod
    def forward(ctx, x, merged_W, bias=None):
        first = in_first_pass()
        need_w = ctx.needs_input_grad[1]
        x_row, x_col = quantize_activation(x, colwise=need_w and not first)
        w_row, w_col = ops.mx_quantize(merged_W.detach().to(BF16).contiguous(), rowwise=True, colwise=not first)
        y = ops.mx_gemm(x_row, w_row, bias=_bias_bf16(bias))
        if first:
            n_out, k_in = merged_W.shape
            w_col = _placeholder(k_in, n_out, x.device)
            x_col = _placeholder(k_in, x_row.codes.shape[0], x.device) if need_w else None
        ctx.save_for_backward(*_pack(x_col), *_pack(w_col))
        ctx.has_bias, ctx.w_dtype, ctx.in_features = bias is not None, merged_W.dtype, merged_W.shape[1]
        return y.reshape(*x.shape[:-1], merged_W.shape[0]).to(x.dtype)

    @staticmethod
    def backward(ctx, grad_y):
        saved = ctx.saved_tensors
        x_col, w_col = _unpack(*saved[0:2]), _unpack(*saved[2:4])
        gy2 = _flat2d(grad_y)
        g_row, g_col = ops.mx_quantize(gy2, rowwise=True, colwise=x_col is not None)
        grad_x = ops.mx_gemm(g_row, w_col).reshape(*grad_y.shape[:-1], ctx.in_features).to(grad_y.dtype)
        grad_w = None
        if x_col is not None:
            grad_w = ops.mx_gemm(g_col, x_col).to(ctx.w_dtype)          # gy^T @ x
        grad_bias = grad_y.reshape(-1, grad_y.shape[-1]).sum(dim=0) if ctx.has_bias else None
        return grad_x, grad_w, grad_bias


def mxfp8_lokr_linear(x, merged_W, bias=None):
    return MXFP8LoKrLinear.apply(x, merged_W, bias)


FP8LoKrLinear = MXFP8LoKrLinear


def fp8_lokr_linear(x, merged_W, bias):
    return MXFP8LoKrLinear.apply(x, merged_W, bias)


class LoKrLinearFused(torch.autograd.Function):
    """``y = x @ (W + alpha * kron(w1, w2)).T (+ bias)`` without ever writing the merged weight
    or its gradient's Kronecker expansion to HBM as bf16 tensors of their own:

    forward   one kernel builds merged = W + alpha*kron(w1, w2) and emits its row- and
              column-wise MXFP8 operands; x is quantised (both forms) from one read; MXFP8 GEMM.
    backward  grad_y quantised (both forms) from one read; MXFP8 dgrad; MXFP8 wgrad with fp32
              output; one pass over dW gives dw1 and dw2 (the adjoint of torch.kron that the
              reference obtains through autograd, lokr_patch.py:19-21).
    """

    @staticmethod
    def forward(ctx, x, W, bias, w1, w2, alpha: float):
        first = in_first_pass()
        train = ctx.needs_input_grad[3] or ctx.needs_input_grad[4]
        x_row, x_col = quantize_activation(x, colwise=train and not first)
        _, w_row, w_col = ops.lokr_merge_quantize(W.detach(), w1.detach(), w2.detach(), alpha, want_merged=False,
                                                  rowwise=True, colwise=not first)
        y = ops.mx_gemm(x_row, w_row, bias=_bias_bf16(bias))
        if first:
            n_out, k_in = W.shape
            w_col = _placeholder(k_in, n_out, x.device)
            x_col = _placeholder(k_in, x_row.codes.shape[0], x.device) if train else None
        ctx.save_for_backward(w1, w2, *_pack(x_col), *_pack(w_col))
        ctx.alpha, ctx.has_bias, ctx.in_features = float(alpha), bias is not None, W.shape[1]
        return y.reshape(*x.shape[:-1], W.shape[0]).to(x.dtype)

    @staticmethod
    def backward(ctx, grad_y):
        saved = ctx.saved_tensors
        w1, w2 = saved[0:2]
        x_col, w_col = _unpack(*saved[2:4]), _unpack(*saved[4:6])
        gy2 = _flat2d(grad_y)
        g_row, g_col = ops.mx_quantize(gy2, rowwise=True, colwise=x_col is not None)
        grad_x = ops.mx_gemm(g_row, w_col).reshape(*grad_y.shape[:-1], ctx.in_features).to(grad_y.dtype)
        g_w1 = g_w2 = None
        if x_col is not None:
            dw = ops.mx_gemm(g_col, x_col, out_dtype=torch.float32)
            d1, d2 = ops.lokr_kron_backward(dw, w1.detach(), w2.detach(), ctx.alpha)
            g_w1, g_w2 = d1.to(w1.dtype), d2.to(w2.dtype)
        grad_bias = grad_y.reshape(-1, grad_y.shape[-1]).sum(dim=0) if ctx.has_bias else None
        return grad_x, None, grad_bias, g_w1, g_w2, None


def lokr_linear_fused(x, W, bias, w1, w2, alpha: float = 1.0):
    return LoKrLinearFused.apply(x, W, bias, w1, w2, alpha)


# ------------------------------------------------------------------------------ module walkers
def is_quantized(mod: nn.Module) -> bool:
    return getattr(mod, "_mxfp8_W", None) is not None


def _mxfp8_linear_forward(self: nn.Linear, x: torch.Tensor) -> torch.Tensor:
    """Forward bound onto a pre-quantised frozen ``nn.Linear`` (reference :284-310). A leading
    size that is not a multiple of 32 takes the bf16 ``F.linear`` path, as in the reference."""
    W_mx = getattr(self, "_mxfp8_W", None)
    W_bf16 = getattr(self, "_mxfp8_W_bf16", None)
    if W_mx is None or W_bf16 is None:
        return F.linear(x, self.weight, self.bias)
    if (x.numel() // x.shape[-1]) % MXFP8_BLOCK != 0:
        return F.linear(x, W_bf16, self.bias)
    return MXFP8FrozenLinear.apply(x, W_mx, W_bf16, self.bias)


def quantize_frozen_linears(
    dit: nn.Module,
    skip: Iterable[nn.Module] = (),
    min_size: int = 256 * 256,
    skip_name_substrings: tuple[str, ...] = ("adaln_modulation", "t_embedder", "FinalLayer"),
) -> int:
    """Pre-quantise every frozen ``nn.Linear`` of ``dit`` and rebind its forward (reference
    :313-405, same skip rules: explicit ``skip`` set, name substrings, trainable weights, fewer
    than ``min_size`` elements, a dimension not divisible by 32). The MXFP8 copies are plain
    attributes, never buffers, so they stay out of ``state_dict``. Idempotent; returns the count."""
    skip_ids = {id(m) for m in skip}
    for name, mod in dit.named_modules():
        if isinstance(mod, nn.Linear) and any(s in name for s in skip_name_substrings):
            skip_ids.add(id(mod))
    count = 0
    for mod in dit.modules():
        if not isinstance(mod, nn.Linear) or id(mod) in skip_ids:
            continue
        if mod.weight.requires_grad or is_quantized(mod):
            continue
        out_dim, in_dim = mod.weight.shape
        if out_dim * in_dim < min_size or out_dim % MXFP8_BLOCK or in_dim % MXFP8_BLOCK:
            continue
        W = mod.weight.detach().contiguous()
        mod._mxfp8_W = quantize_weight(W)
        mod._mxfp8_W_bf16 = W
        mod.forward = types.MethodType(_mxfp8_linear_forward, mod)
        count += 1
    return count


def collect_lokr_wrapped_linears(network: nn.Module) -> list[nn.Linear]:
    """The ``nn.Linear`` instances wrapped by LoKr modules of ``network`` (reference :408-421):
    any module exposing ``org_module[0]`` and ``lokr_w1``."""
    wrapped = []
    for mod in network.modules():
        org = getattr(mod, "org_module", None)
        if org is not None and hasattr(mod, "lokr_w1") and isinstance(org[0], nn.Linear):
            wrapped.append(org[0])
    return wrapped


def quantize_tlokr_base_weights(network: nn.Module) -> int:
    """Pre-quantise the frozen base Linear of every T-LoKr module once (reference :583-613).
    MXFP8 needs both dimensions divisible by 32; a mismatch raises, as the reference does for
    its 128-alignment."""
    count = 0
    for module in network.modules():
        if not getattr(module, "_tlokr_enabled", False) or not hasattr(module, "org_module"):
            continue
        if getattr(module, "_tlokr_fp8_base_weight", None) is not None:
            continue
        inner = module.org_module[0]
        if not isinstance(inner, nn.Linear):
            raise TypeError(f"{getattr(module, 'lora_name', module)}: T-LoKr base must be nn.Linear")
        out_dim, in_dim = inner.weight.shape
        if out_dim % MXFP8_BLOCK or in_dim % MXFP8_BLOCK:
            raise ValueError(f"{getattr(module, 'lora_name', module)}: base shape "
                             f"{tuple(inner.weight.shape)} is not 32-aligned")
        module._tlokr_fp8_base_weight = quantize_weight(inner.weight)
        count += 1
    return count
