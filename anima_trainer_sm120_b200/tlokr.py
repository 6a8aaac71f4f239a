"""Timestep-aware LoKr (T-LoKr) with the call surface of anima-trainer's ``tlokr.py``.

``W2`` of a full-matrix LoKr adapter is factored as ``A @ B`` (rank r) and a per-sample prefix
of that rank is active: ``active(t) = floor((r - r_min) * (1 - t) + r_min)`` (reference
``active_rank_for_timestep`` :40-57, mask :84-92). The adapter output for a linear input is
evaluated structurally (reference :472-492), never forming ``kron(W1, A @ B)``:

    grouped = x.view(B, L*, uq, vq);  hidden = grouped @ B.T;  mixed = W1 @ (hidden * mask)
    out = mixed @ A.T  ->  (B, L*, up * vp)

Mirrored interface: ``active_rank_for_timestep``, ``set_timestep`` / ``clear_timestep`` (:110-130),
``install_root_timestep_hooks`` (:270-292), ``convert_network`` (:330-448), ``_StructuredLoKr``
(:451-540), ``_FP8StructuredLoKr`` (:543-676, here MXFP8), ``forward`` (:738-759).

Kernels: the 8x8 mix, its transpose and its fp32 weight gradient run in ``csrc/tlokr_mix.cu``;
in the quantised variant the factor GEMMs (2 forward, 2 recomputed + 4 in backward) run as
MXFP8 tcgen05 GEMMs with the quantiser producing both operand forms per tensor. The bf16
variant uses ``torch.matmul`` for the factor GEMMs (a library GEMM, as in the reference).
"""
from __future__ import annotations

import math
import os
from contextvars import ContextVar
from dataclasses import dataclass, field
from types import MethodType

from typing import NamedTuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import ops
from .tlokr_kernels import rank_mix, rank_mix_wgrad

_FORMAT_VERSION = 1
BF16 = torch.bfloat16


def active_rank_for_timestep(timestep: float, *, max_rank: int, min_rank: int) -> int:
    """Prefix rank for a scalar flow timestep (t = 1 is the noisiest point)."""
    if max_rank <= 0:
        raise ValueError(f"max_rank must be positive; got {max_rank}")
    if not 1 <= min_rank <= max_rank:
        raise ValueError(f"min_rank must be in [1, {max_rank}]; got {min_rank}")
    t = min(1.0, max(0.0, float(timestep)))
    return max(min_rank, min(max_rank, math.floor((max_rank - min_rank) * (1.0 - t) + min_rank)))


@dataclass
class _TimestepState:
    timesteps: torch.Tensor
    uniform_timestep: float | None = None   # known single timestep: factors are sliced, no mask
    masks: dict = field(default_factory=dict)

    def mask(self, *, max_rank: int, min_rank: int, dtype: torch.dtype, device: torch.device) -> torch.Tensor:
        """[B, max_rank] 0/1 prefix mask; built once per forward and shared by all modules."""
        key = (max_rank, min_rank, dtype, device)
        hit = self.masks.get(key)
        if hit is None:
            t = self.timesteps.detach().to(device=device, dtype=torch.float32).reshape(-1)
            active = torch.floor((max_rank - min_rank) * (1.0 - t.clamp(0.0, 1.0)) + min_rank).to(torch.int64)
            active.clamp_(min=min_rank, max=max_rank)
            hit = (torch.arange(max_rank, device=device).unsqueeze(0) < active.unsqueeze(1)).to(dtype)
            self.masks[key] = hit
        return hit


_STATE: ContextVar[_TimestepState | None] = ContextVar("anima_b200_tlokr_state", default=None)


def set_timestep(timesteps: torch.Tensor, *, uniform_timestep: float | None = None) -> None:
    """Set the timestep context for every T-LoKr module; it stays live through backward because
    activation checkpointing re-runs adapter forwards there. Pair with :func:`clear_timestep`."""
    if not torch.is_tensor(timesteps):
        raise TypeError("T-LoKr timesteps must be a torch.Tensor")
    _STATE.set(_TimestepState(timesteps=timesteps, uniform_timestep=uniform_timestep))


def clear_timestep() -> None:
    _STATE.set(None)


def _current_state() -> _TimestepState:
    state = _STATE.get()
    if state is None:
        raise RuntimeError("T-LoKr forward has no timestep context; call "
                           "anima_trainer_sm120_b200.tlokr.set_timestep() around the DiT forward")
    return state


def install_root_timestep_hooks(dit: nn.Module) -> None:
    """Derive a context from the root forward's ``timesteps`` argument when none was set explicitly,
    restore the previous one afterwards, and keep it alive for checkpoint recomputation: each
    block's ``_forward`` is wrapped so the callable the checkpoint retains re-enters the state."""
    if getattr(dit, "_tlokr_timestep_hooks_installed", False):
        return

    def pre(_m, args, kwargs):
        if _STATE.get() is not None:
            dit._tlokr_tokens.append(None)
            return
        t = next((kwargs[k] for k in ("timesteps", "timesteps_B_T", "timestep") if kwargs.get(k) is not None), None)
        if t is None and len(args) >= 2:
            t = args[1]
        if not torch.is_tensor(t):
            raise RuntimeError("T-LoKr could not derive a tensor timestep from the DiT forward arguments")
        dit._tlokr_tokens.append(_STATE.set(_TimestepState(timesteps=t)))

    def post(_m, _args, _kwargs, _out):
        token = dit._tlokr_tokens.pop() if dit._tlokr_tokens else None
        if token is not None:
            _STATE.reset(token)

    dit._tlokr_tokens = []
    dit.register_forward_pre_hook(pre, with_kwargs=True)
    dit.register_forward_hook(post, with_kwargs=True, always_call=True)
    for blk in dit.modules():
        if hasattr(blk, "_forward") and hasattr(blk, "gradient_checkpointing") and "_forward" not in blk.__dict__:

            def contextual(self_blk, *a, **kw):
                # the class attribute is looked up at call time so that a later adaln_patch.install() is honoured
                inner = type(self_blk)._forward
                captured = getattr(self_blk, "_tlokr_captured_state", None)
                if _STATE.get() is not None or captured is None:
                    self_blk._tlokr_captured_state = _STATE.get()
                    return inner(self_blk, *a, **kw)
                token = _STATE.set(captured)        # recomputation during backward, on autograd's thread
                try:
                    return inner(self_blk, *a, **kw)
                finally:
                    _STATE.reset(token)

            object.__setattr__(blk, "_forward", MethodType(contextual, blk))
    dit._tlokr_timestep_hooks_installed = True


def convert_network(network: nn.Module, *, rank: int, min_rank_ratio: float) -> int:
    """Convert freshly created full-matrix LoKr adapters in place: ``lokr_w2`` becomes the pair
    ``lokr_w2_a`` (kaiming-uniform) / ``lokr_w2_b`` (zeros), so the adapted model starts at the base
    model exactly. Returns the number of converted modules."""
    from .lokr import LokrModule

    if rank <= 0:
        raise ValueError(f"T-LoKr rank must be positive; got {rank}")
    if not 0.0 < min_rank_ratio <= 1.0:
        raise ValueError(f"T-LoKr min_rank_ratio must be in (0, 1]; got {min_rank_ratio}")
    min_rank = max(1, min(rank, math.ceil(rank * min_rank_ratio)))
    pending = list(getattr(network, "unet_loras", ()))
    converted = 0
    for module in (pending if pending else list(network.modules())):
        if not isinstance(module, LokrModule):
            continue
        if module.module_type != "linear":
            raise TypeError(f"T-LoKr supports Linear targets only; {module.lora_name} wraps {module.module_type}")
        if not module.use_w1 or not module.use_w2:
            raise ValueError(f"{module.lora_name}: T-LoKr conversion requires full_matrix=true")
        if module.wd or module.bypass_mode:
            raise ValueError(f"{module.lora_name}: T-LoKr does not support weight decomposition or bypass mode")
        if module.rank_dropout or module.dropout:
            raise ValueError(f"{module.lora_name}: T-LoKr does not support rank/dropout")
        old = module.lokr_w2
        vp, vq = old.shape
        if rank > min(vp, vq):
            raise ValueError(f"T-LoKr rank {rank} exceeds the large Kronecker factor {tuple(old.shape)} "
                             f"in {module.lora_name}")
        del module.lokr_w2
        a = nn.Parameter(torch.empty(vp, rank, device=old.device, dtype=old.dtype))
        b = nn.Parameter(torch.zeros(rank, vq, device=old.device, dtype=old.dtype))
        nn.init.kaiming_uniform_(a, a=math.sqrt(5))
        module.register_parameter("lokr_w2_a", a)
        module.register_parameter("lokr_w2_b", b)
        module.use_w2 = False
        module.full_matrix = False
        module.lora_dim = rank
        module._tlokr_enabled, module._tlokr_rank, module._tlokr_min_rank = True, rank, min_rank
        scalar = module.scalar.item() if torch.is_tensor(module.scalar) else module.scalar
        module._tlokr_alpha = float(module.scale) * float(scalar) * float(module.multiplier)
        module.register_buffer("tlokr_schedule", torch.tensor([_FORMAT_VERSION, rank, min_rank], dtype=torch.int32))
        converted += 1
    if converted == 0:
        raise RuntimeError("T-LoKr conversion found no LoKr modules")
    network._tlokr_enabled, network._tlokr_rank, network._tlokr_min_rank = True, rank, min_rank
    return converted


def _grouped(x: torch.Tensor, uq: int) -> torch.Tensor:
    return x.reshape(x.shape[0], -1, uq, x.shape[-1] // uq)


class _StructuredLoKr(torch.autograd.Function):
    """bf16 structured delta with manual backward; saves only x and the small factors and
    recomputes the rank-space intermediates per module in backward (reference :451-540)."""

    @staticmethod
    def forward(ctx, x, w1, w2_a, w2_b, mask):
        dt = x.dtype
        c, a, b = w1.to(dt), w2_a.to(dt), w2_b.to(dt)
        hidden = torch.matmul(_grouped(x, c.shape[1]), b.t())
        out = torch.matmul(rank_mix(hidden, c, mask), a.t())
        ctx.save_for_backward(x, w1, w2_a, w2_b, *(() if mask is None else (mask,)))
        ctx.has_mask = mask is not None
        return out.reshape(*x.shape[:-1], -1)

    @staticmethod
    def backward(ctx, grad_output):
        saved = ctx.saved_tensors        # read once: activation checkpointing unpacks on access
        x, w1, w2_a, w2_b = saved[:4]
        mask = saved[4] if ctx.has_mask else None
        dt = x.dtype
        c, a, b = w1.to(dt), w2_a.to(dt), w2_b.to(dt)
        up, uq = c.shape
        vp = a.shape[0]
        grouped = _grouped(x, uq)
        hidden = torch.matmul(grouped, b.t())
        mixed = rank_mix(hidden, c, mask)
        g_blocks = grad_output.to(dt).reshape(x.shape[0], -1, up, vp)
        g_a = g_blocks.reshape(-1, vp).t() @ mixed.reshape(-1, mixed.shape[-1])
        g_mixed = torch.matmul(g_blocks, a)
        g_c = rank_mix_wgrad(g_mixed, hidden, mask)
        g_hidden = rank_mix(g_mixed, c, mask, transpose=True)
        g_b = g_hidden.reshape(-1, g_hidden.shape[-1]).t() @ grouped.reshape(-1, grouped.shape[-1])
        g_x = torch.matmul(g_hidden, b).reshape(x.shape)
        return g_x.to(x.dtype), g_c.to(w1.dtype), g_a.to(w2_a.dtype), g_b.to(w2_b.dtype), None


def _capturing(p: torch.Tensor) -> bool:
    """Inside a CUDA-graph capture the factor conversions must be recorded with the rest of the step: a form kept
    from an earlier call would be baked into the graph and every replay would multiply by the factors of the step
    that was captured."""
    return p.is_cuda and torch.cuda.is_current_stream_capturing()


def _factor_forms(p: torch.Tensor, *, quantise: bool):
    """bf16 copy (``quantise=False``) or both MXFP8 operands (``quantise=True``) of a small adapter factor.

    A checkpointed step reads every factor three times with the same values (first pass, recomputation,
    backward); for a leaf parameter the result is kept on the parameter object, keyed on its in-place version
    counter and storage address (an optimizer step or a reassigned ``.data`` invalidates it), which removes two
    thirds of these tiny launches. Sliced or computed factors are converted on every call."""
    cacheable = p.is_leaf and isinstance(p, nn.Parameter) and not _capturing(p)
    slot = "_anima_mx_forms" if quantise else "_anima_bf16_form"
    key = (p._version, p.data_ptr())
    if cacheable:
        hit = getattr(p, slot, None)
        if hit is not None and hit[0] == key:
            return hit[1]
    with torch.no_grad():
        val = _q(p.detach(), col=True) if quantise else p.detach().to(BF16).contiguous()
    if cacheable:
        setattr(p, slot, (key, val))
    return val


def _scaled_row_form(p: torch.Tensor, alpha: float) -> ops.MXOperand:
    """Row-wise MXFP8 operand of ``alpha * p`` rounded to bf16 (the factor a folded delta multiplies by), kept on
    a leaf parameter like :func:`_factor_forms`."""
    cacheable = p.is_leaf and isinstance(p, nn.Parameter) and not _capturing(p)
    key = (p._version, p.data_ptr(), float(alpha))
    if cacheable:
        hit = getattr(p, "_anima_mx_scaled_row", None)
        if hit is not None and hit[0] == key:
            return hit[1]
    with torch.no_grad():
        val = ops.mx_quantize((p.detach().float() * float(alpha)).to(BF16).contiguous(), rowwise=True)[0]
    if cacheable:
        p._anima_mx_scaled_row = (key, val)
    return val


# Fold the structured delta into the base GEMMs as extra K-blocks (``ops.mx_gemm_delta``) where the shapes allow:
# the base projection and ``+ alpha * delta`` (forward), the base input gradient and ``+ grad_hidden @ B``
# (backward) are then one GEMM each, and the output is neither re-read nor rounded twice. False keeps the
# separate add-GEMMs (for comparison; ANIMA_TLOKR_FOLD_DELTA=0 sets it at import).
FOLD_DELTA = os.environ.get("ANIMA_TLOKR_FOLD_DELTA", "1") != "0"


# Compute hidden, the mix and the quantisation of the mixed tensor in one kernel in the forward chain
# (``ops.tlokr_hidden_mix_planes``); False runs the factor GEMM and the quantising mix as two kernels (same bits).
FUSE_HIDDEN_MIX = os.environ.get("ANIMA_TLOKR_FUSE_HIDDEN_MIX", "1") != "0"


def _can_fold(rows: int, n_cols: int, factor_dim: int, batch: int, rank: int) -> bool:
    return (FOLD_DELTA and factor_dim == 8 and ops.can_fold_delta(rows, n_cols) and rows % batch == 0
            and ops.can_mix_to_planes(batch, rows // batch, rank))


def _q(t2d: torch.Tensor, *, col: bool = False):
    return ops.mx_quantize(t2d.contiguous() if t2d.dtype == BF16 else t2d.to(BF16).contiguous(),
                           rowwise=True, colwise=col)


class _MXStructuredLoKr(torch.autograd.Function):
    """The same delta with every factor GEMM in MXFP8 on the tensor cores (the reference's
    ``_FP8StructuredLoKr`` uses TE block-FP8 for them); the 8x8 mix stays in bf16.

    With ``base`` given the result is ``base + alpha * delta``, formed in the epilogue of the last GEMM
    (the reference's separate ``torch.add(base, delta, alpha=)``, ``tlokr.py:757-759``)."""

    @staticmethod
    def forward(ctx, x, w1, w2_a, w2_b, mask, base=None, alpha: float = 1.0):
        c = w1.to(BF16)
        aq, aq_col = _q(w2_a.detach(), col=True)      # A [vp, r]: row form for out, column form for dgrad
        bq, bq_col = _q(w2_b.detach(), col=True)      # B [r, vq]
        grouped = _grouped(x, c.shape[1])
        g2 = grouped.reshape(-1, grouped.shape[-1])
        gq, _ = _q(g2)
        hidden = ops.mx_gemm(gq, bq).view(*grouped.shape[:-1], w2_b.shape[0])
        mixed = rank_mix(hidden, c, mask)
        mq, _ = _q(mixed.reshape(-1, mixed.shape[-1]))
        ctx.save_for_backward(x, w1, w2_a, w2_b, *(() if mask is None else (mask,)))
        ctx.has_mask, ctx.ops = mask is not None, (aq_col, bq, bq_col)
        ctx.has_base, ctx.alpha = base is not None, float(alpha) if base is not None else 1.0
        if base is None:
            return ops.mx_gemm(mq, aq).view(*x.shape[:-1], -1).to(x.dtype)
        # base (bf16, contiguous) is updated in place: base += alpha * delta, added by the GEMM's stores
        res = base.view(-1, w2_a.shape[0])
        ops.mx_gemm(mq, aq, residual=res, alpha=float(alpha), out=res)
        ctx.mark_dirty(base)
        return base

    @staticmethod
    def backward(ctx, grad_output):
        saved = ctx.saved_tensors        # read once: activation checkpointing unpacks on access
        x, w1, w2_a, w2_b = saved[:4]
        mask = saved[4] if ctx.has_mask else None
        aq_col, bq, bq_col = ctx.ops
        c = w1.to(BF16)
        up, uq = c.shape
        vp, rank = w2_a.shape
        grouped = _grouped(x, uq)
        g2 = grouped.reshape(-1, grouped.shape[-1])
        gq, gq_col = _q(g2, col=True)
        hidden = ops.mx_gemm(gq, bq).view(*grouped.shape[:-1], rank)
        mixed = rank_mix(hidden, c, mask)
        _, mq_col = _q(mixed.reshape(-1, rank), col=True)
        gb2 = grad_output.reshape(-1, vp)
        gbq, gbq_col = _q(gb2, col=True)
        g_a = ops.mx_gemm(gbq_col, mq_col, out_dtype=torch.float32, alpha=ctx.alpha)   # alpha * grad_blocks^T @ mixed [vp, r]
        g_mixed = ops.mx_gemm(gbq, aq_col, alpha=ctx.alpha).view(*mixed.shape)         # alpha * grad_blocks @ A       [.., r]
        g_c = rank_mix_wgrad(g_mixed, hidden, mask)
        g_hidden = rank_mix(g_mixed, c, mask, transpose=True)
        ghq, ghq_col = _q(g_hidden.reshape(-1, rank), col=True)
        g_b = ops.mx_gemm(ghq_col, gq_col, out_dtype=torch.float32)          # grad_hidden^T @ grouped [r, vq]
        g_x = ops.mx_gemm(ghq, bq_col).view(x.shape)                         # grad_hidden @ B
        return (g_x.to(x.dtype), g_c.to(w1.dtype), g_a.to(w2_a.dtype), g_b.to(w2_b.dtype), None,
                grad_output if ctx.has_base else None, None)


_FP8StructuredLoKr = _MXStructuredLoKr  # name used by anima-trainer


def _delta_plan(module, x: torch.Tensor, *, fp8: bool):
    """(autograd function, A, B, mask) of the structured delta for the current timestep context
    (the dispatch of reference :679-735)."""
    state = _current_state()
    rank, min_rank = module._tlokr_rank, module._tlokr_min_rank
    w1 = module.lokr_w1
    if x.shape[-1] % w1.shape[1]:
        raise RuntimeError(f"{module.lora_name}: input width {x.shape[-1]} is not divisible by the W1 "
                           f"input factor {w1.shape[1]}")
    if state.uniform_timestep is not None:
        # One known timestep for the whole batch: slice the factors to the active prefix, which drops the
        # mask and the inactive-rank work. The mix kernel wants the rank in multiples of 8 (the MXFP8 GEMMs in
        # multiples of 32); other prefixes keep the full factors and use an equivalent uniform mask.
        active = active_rank_for_timestep(state.uniform_timestep, max_rank=rank, min_rank=min_rank)
        if active % 8 == 0:
            fn = _MXStructuredLoKr if fp8 and active % 32 == 0 else _StructuredLoKr
            return fn, module.lokr_w2_a[:, :active], module.lokr_w2_b[:active], None
        key = ("uniform", rank, active, x.dtype, x.device, x.shape[0])
        mask = state.masks.get(key)
        if mask is None:
            mask = (torch.arange(rank, device=x.device) < active).to(x.dtype).expand(x.shape[0], rank).contiguous()
            state.masks[key] = mask
        return (_MXStructuredLoKr if fp8 else _StructuredLoKr), module.lokr_w2_a, module.lokr_w2_b, mask
    mask = state.mask(max_rank=rank, min_rank=min_rank, dtype=x.dtype, device=x.device)
    if x.shape[0] != mask.shape[0]:
        raise RuntimeError(f"{module.lora_name}: activation batch {x.shape[0]} does not match timestep "
                           f"batch {mask.shape[0]}")
    return (_MXStructuredLoKr if fp8 else _StructuredLoKr), module.lokr_w2_a, module.lokr_w2_b, mask


def _structured_delta(module, x: torch.Tensor, *, fp8: bool, base: torch.Tensor | None = None,
                      alpha: float = 1.0) -> torch.Tensor:
    """``x @ kron(W1, A @ B).T`` for the current timestep context; with ``base`` given,
    ``base + alpha * delta`` (fused into the last GEMM on the quantised path)."""
    fn, w2_a, w2_b, mask = _delta_plan(module, x, fp8=fp8)
    args = (x, module.lokr_w1, w2_a, w2_b, mask)
    if base is None:
        return fn.apply(*args)
    if fn is _MXStructuredLoKr and base.dtype == BF16 and base.is_contiguous() and base.requires_grad:
        return fn.apply(*args, base, alpha)
    return torch.add(base, fn.apply(*args), alpha=alpha)


def _mix_operands(hidden, c, mask, transpose: bool, *, row: bool, col: bool):
    """MXFP8 operands (row form, column form) of ``rank_mix(hidden, c, mask, transpose=...)`` viewed as
    ``[-1, rank]``. The mix kernel writes them itself where the shape allows, so the mixed tensor never exists in
    bf16; otherwise the mix is followed by a quantiser launch. Same bits either way."""
    batch, n, _, rank = hidden.shape
    # at [8, 4096, 8, 128] the kernel's row form beats mix + quantiser (38.4 against 28.7 + 18.9 us); its column
    # forms do not (46.6 against 28.7 + 16.9, 62.0 against 28.7 + 30.7), so those keep the two kernels
    if not col and ops.can_quantise_rank_mix(batch, n, rank):
        m = None if mask is None else mask.contiguous().to(BF16)
        r, cl, _ = ops.tlokr_rank_mix_quant(hidden.contiguous(), c.contiguous(), m, transpose, rowwise=row, colwise=col)
        return r, cl
    mixed = rank_mix(hidden, c, mask, transpose=transpose)
    return ops.mx_quantize(mixed.reshape(-1, rank), rowwise=row, colwise=col)


def _mx_linear_fwd(x_row, gq, lead_shape, W_mx, bias, w1, w2_a, w2_b, mask, alpha):
    """``y = x W^T + bias + alpha * delta(x)`` from the row-wise MXFP8 operand of x viewed as ``[rows, K]``
    (``x_row``) and as the grouped ``[rows * uq, K / uq]`` (``gq``): the same code bytes under two scale tilings.
    Returns (y, small factor operands kept for backward)."""
    from .fp8_quant import _bias_bf16
    c = _factor_forms(w1, quantise=False)
    uq = c.shape[1]
    vp, rank = w2_a.shape
    n_out = W_mx.row.rows
    aq, aq_col = _factor_forms(w2_a, quantise=True)      # A [vp, r]: row form for out, column form for dgrad
    bq, bq_col = _factor_forms(w2_b, quantise=True)      # B [r, vq]
    y = torch.empty(*lead_shape, n_out, dtype=BF16, device=x_row.codes.device)
    if _can_fold(x_row.rows, n_out, c.shape[0], lead_shape[0], rank) and n_out == c.shape[0] * vp and uq == 8:
        # Two kernels for the whole linear: (1) hidden = grouped . B^T, the 8x8 mix, the mask and the quantisation
        # of the mixed tensor, which leaves as eight e4m3 planes (hidden itself stays on the SM); (2) ONE GEMM in
        # which those planes times alpha * A enter as extra K-blocks of the base projection.
        m = None if mask is None else mask.contiguous().to(BF16)
        if FUSE_HIDDEN_MIX:
            planes, _ = ops.tlokr_hidden_mix_planes(gq, bq, c, m, lead_shape[0], False)
        else:
            hidden = ops.mx_gemm(gq, bq).view(lead_shape[0], -1, uq, rank)
            planes, _ = ops.tlokr_rank_mix_quant_planes(hidden, c, m, False)
        ops.mx_gemm_delta(x_row, W_mx.row, planes, _scaled_row_form(w2_a, alpha), bias=_bias_bf16(bias),
                          out=y.view(-1, n_out))
        return y, (aq_col, bq, bq_col)
    hidden = ops.mx_gemm(gq, bq).view(lead_shape[0], -1, uq, rank)
    ops.mx_gemm(x_row, W_mx.row, bias=_bias_bf16(bias), out=y.view(-1, n_out))
    mq, _ = _mix_operands(hidden, c, mask, False, row=True, col=False)
    res = y.view(-1, vp)
    ops.mx_gemm(mq, aq, residual=res, alpha=float(alpha), out=res)       # y += alpha * delta
    return y, (aq_col, bq, bq_col)


def _input_operands(quantise, rows: int, K: int, uq: int, keep: bool, device):
    """MXFP8 operands of a layer input for forward and backward. ``quantise(r, k, col)`` quantises the input viewed
    as ``[r, k]``. With ``keep`` (a pass whose saved tensors backward will read) the grouped view is quantised in both
    forms once, so that backward needs neither the bf16 input nor another pass over it; otherwise only the row form
    is made and uninitialised buffers of the same shapes stand in for what a checkpoint drops anyway.
    Returns (x_row [rows, K], gq [rows * uq, K / uq], gq_col [K / uq, rows * uq])."""
    from .fp8_quant import _placeholder
    if keep:
        gq, gq_col = quantise(rows * uq, K // uq, True)
        return ops.mx_regroup(gq, rows, K), gq, gq_col
    x_row, _ = quantise(rows, K, False)
    return x_row, ops.mx_regroup(x_row, rows * uq, K // uq), _placeholder(K // uq, rows * uq, device)


def _mx_linear_bwd(quant_grad, quant_grouped, lead_shape, K, W_mx, w1, w2_a, w2_b, mask, alpha, factor_ops):
    """Backward of :func:`_mx_linear_fwd`. ``quant_grad(rows, k)`` returns the (row, column) MXFP8 operands of the
    incoming gradient viewed as ``[rows, k]``, so a caller can fold an elementwise op (the derivative of the MLP
    activation) into that quantisation; ``quant_grouped(rows, k)`` returns the operands of the layer input in its
    grouped view (saved by the forward pass). Returns (grad_x bf16 [*lead, K], grad_w1, grad_A, grad_B)."""
    aq_col, bq, bq_col = factor_ops
    c = _factor_forms(w1, quantise=False)
    up, uq = c.shape
    vp, rank = w2_a.shape
    vq = K // uq
    rows = 1
    for d in lead_shape:
        rows *= d
    gbq, gbq_col = quant_grad(rows * up, vp)                                        # grad as [rows * up, vp]
    g_x = torch.empty(*lead_shape, K, dtype=BF16, device=gbq.codes.device)
    fold = _can_fold(rows, K, uq, lead_shape[0], rank) and K == uq * vq
    if not fold:
        ops.mx_gemm(ops.mx_regroup(gbq, rows, up * vp), W_mx.col, out=g_x.view(rows, K))   # base dgrad
    gq, gq_col = quant_grouped(rows * uq, vq)
    hidden = ops.mx_gemm(gq, bq).view(lead_shape[0], -1, uq, rank)
    _, mq_col = _mix_operands(hidden, c, mask, False, row=False, col=True)
    g_a = ops.mx_gemm(gbq_col, mq_col, out_dtype=torch.float32, alpha=alpha)        # alpha * grad^T @ mixed  [vp, r]
    g_mixed = ops.mx_gemm(gbq, aq_col, alpha=alpha).view(*hidden.shape)             # alpha * grad @ A        [.., r]
    g_c = rank_mix_wgrad(g_mixed, hidden, mask)
    if fold:
        # grad_hidden leaves as eight planes + its column form; base dgrad and + grad_hidden @ B are one GEMM
        gh_planes, ghq_col = ops.tlokr_rank_mix_quant_planes(
            g_mixed, c, None if mask is None else mask.contiguous().to(BF16), True, colwise=True)
        g_b = ops.mx_gemm(ghq_col, gq_col, out_dtype=torch.float32)                 # grad_hidden^T @ grouped [r, vq]
        ops.mx_gemm_delta(ops.mx_regroup(gbq, rows, up * vp), W_mx.col, gh_planes, bq_col, out=g_x.view(rows, K))
        return g_x, g_c.to(w1.dtype), g_a.to(w2_a.dtype), g_b.to(w2_b.dtype)
    ghq, ghq_col = _mix_operands(g_mixed, c, mask, True, row=True, col=True)        # of grad_hidden
    g_b = ops.mx_gemm(ghq_col, gq_col, out_dtype=torch.float32)                     # grad_hidden^T @ grouped [r, vq]
    res = g_x.view(-1, vq)
    ops.mx_gemm(ghq, bq_col, residual=res, out=res)                                 # g_x += grad_hidden @ B
    return g_x, g_c.to(w1.dtype), g_a.to(w2_a.dtype), g_b.to(w2_b.dtype)


def _bf16c(t: torch.Tensor) -> torch.Tensor:
    return t.contiguous() if t.dtype == BF16 else t.to(BF16).contiguous()


class _MXTLoKrLinear(torch.autograd.Function):
    """The whole quantised T-LoKr linear, ``x W^T + bias + alpha * delta(x)``, as ONE autograd node.

    The reference runs a frozen FP8 base projection (``fp8_frozen_linear``, ``tlokr.py:743``), the
    structured delta (``_FP8StructuredLoKr``, :543-676) and ``torch.add(base, delta, alpha=)`` (:757-759) as
    three nodes, each quantising its own inputs. As one node:

    * x is quantised row-wise ONCE: the base GEMM contracts it as [rows, K], the delta as the grouped view
      [rows * uq, K / uq]; the code bytes are the same, only the scales are re-tiled (``ops.mx_regroup``);
      likewise the incoming gradient serves the base dgrad and the delta chain from one quantisation;
    * ``+ alpha * delta`` and, in backward, ``+ grad_x(delta)`` are added by the stores of the last GEMM of
      each chain into the buffer the base GEMM wrote: no separate add kernels, no autograd sum.

    What is saved for backward are the MXFP8 operands of x in its grouped view (both forms, made by one pass
    over x in the forward that backward will use) and the small factors; the rank-space intermediates are
    recomputed in backward, as in the reference."""

    @staticmethod
    def forward(ctx, x, W_mx, bias, w1, w2_a, w2_b, mask, alpha: float):
        from .fp8_quant import _pack, in_first_pass, quantize_activation
        K, uq = x.shape[-1], w1.shape[1]
        rows = x.numel() // K
        train = any(ctx.needs_input_grad[i] for i in (0, 3, 4, 5))
        keep = train and not in_first_pass()

        def quantise(r, k, col):
            if not col and (r, k) == (rows, K):
                return quantize_activation(x, colwise=False)        # shared with other consumers of x
            return _q(x.reshape(r, k), col=col)

        x_row, gq, gq_col = _input_operands(quantise, rows, K, uq, keep, x.device)
        y, factor_ops = _mx_linear_fwd(x_row, gq, x.shape[:-1], W_mx, bias, w1, w2_a, w2_b, mask, alpha)
        ctx.save_for_backward(w1, w2_a, w2_b, *_pack(gq), *_pack(gq_col), *(() if mask is None else (mask,)))
        ctx.has_mask, ctx.ops, ctx.W_mx = mask is not None, factor_ops, W_mx
        ctx.alpha, ctx.bias_grad, ctx.x_shape = float(alpha), bias is not None and bias.requires_grad, x.shape
        return y

    @staticmethod
    def backward(ctx, grad_output):
        from .fp8_quant import _unpack
        saved = ctx.saved_tensors        # read once: activation checkpointing unpacks on access
        w1, w2_a, w2_b = saved[:3]
        gq, gq_col = _unpack(*saved[3:5]), _unpack(*saved[5:7])
        mask = saved[7] if ctx.has_mask else None
        gy = _bf16c(grad_output)
        g_x, g_c, g_a, g_b = _mx_linear_bwd(
            lambda r, k: _q(gy.view(r, k), col=True), lambda r, k: (gq, gq_col),
            ctx.x_shape[:-1], ctx.x_shape[-1], ctx.W_mx, w1, w2_a, w2_b, mask, ctx.alpha, ctx.ops)
        g_bias = gy.reshape(-1, gy.shape[-1]).sum(dim=0) if ctx.bias_grad else None
        return g_x, None, g_bias, g_c, g_a, g_b, None, None


class _MXTLoKrMLP(torch.autograd.Function):
    """``layer2(gelu(layer1(x)))`` with both layers quantised T-LoKr linears, as one node: the activation and
    its derivative are evaluated inside the quantiser (``ops.mx_quantize_gelu``), so neither ``gelu(h)`` nor
    ``grad * gelu'(h)`` is ever written as a bf16 tensor. Saves the pre-activation h, the grouped MXFP8 operands of
    both layer inputs and the factors."""

    @staticmethod
    def forward(ctx, x, W1, b1, w1_1, a_1, b_1, mask1, alpha1: float, W2, b2, w1_2, a_2, b_2, mask2, alpha2: float):
        from .fp8_quant import _pack, in_first_pass, quantize_activation
        K, lead = x.shape[-1], x.shape[:-1]
        rows = x.numel() // K
        train = any(ctx.needs_input_grad[i] for i in (0, 3, 4, 5, 10, 11, 12))
        keep = train and not in_first_pass()

        def quantise_x(r, k, col):
            if not col and (r, k) == (rows, K):
                return quantize_activation(x, colwise=False)
            return _q(x.reshape(r, k), col=col)

        x_row, gq1, gq1_col = _input_operands(quantise_x, rows, K, w1_1.shape[1], keep, x.device)
        h, ops1 = _mx_linear_fwd(x_row, gq1, lead, W1, b1, w1_1, a_1, b_1, mask1, alpha1)
        hid = h.shape[-1]
        act_row, gq2, gq2_col = _input_operands(
            lambda r, k, col: ops.mx_quantize_gelu(h.view(r, k), rowwise=True, colwise=col),
            rows, hid, w1_2.shape[1], keep, x.device)
        y, ops2 = _mx_linear_fwd(act_row, gq2, lead, W2, b2, w1_2, a_2, b_2, mask2, alpha2)
        masks = tuple(m for m in (mask1, mask2) if m is not None)
        ctx.save_for_backward(h, w1_1, a_1, b_1, w1_2, a_2, b_2, *_pack(gq1), *_pack(gq1_col), *_pack(gq2),
                              *_pack(gq2_col), *masks)
        ctx.has_masks = (mask1 is not None, mask2 is not None)
        ctx.ops, ctx.W = (ops1, ops2), (W1, W2)
        ctx.alphas, ctx.x_shape = (float(alpha1), float(alpha2)), x.shape
        return y

    @staticmethod
    def backward(ctx, grad_output):
        from .fp8_quant import _unpack
        saved = ctx.saved_tensors
        h, w1_1, a_1, b_1, w1_2, a_2, b_2 = saved[:7]
        gq1, gq1_col, gq2, gq2_col = (_unpack(*saved[i:i + 2]) for i in (7, 9, 11, 13))
        rest = list(saved[15:])
        mask1 = rest.pop(0) if ctx.has_masks[0] else None
        mask2 = rest.pop(0) if ctx.has_masks[1] else None
        gy = _bf16c(grad_output)
        lead = ctx.x_shape[:-1]
        # layer 2: its input gelu(h) was quantised straight from h by the forward pass
        g_act, g_c2, g_a2, g_b2 = _mx_linear_bwd(
            lambda r, k: _q(gy.view(r, k), col=True), lambda r, k: (gq2, gq2_col),
            lead, h.shape[-1], ctx.W[1], w1_2, a_2, b_2, mask2, ctx.alphas[1], ctx.ops[1])
        # layer 1: its incoming gradient is g_act * gelu'(h), formed inside the quantiser
        g_x, g_c1, g_a1, g_b1 = _mx_linear_bwd(
            lambda r, k: ops.mx_quantize_gelu(h.view(r, k), g_act.view(r, k), rowwise=True, colwise=True),
            lambda r, k: (gq1, gq1_col),
            lead, ctx.x_shape[-1], ctx.W[0], w1_1, a_1, b_1, mask1, ctx.alphas[0], ctx.ops[0])
        return (g_x, None, None, g_c1, g_a1, g_b1, None, None,
                None, None, g_c2, g_a2, g_b2, None, None)


class _ActSpec(NamedTuple):
    """Shape, dtype and device of an activation: all the dispatch looks at."""
    shape: tuple
    dtype: torch.dtype
    device: torch.device


def single_node_plan(module, x):
    """Arguments ``(W_mx, bias, w1, A, B, mask, alpha)`` of the one-node quantised T-LoKr linear for an input
    ``x`` (a tensor or an :class:`_ActSpec`), or None when the call has to take the general path (no
    pre-quantised base, rows not a multiple of 32, input not bf16 on CUDA, a factor other than 8 x 8, or an active
    rank the MXFP8 GEMMs cannot contract)."""
    base_q = getattr(module, "_tlokr_fp8_base_weight", None)
    rows = 1
    for d in x.shape[:-1]:
        rows *= d
    if (base_q is None or base_q.col is None or x.device.type != "cuda" or x.dtype != BF16
            or rows % 32 or tuple(module.lokr_w1.shape) != (8, 8)):
        return None
    fn, w2_a, w2_b, mask = _delta_plan(module, x, fp8=True)
    if fn is not _MXStructuredLoKr:
        return None
    return base_q, module.org_module[0].bias, module.lokr_w1, w2_a, w2_b, mask, module._tlokr_alpha


# Precision of the structured delta when the base projection is quantised: "mxfp8" (every factor GEMM on the
# MXFP8 tensor path, the reference's FP8 mode) or "bf16" (the HBM-bound factor chain stays in bf16 and skips its
# quantisation passes; the base projection stays MXFP8).
DELTA_PRECISION = "mxfp8"


def forward(module, x: torch.Tensor) -> torch.Tensor:
    """T-LoKr forward called by ``lokr_patch``: frozen base projection (quantised once when
    ``fp8_quant.quantize_tlokr_base_weights`` ran) plus ``alpha`` times the structured delta."""
    org = module.org_module[0]
    base_q = getattr(module, "_tlokr_fp8_base_weight", None)
    quantised = base_q is not None and x.is_cuda and (x.numel() // x.shape[-1]) % 32 == 0
    plan = single_node_plan(module, x) if DELTA_PRECISION == "mxfp8" else None
    if plan is not None:
        return _MXTLoKrLinear.apply(x.contiguous(), *plan)
    if quantised:
        from .fp8_quant import fp8_frozen_linear
        base = fp8_frozen_linear(x, base_q, org.weight, org.bias)
    else:
        base = F.linear(x, org.weight, org.bias)
    return _structured_delta(module, x, fp8=quantised and DELTA_PRECISION == "mxfp8", base=base,
                             alpha=module._tlokr_alpha)
