"""Fused per-head RMSNorm + rotary embedding for the attention q / k vectors.

anima-trainer swaps two third-party kernels in at this point of the DiT: Liger's RMSNorm for the
``q_norm`` / ``k_norm`` modules (``liger_patch.py:31-47``) and Transformer Engine's fused RoPE for
``apply_rotary_pos_emb`` (``rope_patch.py:28-56``). Here both run as ONE sm_100a kernel per tensor
(``csrc/rmsnorm_rope.cu``): q and k are read once and written once, instead of the ~10 eager
elementwise launches of the unpatched path. ``install`` patches ``Attention._prepare_qk`` the same
way the reference's patches replace module methods; ``uninstall`` restores it.

The fused path needs CUDA bf16 tensors with head width 128 and a frozen norm weight (adapter
training); any other call keeps the original eager method.
"""
from __future__ import annotations

import weakref

import torch

from . import ops

_PATCHED: dict[type, object] = {}
_tables: tuple[weakref.ref, torch.Tensor, torch.Tensor] | None = None


def rope_tables(rope_emb: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """fp32 cos / sin tables [L, d] of an angle tensor (L, 1, 1, d); memoised for the last tensor seen."""
    global _tables
    if _tables is not None and _tables[0]() is rope_emb:
        return _tables[1], _tables[2]
    ang = rope_emb.detach().reshape(rope_emb.shape[0], rope_emb.shape[-1]).float()
    cos, sin = ang.cos().contiguous(), ang.sin().contiguous()
    _tables = (weakref.ref(rope_emb), cos, sin)
    return cos, sin


class FusedRMSNormRoPE(torch.autograd.Function):
    """out = rope(rmsnorm(x) * weight); x (B, L, H, 128) bf16. Gradient for x only."""

    @staticmethod
    def forward(ctx, x, weight, cos, sin, eps):
        x = x.contiguous()
        w = weight.detach().float().contiguous()
        out, rstd = ops.rmsnorm_rope_fwd(x, w, cos, sin, eps)
        ctx.save_for_backward(x, w, rstd)
        ctx.tables = (cos, sin)
        return out

    @staticmethod
    def backward(ctx, dout):
        x, w, rstd = ctx.saved_tensors
        cos, sin = ctx.tables
        return ops.rmsnorm_rope_bwd(dout.contiguous(), x, w, cos, sin, rstd), None, None, None, None


def _fusable(t: torch.Tensor, norm) -> bool:
    return (t.is_cuda and t.dtype == torch.bfloat16 and t.shape[-1] == 128 and t.dim() == 4
            and not norm.weight.requires_grad)


def _patched_prepare_qk(self, q, k, rope_emb):
    if not (_fusable(q, self.q_norm) and _fusable(k, self.k_norm)):
        return _PATCHED[type(self)](self, q, k, rope_emb)
    cos = sin = None
    if rope_emb is not None:
        if rope_emb.shape[0] != q.shape[1] or k.shape[1] != q.shape[1]:
            raise ValueError(f"rope table of {rope_emb.shape[0]} positions for sequences of {q.shape[1]} / {k.shape[1]}")
        cos, sin = rope_tables(rope_emb)
    return (FusedRMSNormRoPE.apply(q, self.q_norm.weight, cos, sin, self.q_norm.eps),
            FusedRMSNormRoPE.apply(k, self.k_norm.weight, cos, sin, self.k_norm.eps))


def install(attn_cls: type | None = None) -> None:
    """Patch ``attn_cls._prepare_qk`` (default: the stand-in ``anima_dit.Attention``). Idempotent."""
    if attn_cls is None:
        from .anima_dit import Attention as attn_cls
    if attn_cls in _PATCHED:
        return
    _PATCHED[attn_cls] = attn_cls._prepare_qk
    attn_cls._prepare_qk = _patched_prepare_qk


def uninstall(attn_cls: type | None = None) -> None:
    if attn_cls is None:
        from .anima_dit import Attention as attn_cls
    orig = _PATCHED.pop(attn_cls, None)
    if orig is not None:
        attn_cls._prepare_qk = orig
