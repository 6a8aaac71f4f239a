"""Merge a Block's three AdaLN-modulation MLPs into one SiLU, one first Linear and one batched
second matmul — the call surface of anima-trainer's ``adaln_merge.py``
(``merge_adaln_modulation`` :173-199, ``apply_merged_adaln`` :202-248).

Original layout per Block (``use_adaln_lora=True``): three ``Sequential(SiLU, Linear(D, r),
Linear(r, 3D))`` applied to the same ``emb_B_T_D``. Merged: ``adaln_modulation_silu``,
``adaln_modulation_l1 = Linear(D, 3r)`` (row-concatenated first weights) and the non-persistent
buffer ``adaln_modulation_l2_stack`` ``(3, r, 3D)`` (transposed second weights) used by one ``bmm``.
Without adaln-lora the three ``Linear(D, 3D)`` collapse into one ``Linear(D, 9D)``.
The merged modules keep ``adaln_modulation`` in their names, so the frozen-Linear walkers of
``fp8_quant`` keep skipping them. These are tiny (B*T rows) eager ops: glue, not a kernel.
"""
from __future__ import annotations

import torch
import torch.nn as nn

_TAG = "_adaln_modulation_merged"
_NAMES = ("adaln_modulation_self_attn", "adaln_modulation_cross_attn", "adaln_modulation_mlp")


def _is_block(mod: nn.Module) -> bool:
    return all(hasattr(mod, n) for n in _NAMES) and hasattr(mod, "use_adaln_lora")


def _merge_block(block: nn.Module) -> bool:
    if getattr(block, _TAG, False):
        return False
    seqs = [getattr(block, n) for n in _NAMES]
    lora = bool(block.use_adaln_lora)
    want = 3 if lora else 2
    if any(len(s) != want or not isinstance(s[0], nn.SiLU) for s in seqs):
        return False
    firsts = [s[1] for s in seqs]
    if any(not isinstance(l, nn.Linear) or l.bias is not None for s in seqs for l in list(s)[1:]):
        return False
    D = firsts[0].in_features
    dev, dt = firsts[0].weight.device, firsts[0].weight.dtype
    l1 = nn.Linear(D, sum(l.out_features for l in firsts), bias=False, device=dev, dtype=dt)
    with torch.no_grad():
        l1.weight.copy_(torch.cat([l.weight.detach() for l in firsts], dim=0))
    l1.weight.requires_grad_(False)
    block.adaln_modulation_silu = nn.SiLU()
    block.adaln_modulation_l1 = l1
    if lora:
        seconds = [s[2] for s in seqs]
        r, three_D = seconds[0].in_features, seconds[0].out_features
        stack = torch.stack([l.weight.detach().t().contiguous() for l in seconds], dim=0)   # (3, r, 3D)
        block.register_buffer("adaln_modulation_l2_stack", stack, persistent=False)
        block._adaln_merged_dims = (D, r, three_D)
    else:
        block._adaln_merged_dims = (D, None, firsts[0].out_features)
    for n in _NAMES:
        delattr(block, n)
    setattr(block, _TAG, True)
    return True


def merge_adaln_modulation(dit: nn.Module) -> int:
    """Merge every Block of ``dit`` (idempotent). Returns the number of Blocks merged."""
    return sum(int(_merge_block(m)) for m in list(dit.modules()) if _is_block(m))


def apply_merged_adaln(block: nn.Module, emb_B_T_D: torch.Tensor, adaln_lora_B_T_3D: torch.Tensor | None):
    """((shift, scale, gate) for self-attn, cross-attn, mlp), each ``(B, T, D)`` (views of one tensor)."""
    D, r, three_D = block._adaln_merged_dims
    B, T, _ = emb_B_T_D.shape
    h = block.adaln_modulation_silu(emb_B_T_D)
    if r is None:
        out = block.adaln_modulation_l1(h)
        if adaln_lora_B_T_3D is not None:
            out = out + adaln_lora_B_T_3D.repeat(1, 1, 3)
        c = out.chunk(9, dim=-1)
        return (c[0], c[1], c[2]), (c[3], c[4], c[5]), (c[6], c[7], c[8])
    h1 = block.adaln_modulation_l1(h).view(B, T, 3, r).permute(2, 0, 1, 3).reshape(3, B * T, r)
    out = torch.bmm(h1, block.adaln_modulation_l2_stack.to(h1.dtype)).view(3, B, T, three_D)
    if adaln_lora_B_T_3D is not None:
        out = out + adaln_lora_B_T_3D.unsqueeze(0)
    return tuple(tuple(o.chunk(3, dim=-1)) for o in out.unbind(0))
