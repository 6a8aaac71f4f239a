"""Replace a DiT ``Block._forward`` with one that runs the AdaLN modulation
``LayerNorm(x) * (1 + scale) + shift`` and the gated residual ``x + gate * sublayer(...)`` on the
fused sm_100a kernels — the call surface of anima-trainer's ``adaln_patch.py`` (``_patched_forward``
:42-153, ``install`` :156-166, ``uninstall`` :169-177). One FusedAdaLN, two FusedGatedAddAdaLN (the reference's FusedGatedAdd + FusedAdaLN pair) and one
FusedGatedAdd call per block; control flow and argument list are those of the patched upstream method.
"""
from __future__ import annotations

import contextlib
from typing import Optional

import torch

from .adaln_kernel import FusedAdaLN, FusedGatedAdd, FusedGatedAddAdaLN
from .adaln_merge import apply_merged_adaln

_PATCHED: dict[type, object] = {}


def _five(t: torch.Tensor) -> torch.Tensor:
    return t[:, :, None, None, :]          # (B, T, D) -> (B, T, 1, 1, D)


def _patched_forward(self, x_B_T_H_W_D: torch.Tensor, emb_B_T_D: torch.Tensor, crossattn_emb: torch.Tensor,
                     attn_params=None, use_fp32: bool = False, rope_emb_L_1_1_D: Optional[torch.Tensor] = None,
                     adaln_lora_B_T_3D: Optional[torch.Tensor] = None,
                     extra_per_block_pos_emb: Optional[torch.Tensor] = None) -> torch.Tensor:
    if use_fp32 or x_B_T_H_W_D.dtype != torch.bfloat16:
        # The fused kernels read and write bf16. A caller that wants the residual stream carried in fp32
        # (``use_fp32``; the reference's kernels keep x.dtype, adaln_kernel.py:185-187) gets the block's own
        # unpatched forward instead of a silently bf16-rounded stream.
        orig = next((f for cls, f in _PATCHED.items() if isinstance(self, cls)), None)
        if orig is None:
            raise TypeError("adaln_patch: the fused Block forward needs a bfloat16 residual stream")
        return orig(self, x_B_T_H_W_D, emb_B_T_D, crossattn_emb, attn_params, use_fp32, rope_emb_L_1_1_D,
                    adaln_lora_B_T_3D, extra_per_block_pos_emb)
    x = x_B_T_H_W_D
    if extra_per_block_pos_emb is not None:
        x = x + extra_per_block_pos_emb
    ctx = contextlib.nullcontext()
    lora = adaln_lora_B_T_3D if self.use_adaln_lora else None
    with ctx:
        if getattr(self, "_adaln_modulation_merged", False):
            mods = apply_merged_adaln(self, emb_B_T_D, lora)
        else:
            mods = []
            for seq in (self.adaln_modulation_self_attn, self.adaln_modulation_cross_attn, self.adaln_modulation_mlp):
                out = seq(emb_B_T_D)
                mods.append((out + lora if lora is not None else out).chunk(3, dim=-1))
    (sh_s, sc_s, g_s), (sh_c, sc_c, g_c), (sh_m, sc_m, g_m) = mods
    B, T, H, W, D = x.shape

    # The residual update of a sublayer and the modulation of the next one are one kernel (one read of x and of
    # the sublayer output); the values are those of FusedGatedAdd followed by FusedAdaLN.
    n = FusedAdaLN.apply(x, _five(sc_s), _five(sh_s), self.layer_norm_self_attn.eps)
    r = self.self_attn(n.reshape(B, T * H * W, D), attn_params, None, rope_emb=rope_emb_L_1_1_D)
    x, n = FusedGatedAddAdaLN.apply(x, _five(g_s), r.view(B, T, H, W, D), _five(sc_c), _five(sh_c),
                                    self.layer_norm_cross_attn.eps)

    r = self.cross_attn(n.reshape(B, T * H * W, D), attn_params, crossattn_emb, rope_emb=rope_emb_L_1_1_D)
    x, n = FusedGatedAddAdaLN.apply(x, _five(g_c), r.view(B, T, H, W, D), _five(sc_m), _five(sh_m),
                                    self.layer_norm_mlp.eps)

    return FusedGatedAdd.apply(x, _five(g_m), self.mlp(n))


def install(block_cls: type | None = None) -> None:
    """Patch ``block_cls._forward`` (default: the stand-in ``anima_dit.Block``). Idempotent."""
    if block_cls is None:
        from .anima_dit import Block as block_cls
    if block_cls in _PATCHED:
        return
    _PATCHED[block_cls] = block_cls._forward
    block_cls._forward = _patched_forward


def uninstall(block_cls: type | None = None) -> None:
    if block_cls is None:
        from .anima_dit import Block as block_cls
    orig = _PATCHED.pop(block_cls, None)
    if orig is not None:
        block_cls._forward = orig
