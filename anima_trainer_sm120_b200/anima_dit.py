"""Anima-shaped stand-in DiT: the module tree the hot path is embedded in.

The real model (sd-scripts ``library.anima_models``) is not available, so this is a
random-init stand-in assembled from the structural facts the reference's patches rely on
(anima-trainer ``adaln_patch.py:42-153``, ``adaln_merge.py:4-8``, ``liger_patch.py:9-13``,
``rope_patch.py:43-44``, ``tests/bench_attention.py:3-7``, ``lokr.py:56-71``,
``train.py:355-365``): 28 blocks of width 2048, 16 heads x 128, MLP 8192, LayerNorms without
affine (eps 1e-6), AdaLN modulation ``Sequential(SiLU, Linear(D, lora_dim), Linear(lora_dim, 3D))``
plus a shared ``adaln_lora_B_T_3D``, per-head RMSNorm on q / k, RoPE on the self-attention q / k,
cross-attention onto 512 text tokens of width 1024, ``mlp.layer1`` / ``mlp.layer2`` with GELU,
latents (B, 16, T, H, W) + 1 padding-mask channel patchified 1x2x2, flow-matching velocity output.
Attribute and method names follow what the module patches read (``Block._forward`` signature,
``layer_norm_*``, ``adaln_modulation_*``, ``use_adaln_lora``, ``self_attn``, ``cross_attn``,
``mlp``), so ``adaln_patch`` / ``lokr_patch`` / ``fp8_quant`` walkers apply unchanged.

Everything in this file is eager PyTorch (attention is torch SDPA, as in the reference): it is
the "bf16 reference mode" arm and the host of the patched kernels, not itself a kernel.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch.utils.checkpoint import checkpoint as torch_checkpoint


@dataclass(frozen=True)
class AnimaConfig:
    depth: int = 28
    dim: int = 2048
    heads: int = 16
    mlp_dim: int = 8192
    context_dim: int = 1024
    latent_channels: int = 16
    patch: int = 2
    adaln_lora_dim: int = 256
    use_adaln_lora: bool = True
    eps: float = 1e-6

    @property
    def head_dim(self) -> int:
        return self.dim // self.heads


def tiny_config(**kw) -> AnimaConfig:
    """A small configuration with the same structure, for CPU tests."""
    base = dict(depth=2, dim=256, heads=4, mlp_dim=512, context_dim=128, adaln_lora_dim=32)
    base.update(kw)
    return AnimaConfig(**base)


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-6):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim))
        self.eps = eps

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        xf = x.float()
        return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.eps)).to(x.dtype) * self.weight


def apply_rotary_pos_emb(t: torch.Tensor, freqs: torch.Tensor) -> torch.Tensor:
    """t (B, L, H, d); freqs (L, 1, 1, d) angles. Rotate-half convention."""
    cos, sin = freqs.cos().to(t.dtype), freqs.sin().to(t.dtype)
    cos, sin = cos.permute(1, 0, 2, 3), sin.permute(1, 0, 2, 3)  # (1, L, 1, d)
    t1, t2 = t.chunk(2, dim=-1)
    return t * cos + torch.cat((-t2, t1), dim=-1) * sin


class Attention(nn.Module):
    def __init__(self, cfg: AnimaConfig, context_dim: int | None):
        super().__init__()
        self.heads, self.head_dim = cfg.heads, cfg.head_dim
        kv_in = cfg.dim if context_dim is None else context_dim
        self.is_cross = context_dim is not None
        self.q_proj = nn.Linear(cfg.dim, cfg.dim, bias=False)
        self.k_proj = nn.Linear(kv_in, cfg.dim, bias=False)
        self.v_proj = nn.Linear(kv_in, cfg.dim, bias=False)
        self.output_proj = nn.Linear(cfg.dim, cfg.dim, bias=False)
        self.q_norm = RMSNorm(cfg.head_dim, cfg.eps)
        self.k_norm = RMSNorm(cfg.head_dim, cfg.eps)

    def _prepare_qk(self, q, k, rope_emb):
        """Per-head RMSNorm, then RoPE on self-attention. ``qk_norm_rope.install`` swaps in one fused kernel."""
        q, k = self.q_norm(q), self.k_norm(k)
        if rope_emb is not None:
            q, k = apply_rotary_pos_emb(q, rope_emb), apply_rotary_pos_emb(k, rope_emb)
        return q, k

    def forward(self, x, attn_params=None, context=None, rope_emb=None):
        B, L, _ = x.shape
        ctx = x if context is None else context
        q = self.q_proj(x).view(B, L, self.heads, self.head_dim)
        k = self.k_proj(ctx).view(B, ctx.shape[1], self.heads, self.head_dim)
        v = self.v_proj(ctx).view(B, ctx.shape[1], self.heads, self.head_dim)
        q, k = self._prepare_qk(q, k, None if self.is_cross else rope_emb)
        out = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2))
        return self.output_proj(out.transpose(1, 2).reshape(B, L, -1))


class GPT2FeedForward(nn.Module):
    def __init__(self, cfg: AnimaConfig):
        super().__init__()
        self.layer1 = nn.Linear(cfg.dim, cfg.mlp_dim, bias=False)
        self.layer2 = nn.Linear(cfg.mlp_dim, cfg.dim, bias=False)
        self.activation = nn.GELU()

    def forward(self, x):
        return self.layer2(self.activation(self.layer1(x)))


def _modulation(cfg: AnimaConfig) -> nn.Sequential:
    if cfg.use_adaln_lora:
        return nn.Sequential(nn.SiLU(), nn.Linear(cfg.dim, cfg.adaln_lora_dim, bias=False),
                             nn.Linear(cfg.adaln_lora_dim, 3 * cfg.dim, bias=False))
    return nn.Sequential(nn.SiLU(), nn.Linear(cfg.dim, 3 * cfg.dim, bias=False))


def _adaln(x, norm: nn.LayerNorm, scale, shift):
    return norm(x) * (1 + scale[:, :, None, None, :]) + shift[:, :, None, None, :]


class Block(nn.Module):
    """One DiT block; ``_forward`` has the signature ``adaln_patch`` replaces."""

    def __init__(self, cfg: AnimaConfig):
        super().__init__()
        D = cfg.dim
        self.use_adaln_lora = cfg.use_adaln_lora
        self.gradient_checkpointing = False
        self.layer_norm_self_attn = nn.LayerNorm(D, elementwise_affine=False, eps=cfg.eps)
        self.layer_norm_cross_attn = nn.LayerNorm(D, elementwise_affine=False, eps=cfg.eps)
        self.layer_norm_mlp = nn.LayerNorm(D, elementwise_affine=False, eps=cfg.eps)
        self.adaln_modulation_self_attn = _modulation(cfg)
        self.adaln_modulation_cross_attn = _modulation(cfg)
        self.adaln_modulation_mlp = _modulation(cfg)
        self.self_attn = Attention(cfg, None)
        self.cross_attn = Attention(cfg, cfg.context_dim)
        self.mlp = GPT2FeedForward(cfg)

    def forward(self, *args, **kwargs):
        if self.training and self.gradient_checkpointing:
            from .fp8_quant import first_pass      # this pass's saved tensors are dropped and recomputed
            with first_pass():
                return torch_checkpoint(self._forward, *args, use_reentrant=False, preserve_rng_state=False, **kwargs)
        return self._forward(*args, **kwargs)

    def _mod(self, seq, emb, adaln_lora):
        out = seq(emb)
        if self.use_adaln_lora and adaln_lora is not None:
            out = out + adaln_lora
        return out.chunk(3, dim=-1)

    def _forward(self, x_B_T_H_W_D, emb_B_T_D, crossattn_emb, attn_params=None, use_fp32=False,
                 rope_emb_L_1_1_D=None, adaln_lora_B_T_3D=None, extra_per_block_pos_emb=None):
        x = x_B_T_H_W_D.float() if use_fp32 else x_B_T_H_W_D     # fp32 residual stream on request
        if extra_per_block_pos_emb is not None:
            x = x + extra_per_block_pos_emb
        B, T, H, W, D = x.shape
        shift, scale, gate = self._mod(self.adaln_modulation_self_attn, emb_B_T_D, adaln_lora_B_T_3D)
        h = _adaln(x, self.layer_norm_self_attn, scale, shift).reshape(B, T * H * W, D)
        h = self.self_attn(h, attn_params, None, rope_emb=rope_emb_L_1_1_D).view(B, T, H, W, D)
        x = x + gate[:, :, None, None, :] * h
        shift, scale, gate = self._mod(self.adaln_modulation_cross_attn, emb_B_T_D, adaln_lora_B_T_3D)
        h = _adaln(x, self.layer_norm_cross_attn, scale, shift).reshape(B, T * H * W, D)
        h = self.cross_attn(h, attn_params, crossattn_emb, rope_emb=rope_emb_L_1_1_D).view(B, T, H, W, D)
        x = x + gate[:, :, None, None, :] * h
        shift, scale, gate = self._mod(self.adaln_modulation_mlp, emb_B_T_D, adaln_lora_B_T_3D)
        h = self.mlp(_adaln(x, self.layer_norm_mlp, scale, shift))
        return x + gate[:, :, None, None, :] * h


class TimestepEmbedder(nn.Module):
    def __init__(self, cfg: AnimaConfig):
        super().__init__()
        self.dim = cfg.dim
        self.linear_1 = nn.Linear(cfg.dim, cfg.dim, bias=False)
        self.linear_2 = nn.Linear(cfg.dim, 3 * cfg.dim if cfg.use_adaln_lora else cfg.dim, bias=False)
        self.use_adaln_lora = cfg.use_adaln_lora
        self.t_embedding_norm = RMSNorm(cfg.dim, cfg.eps)

    def forward(self, t_B_T: torch.Tensor, dtype):
        half = self.dim // 2
        freqs = torch.exp(-math.log(10000.0) * torch.arange(half, device=t_B_T.device, dtype=torch.float32) / half)
        ang = t_B_T.float()[..., None] * 1000.0 * freqs
        base = torch.cat([ang.cos(), ang.sin()], dim=-1).to(dtype)            # (B, T, D)
        out = self.linear_2(F.silu(self.linear_1(base)))
        emb = self.t_embedding_norm(base)
        return (emb, out) if self.use_adaln_lora else (emb + out, None)


class FinalLayer(nn.Module):
    def __init__(self, cfg: AnimaConfig):
        super().__init__()
        self.layer_norm = nn.LayerNorm(cfg.dim, elementwise_affine=False, eps=cfg.eps)
        self.adaln_modulation = nn.Sequential(nn.SiLU(), nn.Linear(cfg.dim, 2 * cfg.dim, bias=False))
        self.linear = nn.Linear(cfg.dim, cfg.patch * cfg.patch * cfg.latent_channels, bias=False)

    def forward(self, x, emb):
        shift, scale = self.adaln_modulation(emb).chunk(2, dim=-1)
        return self.linear(_adaln(x, self.layer_norm, scale, shift))


class AnimaDiT(nn.Module):
    """``dit(noisy_B_C_T_H_W, timesteps_B, crossattn_emb_B_L_C) -> velocity (B, C, T, H, W)``."""

    def __init__(self, cfg: AnimaConfig = AnimaConfig()):
        super().__init__()
        self.cfg = cfg
        in_ch = (cfg.latent_channels + 1) * cfg.patch * cfg.patch   # + padding-mask channel: 68 at patch 2
        self.x_embedder = nn.Linear(in_ch, cfg.dim, bias=False)
        self.t_embedder = TimestepEmbedder(cfg)
        self.blocks = nn.ModuleList(Block(cfg) for _ in range(cfg.depth))
        self.final_layer = FinalLayer(cfg)
        self.reset_parameters()

    def reset_parameters(self) -> None:
        for m in self.modules():
            if isinstance(m, nn.Linear):
                nn.init.normal_(m.weight, std=0.02)

    def enable_gradient_checkpointing(self, on: bool = True) -> None:
        for b in self.blocks:
            b.gradient_checkpointing = on

    def _rope(self, T, H, W, device):
        d = self.cfg.head_dim
        pos = torch.stack(torch.meshgrid(torch.arange(T, device=device), torch.arange(H, device=device),
                                         torch.arange(W, device=device), indexing="ij"), -1).reshape(-1, 3).float()
        n = d // 6
        inv = 1.0 / (10000.0 ** (torch.arange(n, device=device, dtype=torch.float32) / n))
        ang = torch.cat([pos[:, i:i + 1] * inv for i in range(3)], dim=-1)          # (L, 3n)
        ang = F.pad(ang, (0, d // 2 - ang.shape[-1]))
        return torch.cat([ang, ang], dim=-1)[:, None, None, :]                       # (L, 1, 1, d)

    def forward(self, x_B_C_T_H_W, timesteps_B, crossattn_emb, padding_mask=None):
        cfg = self.cfg
        B, C, T, H, W = x_B_C_T_H_W.shape
        p = cfg.patch
        mask = torch.zeros(B, 1, T, H, W, device=x_B_C_T_H_W.device, dtype=x_B_C_T_H_W.dtype) \
            if padding_mask is None else padding_mask
        x = torch.cat([x_B_C_T_H_W, mask], dim=1)
        x = x.view(B, C + 1, T, H // p, p, W // p, p).permute(0, 2, 3, 5, 1, 4, 6).reshape(B, T, H // p, W // p, -1)
        x = self.x_embedder(x)
        emb, adaln_lora = self.t_embedder(timesteps_B.view(B, 1).expand(B, T), x.dtype)
        rope = self._rope(T, H // p, W // p, x.device)
        for blk in self.blocks:
            x = blk(x, emb, crossattn_emb, None, False, rope, adaln_lora, None)
        out = self.final_layer(x, emb)                                                # (B, T, h, w, p*p*C)
        out = out.view(B, T, H // p, W // p, cfg.latent_channels, p, p).permute(0, 4, 1, 2, 5, 3, 6)
        return out.reshape(B, cfg.latent_channels, T, H, W)
