"""GPU parity of the fused per-head RMSNorm + RoPE kernel against a plain fp32 PyTorch statement of
the same op (forward and the x-gradient), and of the patched ``Attention`` against the eager one.
Tolerance: bf16 output rounding, rtol 1e-2 / atol 2e-2."""
from __future__ import annotations

import pytest
import torch

pytestmark = pytest.mark.gpu
BF16 = torch.bfloat16
DEV = "cuda"


def _reference(x, w, ang, eps):
    """fp32: n = x * rsqrt(mean x^2 + eps) * w; out = n cos + rotate_half(n) sin."""
    xf = x.float()
    n = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * w
    if ang is None:
        return n
    cos, sin = ang.cos()[None, :, None, :], ang.sin()[None, :, None, :]
    n1, n2 = n.chunk(2, dim=-1)
    return n * cos + torch.cat((-n2, n1), dim=-1) * sin


@pytest.mark.parametrize("B,L,H", [(2, 64, 16), (1, 37, 3), (3, 1, 1), (2, 512, 16)])
@pytest.mark.parametrize("rope", [True, False])
def test_forward_backward_vs_fp32(B, L, H, rope):
    from anima_trainer_sm120_b200 import ops
    torch.manual_seed(B * 1000 + L + H)
    x = (torch.randn(B, L, H, 128, device=DEV) * 1.7).to(BF16)
    w = 1 + 0.2 * torch.randn(128, device=DEV)
    ang = torch.rand(L, 128, device=DEV) * 50 if rope else None
    cos, sin = (ang.cos().contiguous(), ang.sin().contiguous()) if rope else (None, None)
    g = torch.randn(B, L, H, 128, device=DEV).to(BF16)

    out, rstd = ops.rmsnorm_rope_fwd(x, w, cos, sin, 1e-6)
    dx = ops.rmsnorm_rope_bwd(g, x, w, cos, sin, rstd)

    xr = x.float().requires_grad_(True)
    ref = _reference(xr, w, ang, 1e-6)
    ref.backward(g.float())
    torch.testing.assert_close(out.float(), ref.detach(), rtol=1e-2, atol=2e-2)
    torch.testing.assert_close(dx.float(), xr.grad, rtol=1e-2, atol=2e-2)
    want_rstd = torch.rsqrt(x.float().pow(2).mean(-1) + 1e-6).reshape(-1)
    torch.testing.assert_close(rstd, want_rstd, rtol=1e-5, atol=1e-6)


def test_rejects_other_head_widths_and_ragged_sequences():
    from anima_trainer_sm120_b200 import ops
    w = torch.ones(64, device=DEV)
    with pytest.raises(NotImplementedError):
        ops.rmsnorm_rope_fwd(torch.zeros(1, 4, 2, 64, device=DEV, dtype=BF16), w, None, None, 1e-6)
    tab = torch.zeros(3, 128, device=DEV)
    with pytest.raises(ValueError):
        ops.rmsnorm_rope_fwd(torch.zeros(1, 4, 2, 128, device=DEV, dtype=BF16), torch.ones(128, device=DEV), tab, tab, 1e-6)
    out, rstd = ops.rmsnorm_rope_fwd(torch.zeros(0, 4, 2, 128, device=DEV, dtype=BF16), torch.ones(128, device=DEV),
                                     None, None, 1e-6)
    assert out.numel() == 0 and rstd.numel() == 0


def test_patched_attention_matches_eager_attention():
    from anima_trainer_sm120_b200 import qk_norm_rope
    from anima_trainer_sm120_b200.anima_dit import AnimaConfig, Attention
    torch.manual_seed(1)
    cfg = AnimaConfig(depth=1, dim=512, heads=4, mlp_dim=1024, context_dim=256, adaln_lora_dim=32)
    results = {}
    for cross in (False, True):
        attn = Attention(cfg, cfg.context_dim if cross else None).to(DEV, BF16).requires_grad_(False)
        with torch.no_grad():
            attn.q_norm.weight.add_(0.1 * torch.randn_like(attn.q_norm.weight))
            attn.k_norm.weight.add_(0.1 * torch.randn_like(attn.k_norm.weight))
        x = torch.randn(2, 96, 512, device=DEV, dtype=BF16)
        ctx = torch.randn(2, 24, 256, device=DEV, dtype=BF16) if cross else None
        rope = (torch.rand(96, 1, 1, 128, device=DEV) * 30)
        gy = torch.randn(2, 96, 512, device=DEV, dtype=BF16)
        for fused in (False, True):
            qk_norm_rope.install(Attention) if fused else qk_norm_rope.uninstall(Attention)
            try:
                xi = x.clone().requires_grad_(True)
                y = attn(xi, None, ctx, rope_emb=rope)
                y.backward(gy)
                results[(cross, fused)] = (y.detach().float(), xi.grad.float())
            finally:
                qk_norm_rope.uninstall(Attention)
        for a, b in zip(results[(cross, False)], results[(cross, True)]):
            assert float((a - b).abs().max() / (a.abs().max() + 1e-9)) < 3e-2
