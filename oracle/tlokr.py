"""Oracle: T-LoKr schedule, rank mix and structured delta (CPU torch / python).

Follows anima-trainer ``src/anima_trainer/tlokr.py`` (schedule :40-57, mask :84-92,
structured forward :472-492, manual backward :495-540) and
``tlokr_kernels.py`` (rank_mix :15-82 / :134-146, rank_mix_wgrad :85-122 / :175-185),
plus the explicit-Kronecker form of ``tests/test_tlokr.py:137-156``.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F


def active_rank_for_timestep(timestep: float, *, max_rank: int, min_rank: int) -> int:
    """tlokr.py:40-57: floor((rmax - rmin) * (1 - clamp(t)) + rmin), clamped to [rmin, rmax]."""
    if max_rank <= 0:
        raise ValueError(f"max_rank must be positive; got {max_rank}")
    if not 1 <= min_rank <= max_rank:
        raise ValueError(f"min_rank must be in [1, {max_rank}]; got {min_rank}")
    t = min(1.0, max(0.0, float(timestep)))
    return max(min_rank, min(max_rank, math.floor((max_rank - min_rank) * (1.0 - t) + min_rank)))


def rank_mask(timesteps: torch.Tensor, *, max_rank: int, min_rank: int, dtype=torch.float32) -> torch.Tensor:
    """tlokr.py:84-92: [B, rmax] prefix mask, fp32 arithmetic on the timesteps."""
    t = timesteps.detach().to(torch.float32).reshape(-1)
    active = torch.floor((max_rank - min_rank) * (1.0 - t.clamp(0.0, 1.0)) + min_rank).to(torch.int64)
    active.clamp_(min=min_rank, max=max_rank)
    return (torch.arange(max_rank).unsqueeze(0) < active.unsqueeze(1)).to(dtype)


def rank_mix_fp32(hidden, weight, mask, transpose=False):
    """out[b,n,i,r] = (sum_j W[i,j] * hidden[b,n,j,r]) * mask[b,r], fp32, j ascending
    (tlokr_kernels.py:42-73; W = weight.T when transpose)."""
    h = hidden.float()
    w = weight.float().t() if transpose else weight.float()
    out = torch.zeros_like(h)
    for i in range(w.shape[0]):
        acc = torch.zeros_like(h[:, :, 0, :])
        for j in range(w.shape[1]):
            acc = acc + h[:, :, j, :] * w[i, j]
        out[:, :, i, :] = acc
    if mask is not None:
        out = out * mask.float()[:, None, None, :]
    return out


def rank_mix_wgrad_fp64(grad_mixed, hidden, mask):
    """dC[i,j] = sum_{b,n,r} g[b,n,i,r] * hidden[b,n,j,r] * mask[b,r] (tlokr_kernels.py:97-122),
    accumulated in float64 as ground truth for the fp32 kernel."""
    h = hidden.double()
    if mask is not None:
        h = h * mask.double()[:, None, None, :]
    return torch.einsum("bnir,bnjr->ij", grad_mixed.double(), h)


def structured_delta_fwd(x, w1, w2_a, w2_b, mask):
    """tlokr.py:472-492 in the dtype of x: delta = x @ kron(w1, (A*mask) @ B).T per sample."""
    c, a, b = w1.to(x.dtype), w2_a.to(x.dtype), w2_b.to(x.dtype)
    uq = c.shape[1]
    grouped = x.reshape(x.shape[0], -1, uq, x.shape[-1] // uq)
    hidden = torch.matmul(grouped, b.t())                                  # :479
    masked = hidden if mask is None else hidden * mask[:, None, None, :].to(x.dtype)
    mixed = torch.matmul(c, masked)                                        # :483 (rank_mix)
    out = torch.matmul(mixed, a.t())                                       # :484
    return out.reshape(*x.shape[:-1], -1)


def structured_delta_bwd(x, w1, w2_a, w2_b, mask, grad_output):
    """tlokr.py:495-540: (grad_x, grad_w1, grad_w2_a, grad_w2_b)."""
    dt = x.dtype
    c, a, b = w1.to(dt), w2_a.to(dt), w2_b.to(dt)
    batch, uq, up, vp = x.shape[0], c.shape[1], c.shape[0], a.shape[0]
    m4 = None if mask is None else mask[:, None, None, :].to(dt)
    grouped = x.reshape(batch, -1, uq, x.shape[-1] // uq)
    hidden = torch.matmul(grouped, b.t())
    masked = hidden if m4 is None else hidden * m4
    mixed = torch.matmul(c, masked)
    g_blocks = grad_output.to(dt).reshape(batch, -1, up, vp)
    g_a = g_blocks.reshape(-1, vp).t() @ mixed.reshape(-1, mixed.shape[-1])   # :519-522
    g_mixed = torch.matmul(g_blocks, a)                                         # :523
    g_c = torch.einsum("bnir,bnjr->ij", g_mixed.float(), masked.float())       # :524
    g_hidden = torch.matmul(c.t(), g_mixed if m4 is None else g_mixed * m4)    # :525
    g_b = g_hidden.reshape(-1, g_hidden.shape[-1]).t() @ grouped.reshape(-1, grouped.shape[-1])  # :527-530
    g_x = torch.matmul(g_hidden, b).reshape(x.shape)                            # :531-532
    return g_x, g_c.to(w1.dtype), g_a.to(w2_a.dtype), g_b.to(w2_b.dtype)


def explicit_kron_linear(x, base_w, base_b, w1, w2_a, w2_b, timesteps, *, rank, min_rank, scale):
    """tests/test_tlokr.py:137-156: per-sample F.linear with W + kron(w1, A[:, :a] @ B[:a]) * scale."""
    rows = []
    for i, t in enumerate(timesteps.tolist()):
        act = active_rank_for_timestep(t, max_rank=rank, min_rank=min_rank)
        w2 = w2_a[:, :act] @ w2_b[:act, :]
        rows.append(F.linear(x[i], base_w + torch.kron(w1, w2) * scale, base_b))
    return torch.stack(rows)
