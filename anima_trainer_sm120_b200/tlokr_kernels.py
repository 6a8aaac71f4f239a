"""T-LoKr rank-space ops with the call surface of anima-trainer's
``tlokr_kernels.py`` (``rank_mix`` :125, ``rank_mix_wgrad`` :168), backed by
``csrc/tlokr_mix.cu``.

``hidden`` is ``[batch, n, 8, rank]`` bf16, ``weight`` the 8x8 Kronecker factor,
``mask`` the per-sample ``[batch, rank]`` 0/1 prefix mask or ``None``. Shapes the
kernels do not cover (factor other than 8, rank not a multiple of 8, non-bf16
input) raise instead of silently running elsewhere.
"""
from __future__ import annotations

import torch

from . import ops

BF16 = torch.bfloat16


def _check(hidden: torch.Tensor, mask: torch.Tensor | None) -> None:
    if not hidden.is_cuda:
        raise RuntimeError("rank_mix needs CUDA tensors (no CPU path)")
    if hidden.dim() != 4 or hidden.shape[-2] != 8:
        raise NotImplementedError(f"rank_mix supports [batch, n, 8, rank]; got {tuple(hidden.shape)}")
    if hidden.shape[-1] % 8:
        raise NotImplementedError(f"rank {hidden.shape[-1]} must be a multiple of 8")
    if mask is not None and mask.shape != (hidden.shape[0], hidden.shape[-1]):
        raise ValueError(f"mask {tuple(mask.shape)} does not match hidden {tuple(hidden.shape)}")


def rank_mix(hidden: torch.Tensor, weight: torch.Tensor, mask: torch.Tensor | None, *,
             transpose: bool = False) -> torch.Tensor:
    """``weight[.T] @ (hidden * mask)`` for an 8x8 ``weight``."""
    _check(hidden, mask)
    if weight.shape != (8, 8):
        raise NotImplementedError(f"rank_mix supports an 8x8 factor; got {tuple(weight.shape)}")
    out = ops.tlokr_rank_mix(hidden.contiguous().to(BF16), weight.contiguous().to(BF16),
                             None if mask is None else mask.contiguous().to(BF16), transpose)
    return out.to(hidden.dtype)


def rank_mix_wgrad(grad_mixed: torch.Tensor, hidden: torch.Tensor, mask: torch.Tensor | None
                   ) -> torch.Tensor:
    """fp32 ``einsum('bnir,bnjr->ij', grad_mixed, hidden * mask)``."""
    _check(hidden, mask)
    if grad_mixed.shape != hidden.shape:
        raise ValueError("grad_mixed and hidden must have the same shape")
    return ops.tlokr_rank_mix_wgrad(grad_mixed.contiguous().to(BF16), hidden.contiguous().to(BF16),
                                    None if mask is None else mask.contiguous().to(BF16))
