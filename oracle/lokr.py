"""Oracle: LoKr merged-weight linear, bf16 reference mode (CPU torch).

Follows anima-trainer ``src/anima_trainer/lokr_patch.py:76-94`` (merged = W + alpha * diff,
one F.linear) with ``diff = kron(w1, w2) * scale`` as pinned by
``tests/test_tlokr.py:148``; backward is what autograd derives (docstring :19-21):
``dX = dY @ merged``, ``dW = dY.T @ X``, then the Kronecker adjoint to w1 / w2.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F


def merged_weight(w, w1, w2, alpha: float):
    """bf16 merged weight exactly as the eager path rounds it: the Kronecker product in the
    weight dtype (one rounding), then W + alpha * diff evaluated in fp32 and rounded once
    (torch.add(W, diff, alpha=alpha); alpha == 1 is W + diff), lokr_patch.py:77-84."""
    diff = torch.kron(w1.float(), w2.float()).to(w.dtype)
    return (w.float() + float(alpha) * diff.float()).to(w.dtype)


def kron_backward(dw, w1, w2, alpha: float):
    """Adjoint of diff = alpha * kron(w1, w2) in float64: dw1[i,j] = alpha * sum dW_blk(i,j) * w2,
    dw2[p,q] = alpha * sum_ij dW[i*vp+p, j*vq+q] * w1[i,j]."""
    up, uq = w1.shape
    vp, vq = w2.shape
    blocks = dw.double().reshape(up, vp, uq, vq)
    dw1 = alpha * torch.einsum("ipjq,pq->ij", blocks, w2.double())
    dw2 = alpha * torch.einsum("ipjq,ij->pq", blocks, w1.double())
    return dw1, dw2


def lokr_linear_bf16(x, w, bias, w1, w2, alpha: float, grad_y):
    """Config-1 arithmetic: forward y and backward (dx, dw1, dw2) through torch autograd with
    bf16 x / W and the factors in their own dtype, as the reference's bf16 mode runs it."""
    x = x.detach().clone().requires_grad_(True)
    w1 = w1.detach().clone().requires_grad_(True)
    w2 = w2.detach().clone().requires_grad_(True)
    diff = torch.kron(w1, w2).to(w.dtype)
    merged = w + diff if alpha == 1.0 else torch.add(w, diff, alpha=alpha)
    y = F.linear(x, merged, bias)
    y.backward(grad_y)
    return y.detach(), x.grad, w1.grad, w2.grad
