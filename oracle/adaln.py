"""Oracle: fused AdaLN and gated residual (CPU torch).

Two forms of each op:
* ``*_fp32`` — the arithmetic of anima-trainer's kernels (``adaln_kernel.py``:
  forward :52-68, dx :90-103, dscale/dshift :141-154, gated add :290-295, dgate
  :321-329): fp32 statistics and elementwise math, one rounding to bf16 at the end.
* ``*_eager`` — the eager PyTorch expression the reference tests compare against
  (``tests/sanity_adaln_kernel.py:21-23``; ``adaln_kernel.py:342-346``), evaluated in
  the input dtype with autograd.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F


def adaln_fwd_fp32(x, scale, shift, eps, hw):
    """x [rows, d], scale/shift [rows/hw, d] (any float dtype) -> (y fp32, mean, rstd)."""
    xf = x.float()
    rows, d = xf.shape
    mean = xf.sum(dim=1) / d                                   # adaln_kernel.py:54
    xc = xf - mean[:, None]
    var = (xc * xc).sum(dim=1) / d                             # :58
    rstd = 1.0 / torch.sqrt(var + eps)                         # :59
    s = scale.float().repeat_interleave(hw, dim=0)             # bt = row // HW, :47
    b = shift.float().repeat_interleave(hw, dim=0)
    y = xc * rstd[:, None] * (1.0 + s) + b                     # :60-64
    return y, mean, rstd


def adaln_bwd_fp32(dy, x, scale, mean, rstd, hw):
    """-> (dx, dscale, dshift) in fp32. adaln_kernel.py:77-83 and :112-116."""
    dyf, xf = dy.float(), x.float()
    rows, d = xf.shape
    s = scale.float().repeat_interleave(hw, dim=0)
    xhat = (xf - mean[:, None]) * rstd[:, None]                # :96
    dxhat = dyf * (1.0 + s)                                    # :97
    c1 = dxhat.sum(dim=1, keepdim=True) / d                    # :99
    c2 = (dxhat * xhat).sum(dim=1, keepdim=True) / d           # :100
    dx = rstd[:, None] * (dxhat - c1 - xhat * c2)              # :101
    dscale = (dyf * xhat).view(rows // hw, hw, d).sum(dim=1)   # :150
    dshift = dyf.view(rows // hw, hw, d).sum(dim=1)            # :151
    return dx, dscale, dshift


def adaln_eager(x5, scale5, shift5, eps):
    """tests/sanity_adaln_kernel.py:21-23 on (B,T,H,W,D) / (B,T,1,1,D) tensors."""
    n = F.layer_norm(x5, [x5.shape[-1]], None, None, eps)
    return n * (1 + scale5) + shift5


def gated_add_fwd_fp32(x, gate, y, hw):
    """out = x + gate[row // hw] * y in fp32 (adaln_kernel.py:290-295 computes it in the
    input dtype; the product of two bf16 values is exact in fp32, so fp32 evaluation followed
    by one rounding is the value closest to the exact result)."""
    return x.float() + gate.float().repeat_interleave(hw, dim=0) * y.float()


def gated_add_bwd_fp32(dout, y, gate, hw):
    """-> (dy, dgate) fp32: dy = gate * dout (:399), dgate = sum_hw dout * y (:321-329)."""
    rows, d = y.shape
    dy = gate.float().repeat_interleave(hw, dim=0) * dout.float()
    dgate = (dout.float() * y.float()).view(rows // hw, hw, d).sum(dim=1)
    return dy, dgate


def gated_add_eager(x5, gate5, y5):
    """adaln_kernel.py:342-346: out = x + gate * y with broadcasting."""
    return x5 + gate5 * y5
