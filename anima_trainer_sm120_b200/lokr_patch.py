"""Patched ``LokrModule.forward``: one merged-weight GEMM per wrapped Linear, with the call
surface of anima-trainer's ``lokr_patch.py`` (``_patched_forward`` :47-94, ``enable_fp8`` :129-135,
``install`` :138-147).

Dispatch order is the reference's: module dropout -> T-LoKr -> bypass -> weight-decomposition
fall-backs, then the merged path. Two merged paths exist:

* quantised (after ``enable_fp8(network)``, for CUDA inputs of eligible modules): the fused
  operator ``fp8_quant.lokr_linear_fused`` — W + alpha*kron(w1, w2) is built and quantised in
  one kernel, forward / dgrad / wgrad are MXFP8 tensor-core GEMMs and the adapter gradients
  come from one pass over dW. Nothing [N, K]-sized is materialised in bf16.
* bf16 reference mode (default; also what CPU tensors take): ``merged = W + alpha * diff``
  then ``self.op(x, merged, bias)``, exactly the reference's arithmetic (:76-94).
"""
from __future__ import annotations

import torch

from .lokr import LokrModule

_PATCHED = False
_ORIG_FORWARD = None
_ORIG_CUSTOM_STATE_DICT = None
# Module-global switch, flipped by enable_fp8() / disable_fp8() (reference name: _FP8_ACTIVE).
_FP8_ACTIVE = False
MX_ALIGN = 32  # both dimensions of the wrapped Linear and the token count must divide by 32


def _alpha(self) -> float:
    alpha = getattr(self, "_fused_alpha", None)
    if alpha is None:
        scalar = self.scalar.item() if torch.is_tensor(self.scalar) else self.scalar
        alpha = float(scalar) * float(self.multiplier)
        self._fused_alpha = alpha  # cached python float: no per-call device sync (reference :65-74)
    return alpha


def _patched_forward(self, x: torch.Tensor, *args, **kwargs):
    if self.module_dropout and self.training:
        if torch.rand(1) < self.module_dropout:
            return self.org_forward(x, *args, **kwargs)
    if getattr(self, "_tlokr_enabled", False):
        from .tlokr import forward as tlokr_forward
        return tlokr_forward(self, x)
    if self.bypass_mode:
        return self.bypass_forward(x, self.multiplier)
    if self.wd:
        return _ORIG_FORWARD(self, x, *args, **kwargs)

    org = self.org_module[0]
    alpha = _alpha(self)
    if (_FP8_ACTIVE and getattr(self, "_fp8_ok", False) and x.is_cuda
            and (x.numel() // x.shape[-1]) % MX_ALIGN == 0):
        from .fp8_quant import lokr_linear_fused
        return lokr_linear_fused(x, org.weight, org.bias, self.lokr_w1, self.lokr_w2, alpha * self.scale)

    diff_weight = self.get_weight(self.shape)
    if diff_weight.dtype != org.weight.dtype:
        diff_weight = diff_weight.to(org.weight.dtype)
    merged = org.weight + diff_weight if alpha == 1.0 else torch.add(org.weight, diff_weight, alpha=alpha)
    return self.op(x, merged, org.bias, **self.kw_dict)


def _patched_custom_state_dict(self):
    state = _ORIG_CUSTOM_STATE_DICT(self)
    if getattr(self, "_tlokr_enabled", False):
        state["tlokr_schedule"] = self.tlokr_schedule
    return state


def _mark_fp8_eligible(network) -> int:
    """Tag adapters whose wrapped Linear can take the quantised path (both dims % 32, factor <= 8,
    w2's inner width % 8); T-LoKr modules have their own path. Returns the eligible count."""
    count = 0
    for mod in network.modules():
        if not isinstance(mod, LokrModule):
            continue
        ok = False
        if not getattr(mod, "_tlokr_enabled", False) and isinstance(mod.org_module[0], torch.nn.Linear):
            out_dim, in_dim = mod.org_module[0].weight.shape
            up, uq = mod.lokr_w1.shape
            ok = (out_dim % MX_ALIGN == 0 and in_dim % MX_ALIGN == 0 and up <= 8 and uq <= 8
                  and (in_dim // uq) % 8 == 0)
        mod._fp8_ok = ok
        count += int(ok)
    return count


def enable_fp8(network) -> int:
    """Switch eligible adapters to the quantised path. Call after ``install()``."""
    global _FP8_ACTIVE
    n = _mark_fp8_eligible(network)
    _FP8_ACTIVE = True
    return n


def disable_fp8() -> None:
    global _FP8_ACTIVE
    _FP8_ACTIVE = False


def install() -> None:
    """Replace ``LokrModule.forward`` / ``custom_state_dict`` globally. Idempotent."""
    global _PATCHED, _ORIG_FORWARD, _ORIG_CUSTOM_STATE_DICT
    if _PATCHED:
        return
    _ORIG_FORWARD = LokrModule.forward
    _ORIG_CUSTOM_STATE_DICT = LokrModule.custom_state_dict
    LokrModule.forward = _patched_forward
    LokrModule.custom_state_dict = _patched_custom_state_dict
    _PATCHED = True


def uninstall() -> None:
    global _PATCHED
    if not _PATCHED:
        return
    LokrModule.forward = _ORIG_FORWARD
    LokrModule.custom_state_dict = _ORIG_CUSTOM_STATE_DICT
    _PATCHED = False
