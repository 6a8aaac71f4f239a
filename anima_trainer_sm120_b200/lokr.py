"""LoKr adapter modules and ``attach_lokr`` for the stand-in DiT.

anima-trainer creates its adapters through LyCORIS (``lokr.py:78-142``: algo=lokr, factor 8,
``full_matrix``, presets ``anima-full`` / ``anima-cross-mlp`` at :45-71). LyCORIS is not a
dependency here, so :class:`LokrModule` is a minimal module with the attributes the reference's
patches read (``lokr_patch.py:47-94``, ``tlokr.py:330-448``): ``org_module``, ``lokr_w1``,
``lokr_w2``, ``scale``, ``scalar``, ``multiplier``, ``shape``, ``get_weight``, ``op``,
``kw_dict``, ``module_dropout``, ``bypass_mode``, ``wd``, ``use_w1`` / ``use_w2``,
``module_type``, ``lora_name``. Its stock ``forward`` is the un-patched two-matmul LyCORIS
form (base output + delta output); ``lokr_patch.install()`` replaces it.

Delta definition (pinned by the reference's ``tests/test_tlokr.py:148``):
``delta_W = kron(lokr_w1, lokr_w2) * scale`` with ``scale = alpha / lora_dim``; ``lokr_w2`` is
zero-initialised so the adapted model starts exactly at the base model.
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F

PRESETS = {
    # suffixes of the wrapped Linears inside each Block (anima-trainer lokr.py:56-71)
    "anima-cross-mlp": ("cross_attn.q_proj", "cross_attn.k_proj", "cross_attn.v_proj", "cross_attn.output_proj",
                        "mlp.layer1", "mlp.layer2"),
    "anima-full": ("self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj", "self_attn.output_proj",
                   "cross_attn.q_proj", "cross_attn.k_proj", "cross_attn.v_proj", "cross_attn.output_proj",
                   "mlp.layer1", "mlp.layer2"),
}


def factorization(dimension: int, factor: int) -> tuple[int, int]:
    """(small, large) with small * large == dimension and small == factor when it divides."""
    if factor > 0 and dimension % factor == 0:
        return factor, dimension // factor
    m = int(math.isqrt(dimension))
    while dimension % m:
        m -= 1
    return m, dimension // m


class LokrModule(nn.Module):
    """Full-matrix LoKr adapter around one ``nn.Linear`` (kept in a list so it is not a submodule)."""

    module_type = "linear"

    def __init__(self, lora_name: str, org_module: nn.Linear, multiplier: float = 1.0, lora_dim: int = 128,
                 alpha: float = 128.0, factor: int = 8, full_matrix: bool = True, dtype=torch.float32):
        super().__init__()
        if not isinstance(org_module, nn.Linear):
            raise TypeError("LokrModule wraps nn.Linear only")
        self.lora_name = lora_name
        self.org_module = [org_module]
        out_dim, in_dim = org_module.weight.shape
        self.shape = (out_dim, in_dim)
        up, vp = factorization(out_dim, factor)
        uq, vq = factorization(in_dim, factor)
        dev = org_module.weight.device
        self.lokr_w1 = nn.Parameter(torch.empty(up, uq, device=dev, dtype=dtype))
        self.lokr_w2 = nn.Parameter(torch.zeros(vp, vq, device=dev, dtype=dtype))
        nn.init.kaiming_uniform_(self.lokr_w1, a=math.sqrt(5))
        self.use_w1 = self.use_w2 = True
        self.full_matrix = full_matrix
        self.lora_dim = lora_dim
        self.scale = float(alpha) / float(lora_dim)
        self.multiplier = multiplier
        self.register_buffer("scalar", torch.tensor(1.0), persistent=False)
        self.module_dropout = self.rank_dropout = self.dropout = 0.0
        self.bypass_mode = False
        self.wd = False
        self.op = F.linear
        self.kw_dict: dict = {}

    def get_weight(self, shape=None) -> torch.Tensor:
        w = torch.kron(self.lokr_w1, self.lokr_w2) * self.scale
        return w if shape is None else w.view(shape)

    def org_forward(self, x, *a, **kw):
        return self._org_forward(x)

    def apply_to(self) -> None:
        """Route the wrapped Linear's forward through this adapter (as LyCORIS ``apply_to`` does)."""
        lin = self.org_module[0]
        self._org_forward = lin.forward
        lin.forward = self.forward

    def forward(self, x, *args, **kwargs):
        org = self.org_module[0]
        base = F.linear(x, org.weight, org.bias)
        delta = self.get_weight(self.shape).to(org.weight.dtype) * (float(self.scalar) * self.multiplier)
        return base + F.linear(x, delta, None)

    def custom_state_dict(self) -> dict:
        state = {"lokr_w1": self.lokr_w1, "alpha": torch.tensor(self.scale * self.lora_dim)}
        if hasattr(self, "lokr_w2"):
            state["lokr_w2"] = self.lokr_w2
        else:                                   # T-LoKr: the large factor is stored as A @ B
            state["lokr_w2_a"], state["lokr_w2_b"] = self.lokr_w2_a, self.lokr_w2_b
        return state


class LokrNetwork(nn.Module):
    """The adapters of one model; parameters live here, the base model stays frozen."""

    def __init__(self, loras: list[LokrModule]):
        super().__init__()
        self.unet_loras = nn.ModuleList(loras)

    def apply_to(self) -> None:
        for m in self.unet_loras:
            m.apply_to()


def attach_lokr(dit: nn.Module, *, preset: str = "anima-cross-mlp", factor: int = 8, dim: int = 128,
                alpha: float = 128.0, full_matrix: bool = True, variant: str = "lokr",
                timestep_min_rank_ratio: float = 0.5, dtype=torch.float32) -> LokrNetwork:
    """Freeze ``dit``, wrap the preset's Linears, optionally convert to T-LoKr, install the patched
    forward and hook the adapters in (reference ``lokr.py:78-142``)."""
    from . import lokr_patch, tlokr

    if preset not in PRESETS:
        raise ValueError(f"unknown preset {preset!r}")
    dit.requires_grad_(False)
    loras = []
    for name, mod in dit.named_modules():
        if isinstance(mod, nn.Linear) and ".blocks." in f".{name}" and name.endswith(PRESETS[preset]):
            loras.append(LokrModule("lokr_" + name.replace(".", "_"), mod, lora_dim=dim, alpha=alpha, factor=factor,
                                    full_matrix=full_matrix, dtype=dtype))
    if not loras:
        raise RuntimeError("attach_lokr found no target Linear")
    network = LokrNetwork(loras)
    lokr_patch.install()
    if variant == "tlokr":
        tlokr.convert_network(network, rank=dim, min_rank_ratio=timestep_min_rank_ratio)
    elif variant != "lokr":
        raise ValueError(f"unknown variant {variant!r}")
    network.apply_to()
    return network
