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

    # A LyCORIS network serialises ``{lora_name}.{key}`` from every module's ``custom_state_dict()`` (which the
    # forward patch extends with the T-LoKr marker); this is the key set the adapter file carries.
    def state_dict(self, *args, destination=None, prefix: str = "", keep_vars: bool = False):
        sd = {} if destination is None else destination
        for m in self.unet_loras:
            for k, v in m.custom_state_dict().items():
                sd[f"{prefix}{m.lora_name}.{k}"] = v if keep_vars else v.detach()
        return sd

    def load_state_dict(self, state_dict, strict: bool = True, assign: bool = False):
        """Copy an adapter state into the modules. ``alpha`` updates the module's scale; a ``tlokr_schedule``
        that differs from the module's is an error (anima-trainer ``tlokr.py:305-327``), as are shape
        mismatches and, with ``strict``, missing or unexpected keys."""
        from torch.nn.modules.module import _IncompatibleKeys

        expected = self.state_dict(keep_vars=True)
        missing = [k for k in expected if k not in state_dict]
        unexpected = [k for k in state_dict if k not in expected]
        errors: list[str] = []
        by_name = {m.lora_name: m for m in self.unet_loras}
        with torch.no_grad():
            for key, dst in expected.items():
                src = state_dict.get(key)
                if src is None:
                    continue
                name, leaf = key.rsplit(".", 1)
                mod = by_name[name]
                if leaf == "tlokr_schedule":
                    want = dst.detach().to("cpu", torch.int64)
                    got = src.detach().to("cpu", torch.int64)
                    if got.shape != want.shape or not torch.equal(got, want):
                        errors.append(f"{key} is incompatible: checkpoint has {got.tolist()}, "
                                      f"model expects {want.tolist()}")
                    continue
                if leaf == "alpha":
                    if src.numel() != 1:
                        errors.append(f"{key}: alpha must be a scalar, got shape {tuple(src.shape)}")
                        continue
                    mod.scale = float(src) / float(mod.lora_dim)
                    if getattr(mod, "_tlokr_enabled", False):
                        scalar = mod.scalar.item() if torch.is_tensor(mod.scalar) else mod.scalar
                        mod._tlokr_alpha = float(mod.scale) * float(scalar) * float(mod.multiplier)
                    continue
                if tuple(src.shape) != tuple(dst.shape):
                    errors.append(f"size mismatch for {key}: checkpoint {tuple(src.shape)}, model {tuple(dst.shape)}")
                    continue
                dst.copy_(src.to(device=dst.device, dtype=dst.dtype))
        if strict:
            if unexpected:
                errors.insert(0, "Unexpected key(s) in state_dict: " + ", ".join(map(repr, unexpected)))
            if missing:
                errors.insert(0, "Missing key(s) in state_dict: " + ", ".join(map(repr, missing)))
        if errors:
            raise RuntimeError("Error(s) in loading state_dict for LokrNetwork:\n\t" + "\n\t".join(errors))
        return _IncompatibleKeys(missing, unexpected)


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
