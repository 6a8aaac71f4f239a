"""Precision modes of the DiT forward, with the call surface of anima-trainer's ``precision.py``.

Mirrored interface (anima-trainer ``src/anima_trainer/precision.py``): ``Mode`` (:35), ``torch_dtype``
(:38-44), ``autocast_for`` (:47-55), ``fp8_autocast_for`` (:58-66), ``quantize_dit_in_place`` (:69-77).

All three modes store activations, adapter deltas and base weights in bf16 and run the forward under bf16
autocast. ``mxfp8`` and ``fp8`` both mean "the quantised linears of this package": there is no block-FP8 /
Transformer Engine path on B200 here, every quantised GEMM is an MXFP8 tcgen05 GEMM that the patched modules
call explicitly (``fp8_quant``), so the FP8 gate the reference opens around the forward
(``te.fp8_autocast``) has nothing to switch and is a no-op context for every mode.
"""
from __future__ import annotations

from contextlib import contextmanager, nullcontext
from typing import Literal

import torch
import torch.nn as nn

Mode = Literal["bf16", "mxfp8", "fp8"]
MODES: tuple[str, ...] = ("bf16", "mxfp8", "fp8")


def _check(mode: str) -> None:
    if mode not in MODES:
        raise NotImplementedError(f"precision={mode!r}: only 'bf16', 'mxfp8', or 'fp8' is supported")


def torch_dtype(mode: Mode) -> torch.dtype:
    """Storage dtype of activations, adapter deltas and the base weights that get pre-quantised."""
    _check(mode)
    return torch.bfloat16


@contextmanager
def autocast_for(mode: Mode, device_type: str = "cuda"):
    """bf16 autocast for every mode; the quantised GEMMs are called explicitly by the patched modules."""
    _check(mode)
    with torch.autocast(device_type=device_type, dtype=torch.bfloat16):
        yield


def fp8_autocast_for(mode: Mode):
    """The gate a training loop opens around every DiT forward (train and sample). The reference enables
    Transformer Engine's FP8 autocast for ``fp8``; the MXFP8 operators here need no ambient state, so the gate
    validates the mode and returns a null context."""
    _check(mode)
    return nullcontext()


def quantize_dit_in_place(dit: nn.Module, mode: Mode, **_kwargs) -> None:
    """No-op for all modes: weights are quantised after the adapters are attached
    (``fp8_quant.quantize_frozen_linears`` / ``quantize_tlokr_base_weights``)."""
    _check(mode)
