"""Adapter wire format: the ``*.safetensors`` file a LoKr / T-LoKr run publishes, and its loader.

Format, as anima-trainer writes it (``src/anima_trainer/train.py:508-545``):
* tensors = ``network.state_dict()``; floating tensors cast to bf16, integer tensors kept (the T-LoKr marker
  ``tlokr_schedule = [format, rank, min_rank]`` stays int32, ``tlokr.py:436-440``);
* keys ``{lora_name}.lokr_w1 / .lokr_w2 / .alpha`` for LoKr (``tests/sanity_save_bf16.py:78``) and
  ``{lora_name}.lokr_w1 / .lokr_w2_a / .lokr_w2_b / .alpha / .tlokr_schedule`` for T-LoKr
  (``docs/tlokr-melted1-fp8-ab.md:116-122``);
* metadata ``anima_adapter_type`` ("lokr" | "tlokr") and ``anima_adapter_format`` ("1");
* publication is atomic: uniquely named temp file in the target directory -> fsync -> ``os.replace`` -> fsync of
  the directory; a crash leaves the previous file or the new one, never a torn one, and no temp file survives.

Data-parallel use: adapters are replicated, so only rank 0 writes; every rank then waits at a barrier, after
which the file is complete for all of them. Loading is done by every rank from the same file, and a T-LoKr file
whose schedule differs from the network's is rejected (the reference's ``_validate_schedule_on_load``,
``tlokr.py:305-327``).
"""
from __future__ import annotations

import os
from pathlib import Path
from uuid import uuid4

import torch
import torch.distributed as dist

ADAPTER_FORMAT = "1"


def _dist_on() -> bool:
    return dist.is_available() and dist.is_initialized()


def adapter_tensors(network: torch.nn.Module) -> dict[str, torch.Tensor]:
    """The tensors that go on the wire: floats as bf16 on the CPU, integer tensors unchanged."""
    return {k: (v.detach().to(torch.bfloat16).cpu() if v.is_floating_point() else v.detach().cpu()).contiguous()
            for k, v in network.state_dict().items()}


def save_adapter(network: torch.nn.Module, path: str | os.PathLike, *, all_ranks: bool = False) -> int:
    """Publish the adapter atomically; returns the number of parameters written (0 on ranks that do not write).
    With a process group only rank 0 writes (``all_ranks=True`` lets every rank write its own ``path``); every
    rank leaves through a barrier, so the file exists for all of them on return."""
    from safetensors.torch import save_file

    path = Path(path)
    rank = dist.get_rank() if _dist_on() else 0
    written = 0
    try:
        if rank == 0 or all_ranks:
            sd = adapter_tensors(network)
            adapter_type = "tlokr" if getattr(network, "_tlokr_enabled", False) else "lokr"
            temp = path.with_name(f".{path.name}.tmp-{os.getpid()}-{uuid4().hex}")
            try:
                save_file(sd, str(temp), metadata={"anima_adapter_type": adapter_type,
                                                   "anima_adapter_format": ADAPTER_FORMAT})
                with temp.open("rb") as handle:
                    os.fsync(handle.fileno())
                os.replace(temp, path)
                try:
                    fd = os.open(path.parent, os.O_RDONLY | getattr(os, "O_DIRECTORY", 0))
                except OSError:
                    fd = None
                if fd is not None:
                    try:
                        os.fsync(fd)
                    finally:
                        os.close(fd)
            finally:
                temp.unlink(missing_ok=True)
            written = sum(t.numel() for t in sd.values())
    finally:
        if _dist_on():
            dist.barrier()
    return written


_save_lora = save_adapter   # the reference's name (train.py:508)


def read_adapter(path: str | os.PathLike) -> tuple[dict[str, torch.Tensor], dict[str, str]]:
    """(tensors, metadata) of an adapter file."""
    from safetensors import safe_open

    tensors: dict[str, torch.Tensor] = {}
    with safe_open(str(path), framework="pt", device="cpu") as f:
        meta = dict(f.metadata() or {})
        for k in f.keys():
            tensors[k] = f.get_tensor(k)
    return tensors, meta


def load_adapter(network: torch.nn.Module, path: str | os.PathLike, *, strict: bool = True) -> dict[str, str]:
    """Load an adapter file into ``network`` (every rank reads the same file). Rejects a file of the other adapter
    type, an unknown format number, and - through ``network.load_state_dict`` - missing / unexpected keys,
    shape mismatches and a T-LoKr schedule that differs from the network's. Returns the file's metadata."""
    tensors, meta = read_adapter(path)
    want = "tlokr" if getattr(network, "_tlokr_enabled", False) else "lokr"
    got = meta.get("anima_adapter_type")
    if got is not None and got != want:
        raise RuntimeError(f"{path}: adapter type {got!r} cannot be loaded into a {want!r} network")
    fmt = meta.get("anima_adapter_format")
    if fmt is not None and fmt != ADAPTER_FORMAT:
        raise RuntimeError(f"{path}: adapter format {fmt!r} is not supported (expected {ADAPTER_FORMAT!r})")
    network.load_state_dict(tensors, strict=strict)
    return meta
