"""Per-rank RNG capture and restore for the data-parallel training step.

anima-trainer is single-process: ``capture_rng_state`` / ``restore_rng_state``
(``src/anima_trainer/training_state.py:239-278``) snapshot the CPU generator, EVERY visible CUDA device's
generator, Python's and numpy's, and refuse a checkpoint when the CUDA device count changed (:262-266). Under
one process per GPU that rule has to become per rank:

* a rank captures only the generator of ITS device, tagged with ``(rank, world_size)``;
* :func:`gather_rng_states` collects the ranks' snapshots on rank 0 so they go into one checkpoint payload;
* :func:`restore_rng_state` gives each rank its own snapshot back when the world size is unchanged; a changed
  world size raises :class:`TrainingStateError` (the reference's behaviour) unless the caller asks for
  ``on_world_change="reseed"``, in which case every rank derives a fresh seed from the checkpoint's rank-0 CPU
  state and its new rank - deterministic, but explicitly not a bit-exact continuation.

The rest of the reference module (payload files, manifests, dataset fingerprints) is its storage engine and is
not part of this package.
"""
from __future__ import annotations

import hashlib
import io
import random
from typing import Any

import numpy as np
import torch
import torch.distributed as dist


class TrainingStateError(RuntimeError):
    """Saved state is incompatible with this process group or cannot be restored safely."""


def _world() -> tuple[int, int]:
    if dist.is_available() and dist.is_initialized():
        return dist.get_rank(), dist.get_world_size()
    return 0, 1


def capture_rng_state(device: torch.device | None = None) -> dict[str, Any]:
    """This rank's generators: torch CPU, torch CUDA of ``device`` (default: the current device, if CUDA is
    initialised), Python ``random`` and numpy's global state."""
    rank, world = _world()
    np_name, np_keys, np_pos, np_has_gauss, np_cached = np.random.get_state()
    cuda_state = None
    if torch.cuda.is_available() and torch.cuda.is_initialized():
        dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        if dev.type == "cuda":
            cuda_state = torch.cuda.get_rng_state(dev).clone().cpu()
    return {
        "rank": rank,
        "world_size": world,
        "torch_cpu": torch.get_rng_state().clone(),
        "torch_cuda": cuda_state,
        "python": random.getstate(),
        "numpy": {"name": np_name, "keys": torch.from_numpy(np_keys.copy()), "pos": int(np_pos),
                  "has_gauss": int(np_has_gauss), "cached_gaussian": float(np_cached)},
    }


def gather_rng_states(device: torch.device | None = None) -> dict[str, Any] | None:
    """Every rank calls this; rank 0 gets ``{"world_size": W, "ranks": [state_0, ..., state_{W-1}]}`` to put
    into the checkpoint it writes, the other ranks get None."""
    rank, world = _world()
    mine = capture_rng_state(device)
    if world == 1:
        return {"world_size": 1, "ranks": [mine]}
    # the snapshot travels as one bytes object: tensors nested in pickled objects do not survive every backend
    buf = io.BytesIO()
    torch.save(mine, buf)
    bucket = [None] * world if rank == 0 else None
    dist.gather_object(buf.getvalue(), bucket, dst=0)
    if rank != 0:
        return None
    return {"world_size": world, "ranks": [torch.load(io.BytesIO(b), weights_only=False) for b in bucket]}


def _reseed(payload: dict[str, Any], rank: int, device: torch.device | None) -> None:
    digest = hashlib.sha256(payload["ranks"][0]["torch_cpu"].numpy().tobytes()).digest()
    seed = (int.from_bytes(digest[:8], "little") + 0x9E3779B97F4A7C15 * (rank + 1)) % (2 ** 63)
    torch.manual_seed(seed)
    if torch.cuda.is_available() and torch.cuda.is_initialized():
        dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        if dev.type == "cuda":
            idx = dev.index if dev.index is not None else torch.cuda.current_device()
            torch.cuda.default_generators[idx].manual_seed(seed)
    random.seed(seed)
    np.random.seed(seed % (2 ** 32))


def restore_rng_state(payload: dict[str, Any], device: torch.device | None = None, *,
                      on_world_change: str = "error") -> str:
    """Restore this rank's generators from a payload made by :func:`gather_rng_states` (or from one rank's
    :func:`capture_rng_state` dict in a single-process run). Returns ``"restored"`` or ``"reseeded"``.

    ``on_world_change``: ``"error"`` (default) raises when the payload was written by a different number of
    ranks, as the reference raises on a changed device count; ``"reseed"`` accepts it and seeds every rank
    afresh from the checkpoint (deterministic in (checkpoint, rank), not a continuation of any saved stream)."""
    if on_world_change not in ("error", "reseed"):
        raise ValueError("on_world_change must be 'error' or 'reseed'")
    if "ranks" not in payload:                      # a bare single-rank snapshot
        payload = {"world_size": payload.get("world_size", 1), "ranks": [payload]}
    rank, world = _world()
    saved_world = int(payload["world_size"])
    if saved_world != world or len(payload["ranks"]) != saved_world:
        if on_world_change == "error":
            raise TrainingStateError(f"world size changed: checkpoint has RNG state of {saved_world} rank(s), "
                                     f"this job runs {world}; pass on_world_change='reseed' to continue with "
                                     "fresh per-rank seeds")
        _reseed(payload, rank, device)
        return "reseeded"
    state = payload["ranks"][rank]
    if int(state.get("rank", rank)) != rank:
        raise TrainingStateError(f"RNG snapshot {rank} of the checkpoint belongs to rank {state.get('rank')}")
    torch.set_rng_state(state["torch_cpu"].cpu())
    cuda_state = state.get("torch_cuda")
    if cuda_state is not None:
        if not torch.cuda.is_available():
            raise TrainingStateError("saved state contains CUDA RNG state but CUDA is unavailable")
        dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        torch.cuda.set_rng_state(cuda_state.cpu(), dev)
    random.setstate(state["python"])
    n = state["numpy"]
    np.random.set_state((n["name"], n["keys"].cpu().numpy().astype(np.uint32, copy=True), int(n["pos"]),
                         int(n["has_gauss"]), float(n["cached_gaussian"])))
    return "restored"
