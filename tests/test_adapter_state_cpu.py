"""CPU tests of the adapter wire format, the per-rank RNG state, the precision gate and the status check.

The cases follow the reference's own tests where it has them: atomic, replaceable adapter file that leaves no
temp file behind (``tests/test_checkpoint.py:14-33``), bf16-only tensors and the LoKr key set
(``tests/sanity_save_bf16.py:60-85``), the T-LoKr key set and int32 schedule marker
(``src/anima_trainer/tlokr.py:434-441``), rejection of a different schedule (``tlokr.py:305-327``), rejection of
a changed device count by the RNG restore (``training_state.py:260-267``; here: world size)."""
from __future__ import annotations

import os
import random
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
from safetensors import safe_open
from safetensors.torch import load_file

from anima_trainer_sm120_b200 import adapter_io, precision, training_state
from anima_trainer_sm120_b200.anima_dit import AnimaDiT, tiny_config
from anima_trainer_sm120_b200.lokr import attach_lokr

ROOT = Path(__file__).resolve().parents[1]


def _network(variant: str, rank: int = 8, ratio: float = 0.5):
    torch.manual_seed(3)
    dit = AnimaDiT(tiny_config(dim=128, heads=2, mlp_dim=256, context_dim=64, adaln_lora_dim=16, depth=2))
    net = attach_lokr(dit, preset="anima-cross-mlp", factor=8, dim=rank, alpha=rank, variant=variant,
                      timestep_min_rank_ratio=ratio)
    with torch.no_grad():
        for p in net.parameters():
            p.normal_(std=0.1)
    return dit, net


def test_reference_save_is_atomic_replaceable_and_bf16(tmp_path):
    # the reference's own case: any module, saved twice to the same path
    path = tmp_path / "adapter.safetensors"
    lin = torch.nn.Linear(3, 2)
    assert adapter_io._save_lora(lin, path) == 8
    first = load_file(path)
    assert first and all(t.dtype == torch.bfloat16 for t in first.values())
    with torch.no_grad():
        lin.weight.fill_(7)
    adapter_io.save_adapter(lin, path)
    second = load_file(path)
    torch.testing.assert_close(second["weight"], torch.full_like(second["weight"], 7), rtol=0, atol=0)
    assert list(tmp_path.glob(".adapter.safetensors.tmp-*")) == []


def test_failed_write_keeps_the_previous_file_and_no_temp(tmp_path, monkeypatch):
    path = tmp_path / "adapter.safetensors"
    lin = torch.nn.Linear(3, 2)
    adapter_io.save_adapter(lin, path)
    before = path.read_bytes()

    def boom(src, dst):
        raise OSError("disk full")
    monkeypatch.setattr(os, "replace", boom)
    with pytest.raises(OSError):
        adapter_io.save_adapter(lin, path)
    assert path.read_bytes() == before
    assert list(tmp_path.glob(".adapter.safetensors.tmp-*")) == []


def test_lokr_key_set_dtypes_and_metadata(tmp_path):
    _, net = _network("lokr")
    path = tmp_path / "a.safetensors"
    n = adapter_io.save_adapter(net, path)
    with safe_open(str(path), framework="pt") as f:
        keys, meta = set(f.keys()), f.metadata()
        tensors = {k: f.get_tensor(k) for k in keys}
    names = [m.lora_name for m in net.unet_loras]
    assert len(names) == 12 and all(nm.startswith("lokr_blocks_") for nm in names)
    assert keys == {f"{nm}.{leaf}" for nm in names for leaf in ("lokr_w1", "lokr_w2", "alpha")}
    assert all(t.dtype == torch.bfloat16 for t in tensors.values())
    assert not any("_mxfp8" in k for k in keys)
    assert meta == {"anima_adapter_type": "lokr", "anima_adapter_format": "1"}
    assert n == sum(t.numel() for t in tensors.values())


def test_tlokr_key_set_schedule_marker_and_round_trip(tmp_path):
    _, net = _network("tlokr", rank=8, ratio=0.5)
    path = tmp_path / "t.safetensors"
    adapter_io.save_adapter(net, path)
    tensors, meta = adapter_io.read_adapter(path)
    names = [m.lora_name for m in net.unet_loras]
    leaves = ("lokr_w1", "lokr_w2_a", "lokr_w2_b", "alpha", "tlokr_schedule")
    assert set(tensors) == {f"{nm}.{leaf}" for nm in names for leaf in leaves}
    assert meta["anima_adapter_type"] == "tlokr"
    for k, t in tensors.items():
        if k.endswith("tlokr_schedule"):
            assert t.dtype == torch.int32 and t.tolist() == [1, 8, 4]
        else:
            assert t.dtype == torch.bfloat16
    # round trip into a fresh network: values equal the bf16-rounded originals
    _, fresh = _network("tlokr", rank=8, ratio=0.5)
    with torch.no_grad():
        for p in fresh.parameters():
            p.zero_()
    adapter_io.load_adapter(fresh, path)
    for a, b in zip(net.parameters(), fresh.parameters()):
        assert torch.equal(a.detach().to(torch.bfloat16).float(), b.detach())


def test_loader_rejects_other_schedule_type_shape_and_keys(tmp_path):
    _, net = _network("tlokr", rank=8, ratio=0.5)
    path = tmp_path / "t.safetensors"
    adapter_io.save_adapter(net, path)
    _, other_sched = _network("tlokr", rank=8, ratio=1.0)        # min rank 8 instead of 4
    with pytest.raises(RuntimeError, match="tlokr_schedule is incompatible"):
        adapter_io.load_adapter(other_sched, path)
    _, plain = _network("lokr")
    with pytest.raises(RuntimeError, match="adapter type 'tlokr'"):
        adapter_io.load_adapter(plain, path)
    with pytest.raises(RuntimeError, match="Missing key"):
        plain.load_state_dict(adapter_io.read_adapter(path)[0], strict=True)
    lokr_path = tmp_path / "l.safetensors"
    adapter_io.save_adapter(plain, lokr_path)
    _, wide = _network("lokr", rank=16)
    sd = adapter_io.read_adapter(lokr_path)[0]
    key = next(k for k in sd if k.endswith("lokr_w2"))
    sd[key] = sd[key][:, :-1].contiguous()
    with pytest.raises(RuntimeError, match="size mismatch"):
        wide.load_state_dict(sd)
    sd = adapter_io.read_adapter(lokr_path)[0]
    sd["stray.lokr_w1"] = torch.zeros(1)
    with pytest.raises(RuntimeError, match="Unexpected key"):
        wide.load_state_dict(sd)
    assert wide.load_state_dict(sd, strict=False).unexpected_keys == ["stray.lokr_w1"]


def test_alpha_round_trips_into_the_scale(tmp_path):
    _, net = _network("lokr", rank=8)
    sd = {k: v.clone() for k, v in net.state_dict().items()}
    for k in sd:
        if k.endswith(".alpha"):
            sd[k] = torch.tensor(4.0)
    net.load_state_dict(sd)
    assert all(abs(m.scale - 0.5) < 1e-12 for m in net.unet_loras)


def test_rng_state_round_trip_single_process():
    torch.manual_seed(11); random.seed(11); np.random.seed(11)
    snap = training_state.capture_rng_state()
    want = (torch.rand(3), random.random(), np.random.rand(2))
    torch.rand(100); random.random(); np.random.rand(5)
    assert training_state.restore_rng_state(snap) == "restored"
    got = (torch.rand(3), random.random(), np.random.rand(2))
    assert torch.equal(want[0], got[0]) and want[1] == got[1] and np.array_equal(want[2], got[2])
    assert snap["rank"] == 0 and snap["world_size"] == 1 and snap["torch_cuda"] is None


def test_rng_restore_rejects_changed_world_size_unless_told_to_reseed():
    payload = {"world_size": 4, "ranks": [training_state.capture_rng_state() for _ in range(4)]}
    with pytest.raises(training_state.TrainingStateError, match="world size changed"):
        training_state.restore_rng_state(payload)
    assert training_state.restore_rng_state(payload, on_world_change="reseed") == "reseeded"
    a = torch.rand(4)
    assert training_state.restore_rng_state(payload, on_world_change="reseed") == "reseeded"
    assert torch.equal(a, torch.rand(4))                       # deterministic in (checkpoint, rank)
    with pytest.raises(ValueError):
        training_state.restore_rng_state(payload, on_world_change="ignore")


def test_precision_modes_and_errors():
    for mode in ("bf16", "mxfp8", "fp8"):
        assert precision.torch_dtype(mode) is torch.bfloat16
        with precision.autocast_for(mode, "cpu"), precision.fp8_autocast_for(mode):
            y = torch.nn.functional.linear(torch.randn(2, 4), torch.randn(3, 4))
        assert y.dtype is torch.bfloat16
        precision.quantize_dit_in_place(torch.nn.Identity(), mode)
    for fn in (precision.torch_dtype, precision.fp8_autocast_for,
               lambda m: precision.quantize_dit_in_place(torch.nn.Identity(), m)):
        with pytest.raises(NotImplementedError):
            fn("fp4")
    with pytest.raises(NotImplementedError):
        with precision.autocast_for("int8", "cpu"):
            pass


def test_nonzero_status_words_raise(monkeypatch):
    from anima_trainer_sm120_b200 import _lib

    class FakeWord:
        def __init__(self, v): self.v = v
        def item(self): return self.v
        def zero_(self): self.v = 0
    dev = torch.device("cuda", 0)
    monkeypatch.setitem(_lib._status_words, 0, FakeWord(1))
    with pytest.raises(RuntimeError, match="bounded wait"):
        _lib.check_status_word(dev)
    _lib.check_status_word(dev)                                 # cleared by the failed check

    class FakeLib:
        def __init__(self, rc): self.rc = rc
        def anima_mx_quantize_status(self): return self.rc
        def anima_last_error(self): return b"mx_quantize_status: boom"
    monkeypatch.setattr(_lib, "load", lambda: FakeLib(1))
    with pytest.raises(RuntimeError, match="timed out"):
        _lib.check_quantize_status()
    monkeypatch.setattr(_lib, "load", lambda: FakeLib(0))
    _lib.check_quantize_status()
    monkeypatch.setattr(_lib, "load", lambda: FakeLib(-4))
    with pytest.raises(RuntimeError, match="boom"):
        _lib.check_quantize_status()


def _torchrun(script: Path, args: list[str], port: int, timeout: int = 600):
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", OMP_NUM_THREADS="2")
    return subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                           "--master-addr", "127.0.0.1", "--master-port", str(port), str(script), *args],
                          capture_output=True, text=True, env=env, timeout=timeout, cwd=ROOT)


def test_two_ranks_rank0_writes_and_reload_reproduces_next_step(tmp_path):
    """world_size 2 (gloo): after one step only rank 0 has written the adapter file; both ranks reload it and
    the RNG payload into fresh trainers and the next step gives bit-identical adapters and losses to the run
    that simply continued (from the same bf16-rounded adapters and optimizer state)."""
    res = _torchrun(ROOT / "tests" / "dp_resume_worker.py", [str(tmp_path)], 29533)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
    out = [torch.load(tmp_path / f"resume_rank{r}.pt") for r in (0, 1)]
    assert out[0]["writers"] == [0]
    for o in out:
        assert o["rng"] == "restored" and o["world_change"] == "TrainingStateError"
        assert o["loss_continued"] == o["loss_resumed"]
        for a, b in zip(o["continued"], o["resumed"]):
            assert torch.equal(a, b)
    for a, b in zip(out[0]["resumed"], out[1]["resumed"]):
        assert torch.equal(a, b)


def test_a_rank_that_fails_before_the_exchange_gives_the_survivor_a_clean_error(tmp_path):
    """Rank 1 raises before its all-reduce; rank 0's exchange ends with an error within the process group's
    short timeout instead of hanging (host-side failure only: gloo on CPU)."""
    res = _torchrun(ROOT / "tests" / "dp_failure_worker.py", [str(tmp_path)], 29535, timeout=300)
    note = (tmp_path / "survivor.txt")
    assert note.exists(), res.stdout[-2000:] + res.stderr[-2000:]
    kind, seconds = note.read_text().split("|")[:2]
    assert kind in ("RuntimeError", "DistBackendError", "DistNetworkError"), kind
    assert float(seconds) < 60.0
