"""CPU tests of the host-side module layer (no kernel calls): T-LoKr schedule / context / conversion,
AdaLN-modulation merge, the LoKr patch's bf16 path, preset coverage, and the data-parallel step on
two gloo ranks. Known answers and expectations follow the reference's ``tests/test_tlokr.py``."""
from __future__ import annotations

import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

from anima_trainer_sm120_b200 import adaln_merge, lokr_patch, tlokr
from anima_trainer_sm120_b200.anima_dit import AnimaConfig, AnimaDiT, tiny_config
from anima_trainer_sm120_b200.lokr import LokrModule, LokrNetwork, attach_lokr

ROOT = Path(__file__).resolve().parents[1]


def test_schedule_known_answers(golden):
    # tests/test_tlokr.py:59-76 of the reference
    assert tlokr.active_rank_for_timestep(1.0, max_rank=128, min_rank=64) == 64
    assert tlokr.active_rank_for_timestep(0.5, max_rank=128, min_rank=64) == 96
    assert tlokr.active_rank_for_timestep(0.0, max_rank=128, min_rank=64) == 128
    assert tlokr.active_rank_for_timestep(2.0, max_rank=8, min_rank=4) == 4
    assert tlokr.active_rank_for_timestep(-1.0, max_rank=8, min_rank=4) == 8
    g = golden("tlokr")
    for (t, a, b), want in zip(g["sched_cases"], g["sched_out"]):
        assert tlokr.active_rank_for_timestep(t, max_rank=int(a), min_rank=int(b)) == int(want)
    with pytest.raises(ValueError):
        tlokr.active_rank_for_timestep(0.5, max_rank=0, min_rank=1)
    with pytest.raises(ValueError):
        tlokr.active_rank_for_timestep(0.5, max_rank=4, min_rank=5)
    st = tlokr._TimestepState(timesteps=torch.from_numpy(g["mask_t"]))
    m = st.mask(max_rank=128, min_rank=64, dtype=torch.float32, device=torch.device("cpu"))
    assert np.array_equal(m.numpy(), g["mask"])
    assert st.mask(max_rank=128, min_rank=64, dtype=torch.float32, device=torch.device("cpu")) is m  # cached


def _module(in_f=16, out_f=16, factor=2, rank=4):
    torch.manual_seed(7)
    lin = torch.nn.Linear(in_f, out_f, bias=True).requires_grad_(False)
    mod = LokrModule("test_lokr", lin, lora_dim=rank, alpha=rank, factor=factor)
    net = LokrNetwork([mod])
    lokr_patch.install()
    return net, mod, lin


def test_conversion_and_context_errors():
    net, mod, lin = _module()
    assert tlokr.convert_network(net, rank=4, min_rank_ratio=0.5) == 1
    assert not hasattr(mod, "lokr_w2") and mod.lokr_w2_a.shape == (8, 4) and mod.lokr_w2_b.shape == (4, 8)
    assert not mod.lokr_w2_b.any() and mod._tlokr_min_rank == 2 and mod._tlokr_rank == 4
    assert mod.tlokr_schedule.tolist() == [1, 4, 2] and mod.tlokr_schedule.dtype == torch.int32
    assert "tlokr_schedule" in mod.custom_state_dict()
    tlokr.clear_timestep()
    with pytest.raises(RuntimeError, match="timestep context"):
        mod(torch.randn(2, 3, 16))
    with pytest.raises(TypeError):
        tlokr.set_timestep([0.1, 0.2])
    with pytest.raises(ValueError):
        tlokr.convert_network(LokrNetwork([_module()[1]]), rank=64, min_rank_ratio=0.5)   # exceeds factor capacity
    with pytest.raises(ValueError):
        tlokr.convert_network(LokrNetwork([_module()[1]]), rank=4, min_rank_ratio=0.0)
    with pytest.raises(RuntimeError):
        tlokr.convert_network(torch.nn.Module(), rank=4, min_rank_ratio=0.5)
    # batch / timestep mismatch is reported before any kernel runs
    tlokr.set_timestep(torch.tensor([0.1, 0.2, 0.3]))
    try:
        with pytest.raises(RuntimeError, match="does not match timestep batch"):
            mod(torch.randn(2, 3, 16))
    finally:
        tlokr.clear_timestep()


def test_lokr_patch_bf16_path_matches_stock_forward():
    net, mod, lin = _module()
    with torch.no_grad():
        mod.lokr_w2.normal_(std=0.2)
    x = torch.randn(2, 5, 16)
    want = lin(x) + torch.nn.functional.linear(x, torch.kron(mod.lokr_w1, mod.lokr_w2) * mod.scale)
    torch.testing.assert_close(mod(x), want, rtol=1e-5, atol=1e-6)
    mod.apply_to()
    torch.testing.assert_close(lin(x), want, rtol=1e-5, atol=1e-6)     # wrapped Linear now routes through the adapter
    # zero-initialised delta leaves the base output exact
    net2, mod2, lin2 = _module()
    assert torch.equal(mod2(x), torch.nn.functional.linear(x, lin2.weight, lin2.bias))
    assert lokr_patch._mark_fp8_eligible(net) == 0          # 16 x 16 is not 32-aligned


@pytest.mark.parametrize("lora", [True, False])
def test_adaln_merge_is_exact(lora):
    torch.manual_seed(0)
    dit = AnimaDiT(tiny_config(use_adaln_lora=lora)).eval()
    blk = dit.blocks[0]
    emb = torch.randn(2, 1, 256)
    al = torch.randn(2, 1, 768) if lora else None
    want = [blk._mod(getattr(blk, n), emb, al) for n in adaln_merge._NAMES]
    assert adaln_merge.merge_adaln_modulation(dit) == 2 and adaln_merge.merge_adaln_modulation(dit) == 0
    got = adaln_merge.apply_merged_adaln(blk, emb, al)
    for w3, g3 in zip(want, got):
        for w, g in zip(w3, g3):
            torch.testing.assert_close(g, w, rtol=1e-5, atol=1e-6)
    assert "adaln_modulation_l2_stack" not in dit.state_dict() or not lora


def test_preset_covers_168_modules_at_production_shape():
    with torch.device("meta"):
        dit = AnimaDiT(AnimaConfig())
        net = attach_lokr(dit, preset="anima-cross-mlp")
    mods = list(net.unet_loras)
    assert len(mods) == 168                                     # 28 blocks x (cross q,k,v,o + mlp.layer1,2)
    shapes = {tuple(m.lokr_w2.shape) for m in mods}
    assert shapes == {(256, 256), (256, 128), (1024, 256), (256, 1024)}
    assert all(tuple(m.lokr_w1.shape) == (8, 8) for m in mods)
    n_params = sum(p.numel() for p in net.parameters())
    assert n_params == 20_195_840                               # the reference's LoKr parameter count
    assert not any(p.requires_grad for p in dit.parameters())
    assert lokr_patch._mark_fp8_eligible(net) == 168


def test_data_parallel_step_two_gloo_ranks(tmp_path):
    """world_size 2 on CPU (gloo, bf16 arm): after a step both ranks hold identical adapters, equal to a
    single process that averages the two ranks' gradients by hand."""
    script = ROOT / "tests" / "dp_worker.py"
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", OMP_NUM_THREADS="2")
    res = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                          "--master-addr", "127.0.0.1", "--master-port", "29531", str(script), str(tmp_path)],
                         capture_output=True, text=True, env=env, timeout=600, cwd=ROOT)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
    r0, r1, ref = (torch.load(tmp_path / f"{n}.pt") for n in ("rank0", "rank1", "single"))
    assert r0["losses"] != r1["losses"]                         # different shards
    for a, b in zip(r0["params"], r1["params"]):
        assert torch.equal(a, b)
    for a, b in zip(r0["params"], ref["params"]):
        torch.testing.assert_close(a, b, rtol=1e-4, atol=1e-6)
