"""Host-side logic that needs no GPU: the activation-quantisation memo, the checkpoint first-pass flag, the
T-LoKr dispatch plan, and the fall-through of the MLP / q-k patches on CPU tensors."""
from __future__ import annotations

import gc

import pytest
import torch

from anima_trainer_sm120_b200 import fp8_quant, mlp_patch, ops, qk_norm_rope, tlokr
from anima_trainer_sm120_b200.anima_dit import Attention, GPT2FeedForward, tiny_config


@pytest.fixture
def fake_quantiser(monkeypatch):
    """Replace the CUDA quantiser by a counter that returns distinguishable operands."""
    calls = []

    def fake(x2d, *, rowwise=True, colwise=False, layout=1):
        calls.append((tuple(x2d.shape), rowwise, colwise))
        row = ops.MXOperand(torch.zeros(1, dtype=torch.uint8), torch.tensor([len(calls)], dtype=torch.uint8), layout)
        col = ops.MXOperand(torch.ones(1, dtype=torch.uint8), torch.tensor([len(calls)], dtype=torch.uint8), layout)
        return row, (col if colwise else None)

    monkeypatch.setattr(ops, "mx_quantize", fake)
    fp8_quant.clear_activation_memo()
    fp8_quant.act_memo_stats.update(hits=0, misses=0, adopted=0)
    yield calls
    fp8_quant.clear_activation_memo()


def test_memo_hits_on_the_tensor_and_on_contiguous_views_of_all_of_it(fake_quantiser):
    x = torch.zeros(64, 32, dtype=torch.bfloat16)
    r1, c1 = fp8_quant.quantize_activation(x, colwise=False)
    r2, _ = fp8_quant.quantize_activation(x, colwise=False)
    assert r2 is r1 and c1 is None and len(fake_quantiser) == 1
    r3, _ = fp8_quant.quantize_activation(x.view(2, 32, 32), colwise=False)   # same bytes, same row length
    assert r3 is r1 and len(fake_quantiser) == 1
    fp8_quant.quantize_activation(x.view(32, 64), colwise=False)              # other row length: other operand
    assert len(fake_quantiser) == 2
    fp8_quant.quantize_activation(x[:32], colwise=False)                      # part of the tensor
    assert len(fake_quantiser) == 3
    fp8_quant.quantize_activation(torch.zeros(64, 32, dtype=torch.bfloat16), colwise=False)   # equal values, other tensor
    assert len(fake_quantiser) == 4
    assert fp8_quant.act_memo_stats == {"hits": 2, "misses": 4, "adopted": 0}


def test_memo_adopts_an_operand_made_by_the_producer(fake_quantiser):
    y = torch.zeros(2, 64, 32, dtype=torch.bfloat16)
    made = ops.MXOperand(torch.zeros(128, 32, dtype=torch.uint8), torch.zeros(512, dtype=torch.uint8), 1)
    fp8_quant.adopt_row_operand(y, made)
    row, col = fp8_quant.quantize_activation(y.reshape(2, 64, 32).view(128, 32), colwise=False)
    assert row is made and col is None and len(fake_quantiser) == 0
    row, col = fp8_quant.quantize_activation(y, colwise=True)                 # only the missing form is made
    assert row is made and col is not None and fake_quantiser == [((128, 32), False, True)]
    y.mul_(2)
    fp8_quant.quantize_activation(y, colwise=False)                           # stale after an in-place change
    assert len(fake_quantiser) == 2
    with pytest.raises(ValueError):
        fp8_quant.adopt_row_operand(y.transpose(0, 1), made)


def test_memo_misses_after_in_place_change_and_when_a_form_is_missing(fake_quantiser):
    x = torch.zeros(64, 32, dtype=torch.bfloat16)
    fp8_quant.quantize_activation(x, colwise=False)
    _, col = fp8_quant.quantize_activation(x, colwise=True)             # entry has no column form: make that one
    assert col is not None and fake_quantiser[1] == ((64, 32), False, True)
    row, col2 = fp8_quant.quantize_activation(x, colwise=True)          # now both forms are there
    assert col2 is col and len(fake_quantiser) == 2
    row_only, none = fp8_quant.quantize_activation(x, colwise=False)    # a richer entry serves a poorer request
    assert row_only is row and none is None and len(fake_quantiser) == 2
    x.add_(1)
    fp8_quant.quantize_activation(x, colwise=False)
    assert len(fake_quantiser) == 3


def test_memo_keeps_two_tensors_and_forgets_dead_ones(fake_quantiser):
    a, b, c = (torch.zeros(32, 32, dtype=torch.bfloat16) for _ in range(3))
    for t in (a, b):
        fp8_quant.quantize_activation(t, colwise=False)
    fp8_quant.quantize_activation(a, colwise=False)                     # a and b both still held
    fp8_quant.quantize_activation(b, colwise=False)
    assert len(fake_quantiser) == 2
    fp8_quant.quantize_activation(c, colwise=False)                     # evicts the least recently used (a)
    fp8_quant.quantize_activation(a, colwise=False)
    assert len(fake_quantiser) == 4
    del c
    gc.collect()
    fresh = torch.zeros(32, 32, dtype=torch.bfloat16)                   # may reuse c's address: must not hit
    fp8_quant.quantize_activation(fresh, colwise=False)
    assert len(fake_quantiser) == 5


def test_first_pass_flag_nests_and_resets():
    assert not fp8_quant.in_first_pass()
    with fp8_quant.first_pass():
        assert fp8_quant.in_first_pass()
        with fp8_quant.first_pass():
            assert fp8_quant.in_first_pass()
        assert fp8_quant.in_first_pass()
    assert not fp8_quant.in_first_pass()
    with pytest.raises(RuntimeError):
        with fp8_quant.first_pass():
            raise RuntimeError("boom")
    assert not fp8_quant.in_first_pass()


def _tlokr_module(in_f=256, out_f=256, rank=16):
    from anima_trainer_sm120_b200 import lokr_patch
    from anima_trainer_sm120_b200.lokr import LokrModule, LokrNetwork
    lin = torch.nn.Linear(in_f, out_f, bias=False).requires_grad_(False)
    mod = LokrModule("t", lin, lora_dim=rank, alpha=rank, factor=8)
    net = LokrNetwork([mod])
    lokr_patch.install()
    tlokr.convert_network(net, rank=rank, min_rank_ratio=0.5)
    return mod


def test_delta_plan_follows_the_timestep_context():
    mod = _tlokr_module()
    x = torch.zeros(2, 8, 256, dtype=torch.bfloat16)
    try:
        tlokr.set_timestep(torch.tensor([0.1, 0.9]))
        fn, a, b, mask = tlokr._delta_plan(mod, x, fp8=False)
        assert fn is tlokr._StructuredLoKr and a is mod.lokr_w2_a and tuple(mask.shape) == (2, 16)
        spec = tlokr._ActSpec((2, 8, 256), torch.bfloat16, torch.device("cpu"))      # a shape stands in for a tensor
        fn2, _, _, mask2 = tlokr._delta_plan(mod, spec, fp8=False)
        assert fn2 is fn and torch.equal(mask2, mask)
        tlokr.set_timestep(torch.tensor([1.0, 1.0]), uniform_timestep=1.0)           # 8 active ranks: sliced factors
        fn, a, b, mask = tlokr._delta_plan(mod, x, fp8=True)
        assert mask is None and a.shape[1] == 8 and b.shape[0] == 8
        assert fn is tlokr._StructuredLoKr                                             # 8 % 32 != 0: no MXFP8 GEMM
        with pytest.raises(RuntimeError):                                              # width not divisible by 8
            tlokr._delta_plan(mod, torch.zeros(2, 8, 252, dtype=torch.bfloat16), fp8=False)
    finally:
        tlokr.clear_timestep()
    assert tlokr.single_node_plan(mod, x) is None                                      # CPU tensor, no quantised base


def test_patches_fall_through_on_cpu():
    cfg = tiny_config(dim=256, heads=2, mlp_dim=512)
    mlp = GPT2FeedForward(cfg)
    x = torch.randn(2, 8, 256)
    ref = mlp(x)
    mlp_patch.install(GPT2FeedForward)
    try:
        assert torch.equal(mlp(x), ref)
    finally:
        mlp_patch.uninstall(GPT2FeedForward)
    attn = Attention(cfg, None)
    rope = torch.rand(8, 1, 1, 128)
    ref = attn(x, None, None, rope_emb=rope)
    qk_norm_rope.install(Attention)
    try:
        assert torch.equal(attn(x, None, None, rope_emb=rope), ref)
    finally:
        qk_norm_rope.uninstall(Attention)


def test_producer_side_quantisation_is_offered_only_for_shapes_the_kernels_tile():
    from anima_trainer_sm120_b200 import adaln_kernel
    assert ops.can_emit_row_codes(32768, 2048) and ops.can_emit_row_codes(128, 128)
    assert not ops.can_emit_row_codes(0, 2048)            # nothing to do
    assert not ops.can_emit_row_codes(96, 2048)           # tiled scales need whole 128-row chunks
    assert not ops.can_emit_row_codes(128, 2080)          # and whole 128-column chunks
    assert not ops.can_emit_row_codes(128, 8192)          # longer than the AdaLN kernels' longest row
    assert ops.can_quantise_rank_mix(8, 4096, 128) and ops.can_quantise_rank_mix(1, 16, 512)
    assert not ops.can_quantise_rank_mix(8, 4096, 64) and not ops.can_quantise_rank_mix(1, 24, 128)
    x = torch.zeros(1, 1, 8, 16, 256, dtype=torch.bfloat16)
    assert not adaln_kernel._emits(x, 128, 256)           # off unless switched on
    adaln_kernel.emit_row_operand(True)
    try:
        assert adaln_kernel._emits(x, 128, 256)
        assert not adaln_kernel._emits(x.float(), 128, 256)   # the fp32 path returns a cast copy: nothing to adopt
        assert not adaln_kernel._emits(x, 120, 256)
    finally:
        adaln_kernel.emit_row_operand(False)


def test_factor_forms_are_kept_per_parameter_version(monkeypatch):
    calls = []

    def fake_q(t, *, col=False):
        calls.append(tuple(t.shape))
        return ("row", len(calls)), ("col", len(calls))

    monkeypatch.setattr(tlokr, "_q", fake_q)
    p = torch.nn.Parameter(torch.randn(16, 8))
    first = tlokr._factor_forms(p, quantise=True)
    assert tlokr._factor_forms(p, quantise=True) is first and len(calls) == 1      # same values: no new launch
    c = tlokr._factor_forms(p, quantise=False)
    assert c.dtype == torch.bfloat16 and tlokr._factor_forms(p, quantise=False) is c
    with torch.no_grad():
        p.add_(1.0)                                                               # what an optimizer step does
    assert tlokr._factor_forms(p, quantise=True) is not first and len(calls) == 2
    assert tlokr._factor_forms(p, quantise=False) is not c
    assert torch.equal(tlokr._factor_forms(p, quantise=False), p.detach().to(torch.bfloat16))
    sliced = p[:, :4]                                                            # computed factors are never kept
    tlokr._factor_forms(sliced, quantise=True)
    tlokr._factor_forms(sliced, quantise=True)
    assert len(calls) == 4


# ----------------------------------------------------------------------------- GEMM work list (CTA-pair kernel)
def _pair_plan(M, N, K, ws=1):
    import ctypes

    from anima_trainer_sm120_b200 import _lib
    out = (ctypes.c_int32 * 9)()
    rc = _lib.load().anima_mx_gemm_pair_plan(M, N, K, ws, out)
    return rc, dict(zip(("pairs", "n_wide", "narrow", "full_items", "tail_tiles", "splits", "kbs", "shift", "bn"), out))


def _walk_plan(M, N, K, pl):
    """The device-side decode of the work list restated: {(mt, nt): [(kb0, kb1, pair, partial slot)]}."""
    m_tiles, kb = -(-M // 256), -(-K // 128)
    n_tiles = pl["n_wide"] + pl["narrow"]

    def coords(tile):
        if m_tiles < n_tiles:
            return tile % m_tiles, tile // m_tiles
        return tile // n_tiles, tile % n_tiles

    split_items = pl["tail_tiles"] * pl["splits"]
    slots = pl["full_items"] + (pl["shift"] + split_items if split_items else 0)
    cover: dict = {}
    for slot in range(slots):
        pair = slot % pl["pairs"]
        kb0, kb1, part, tile = 0, kb, -1, slot
        if slot >= pl["full_items"]:
            r = slot - pl["full_items"] - pl["shift"]
            if r < 0:
                continue
            t, sp = divmod(r, pl["splits"])
            tile = pl["full_items"] + t
            if pl["splits"] > 1:
                kb0, kb1, part = sp * pl["kbs"], min(kb, (sp + 1) * pl["kbs"]), r
        cover.setdefault(coords(tile), []).append((kb0, kb1, pair, part))
    return cover


@pytest.mark.parametrize("M,N,K", [
    (32768, 2048, 2048), (32768, 6144, 2048), (32768, 8192, 2048), (32768, 2048, 8192),      # forward / dgrad
    (2048, 2048, 32768), (6144, 2048, 32768), (8192, 2048, 32768), (2048, 8192, 32768),      # weight gradients
    (4096, 2048, 1024), (2048, 1024, 4096), (512, 512, 16384), (257, 384, 416), (130, 264, 160), (256, 136, 32),
])
@pytest.mark.parametrize("ws", [0, 1])
@pytest.mark.parametrize("width", [0, 192, 256])
def test_pair_kernel_work_list_covers_every_tile_and_k_block_once(M, N, K, ws, width, monkeypatch):
    if width:
        monkeypatch.setenv("ANIMA_MX_GEMM_BN", str(width))
    rc, pl = _pair_plan(M, N, K, ws)
    assert rc == 0
    bn = pl["bn"]
    assert bn == (width or (256 if K >= 4096 else 192))
    m_tiles, kb = -(-M // 256), -(-K // 128)
    n_cols = pl["n_wide"] + pl["narrow"]
    assert pl["n_wide"] * bn + 128 * pl["narrow"] >= N > (n_cols - 1) * bn
    assert pl["full_items"] % pl["pairs"] == 0 and pl["full_items"] + pl["tail_tiles"] == m_tiles * n_cols
    assert pl["pairs"] <= 74 and (ws or pl["splits"] == 1)
    cover = _walk_plan(M, N, K, pl)
    assert set(cover) == {(mt, nt) for mt in range(m_tiles) for nt in range(n_cols)}
    parts = []
    for ranges in cover.values():
        ranges.sort()
        assert ranges[0][0] == 0 and ranges[-1][1] == kb
        assert all(a[1] == b[0] for a, b in zip(ranges, ranges[1:])) and all(a[0] < a[1] for a in ranges)
        assert (len(ranges) == 1) == (ranges[0][3] < 0)
        parts += [r[3] for r in ranges if r[3] >= 0]
    assert sorted(parts) == list(range(len(parts)))                        # every partial slot written exactly once
    from anima_trainer_sm120_b200 import _lib
    need = _lib.load().anima_mx_gemm_workspace_bytes(M, N, K)
    assert need == (len(parts) * 256 * bn * 4 if ws else need)


def test_pair_kernel_splits_the_partial_round_of_long_contractions_only(monkeypatch):
    # default tile width: 256 from K = 4096 up
    assert _pair_plan(2048, 2048, 32768)[1] | {"kbs": 0} == {
        "pairs": 64, "n_wide": 8, "narrow": 0, "full_items": 64, "tail_tiles": 0, "splits": 1, "kbs": 0, "shift": 0,
        "bn": 256}                                                         # 64 tiles of 256 x 256: one round, no tail
    assert _pair_plan(6144, 2048, 32768)[1]["splits"] > 1                  # 192 tiles on 74 pairs: 44 tail tiles
    assert _pair_plan(32768, 2048, 8192)[1]["bn"] == 256 and _pair_plan(32768, 8192, 2048)[1]["bn"] == 192
    monkeypatch.setenv("ANIMA_MX_GEMM_BN", "192")
    assert _pair_plan(2048, 2048, 32768)[1]["splits"] > 1                  # 88 tiles on 74 pairs, 256 K-blocks each
    assert _pair_plan(2048, 2048, 32768, ws=0)[1]["splits"] == 1
    assert _pair_plan(32768, 2048, 2048)[1]["splits"] == 1                 # 16 K-blocks per tile: a split costs more
    assert _pair_plan(32768, 2048, 8192)[1]["splits"] == 1                 # two tail tiles of 64 K-blocks: the finalize launch costs more
    assert _pair_plan(32768, 2048, 2048)[1]["narrow"] == 1                 # 2048 = 10 x 192 + 128
    assert _pair_plan(32768, 6144, 2048)[1]["narrow"] == 0                 # 6144 = 32 x 192
    assert _pair_plan(128, 2048, 2048)[0] == 1                             # one-CTA kernel's shape
    # the modelled finish time with the split must not exceed the unsplit one: the busiest pair's K-blocks
    for shape, gain in [((2048, 2048, 32768), 0.65), ((6144, 2048, 32768), 0.99), ((2048, 8192, 32768), 0.99)]:
        loads = []
        for ws in (0, 1):
            pl = _pair_plan(*shape, ws)[1]
            per_pair = [0.0] * pl["pairs"]
            for (mt, nt), ranges in _walk_plan(*shape, pl).items():
                for kb0, kb1, pair, _ in ranges:
                    per_pair[pair] += (kb1 - kb0) * (1.0 if nt < pl["n_wide"] else 128.0 / pl["bn"])
            loads.append(max(per_pair))
        assert loads[1] < gain * loads[0], (shape, loads)
