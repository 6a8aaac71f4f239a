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
