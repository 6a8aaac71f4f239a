"""GPU parity of the module layer: T-LoKr structured delta (bf16 kernels and MXFP8 GEMMs) against the
oracle and the explicit-Kronecker form, the patched Block forward against the eager Block, the LoKr
patch's quantised path against its bf16 path, and a few optimizer steps of both precision arms.
The algebra cases mirror the reference's ``tests/test_tlokr.py:117-207``."""
from __future__ import annotations

import pytest
import torch
import torch.nn.functional as F

from oracle import tlokr as OT

pytestmark = pytest.mark.gpu
BF16 = torch.bfloat16
DEV = "cuda"


def _tlokr_module(in_f=256, out_f=512, rank=16, dtype=BF16):
    from anima_trainer_sm120_b200 import lokr_patch, tlokr
    from anima_trainer_sm120_b200.lokr import LokrModule, LokrNetwork
    torch.manual_seed(7)
    lin = torch.nn.Linear(in_f, out_f, bias=True).to(DEV, dtype).requires_grad_(False)
    mod = LokrModule("t", lin, lora_dim=rank, alpha=rank, factor=8).to(DEV)
    net = LokrNetwork([mod])
    lokr_patch.install()
    tlokr.convert_network(net, rank=rank, min_rank_ratio=0.5)
    return net, mod, lin


def _rel(ref, got):
    return float((ref.float() - got.float()).abs().max() / (ref.float().abs().max() + 1e-9))


def test_tlokr_zero_init_is_exact_base_output():
    from anima_trainer_sm120_b200 import tlokr
    _, mod, lin = _tlokr_module()
    x = torch.randn(2, 32, 256, device=DEV, dtype=BF16)
    tlokr.set_timestep(torch.tensor([0.0, 1.0], device=DEV))
    try:
        assert torch.equal(mod(x), F.linear(x, lin.weight, lin.bias))
    finally:
        tlokr.clear_timestep()


def test_tlokr_structured_forward_backward_vs_oracle_and_explicit_kron():
    from anima_trainer_sm120_b200 import tlokr
    _, mod, lin = _tlokr_module()
    with torch.no_grad():
        mod.lokr_w2_b.normal_(std=0.2)
    t = torch.tensor([0.2, 0.9], device=DEV)
    x = torch.randn(2, 32, 256, device=DEV, dtype=BF16, requires_grad=True)
    probe = torch.randn(2, 32, 512, device=DEV, dtype=BF16)
    mask = tlokr._TimestepState(timesteps=t).mask(max_rank=16, min_rank=8, dtype=BF16, device=torch.device(DEV))
    out = tlokr._StructuredLoKr.apply(x, mod.lokr_w1, mod.lokr_w2_a, mod.lokr_w2_b, mask)
    out.backward(probe)
    # oracle in fp32 on the bf16-rounded operands (structured form of tlokr.py:472-540)
    xs = x.detach().float().cpu()
    w1, a, b = (p.detach().to(BF16).float().cpu() for p in (mod.lokr_w1, mod.lokr_w2_a, mod.lokr_w2_b))
    want = OT.structured_delta_fwd(xs, w1, a, b, mask.float().cpu())
    gx, gw1, ga, gb = OT.structured_delta_bwd(xs, w1, a, b, mask.float().cpu(), probe.float().cpu())
    assert _rel(want, out.cpu()) < 2e-2
    assert _rel(gx, x.grad.cpu()) < 2e-2
    for got, ref in ((mod.lokr_w1.grad, gw1), (mod.lokr_w2_a.grad, ga), (mod.lokr_w2_b.grad, gb)):
        assert _rel(ref, got.cpu()) < 3e-2
    # explicit Kronecker statement (tests/test_tlokr.py:137-156)
    base = torch.zeros(512, 256)
    explicit = OT.explicit_kron_linear(xs, base, None, w1, a, b, t.cpu(), rank=16, min_rank=8, scale=1.0)
    assert _rel(explicit, out.cpu()) < 2e-2
    # module forward = base + alpha * delta
    tlokr.set_timestep(t)
    try:
        y = mod(x.detach())
    finally:
        tlokr.clear_timestep()
    ref_y = F.linear(x.detach().float(), lin.weight.float(), lin.bias.float()).cpu() + mod._tlokr_alpha * want
    assert _rel(ref_y, y.cpu()) < 2e-2


def test_tlokr_uniform_sliced_path_matches_masked_path():
    from anima_trainer_sm120_b200 import tlokr
    _, mod, _ = _tlokr_module()
    with torch.no_grad():
        mod.lokr_w2_b.normal_(std=0.2)
    x = torch.randn(1, 64, 256, device=DEV, dtype=BF16)
    t = torch.tensor([0.375], device=DEV)
    try:
        tlokr.set_timestep(t)
        masked = mod(x)
        tlokr.set_timestep(t, uniform_timestep=0.375)
        sliced = mod(x)
    finally:
        tlokr.clear_timestep()
    torch.testing.assert_close(sliced.float(), masked.float(), rtol=2e-2, atol=2e-2)
    try:                                   # t = 1.0 -> 8 active ranks: a multiple of 8, so the factors are really sliced
        tlokr.set_timestep(torch.tensor([1.0], device=DEV))
        masked8 = mod(x)
        tlokr.set_timestep(torch.tensor([1.0], device=DEV), uniform_timestep=1.0)
        sliced8 = mod(x)                   # truly sliced factors (A[:, :8], B[:8]), no mask
    finally:
        tlokr.clear_timestep()
    torch.testing.assert_close(sliced8.float(), masked8.float(), rtol=2e-2, atol=2e-2)


def test_tlokr_mxfp8_structured_matches_bf16_structured():
    from anima_trainer_sm120_b200 import tlokr
    _, mod, _ = _tlokr_module(in_f=2048, out_f=2048, rank=128)
    with torch.no_grad():
        mod.lokr_w2_b.normal_(std=0.05)
    t = torch.rand(4, device=DEV)
    mask = tlokr._TimestepState(timesteps=t).mask(max_rank=128, min_rank=64, dtype=BF16, device=torch.device(DEV))
    x = torch.randn(4, 256, 2048, device=DEV, dtype=BF16)
    probe = torch.randn(4, 256, 2048, device=DEV, dtype=BF16)
    outs = []
    for fn in (tlokr._StructuredLoKr, tlokr._MXStructuredLoKr):
        xi = x.clone().requires_grad_(True)
        for p in (mod.lokr_w1, mod.lokr_w2_a, mod.lokr_w2_b):
            p.grad = None
        y = fn.apply(xi, mod.lokr_w1, mod.lokr_w2_a, mod.lokr_w2_b, mask)
        y.backward(probe)
        outs.append([y.detach(), xi.grad, mod.lokr_w1.grad.clone(), mod.lokr_w2_a.grad.clone(), mod.lokr_w2_b.grad.clone()])
    for ref, got in zip(*outs):
        assert _rel(ref, got) < 0.10       # the reference's acceptance for quantised vs bf16 paths


def test_lokr_patch_quantised_path_vs_bf16_path():
    from anima_trainer_sm120_b200 import lokr_patch
    from anima_trainer_sm120_b200.lokr import LokrModule, LokrNetwork
    torch.manual_seed(3)
    lin = torch.nn.Linear(1024, 2048, bias=False).to(DEV, BF16).requires_grad_(False)
    with torch.no_grad():
        lin.weight.normal_(std=0.02)
    mod = LokrModule("m", lin, lora_dim=128, alpha=128, factor=8).to(DEV)
    with torch.no_grad():
        mod.lokr_w2.normal_(std=0.02)
    net = LokrNetwork([mod])
    lokr_patch.install()
    x = torch.randn(8, 512, 1024, device=DEV, dtype=BF16)
    gy = torch.randn(8, 512, 2048, device=DEV, dtype=BF16)
    res = []
    for quant in (False, True):
        lokr_patch.enable_fp8(net) if quant else lokr_patch.disable_fp8()
        xi = x.clone().requires_grad_(True)
        mod.lokr_w1.grad = mod.lokr_w2.grad = None
        y = mod(xi)
        y.backward(gy)
        res.append([y.detach(), xi.grad, mod.lokr_w1.grad.clone(), mod.lokr_w2.grad.clone()])
    lokr_patch.disable_fp8()
    for ref, got in zip(*res):
        assert _rel(ref, got) < 0.10


def test_patched_block_forward_matches_eager_block():
    from anima_trainer_sm120_b200 import adaln_merge, adaln_patch
    from anima_trainer_sm120_b200.anima_dit import AnimaDiT, Block, tiny_config
    torch.manual_seed(0)
    dit = AnimaDiT(tiny_config(depth=2)).to(DEV, BF16)
    x = torch.randn(2, 16, 1, 32, 32, device=DEV, dtype=BF16)
    t = torch.tensor([0.3, 0.8], device=DEV)
    ctx = torch.randn(2, 24, 128, device=DEV, dtype=BF16)
    for p in dit.parameters():
        p.requires_grad_(True)

    def run():
        dit.zero_grad()
        out = dit(x, t, ctx)
        out.float().pow(2).mean().backward()
        return out.detach(), dit.blocks[0].mlp.layer1.weight.grad.clone(), dit.x_embedder.weight.grad.clone()

    adaln_patch.uninstall(Block)
    ref = run()
    adaln_patch.install(Block)
    try:
        got = run()
        assert adaln_merge.merge_adaln_modulation(dit) == 2
        for p in dit.parameters():
            p.requires_grad_(True)
        got_merged = run()
    finally:
        adaln_patch.uninstall(Block)
    torch.testing.assert_close(got[0].float(), ref[0].float(), rtol=5e-2, atol=5e-2)
    torch.testing.assert_close(got_merged[0].float(), ref[0].float(), rtol=5e-2, atol=5e-2)
    for r, g in zip(ref[1:], got[1:]):
        assert _rel(r, g) < 5e-2


@pytest.mark.parametrize("variant", ["lokr", "tlokr"])
def test_training_arms_track_each_other(variant):
    """Eight optimizer steps of a small-width model in both precision arms from the same seed: per-step
    loss within 2 % (the loss-curve criterion) and the adapters move."""
    from anima_trainer_sm120_b200.anima_dit import tiny_config
    from anima_trainer_sm120_b200.train_step import StepConfig, Trainer
    mcfg = tiny_config(depth=2, dim=512, heads=4, mlp_dim=1024, context_dim=256, adaln_lora_dim=64)
    curves = {}
    for prec in ("bf16", "mxfp8"):
        tr = Trainer(mcfg, StepConfig(precision=prec, variant=variant, lokr_dim=32, lr=2e-3), torch.device(DEV))
        before = [p.detach().clone() for p in tr.params]
        curves[prec] = tr.run(steps=8, batch=4, latent_hw=32, text_tokens=32)
        assert any(not torch.equal(a, b) for a, b in zip(before, tr.params))
    for a, b in zip(curves["bf16"], curves["mxfp8"]):
        assert abs(a - b) / a < 0.02, curves


def test_scale_regroup_equals_quantising_the_reshaped_tensor():
    from anima_trainer_sm120_b200 import ops
    torch.manual_seed(4)
    for rows, K, u in ((96, 512, 8), (1024, 2048, 8), (33, 256, 4), (160, 1024, 8), (256, 8192, 8), (72, 1024, 4)):
        x = (torch.randn(rows, K, device=DEV) * 3).to(BF16)
        row, _ = ops.mx_quantize(x, rowwise=True)
        want, _ = ops.mx_quantize(x.view(rows * u, K // u), rowwise=True)
        got = ops.mx_regroup(row, rows * u, K // u)
        assert torch.equal(got.codes, want.codes) and torch.equal(got.scales, want.scales)
        back = ops.mx_regroup(got, rows, K)
        assert torch.equal(back.scales, row.scales)
    with pytest.raises(ValueError):
        ops.mx_regroup(row, 7, 11)


def test_tlokr_single_node_linear_matches_three_node_composition():
    """``_MXTLoKrLinear`` (one quantisation of x and of the gradient, adds done by GEMM stores) against the
    base projection + ``_MXStructuredLoKr`` + ``torch.add`` composition it replaces."""
    from anima_trainer_sm120_b200 import fp8_quant, tlokr
    _, mod, lin = _tlokr_module(in_f=1024, out_f=2048, rank=64)
    with torch.no_grad():
        mod.lokr_w2_b.normal_(std=0.05)
        lin.weight.normal_(std=0.03)
    Wq = fp8_quant.quantize_weight(lin.weight)
    t = torch.rand(4, device=DEV)
    mask = tlokr._TimestepState(timesteps=t).mask(max_rank=64, min_rank=32, dtype=BF16, device=torch.device(DEV))
    x = torch.randn(4, 128, 1024, device=DEV, dtype=BF16)
    probe = torch.randn(4, 128, 2048, device=DEV, dtype=BF16)
    alpha = 0.6
    res = []
    for single in (False, True):
        xi = x.clone().requires_grad_(True)
        for p in (mod.lokr_w1, mod.lokr_w2_a, mod.lokr_w2_b):
            p.grad = None
        if single:
            y = tlokr._MXTLoKrLinear.apply(xi, Wq, lin.bias, mod.lokr_w1, mod.lokr_w2_a, mod.lokr_w2_b, mask, alpha)
        else:
            base = fp8_quant.fp8_frozen_linear(xi, Wq, lin.weight, lin.bias)
            y = torch.add(base, tlokr._MXStructuredLoKr.apply(xi, mod.lokr_w1, mod.lokr_w2_a, mod.lokr_w2_b, mask),
                          alpha=alpha)
        y.backward(probe)
        res.append([y.detach(), xi.grad, mod.lokr_w1.grad.clone(), mod.lokr_w2_a.grad.clone(), mod.lokr_w2_b.grad.clone()])
    names = ("y", "grad_x", "grad_w1", "grad_A", "grad_B")
    rels = {name: _rel(ref, got) for name, ref, got in zip(names, *res)}
    # the factor gradients are signed sums over every token of products of two quantised tensors; the two
    # forms quantise alpha * grad and grad respectively, so those sums move by a few percent of their maximum
    # (quantisation noise, not accumulation order). The reference's acceptance for quantised paths is 0.10.
    assert all(v < (2e-2 if name in ("y", "grad_x") else 0.10) for name, v in rels.items()), rels


def test_tlokr_mlp_node_matches_two_linears_with_eager_gelu():
    from anima_trainer_sm120_b200 import fp8_quant, tlokr
    _, m1, l1 = _tlokr_module(in_f=512, out_f=2048, rank=64)
    _, m2, l2 = _tlokr_module(in_f=2048, out_f=512, rank=64)
    with torch.no_grad():
        for m, l in ((m1, l1), (m2, l2)):
            m.lokr_w2_b.normal_(std=0.05)
            l.weight.normal_(std=0.03)
    W1, W2 = fp8_quant.quantize_weight(l1.weight), fp8_quant.quantize_weight(l2.weight)
    t = torch.rand(4, device=DEV)
    mask = tlokr._TimestepState(timesteps=t).mask(max_rank=64, min_rank=32, dtype=BF16, device=torch.device(DEV))
    x = torch.randn(4, 128, 512, device=DEV, dtype=BF16)
    probe = torch.randn(4, 128, 512, device=DEV, dtype=BF16)
    params = (m1.lokr_w1, m1.lokr_w2_a, m1.lokr_w2_b, m2.lokr_w1, m2.lokr_w2_a, m2.lokr_w2_b)
    res = []
    for fused in (False, True):
        xi = x.clone().requires_grad_(True)
        for p in params:
            p.grad = None
        a1 = (W1, l1.bias, m1.lokr_w1, m1.lokr_w2_a, m1.lokr_w2_b, mask, 0.8)
        a2 = (W2, l2.bias, m2.lokr_w1, m2.lokr_w2_a, m2.lokr_w2_b, mask, 1.2)
        if fused:
            y = tlokr._MXTLoKrMLP.apply(xi, *a1, *a2)
        else:
            y = tlokr._MXTLoKrLinear.apply(F.gelu(tlokr._MXTLoKrLinear.apply(xi, *a1)), *a2)
        y.backward(probe)
        res.append([y.detach(), xi.grad] + [p.grad.clone() for p in params])
    rels = [_rel(ref, got) for ref, got in zip(*res)]
    assert all(v < (2e-2 if i < 2 else 0.10) for i, v in enumerate(rels)), rels


@pytest.mark.parametrize("variant", ["lokr", "tlokr"])
def test_cuda_graph_replay_reproduces_the_eager_step(variant):
    """Forward + backward captured per input shape and replayed (cuda_graphs.CUDAGraphRunner, the reference's
    cuda_graphs.py:68-234): same seeded steps as the eager trainer, losses and adapters equal; the runner warms up
    eagerly, captures once, then replays."""
    from anima_trainer_sm120_b200.anima_dit import tiny_config
    from anima_trainer_sm120_b200.train_step import StepConfig, Trainer
    mcfg = tiny_config(depth=2, dim=512, heads=4, mlp_dim=1024, context_dim=256, adaln_lora_dim=64)
    runs = {}
    for graph in (False, True):
        tr = Trainer(mcfg, StepConfig(precision="mxfp8", variant=variant, lokr_dim=32, lr=2e-3, cuda_graph=graph),
                     torch.device(DEV))
        losses = tr.run(steps=7, batch=4, latent_hw=32, text_tokens=32)
        runs[graph] = (losses, [p.detach().clone() for p in tr.params])
        if graph:
            assert tr.runner is not None and len(tr.runner._state) == 1
            assert all(tr.runner.captured(k) for k in tr.runner._state)       # steps 4..7 were replays
    (l_e, p_e), (l_g, p_g) = runs[False], runs[True]
    for a, b in zip(l_e, l_g):
        assert abs(a - b) <= 1e-5 * abs(a), (l_e, l_g)
    for a, b in zip(p_e, p_g):
        torch.testing.assert_close(a, b, rtol=1e-4, atol=1e-6)
