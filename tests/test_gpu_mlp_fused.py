"""GPU parity of the GELU-in-the-quantiser kernel against quantising the eager bf16 GELU (and its eager
gradient), and of the fused LoKr MLP node against the unfused chain of two LoKr linears with an eager
GELU between them. The kernel tabulates, per device, the very expressions the eager kernels evaluate, so
codes and scale bytes must be identical bit for bit, for every finite bf16 input."""
from __future__ import annotations

import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu
BF16 = torch.bfloat16
DEV = "cuda"


def _same(a, b):
    assert torch.equal(a.scales, b.scales)
    assert torch.equal(a.codes, b.codes)


@pytest.fixture(params=["1", "2"], ids=["plain-loads", "copy-engine-fed"])
def quantiser_variant(request, monkeypatch):
    """The kernel tests run once per quantiser kernel (the library reads the variable on every call): the tile
    kernel with plain loads, and the persistent kernel fed by bulk tensor copies (whose bounded waits must not
    have given up)."""
    monkeypatch.setenv("ANIMA_MX_QUANTIZE_VARIANT", request.param)
    yield request.param
    from anima_trainer_sm120_b200 import _lib
    assert _lib.load().anima_mx_quantize_status() == 0


def test_quantize_gelu_is_bit_exact_for_every_finite_bf16_input(quantiser_variant):
    from anima_trainer_sm120_b200 import ops
    bits = torch.arange(65536, dtype=torch.int32)
    finite = bits[(bits & 0x7F80) != 0x7F80]                                  # 65280 patterns
    g = torch.Generator().manual_seed(0)
    h = finite[torch.randperm(finite.numel(), generator=g)].to(torch.int16).view(BF16).view(2040, 32).to(DEV)
    act = torch.empty_like(h)
    row, _ = ops.mx_quantize_gelu(h, rowwise=True, act_out=act)
    eager = F.gelu(h)
    assert torch.equal(act.view(torch.int16), eager.view(torch.int16))           # the bf16 activation itself
    want, _ = ops.mx_quantize(eager, rowwise=True)
    _same(row, want)
    for seed in (1, 2):                                                           # the gradient depends on dy too
        dy = torch.randn(2040, 32, generator=torch.Generator().manual_seed(seed)).to(BF16).to(DEV)
        hr = h.clone().requires_grad_(True)
        F.gelu(hr).backward(dy)
        grad = torch.empty_like(h)
        row, _ = ops.mx_quantize_gelu(h, dy, rowwise=True, act_out=grad)
        assert torch.equal(grad.view(torch.int16), hr.grad.view(torch.int16))
        want, _ = ops.mx_quantize(hr.grad, rowwise=True)
        _same(row, want)


@pytest.mark.parametrize("rows,cols", [(256, 512), (96, 160), (1024, 8192), (8192 + 32, 2048 + 32)])
def test_quantize_gelu_forward_and_gradient_match_eager_then_quantise(rows, cols, quantiser_variant):
    from anima_trainer_sm120_b200 import ops
    torch.manual_seed(rows + cols)
    h = (torch.randn(rows, cols, device=DEV) * 2.0).to(BF16)
    h[0, :8] = torch.tensor([0.0, -0.0, 30.0, -30.0, 1e-3, -1e-3, 6.0, -6.0], device=DEV, dtype=BF16)
    g = torch.randn(rows, cols, device=DEV).to(BF16)
    row, col = ops.mx_quantize_gelu(h, rowwise=True, colwise=True)
    want_row, want_col = ops.mx_quantize(F.gelu(h), rowwise=True, colwise=True)
    _same(row, want_row)
    _same(col, want_col)
    hr = h.clone().requires_grad_(True)
    F.gelu(hr).backward(g)
    row, col = ops.mx_quantize_gelu(h, g, rowwise=True, colwise=True)
    want_row, want_col = ops.mx_quantize(hr.grad, rowwise=True, colwise=True)
    _same(row, want_row)
    _same(col, want_col)
    _same(ops.mx_quantize_gelu(h, g, rowwise=False, colwise=True)[1], want_col)      # one form at a time
    _same(ops.mx_quantize_gelu(h, g, rowwise=True, colwise=False)[0], want_row)
    _same(ops.mx_quantize_gelu(h, rowwise=False, colwise=True)[1], ops.mx_quantize(F.gelu(h), rowwise=False, colwise=True)[1])


def test_quantize_gelu_rejects_mismatched_gradient():
    from anima_trainer_sm120_b200 import ops
    h = torch.zeros(64, 64, device=DEV, dtype=BF16)
    with pytest.raises(ValueError):
        ops.mx_quantize_gelu(h, torch.zeros(64, 32, device=DEV, dtype=BF16))


def test_fused_mlp_equals_unfused_chain():
    from anima_trainer_sm120_b200.fp8_quant import lokr_linear_fused
    from anima_trainer_sm120_b200.mlp_patch import LoKrMLPFused
    torch.manual_seed(5)
    D, H, M = 512, 2048, 1024
    W1 = (torch.randn(H, D, device=DEV) * 0.03).to(BF16)
    W2 = (torch.randn(D, H, device=DEV) * 0.03).to(BF16)
    f = lambda *s: (torch.randn(*s, device=DEV) * 0.05).requires_grad_(True)
    w1a, w2a, w1b, w2b = f(8, 8), f(H // 8, D // 8), f(8, 8), f(D // 8, H // 8)
    x = torch.randn(4, M // 4, D, device=DEV, dtype=BF16)
    gy = torch.randn(4, M // 4, D, device=DEV, dtype=BF16)
    results = []
    for fused in (False, True):
        xi = x.clone().requires_grad_(True)
        for p in (w1a, w2a, w1b, w2b):
            p.grad = None
        if fused:
            y = LoKrMLPFused.apply(xi, W1, None, w1a, w2a, 0.7, W2, None, w1b, w2b, 1.3)
        else:
            y = lokr_linear_fused(F.gelu(lokr_linear_fused(xi, W1, None, w1a, w2a, 0.7)), W2, None, w1b, w2b, 1.3)
        y.backward(gy)
        results.append([y.detach(), xi.grad] + [p.grad.clone() for p in (w1a, w2a, w1b, w2b)])
    for ref, got in zip(*results):
        assert torch.equal(ref, got)


def test_mlp_patch_routes_eligible_adapters_and_falls_through_otherwise():
    from anima_trainer_sm120_b200 import lokr_patch, mlp_patch
    from anima_trainer_sm120_b200.anima_dit import GPT2FeedForward, tiny_config
    from anima_trainer_sm120_b200.lokr import LokrModule, LokrNetwork
    torch.manual_seed(9)
    mlp = GPT2FeedForward(tiny_config(dim=256, mlp_dim=1024)).to(DEV, BF16).requires_grad_(False)
    mods = [LokrModule(n, getattr(mlp, n), lora_dim=32, alpha=32, factor=8).to(DEV) for n in ("layer1", "layer2")]
    with torch.no_grad():
        for m in mods:
            m.lokr_w2.normal_(std=0.05)
    net = LokrNetwork(mods)
    lokr_patch.install()
    net.apply_to()
    lokr_patch.enable_fp8(net)
    x = torch.randn(2, 64, 256, device=DEV, dtype=BF16)
    try:
        ref = mlp(x)                                  # two fused linears + eager GELU
        mlp_patch.install(GPT2FeedForward)
        got = mlp(x)
        assert torch.equal(ref, got)
        lokr_patch.disable_fp8()
        bf16 = mlp(x)                                 # patched class, adapters not on the quantised path
        assert float((bf16.float() - ref.float()).abs().max() / ref.float().abs().max()) < 0.1
    finally:
        mlp_patch.uninstall(GPT2FeedForward)
        lokr_patch.disable_fp8()


def test_activation_memo_shares_one_quantisation_between_consumers():
    from anima_trainer_sm120_b200 import fp8_quant, ops
    torch.manual_seed(2)
    x = torch.randn(128, 256, device=DEV, dtype=BF16)
    Ws = [fp8_quant.quantize_weight((torch.randn(256, 256, device=DEV) * 0.05).to(BF16)) for _ in range(3)]
    W_bf16 = torch.zeros(256, 256, device=DEV, dtype=BF16)
    fp8_quant.clear_activation_memo()
    fp8_quant.act_memo_stats.update(hits=0, misses=0, adopted=0)
    ys = [fp8_quant.mxfp8_frozen_linear(x, W, W_bf16) for W in Ws]          # q / k / v pattern: same tensor object
    assert fp8_quant.act_memo_stats == {"hits": 2, "misses": 1, "adopted": 0}
    x_row, _ = ops.mx_quantize(x, rowwise=True)
    for y, W in zip(ys, Ws):
        assert torch.equal(y, ops.mx_gemm(x_row, W.row))
    x.add_(1.0)                                                              # in-place change invalidates the entry
    y = fp8_quant.mxfp8_frozen_linear(x, Ws[0], W_bf16)
    assert fp8_quant.act_memo_stats["misses"] == 2
    assert torch.equal(y, ops.mx_gemm(ops.mx_quantize(x, rowwise=True)[0], Ws[0].row))
    row, col = fp8_quant.quantize_activation(x, colwise=True)               # the entry lacks this form: only it is made
    assert fp8_quant.act_memo_stats["misses"] == 2
    assert torch.equal(col.codes, ops.mx_quantize(x, rowwise=False, colwise=True)[1].codes)
    fp8_quant.clear_activation_memo()
