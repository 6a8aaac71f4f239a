"""GPU parity: fused AdaLN and gated residual through the C ABI vs the CPU oracle, the golden
vectors of the reference kernels, and eager PyTorch. Tolerance for floating-point outputs is
rtol 1e-2 / atol 2e-2 (bf16 I/O); elementwise outputs whose fp32 value is exact are bit-compared.
Cases follow tests/sanity_adaln_kernel.py:105-112 of the reference (shapes, seeds 0 / 1, eps 1e-6,
scale / shift ~ 0.1 N(0,1))."""
from __future__ import annotations

import pytest
import torch

from conftest import bf16_from_bits
from oracle import adaln as OA

pytestmark = pytest.mark.gpu
RTOL, ATOL = 1e-2, 2e-2
BF16 = torch.bfloat16


def _ops():
    from anima_trainer_sm120_b200 import ops
    return ops


def _close(got, want, rtol=RTOL, atol=ATOL):
    torch.testing.assert_close(got.float().cpu(), want.float().cpu(), rtol=rtol, atol=atol)


def _case(BT, HW, D, seed=0):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(BT * HW, D, generator=g).to(BF16)
    s = (torch.randn(BT, D, generator=g) * 0.1).to(BF16)
    b = (torch.randn(BT, D, generator=g) * 0.1).to(BF16)
    gate = (torch.randn(BT, D, generator=g) * 0.1).to(BF16)
    y2 = torch.randn(BT * HW, D, generator=g).to(BF16)
    g1 = torch.Generator().manual_seed(seed + 1)
    dy = torch.randn(BT * HW, D, generator=g1).to(BF16)
    return x, s, b, gate, y2, dy


@pytest.mark.parametrize("BT,HW,D", [(2, 24, 256), (3, 8, 768), (8, 1024, 2048), (4, 256, 1024), (1, 5, 8),
                                       (2, 7, 2056), (2, 33, 4096)])
def test_adaln_forward_backward_vs_oracle(BT, HW, D):
    ops = _ops()
    x, s, b, _, _, dy = _case(BT, HW, D)
    y, mean, rstd = ops.adaln_fwd(x.cuda(), s.cuda(), b.cuda(), 1e-6, HW)
    y_o, mean_o, rstd_o = OA.adaln_fwd_fp32(x, s, b, 1e-6, HW)
    _close(mean, mean_o, 1e-5, 1e-5)
    _close(rstd, rstd_o, 1e-5, 1e-5)
    _close(y, y_o.to(BF16))
    assert (y.cpu().view(torch.int16) != y_o.to(BF16).view(torch.int16)).float().mean() < 0.02
    dx, ds, db = ops.adaln_bwd(dy.cuda(), x.cuda(), s.cuda(), mean, rstd, HW)
    dx_o, ds_o, db_o = OA.adaln_bwd_fp32(dy, x, s, mean.cpu(), rstd.cpu(), HW)
    _close(dx, dx_o.to(BF16))
    # H*W reductions: judged against the fp32 truth rounded to bf16 (sanity_adaln_kernel.py:81-96)
    _close(ds, ds_o.to(BF16))
    _close(db, db_o.to(BF16))


def test_adaln_golden_reference_kernel_outputs(golden):
    ops = _ops()
    g = golden("adaln")
    for n in ("a", "b"):
        BT, HW, D = (int(v) for v in g[f"{n}_shape"])
        x, s, b, gate, y2, dy = (bf16_from_bits(g[f"{n}_{k}"]).cuda() for k in ("x", "s", "b", "gate", "y2", "dy"))
        y, mean, rstd = ops.adaln_fwd(x, s, b, 1e-6, HW)
        _close(y, bf16_from_bits(g[f"{n}_y"]))
        _close(mean, torch.from_numpy(g[f"{n}_mean"]), 1e-5, 1e-5)
        _close(rstd, torch.from_numpy(g[f"{n}_rstd"]), 1e-5, 1e-5)
        dx, ds, db = ops.adaln_bwd(dy, x, s, mean, rstd, HW)
        _close(dx, bf16_from_bits(g[f"{n}_dx"]))
        _close(ds, torch.from_numpy(g[f"{n}_ds"]).to(BF16))
        _close(db, torch.from_numpy(g[f"{n}_db"]).to(BF16))
        out = ops.gated_add_fwd(x, gate, y2, HW)
        _close(out, bf16_from_bits(g[f"{n}_go"]))
        _, dg = ops.gated_add_bwd(dy, y2, gate, HW)
        _close(dg, torch.from_numpy(g[f"{n}_dg"]).to(BF16))


@pytest.mark.parametrize("B,H,W,D", [(8, 32, 32, 2048), (2, 8, 8, 768)])
def test_autograd_ops_vs_eager(B, H, W, D):
    """FusedAdaLN / FusedGatedAdd (the reference's operator signatures) against eager autograd;
    dscale / dshift / dgate (sums over H*W) are held to the reference's own criterion: no further from the fp32 truth than
    1.5x eager's error (tests/sanity_adaln_kernel.py:58-65, 81-96)."""
    from anima_trainer_sm120_b200.adaln_kernel import FusedAdaLN, FusedGatedAdd
    torch.manual_seed(0)
    dev = "cuda"
    x = torch.randn(B, 1, H, W, D, dtype=BF16, device=dev)
    scale = (torch.randn(B, 1, 1, 1, D, device=dev) * 0.1).to(BF16)
    shift = (torch.randn(B, 1, 1, 1, D, device=dev) * 0.1).to(BF16)
    gate = (torch.randn(B, 1, 1, 1, D, device=dev) * 0.1).to(BF16)
    torch.manual_seed(1)
    dy = torch.randn_like(x)

    def run(fn, dtype):
        leaves = [t.detach().to(dtype).clone().requires_grad_(True) for t in (x, scale, shift, gate)]
        xx, ss, bb, gg = leaves
        out = fn(xx, ss, bb, gg)
        out.backward(dy.to(dtype))
        return out.detach(), [t.grad for t in leaves]

    def fused(xx, ss, bb, gg):
        return FusedGatedAdd.apply(xx, gg, FusedAdaLN.apply(xx, ss, bb, 1e-6))

    def eager(xx, ss, bb, gg):
        return OA.gated_add_eager(xx, gg, OA.adaln_eager(xx, ss, bb, 1e-6))

    out_k, grads_k = run(fused, BF16)
    out_e, grads_e = run(eager, BF16)
    out_t, grads_t = run(eager, torch.float32)
    _close(out_k, out_t.to(BF16))
    _close(out_k, out_e, 5e-2, 5e-2)                      # reference's own bf16 tolerance (:105)
    _close(grads_k[0], grads_t[0].to(BF16))               # dx
    for i in (1, 2, 3):                                   # dscale, dshift, dgate: sums over H*W
        err_k = (grads_k[i].float() - grads_t[i]).abs().max().item()
        err_e = (grads_e[i].float() - grads_t[i]).abs().max().item()
        assert err_k <= max(1.5 * err_e, 1e-3), (i, err_k, err_e)


def test_gated_add_elementwise_outputs_bit_exact():
    """x + g*y and g*dout: the product of two bf16 values is exact in fp32, so the kernel must
    reproduce the fp32 oracle bit for bit after the single rounding."""
    ops = _ops()
    x, _, _, gate, y2, dy = _case(4, 96, 1024, seed=3)
    out = ops.gated_add_fwd(x.cuda(), gate.cuda(), y2.cuda(), 96).cpu()
    assert torch.equal(out.view(torch.int16), OA.gated_add_fwd_fp32(x, gate, y2, 96).to(BF16).view(torch.int16))
    d_y, d_g = ops.gated_add_bwd(dy.cuda(), y2.cuda(), gate.cuda(), 96)
    dy_o, dg_o = OA.gated_add_bwd_fp32(dy, y2, gate, 96)
    assert torch.equal(d_y.cpu().view(torch.int16), dy_o.to(BF16).view(torch.int16))
    _close(d_g, dg_o.to(BF16))


def test_reductions_are_bit_reproducible():
    ops = _ops()
    x, s, b, gate, y2, dy = (t.cuda() for t in _case(8, 512, 2048, seed=7))
    _, mean, rstd = ops.adaln_fwd(x, s, b, 1e-6, 512)
    first = ops.adaln_bwd(dy, x, s, mean, rstd, 512)
    g_first = ops.gated_add_bwd(dy, y2, gate, 512)
    for _ in range(3):
        again = ops.adaln_bwd(dy, x, s, mean, rstd, 512)
        assert all(torch.equal(a, b_) for a, b_ in zip(first, again))
        assert all(torch.equal(a, b_) for a, b_ in zip(g_first, ops.gated_add_bwd(dy, y2, gate, 512)))


def test_full_size_config3_properties():
    """Config 3 shape x [8, 4096, 2048]: oracle on one sample, and size-independent properties —
    LN output rows have zero mean / unit variance when scale = shift = 0; dshift equals the column
    sum of dy; linearity of gated add in gate."""
    ops = _ops()
    BT, HW, D = 8, 4096, 2048
    g = torch.Generator(device="cuda").manual_seed(0)
    x = torch.randn(BT * HW, D, generator=g, device="cuda").to(BF16)
    zeros = torch.zeros(BT, D, dtype=BF16, device="cuda")
    y, mean, rstd = ops.adaln_fwd(x, zeros, zeros, 1e-6, HW)
    yf = y.float()
    assert yf.mean(dim=1).abs().max() < 5e-3
    assert (yf.var(dim=1, unbiased=False) - 1).abs().max() < 2e-2
    mod = (torch.randn(BT, 3 * D, generator=g, device="cuda") * 0.1).to(BF16)
    shift, scale, gate = (t.contiguous() for t in mod.chunk(3, dim=-1))
    y, mean, rstd = ops.adaln_fwd(x, scale, shift, 1e-6, HW)
    sl = slice(3 * HW, 3 * HW + 512)
    y_o, _, _ = OA.adaln_fwd_fp32(x[sl].cpu(), scale[3:4].cpu(), shift[3:4].cpu(), 1e-6, 512)
    _close(y[sl], y_o.to(BF16))
    dy = torch.randn(BT * HW, D, generator=g, device="cuda").to(BF16)
    dx, ds, db = ops.adaln_bwd(dy, x, scale, mean, rstd, HW)
    _close(db, dy.float().view(BT, HW, D).sum(dim=1).to(BF16))
    dx_o, _, _ = OA.adaln_bwd_fp32(dy[sl].cpu(), x[sl].cpu(), scale[3:4].cpu(), mean[sl].cpu(), rstd[sl].cpu(), 512)
    _close(dx[sl], dx_o.to(BF16))
    out1 = ops.gated_add_fwd(x, gate, y, HW).float()
    out0 = ops.gated_add_fwd(x, torch.zeros_like(gate), y, HW)
    assert torch.equal(out0, x)
    _close(out1, x.float() + gate.float().repeat_interleave(HW, dim=0) * y.float())


@pytest.mark.parametrize("B,H,W,D", [(2, 8, 8, 256), (1, 5, 7, 2048), (3, 4, 4, 4096)])
def test_gated_add_adaln_one_pass_equals_the_two_ops(B, H, W, D):
    """x_new and y of the one-pass op are bit-identical to FusedGatedAdd followed by FusedAdaLN, and so are
    all five gradients (backward runs the same two backward kernels on the same operands)."""
    from anima_trainer_sm120_b200.adaln_kernel import FusedAdaLN, FusedGatedAdd, FusedGatedAddAdaLN
    g = torch.Generator().manual_seed(B * 100 + D)
    mk = lambda *s, std=1.0: (torch.randn(*s, generator=g) * std).to(torch.bfloat16).cuda()
    x, sub = mk(B, 1, H, W, D), mk(B, 1, H, W, D)
    gate, scale, shift = mk(B, 1, 1, 1, D, std=0.3), mk(B, 1, 1, 1, D, std=0.3), mk(B, 1, 1, 1, D, std=0.3)
    p1, p2 = mk(B, 1, H, W, D), mk(B, 1, H, W, D)
    results = []
    for fused in (False, True):
        leaves = [t.clone().requires_grad_(True) for t in (x, gate, sub, scale, shift)]
        xi, gi, ui, si, bi = leaves
        if fused:
            x_new, y = FusedGatedAddAdaLN.apply(xi, gi, ui, si, bi, 1e-6)
        else:
            x_new = FusedGatedAdd.apply(xi, gi, ui)
            y = FusedAdaLN.apply(x_new, si, bi, 1e-6)
        torch.autograd.backward([x_new, y], [p1, p2])
        results.append([x_new.detach(), y.detach()] + [t.grad for t in leaves])
    for ref, got in zip(*results):
        assert torch.equal(ref, got)


@pytest.mark.parametrize("BT,HW,D", [(2, 64, 128), (1, 128, 384), (3, 128, 1024), (8, 512, 2048), (2, 192, 4096)])
def test_adaln_forward_emits_the_row_operand_of_its_output(BT, HW, D):
    """The quantising forward writes the same y / mean / rstd as the plain one, and codes and scales equal to
    quantising that y afterwards (tiled scales), bit for bit; the same holds for the one-pass residual form and
    when y itself is not written."""
    from anima_trainer_sm120_b200 import _lib
    ops = _ops()
    x, s, b, gate, sub, _ = (t.cuda() for t in _case(BT, HW, D, seed=5))
    y, mean, rstd = ops.adaln_fwd(x, s, b, 1e-6, HW)
    y_q, mean_q, rstd_q, op = ops.adaln_fwd(x, s, b, 1e-6, HW, quant=True)
    want, _ = ops.mx_quantize(y, rowwise=True)
    assert torch.equal(y_q, y) and torch.equal(mean_q, mean) and torch.equal(rstd_q, rstd)
    assert torch.equal(op.codes, want.codes) and torch.equal(op.scales, want.scales)

    x_new, y2, mean2, rstd2 = ops.gated_add_adaln_fwd(x, gate, sub, s, b, 1e-6, HW)
    x_new_q, y2_q, mean2_q, rstd2_q, op2 = ops.gated_add_adaln_fwd(x, gate, sub, s, b, 1e-6, HW, quant=True)
    want2, _ = ops.mx_quantize(y2, rowwise=True)
    assert torch.equal(x_new_q, x_new) and torch.equal(y2_q, y2) and torch.equal(mean2_q, mean2)
    assert torch.equal(op2.codes, want2.codes) and torch.equal(op2.scales, want2.scales)

    # plain scale layout and no bf16 output, through the C ABI directly
    rows = BT * HW
    codes = torch.zeros(rows, D, dtype=torch.uint8, device="cuda")
    scales = torch.zeros(rows, D // 32, dtype=torch.uint8, device="cuda")
    mean3, rstd3 = torch.empty_like(mean), torch.empty_like(rstd)
    rc = _lib.load().anima_adaln_fwd_quant(ops.ptr(x), ops.ptr(s), ops.ptr(b), 1e-6, rows, HW, D, None, ops.ptr(mean3),
                                           ops.ptr(rstd3), ops.ptr(codes), ops.ptr(scales), ops.SCALES_PLAIN,
                                           _lib.stream_ptr(x.device))
    assert rc == 0
    plain, _ = ops.mx_quantize(y, rowwise=True, layout=ops.SCALES_PLAIN)
    assert torch.equal(codes, plain.codes) and torch.equal(scales, plain.scales.view(rows, D // 32))
    assert torch.equal(mean3, mean) and torch.equal(rstd3, rstd)


def test_adaln_quantising_forward_refuses_shapes_it_cannot_tile():
    ops = _ops()
    x, s, b, _, _, _ = (t.cuda() for t in _case(2, 24, 256))
    with pytest.raises(ValueError):
        ops.adaln_fwd(x, s, b, 1e-6, 24, quant=True)          # 48 rows: tiled scales need whole 128-row chunks
    assert not ops.can_emit_row_codes(48, 256) and not ops.can_emit_row_codes(128, 96)


def test_autograd_adaln_hands_its_operand_to_the_quantised_linears():
    """With emission on, a quantised linear fed a reshape of the AdaLN output launches no quantiser and returns
    exactly what it returns with emission off."""
    from anima_trainer_sm120_b200 import adaln_kernel, fp8_quant
    torch.manual_seed(3)
    B, H, W, D = 2, 8, 16, 256
    x = torch.randn(B, 1, H, W, D, device="cuda", dtype=BF16)
    sc = (torch.randn(B, 1, 1, 1, D, device="cuda") * 0.1).to(BF16)
    sh = (torch.randn(B, 1, 1, 1, D, device="cuda") * 0.1).to(BF16)
    Wq = fp8_quant.quantize_weight((torch.randn(384, D, device="cuda") * 0.05).to(BF16))
    W_bf16 = torch.zeros(384, D, device="cuda", dtype=BF16)

    def run():
        fp8_quant.clear_activation_memo()
        fp8_quant.act_memo_stats.update(hits=0, misses=0, adopted=0)
        n = adaln_kernel.fused_adaln(x, sc, sh, 1e-6)
        out = fp8_quant.mxfp8_frozen_linear(n.reshape(B, H * W, D), Wq, W_bf16)
        return n, out, dict(fp8_quant.act_memo_stats)

    try:
        adaln_kernel.emit_row_operand(True)
        n1, out1, stats1 = run()
    finally:
        adaln_kernel.emit_row_operand(False)
    n0, out0, stats0 = run()
    assert stats1 == {"hits": 1, "misses": 0, "adopted": 1} and stats0 == {"hits": 0, "misses": 1, "adopted": 0}
    assert torch.equal(n1, n0) and torch.equal(out1, out0)
    fp8_quant.clear_activation_memo()


@pytest.mark.parametrize("BT,HW,D", [(2, 64, 256), (3, 128, 1024), (4, 1024, 2048), (2, 24, 4096)])
def test_staged_modulation_gives_the_same_bits(BT, HW, D, monkeypatch):
    """The forward kernels convert the sample's modulation row once per CTA (hw % 8 == 0); every output equals
    the kernel that reads it from global memory per row (the library reads the variable on every call)."""
    ops = _ops()
    x, s, b, gate, sub, _ = (t.cuda() for t in _case(BT, HW, D, seed=9))
    outs = {}
    for flag in ("0", "1"):
        monkeypatch.setenv("ANIMA_ADALN_FWD_STAGING", flag)
        outs[flag] = (*ops.gated_add_adaln_fwd(x, gate, sub, s, b, 1e-6, HW), *ops.adaln_fwd(x, s, b, 1e-6, HW))
        if ops.can_emit_row_codes(BT * HW, D):
            *plain, op = ops.gated_add_adaln_fwd(x, gate, sub, s, b, 1e-6, HW, quant=True)
            outs[flag] = (*outs[flag], *plain, op.codes, op.scales)
    assert len(outs["0"]) == len(outs["1"])
    for a, c in zip(outs["0"], outs["1"]):
        assert torch.equal(a, c)
