"""GPU parity at the benchmark configurations' own shapes, through the public operators and the C ABI.

config 1  the LoKr linear x [2048, 2048], W [8192, 2048], w1 [8, 8], w2 [1024, 256], seed 42 through
          ``lokr_linear_fused``: y / dx against the dequantise-then-matmul oracle on the kernels' own codes
          (rtol 1e-2 / atol 2e-2), dw1 / dw2 against the oracle's Kronecker adjoint of the oracle's dW, and all
          four against the reference's bf16 mode (``lokr_patch.py:76-94``) with its own acceptance
          ``max_err / max|ref| < 0.10`` (the violation fraction of rtol 1e-2 / atol 2e-2 against bf16 is printed:
          that tolerance is below the MXFP8 quantisation noise).
config 2  every (N, K) of the sweep at M = 32768 and every direction (forward, dgrad, wgrad): three disjoint
          output tiles of the CTA-pair kernel against the oracle on identical codes.
config 4  the quantised T-LoKr delta (``_MXStructuredLoKr``) and the one-node quantised T-LoKr linear
          (``_MXTLoKrLinear``) at the four module shapes of the 168-module preset, rank 128, min rank 64,
          t ~ U(0, 1) seed 42: every factor GEMM against the oracle on identical codes, the 8x8 mix bit-exact,
          dC against float64, and the whole chain against the reference's structured algebra
          (``tlokr.py:476-540``) evaluated on the dequantised operands.
The reference-signature LoKr linear ``fp8_lokr_linear(x, merged_W, bias)`` (``fp8_quant.py:190-264, 460-516``),
which returns the gradient of the merged weight, is checked the same way.
"""
from __future__ import annotations

import numpy as np
import pytest
import torch
import torch.nn.functional as F

from oracle import lokr as OL
from oracle import mxfp8 as OQ
from oracle import tlokr as OT

pytestmark = pytest.mark.gpu
RTOL, ATOL = 1e-2, 2e-2
BF16 = torch.bfloat16


def _ops():
    from anima_trainer_sm120_b200 import _lib, ops
    return ops, _lib


def _plain_and_tiled(t2d, *, row=True, col=False):
    """(row_plain, row_tiled, col_plain, col_tiled) MXFP8 operands of a bf16 matrix: the PLAIN scales feed the
    oracle, the TILED ones (same codes, same scale values) feed the GEMM."""
    ops, _ = _ops()
    r, c = ops.mx_quantize(t2d.contiguous(), rowwise=row, colwise=col, layout=0)
    return r, (ops.mx_retile(r) if r else None), c, (ops.mx_retile(c) if c else None)


def _np(op):
    return op.codes.cpu().numpy(), op.scales.cpu().numpy()


def _oracle(a, b, *, out_bf16=True, bias=None):
    return OQ.matmul(*_np(a), *_np(b), None if bias is None else bias.float().cpu().numpy(), out_bf16=out_bf16)


def _rel_max(ref, got) -> float:
    ref, got = torch.as_tensor(ref).double(), torch.as_tensor(got).double()
    return float((ref - got).abs().max() / (ref.abs().max() + 1e-30))


def _violations(ref, got) -> float:
    ref, got = torch.as_tensor(ref).double(), torch.as_tensor(got).double()
    return float(((ref - got).abs() > ATOL + RTOL * ref.abs()).double().mean())


def _close(got, want, rtol=RTOL, atol=ATOL):
    np.testing.assert_allclose(torch.as_tensor(got).float().cpu().numpy(), np.asarray(want, dtype=np.float32),
                               rtol=rtol, atol=atol)


def _close_sum(got, term_a, term_b, rtol=RTOL, atol=ATOL):
    """got == term_a + term_b where each term was rounded to bf16 on its own before the bf16 add (as the
    reference's ``torch.add(base, delta, alpha=)`` on bf16 tensors does): the error scales with the terms, not
    with their possibly cancelling sum."""
    got = torch.as_tensor(got).float().cpu().numpy()
    bound = atol + rtol * (np.abs(term_a) + np.abs(term_b))
    err = np.abs(got - (term_a + term_b))
    assert (err <= bound).all(), (float(err.max()), int((err > bound).sum()))


# ----------------------------------------------------------------------------------------------- config 1
def test_config1_lokr_linear_at_its_stated_shape(capsys):
    ops, lib = _ops()
    from anima_trainer_sm120_b200.fp8_quant import clear_activation_memo, lokr_linear_fused
    g = torch.Generator().manual_seed(42)
    x = torch.randn(2048, 2048, generator=g).to(BF16)
    W = (torch.randn(8192, 2048, generator=g) * 0.02).to(BF16)
    w1 = torch.randn(8, 8, generator=g) * 0.1
    w2 = torch.randn(1024, 256, generator=g) * 0.02
    gy = torch.randn(2048, 8192, generator=g).to(BF16)            # the fixed N(0,1) probe of tests/test_tlokr.py:179-181
    alpha = 1.0
    xd = x.cuda().requires_grad_(True)
    w1d, w2d = w1.cuda().requires_grad_(True), w2.cuda().requires_grad_(True)
    clear_activation_memo()
    y = lokr_linear_fused(xd, W.cuda(), None, w1d, w2d, alpha)
    y.backward(gy.cuda())
    torch.cuda.synchronize()
    lib.check_status_word(y.device)

    # the operands the node made, made again (the quantisers are deterministic): PLAIN scales for the oracle
    x_row, _, x_col, _ = _plain_and_tiled(x.cuda(), row=True, col=True)
    _, w_row, w_col = ops.lokr_merge_quantize(W.cuda(), w1.cuda(), w2.cuda(), alpha, want_merged=False, rowwise=True,
                                              colwise=True, layout=0)
    g_row, _, g_col, _ = _plain_and_tiled(gy.cuda(), row=True, col=True)
    # codes and scales of x bit-exact against the oracle quantiser (the merged weight's are covered where
    # the merge kernel is tested)
    codes, scales = OQ.quantize_rowwise(x.float().numpy())
    assert np.array_equal(codes, x_row.codes.cpu().numpy()) and np.array_equal(scales, x_row.scales.cpu().numpy())

    _close(y.detach(), _oracle(x_row, w_row))                                 # y  = x . W'^T
    _close(xd.grad, _oracle(g_row, w_col))                                    # dx = gy . W'
    dW = torch.from_numpy(_oracle(g_col, x_col, out_bf16=False))              # dW = gy^T . x   (fp32, oracle)
    dw1_o, dw2_o = OL.kron_backward(dW, w1, w2, alpha)
    assert _rel_max(dw1_o, w1d.grad.cpu()) < 2e-3
    assert _rel_max(dw2_o, w2d.grad.cpu()) < 2e-3

    # against the reference's bf16 mode on the host
    y_b, dx_b, dw1_b, dw2_b = OL.lokr_linear_bf16(x, W, None, w1, w2, alpha, gy)
    report = {}
    for name, ref, got in (("y", y_b, y.detach()), ("dx", dx_b, xd.grad), ("dw1", dw1_b, w1d.grad),
                           ("dw2", dw2_b, w2d.grad)):
        report[name] = (_rel_max(ref, got.cpu()), _violations(ref, got.cpu()))
        assert report[name][0] < 0.10, (name, report[name])
    with capsys.disabled():
        print("\nconfig 1 vs bf16 mode (rel_max, fraction outside rtol 1e-2 / atol 2e-2): "
              + ", ".join(f"{k} {v[0]:.4f} / {v[1]:.3f}" for k, v in report.items()))


# ----------------------------------------------------------------------------------------------- config 2
def _acts(rows, cols, seed, std=1.0, outliers=True):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(rows, cols, generator=g) * std
    if outliers:
        idx = torch.randperm(cols, generator=g)[: max(1, -(-cols // 1000))]
        x[:, idx] *= 50.0
    return x.to(BF16)


def _tile_checks(c, a_plain, b_plain, tiles, *, out_bf16, rtol, atol):
    for r0, c0 in tiles:
        a = type(a_plain)(a_plain.codes[r0:r0 + 128], a_plain.scales[r0:r0 + 128], 0)
        b = type(b_plain)(b_plain.codes[c0:c0 + 256], b_plain.scales[c0:c0 + 256], 0)
        want = _oracle(a, b, out_bf16=out_bf16)
        _close(c[r0:r0 + 128, c0:c0 + 256], want, rtol, atol)


def _three_tiles(rows, cols):
    return [(0, 0), (rows - 128, cols - 256), ((rows // 2 + 77) // 128 * 128, (cols // 2) // 256 * 256)]


@pytest.mark.parametrize("N,K", [(2048, 2048), (6144, 2048), (8192, 2048), (2048, 8192)])
def test_config2_every_shape_and_direction_against_the_oracle(N, K, monkeypatch):
    monkeypatch.delenv("ANIMA_MX_GEMM_VARIANT", raising=False)     # the shape-chosen kernel: CTA pairs
    ops, lib = _ops()
    M = 32768
    x = _acts(M, K, 100 + N + K).cuda()
    w = _acts(N, K, 101 + N + K, std=0.02, outliers=False).cuda()
    gy = _acts(M, N, 102 + N + K, outliers=False).cuda()
    x_row, x_row_t, x_col, x_col_t = _plain_and_tiled(x, row=True, col=True)
    w_row, w_row_t, w_col, w_col_t = _plain_and_tiled(w, row=True, col=True)
    g_row, g_row_t, g_col, g_col_t = _plain_and_tiled(gy, row=True, col=True)
    del x, w, gy
    y = ops.mx_gemm(x_row_t, w_row_t)                               # forward  [M, N], contraction K
    _tile_checks(y, x_row, w_row, _three_tiles(M, N), out_bf16=True, rtol=RTOL, atol=ATOL)
    del y
    dx = ops.mx_gemm(g_row_t, w_col_t)                              # dgrad    [M, K], contraction N
    _tile_checks(dx, g_row, w_col, _three_tiles(M, K), out_bf16=True, rtol=RTOL, atol=ATOL)
    del dx
    dw = ops.mx_gemm(g_col_t, x_col_t, out_dtype=torch.float32)     # wgrad    [N, K], contraction M = 32768
    again = ops.mx_gemm(g_col_t, x_col_t, out_dtype=torch.float32)
    torch.cuda.synchronize()
    lib.check_status_word(dw.device)
    assert torch.equal(dw, again)                                   # fixed summation order
    _tile_checks(dw, g_col, x_col, _three_tiles(N, K), out_bf16=False, rtol=1e-3, atol=5e-2)


# ----------------------------------------------------------------------------------------------- config 4
# (name, in, out, batch, tokens per sample)
TLOKR_SHAPES = [("cross q/o", 2048, 2048, 8, 4096), ("cross k/v", 1024, 2048, 8, 512),
                ("mlp.layer1", 2048, 8192, 8, 1024), ("mlp.layer2", 8192, 2048, 8, 1024)]
RANK, MIN_RANK = 128, 64


def _tlokr_inputs(d_in, d_out, batch, tokens, seed=42):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(batch, tokens, d_in, generator=g).to(BF16)
    grad = torch.randn(batch, tokens, d_out, generator=g).to(BF16)
    w1 = torch.randn(8, 8, generator=g) * 0.3
    a = (torch.rand(d_out // 8, RANK, generator=g) * 2 - 1) / RANK ** 0.5           # kaiming-uniform-like
    b = torch.randn(RANK, d_in // 8, generator=g) * 0.2                             # re-randomised as the reference's tests do
    t = torch.rand(batch, generator=g)
    mask = OT.rank_mask(t, max_rank=RANK, min_rank=MIN_RANK, dtype=BF16)
    return x, grad, w1, a, b, mask


def _deq(op_plain):
    return torch.from_numpy(OQ.dequantize_rowwise(*_np(op_plain)))


@pytest.mark.parametrize("name,d_in,d_out,batch,tokens", TLOKR_SHAPES)
def test_config4_quantised_delta_chain_against_the_oracle(name, d_in, d_out, batch, tokens, capsys):
    ops, lib = _ops()
    from anima_trainer_sm120_b200 import tlokr
    from anima_trainer_sm120_b200.tlokr_kernels import rank_mix, rank_mix_wgrad
    x, grad, w1, a, b, mask = _tlokr_inputs(d_in, d_out, batch, tokens)
    uq, up, vq, vp = 8, 8, d_in // 8, d_out // 8
    rows8 = batch * tokens * 8
    dev = "cuda"
    c = w1.to(BF16)
    xd, md = x.to(dev), mask.to(dev)

    # ---- forward, stage by stage, every GEMM on identical codes
    a_row, a_row_t, a_col, a_col_t = _plain_and_tiled(a.to(BF16).to(dev), row=True, col=True)
    b_row, b_row_t, b_col, b_col_t = _plain_and_tiled(b.to(BF16).to(dev), row=True, col=True)
    g_row, g_row_t, g_col, g_col_t = _plain_and_tiled(xd.view(rows8, vq), row=True, col=True)
    hidden = ops.mx_gemm(g_row_t, b_row_t)                                           # [rows8, r]
    _close(hidden, _oracle(g_row, b_row))
    hidden4 = hidden.view(batch, tokens, 8, RANK)
    mixed = rank_mix(hidden4, c.to(dev), md)
    want_mix = OT.rank_mix_fp32(hidden4.cpu(), c, mask).to(BF16)
    assert torch.equal(mixed.cpu().view(torch.int16), want_mix.view(torch.int16))
    m_row, m_row_t, m_col, m_col_t = _plain_and_tiled(mixed.view(rows8, RANK), row=True, col=True)
    out = ops.mx_gemm(m_row_t, a_row_t)                                              # [rows8, vp]
    _close(out, _oracle(m_row, a_row))
    # the autograd node is this chain
    xg = xd.clone().requires_grad_(True)
    w1g, ag, bg = (p.to(dev).requires_grad_(True) for p in (w1, a, b))
    node_out = tlokr._MXStructuredLoKr.apply(xg, w1g, ag, bg, md)
    assert torch.equal(node_out.view(rows8, vp), out)
    # whole chain against the reference's structured algebra on the dequantised operands (fp32)
    x_dq = _deq(g_row).view(batch, tokens, d_in)
    a_dq, b_dq = _deq(a_row), _deq(b_row)
    want = OT.structured_delta_fwd(x_dq, c.float(), a_dq, b_dq, mask.float())
    rel_f, vio_f = _rel_max(want, node_out.cpu()), _violations(want, node_out.cpu())
    assert rel_f < 0.05, (name, rel_f)

    # ---- backward, stage by stage
    gd = grad.to(dev)
    node_out.backward(gd)
    gb_row, gb_row_t, gb_col, gb_col_t = _plain_and_tiled(gd.view(rows8, vp), row=True, col=True)
    g_a = ops.mx_gemm(gb_col_t, m_col_t, out_dtype=torch.float32)                    # grad^T @ mixed      [vp, r]
    _close(g_a, _oracle(gb_col, m_col, out_bf16=False), 1e-3, 1e-3 * float(g_a.abs().max()))
    g_mixed = ops.mx_gemm(gb_row_t, a_col_t)                                         # grad @ A            [rows8, r]
    _close(g_mixed, _oracle(gb_row, a_col))
    g_mixed4 = g_mixed.view(batch, tokens, 8, RANK)
    g_c = rank_mix_wgrad(g_mixed4, hidden4, md)
    want_c = OT.rank_mix_wgrad_fp64(g_mixed4.cpu(), hidden4.cpu(), mask)
    assert _rel_max(want_c, g_c.cpu()) < 1e-3
    g_hidden = rank_mix(g_mixed4, c.to(dev), md, transpose=True)
    want_gh = OT.rank_mix_fp32(g_mixed4.cpu(), c, mask, transpose=True).to(BF16)
    assert torch.equal(g_hidden.cpu().view(torch.int16), want_gh.view(torch.int16))
    gh_row, gh_row_t, gh_col, gh_col_t = _plain_and_tiled(g_hidden.view(rows8, RANK), row=True, col=True)
    g_b = ops.mx_gemm(gh_col_t, g_col_t, out_dtype=torch.float32)                    # grad_hidden^T @ grouped [r, vq]
    _close(g_b, _oracle(gh_col, g_col, out_bf16=False), 1e-3, 1e-3 * float(g_b.abs().max()))
    g_x = ops.mx_gemm(gh_row_t, b_col_t)                                             # grad_hidden @ B     [rows8, vq]
    _close(g_x, _oracle(gh_row, b_col))
    torch.cuda.synchronize()
    lib.check_status_word(torch.device(dev))
    # the node's gradients are these
    assert torch.equal(xg.grad.view(rows8, vq), g_x)
    torch.testing.assert_close(w1g.grad, g_c, rtol=0, atol=0)
    torch.testing.assert_close(ag.grad, g_a, rtol=0, atol=0)
    torch.testing.assert_close(bg.grad, g_b, rtol=0, atol=0)
    # and agree with the reference's manual backward on the dequantised operands
    gr_dq = _deq(gb_row).view(batch, tokens, d_out)
    wx, wc, wa, wb = OT.structured_delta_bwd(x_dq, c.float(), a_dq, b_dq, mask.float(), gr_dq)
    rels = {"gx": _rel_max(wx, xg.grad.cpu()), "gC": _rel_max(wc, w1g.grad.cpu()), "gA": _rel_max(wa, ag.grad.cpu()),
            "gB": _rel_max(wb, bg.grad.cpu())}
    with capsys.disabled():
        print(f"\nconfig 4 {name}: fwd rel_max {rel_f:.4f} (outside rtol 1e-2/atol 2e-2: {vio_f:.3f}); bwd "
              + ", ".join(f"{k} {v:.4f}" for k, v in rels.items()))
    assert all(v < 0.10 for v in rels.values()), rels


@pytest.mark.parametrize("name,d_in,d_out,batch,tokens", TLOKR_SHAPES)
def test_config4_one_node_quantised_tlokr_linear(name, d_in, d_out, batch, tokens):
    """``y = x W^T + bias + alpha * delta(x)`` as one node: forward and input gradient against the oracle sums of
    the base GEMM and the delta chain on identical codes; factor gradients against the stand-alone chain."""
    ops, lib = _ops()
    from anima_trainer_sm120_b200 import tlokr
    from anima_trainer_sm120_b200.fp8_quant import clear_activation_memo, quantize_weight
    from anima_trainer_sm120_b200.tlokr_kernels import rank_mix
    x, grad, w1, a, b, mask = _tlokr_inputs(d_in, d_out, batch, tokens, seed=43)
    dev = "cuda"
    alpha = 0.5
    g = torch.Generator().manual_seed(7)
    W = (torch.randn(d_out, d_in, generator=g) * 0.02).to(BF16)
    bias = (torch.randn(d_out, generator=g) * 0.1).to(BF16)
    rows, rows8, vq, vp = batch * tokens, batch * tokens * 8, d_in // 8, d_out // 8
    c = w1.to(BF16)
    xd, md = x.to(dev), mask.to(dev)
    W_mx = quantize_weight(W.to(dev))
    xg = xd.clone().requires_grad_(True)
    w1g, ag, bg = (p.to(dev).requires_grad_(True) for p in (w1, a, b))
    clear_activation_memo()
    y = tlokr._MXTLoKrLinear.apply(xg, W_mx, bias.to(dev), w1g, ag, bg, md, alpha)
    y.backward(grad.to(dev))
    torch.cuda.synchronize()
    lib.check_status_word(torch.device(dev))

    # oracle pieces on identical codes
    w_row, _, w_col, _ = _plain_and_tiled(W.to(dev), row=True, col=True)
    x_row, _, _, _ = _plain_and_tiled(xd.view(rows, d_in))
    a_row, a_row_t, a_col, a_col_t = _plain_and_tiled(a.to(BF16).to(dev), row=True, col=True)
    b_row, b_row_t, b_col, b_col_t = _plain_and_tiled(b.to(BF16).to(dev), row=True, col=True)
    gx_row, gx_row_t, _, _ = _plain_and_tiled(xd.view(rows8, vq))
    hidden4 = ops.mx_gemm(gx_row_t, b_row_t).view(batch, tokens, 8, RANK)
    mixed = rank_mix(hidden4, c.to(dev), md)
    m_row, _, _, _ = _plain_and_tiled(mixed.view(rows8, RANK))
    base = _oracle(x_row, w_row, out_bf16=False) + bias.float().numpy()[None, :]
    delta = _oracle(m_row, a_row, out_bf16=False).reshape(rows, d_out)
    _close_sum(y.detach().view(rows, d_out), base, alpha * delta)
    # input gradient: base dgrad + alpha * chain
    gd = grad.to(dev)
    gy_row, _, _, _ = _plain_and_tiled(gd.view(rows, d_out))
    gb_row, gb_row_t, _, _ = _plain_and_tiled(gd.view(rows8, vp))
    g_mixed4 = ops.mx_gemm(gb_row_t, a_col_t, alpha=alpha).view(batch, tokens, 8, RANK)
    g_hidden = rank_mix(g_mixed4, c.to(dev), md, transpose=True)
    gh_row, _, _, _ = _plain_and_tiled(g_hidden.view(rows8, RANK))
    _close_sum(xg.grad.view(rows, d_in), _oracle(gy_row, w_col, out_bf16=False),
               _oracle(gh_row, b_col, out_bf16=False).reshape(rows, d_in))
    # factor gradients: alpha times the stand-alone chain's
    xs = xd.clone().requires_grad_(True)
    w1s, as_, bs = (p.to(dev).requires_grad_(True) for p in (w1, a, b))
    tlokr._MXStructuredLoKr.apply(xs, w1s, as_, bs, md).backward(gd)
    for got, ref in ((w1g.grad, w1s.grad), (ag.grad, as_.grad), (bg.grad, bs.grad)):
        assert _rel_max(alpha * ref.cpu(), got.cpu()) < 2e-3


# ------------------------------------------------------------------------- reference-signature LoKr linear
@pytest.mark.parametrize("with_bias", [False, True])
def test_reference_signature_lokr_linear_returns_the_merged_weight_gradient(with_bias):
    ops, lib = _ops()
    from anima_trainer_sm120_b200 import fp8_quant
    g = torch.Generator().manual_seed(9)
    rows, K, N = 4096, 1024, 2048
    x = torch.randn(8, rows // 8, K, generator=g).to(BF16)
    W = (torch.randn(N, K, generator=g) * 0.02).to(BF16)
    bias = (torch.randn(N, generator=g) * 0.1).to(BF16) if with_bias else None
    gy = torch.randn(8, rows // 8, N, generator=g).to(BF16)
    res = {}
    for fn in (fp8_quant.fp8_lokr_linear, fp8_quant.mxfp8_lokr_linear):
        xd = x.cuda().requires_grad_(True)
        Wd = W.cuda().requires_grad_(True)
        bd = None if bias is None else bias.cuda().requires_grad_(True)
        fp8_quant.clear_activation_memo()
        y = fn(xd, Wd, bd)
        y.backward(gy.cuda())
        res[fn.__name__] = (y.detach(), xd.grad, Wd.grad, None if bd is None else bd.grad)
    torch.cuda.synchronize()
    lib.check_status_word(torch.device("cuda"))
    for u, v in zip(*res.values()):                                                  # one operator behind both names
        assert (u is None and v is None) or torch.equal(u, v)
    y, dx, dW, db = res["fp8_lokr_linear"]
    assert dW.shape == W.shape and dW.dtype == W.dtype
    x_row, _, x_col, _ = _plain_and_tiled(x.cuda().view(rows, K), row=True, col=True)
    w_row, _, w_col, _ = _plain_and_tiled(W.cuda(), row=True, col=True)
    g_row, _, g_col, _ = _plain_and_tiled(gy.cuda().view(rows, N), row=True, col=True)
    _close(y.view(rows, N), _oracle(x_row, w_row, bias=bias))
    _close(dx.view(rows, K), _oracle(g_row, w_col))
    want_dW = _oracle(g_col, x_col)                                                  # gy^T . x, rounded to bf16 like W
    _close(dW, want_dW, rtol=RTOL, atol=ATOL * float(np.abs(want_dW).max()) / 8)
    if with_bias:
        torch.testing.assert_close(db.float().cpu(), gy.view(rows, N).float().sum(0), rtol=2e-2, atol=0.5)
    # against bf16 autograd of F.linear (the reference's acceptance for the quantised path)
    xr, Wr = x.float().requires_grad_(True), W.float().requires_grad_(True)
    F.linear(xr, Wr, None if bias is None else bias.float()).backward(gy.float())
    assert _rel_max(xr.grad, dx.cpu()) < 0.10 and _rel_max(Wr.grad, dW.cpu()) < 0.10


# ------------------------------------------------------------------------------- a second device in one process
def test_gemm_and_column_quantiser_on_a_second_device():
    """Kernels that opt in to large dynamic shared memory must do so on every device they run on."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two visible GPUs")
    ops, lib = _ops()
    for dev in ("cuda:0", "cuda:1"):
        x = _acts(512, 256, 5).to(dev)
        w = _acts(384, 256, 6, std=0.02, outliers=False).to(dev)
        x_row, x_row_t, x_col, _ = _plain_and_tiled(x, row=True, col=True)      # the column form runs the copy-engine-fed kernel
        w_row, w_row_t, _, _ = _plain_and_tiled(w)
        cq, sq = OQ.quantize_colwise_T(x.float().cpu().numpy())
        assert np.array_equal(cq, x_col.codes.cpu().numpy()) and np.array_equal(sq, x_col.scales.cpu().numpy())
        y = ops.mx_gemm(x_row_t, w_row_t)
        torch.cuda.synchronize(dev)
        lib.check_status_word(torch.device(dev))
        _close(y, _oracle(x_row, w_row))
