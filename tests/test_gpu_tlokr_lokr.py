"""GPU parity: T-LoKr rank mix / its weight gradient and the LoKr merged-weight kernels through
the C ABI vs the CPU oracle and the reference's golden vectors. Tolerances for rank_mix are the
reference's own (tests/test_tlokr.py:94, :105-110) where it is compared with the reference, and
bit-exactness where the fp32 oracle evaluates the same sums in the same order."""
from __future__ import annotations

import numpy as np
import pytest
import torch

from conftest import bf16_from_bits
from oracle import lokr as OL
from oracle import mxfp8 as OQ
from oracle import tlokr as OT

pytestmark = pytest.mark.gpu
BF16 = torch.bfloat16


def _ops():
    from anima_trainer_sm120_b200 import ops
    return ops


def test_rank_mix_golden_and_reference_case(golden):
    """The reference's CUDA test case (tests/test_tlokr.py:80-110): [2,*,8,128] bf16, masks 73/111."""
    from anima_trainer_sm120_b200.tlokr_kernels import rank_mix, rank_mix_wgrad
    g = golden("tlokr")
    hidden, weight, grad, mask = (bf16_from_bits(g[f"mix_{k}"]).cuda() for k in ("hidden", "weight", "grad", "mask"))
    for tr in (False, True):
        got = rank_mix(hidden, weight, mask, transpose=tr)
        torch.testing.assert_close(got.float().cpu(), bf16_from_bits(g[f"mix_cpu_t{int(tr)}"]).float(),
                                   rtol=2e-2, atol=6.25e-2)
        want = OT.rank_mix_fp32(hidden.cpu(), weight.cpu(), mask.cpu(), transpose=tr).to(BF16)
        assert torch.equal(got.cpu().view(torch.int16), want.view(torch.int16))
    got = rank_mix(hidden, weight, None)
    torch.testing.assert_close(got.float().cpu(), bf16_from_bits(g["mix_cpu_nomask"]).float(), rtol=2e-2, atol=6.25e-2)
    dc = rank_mix_wgrad(grad, hidden, mask)
    np.testing.assert_allclose(dc.cpu().numpy(), g["wgrad"], rtol=1e-2, atol=2e-1)       # test_tlokr.py:105-110
    np.testing.assert_allclose(dc.cpu().numpy(), OT.rank_mix_wgrad_fp64(grad.cpu(), hidden.cpu(), mask.cpu()).numpy(),
                               rtol=1e-4, atol=1e-2)


@pytest.mark.parametrize("B,n,r", [(1, 1, 8), (3, 7, 24), (2, 33, 128), (8, 4096, 128)])
def test_rank_mix_shapes_vs_oracle(B, n, r):
    ops = _ops()
    g = torch.Generator().manual_seed(B * 100 + n)
    hidden = torch.randn(B, n, 8, r, generator=g).to(BF16)
    grad = torch.randn(B, n, 8, r, generator=g).to(BF16)
    weight = torch.randn(8, 8, generator=g).to(BF16)
    t = torch.rand(B, generator=g)
    mask = OT.rank_mask(t, max_rank=r, min_rank=max(1, r // 2), dtype=BF16)
    big = B * n * r > 1 << 20
    sl = slice(0, 64) if big else slice(None)
    for m in (mask, None):
        for tr in (False, True):
            got = ops.tlokr_rank_mix(hidden.cuda(), weight.cuda(), None if m is None else m.cuda(), tr).cpu()
            want = OT.rank_mix_fp32(hidden[:, sl], weight, m, transpose=tr).to(BF16)
            assert torch.equal(got[:, sl].view(torch.int16), want.view(torch.int16))
        dc = ops.tlokr_rank_mix_wgrad(grad.cuda(), hidden.cuda(), None if m is None else m.cuda()).cpu()
        if big:  # float64 einsum over 33 M elements is still quick on the host
            pass
        want = OT.rank_mix_wgrad_fp64(grad, hidden, m)
        tol = 1e-3 * float(want.abs().max()) + 1e-3
        assert (dc.double() - want).abs().max() <= tol
        again = ops.tlokr_rank_mix_wgrad(grad.cuda(), hidden.cuda(), None if m is None else m.cuda()).cpu()
        assert torch.equal(dc, again)  # deterministic reduction


@pytest.mark.parametrize("B,n,r", [(2, 64, 128), (1, 16, 256), (3, 16, 512), (8, 512, 128)])
def test_rank_mix_emits_the_operands_of_its_output(B, n, r):
    """The quantising mix writes codes and tiled scales equal to quantising the bf16 mix afterwards, in the row
    form, the transposed column form, or both, with and without mask and transpose; the optional bf16 output is
    the plain kernel's."""
    ops = _ops()
    g = torch.Generator().manual_seed(B + n + r)
    hidden = (torch.randn(B, n, 8, r, generator=g) * 3.0).to(BF16).cuda()
    hidden[0, 0, :, :32] = 0                                  # an all-zero block takes the amax floor
    weight = torch.randn(8, 8, generator=g).to(BF16).cuda()
    mask = OT.rank_mask(torch.rand(B, generator=g), max_rank=r, min_rank=max(1, r // 2), dtype=BF16).cuda()
    for m in (mask, None):
        for tr in (False, True):
            mixed = ops.tlokr_rank_mix(hidden, weight, m, tr)
            want_row, want_col = ops.mx_quantize(mixed.view(-1, r), rowwise=True, colwise=True)
            for row, col in ((True, True), (True, False), (False, True)):
                got_row, got_col, out = ops.tlokr_rank_mix_quant(hidden, weight, m, tr, rowwise=row, colwise=col,
                                                                 want_bf16=row and col)
                if row:
                    assert torch.equal(got_row.codes, want_row.codes) and torch.equal(got_row.scales, want_row.scales)
                if col:
                    assert torch.equal(got_col.codes, want_col.codes) and torch.equal(got_col.scales, want_col.scales)
                assert (out is None) != (row and col)
                if out is not None:
                    assert torch.equal(out, mixed)


def test_rank_mix_quant_refuses_shapes_it_cannot_tile():
    ops = _ops()
    w = torch.eye(8, dtype=BF16, device="cuda")
    assert not ops.can_quantise_rank_mix(1, 16, 64) and not ops.can_quantise_rank_mix(1, 8, 128)
    with pytest.raises(ValueError):
        ops.tlokr_rank_mix_quant(torch.zeros(1, 16, 8, 64, dtype=BF16, device="cuda"), w, None, False)
    with pytest.raises(ValueError):
        ops.tlokr_rank_mix_quant(torch.zeros(1, 8, 8, 128, dtype=BF16, device="cuda"), w, None, False)


def test_rank_mix_rejects_unsupported_shapes():
    from anima_trainer_sm120_b200.tlokr_kernels import rank_mix
    h = torch.zeros(1, 2, 4, 16, dtype=BF16, device="cuda")
    with pytest.raises(NotImplementedError):
        rank_mix(h, torch.eye(4, dtype=BF16, device="cuda"), None)
    with pytest.raises(NotImplementedError):
        rank_mix(torch.zeros(1, 2, 8, 12, dtype=BF16, device="cuda"), torch.eye(8, dtype=BF16, device="cuda"), None)


# ------------------------------------------------------------------------------ LoKr weight kernels
def _lokr_case(N, K, seed, factor_dtype):
    g = torch.Generator().manual_seed(seed)
    w = (torch.randn(N, K, generator=g) * 0.02).to(BF16)
    w1 = (torch.randn(8, 8, generator=g) * 0.1).to(factor_dtype)
    w2 = (torch.randn(N // 8, K // 8, generator=g) * 0.02).to(factor_dtype)
    return w, w1, w2


@pytest.mark.parametrize("N,K", [(256, 256), (1024, 512), (2048, 1024)])
@pytest.mark.parametrize("factor_dtype", [torch.float32, BF16])
@pytest.mark.parametrize("alpha", [1.0, 0.5])
def test_merge_quantize_bit_exact(N, K, factor_dtype, alpha):
    ops = _ops()
    w, w1, w2 = _lokr_case(N, K, 42, factor_dtype)
    merged, row, col = ops.lokr_merge_quantize(w.cuda(), w1.cuda(), w2.cuda(), alpha, want_merged=True,
                                               rowwise=True, colwise=True, layout=0)
    want = OL.merged_weight(w, w1, w2, alpha)
    assert torch.equal(merged.cpu().view(torch.int16), want.view(torch.int16))
    codes, scales = OQ.quantize_rowwise(want.float().numpy())
    assert np.array_equal(row.codes.cpu().numpy(), codes) and np.array_equal(row.scales.cpu().numpy(), scales)
    codes, scales = OQ.quantize_colwise_T(want.float().numpy())
    assert np.array_equal(col.codes.cpu().numpy(), codes) and np.array_equal(col.scales.cpu().numpy(), scales)
    only, _, _ = ops.lokr_merge_quantize(w.cuda(), w1.cuda(), w2.cuda(), alpha, want_merged=True)
    assert torch.equal(only, merged)
    # identical to quantising the materialised merged weight with the plain quantiser
    r2, c2 = ops.mx_quantize(merged, rowwise=True, colwise=True, layout=1)
    _, r1, c1 = ops.lokr_merge_quantize(w.cuda(), w1.cuda(), w2.cuda(), alpha, want_merged=False,
                                        rowwise=True, colwise=True, layout=1)
    assert torch.equal(r1.codes, r2.codes) and torch.equal(r1.scales, r2.scales)
    assert torch.equal(c1.codes, c2.codes) and torch.equal(c1.scales, c2.scales)


def test_zero_delta_leaves_base_weight_exact():
    """LoKr initialises the delta to zero: merged must be W bit for bit (the T-LoKr analogue is
    pinned by tests/test_tlokr.py:117-125)."""
    ops = _ops()
    w, w1, w2 = _lokr_case(512, 512, 1, torch.float32)
    merged, _, _ = ops.lokr_merge_quantize(w.cuda(), w1.cuda(), torch.zeros_like(w2).cuda(), 1.0)
    assert torch.equal(merged.cpu().view(torch.int16), w.view(torch.int16))


@pytest.mark.parametrize("N,K", [(256, 256), (2048, 1024), (8192, 2048)])
@pytest.mark.parametrize("dw_dtype", [torch.float32, BF16])
def test_kron_backward_vs_oracle(N, K, dw_dtype):
    ops = _ops()
    w, w1, w2 = _lokr_case(N, K, 7, torch.float32)
    g = torch.Generator().manual_seed(8)
    dw = torch.randn(N, K, generator=g).to(dw_dtype)
    dw1, dw2 = ops.lokr_kron_backward(dw.cuda(), w1.cuda(), w2.cuda(), 0.5)
    dw1_o, dw2_o = OL.kron_backward(dw, w1, w2, 0.5)
    for got, want in ((dw1, dw1_o), (dw2, dw2_o)):
        tol = 1e-4 * float(want.abs().max()) + 1e-5
        assert (got.cpu().double() - want).abs().max() <= tol
    again = ops.lokr_kron_backward(dw.cuda(), w1.cuda(), w2.cuda(), 0.5)
    assert torch.equal(again[0], dw1) and torch.equal(again[1], dw2)
    # cross-check with autograd through torch.kron, as the reference's bf16 mode derives it
    w1a, w2a = w1.clone().requires_grad_(True), w2.clone().requires_grad_(True)
    (0.5 * torch.kron(w1a, w2a) * dw.float()).sum().backward()
    torch.testing.assert_close(dw1.cpu(), w1a.grad, rtol=1e-3, atol=1e-4 * float(w1a.grad.abs().max()))
    torch.testing.assert_close(dw2.cpu(), w2a.grad, rtol=1e-3, atol=1e-4 * float(w2a.grad.abs().max()))


@pytest.mark.parametrize("batch,n,k", [(1, 128, 128), (2, 192, 256), (8, 512, 1024), (3, 128, 96)])
@pytest.mark.parametrize("transpose", [False, True])
@pytest.mark.parametrize("masked", [True, False])
def test_hidden_gemm_mix_and_quantisation_in_one_kernel(batch, n, k, transpose, masked):
    """anima_tlokr_hidden_mix_planes == the factor GEMM (bf16 output) followed by the quantising mix, bit for bit:
    plane codes, tiled scales and the optional bf16 hidden tensor; and the hidden GEMM against the oracle."""
    ops = _ops()
    from anima_trainer_sm120_b200 import _lib
    g = torch.Generator().manual_seed(batch * 1000 + n + k)
    rows8 = batch * n * 8
    x = (torch.randn(rows8, k, generator=g)).to(BF16).cuda()
    x[5] = 0                                                   # an all-zero row: amax floor in hidden's consumers
    f = (torch.randn(128, k, generator=g) * 0.2).to(BF16).cuda()
    cmat = (torch.randn(8, 8, generator=g) * 0.4).to(BF16).cuda()
    mask = OT.rank_mask(torch.rand(batch, generator=g), max_rank=128, min_rank=64, dtype=BF16).cuda() if masked else None
    xq, _ = ops.mx_quantize(x, rowwise=True)
    fq, _ = ops.mx_quantize(f, rowwise=True)
    hidden = ops.mx_gemm(xq, fq).view(batch, n, 8, 128)
    want_planes, _ = ops.tlokr_rank_mix_quant_planes(hidden, cmat, mask, transpose)
    planes, hid = ops.tlokr_hidden_mix_planes(xq, fq, cmat, mask, batch, transpose, want_hidden=True)
    planes2, none = ops.tlokr_hidden_mix_planes(xq, fq, cmat, mask, batch, transpose)
    torch.cuda.synchronize()
    _lib.check_status_word(x.device)
    assert none is None
    assert torch.equal(hid, hidden)
    assert torch.equal(planes.codes, want_planes.codes) and torch.equal(planes.scales, want_planes.scales)
    assert torch.equal(planes2.codes, planes.codes) and torch.equal(planes2.scales, planes.scales)
    xp, _ = ops.mx_quantize(x, rowwise=True, layout=0)
    fp, _ = ops.mx_quantize(f, rowwise=True, layout=0)
    want_h = OQ.matmul(xp.codes.cpu().numpy(), xp.scales.cpu().numpy(), fp.codes.cpu().numpy(), fp.scales.cpu().numpy())
    np.testing.assert_allclose(hid.float().cpu().numpy().reshape(rows8, 128), want_h, rtol=1e-2, atol=2e-2)
