"""GPU parity: the tcgen05 block-scaled MXFP8 GEMM through the C ABI.

Gate 1 (kernel correctness): kernel vs the dequantise-then-matmul oracle on IDENTICAL codes and
scales, rtol 1e-2 / atol 2e-2 (differences are accumulation order and the bf16 store).
Gate 2 (the reference's own acceptance, tests/sanity_mxfp8_triton.py:29-37, :86-90): quantised
forward / dgrad (and wgrad) vs the bf16 path, max_err / max|ref| < 0.10.
Full-size checks use size-independent properties (linearity in a scale byte, agreement of an
output tile with the oracle, transposition symmetry)."""
from __future__ import annotations

import numpy as np
import pytest
import torch


from oracle import mxfp8 as OQ

pytestmark = pytest.mark.gpu
RTOL, ATOL = 1e-2, 2e-2
BF16 = torch.bfloat16


def _ops():
    from anima_trainer_sm120_b200 import _lib, ops
    return ops, _lib


def _acts(rows, cols, seed, std=1.0, outliers=True):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(rows, cols, generator=g) * std
    if outliers:
        idx = torch.randperm(cols, generator=g)[: max(1, -(-cols // 1000))]
        x[:, idx] *= 50.0
    return x.to(BF16)


def _oracle_product(a, b, bias=None, out_bf16=True):
    """Oracle on the kernel's own operands (PLAIN scales)."""
    return OQ.matmul(a.codes.cpu().numpy(), a.scales.cpu().numpy(), b.codes.cpu().numpy(), b.scales.cpu().numpy(),
                     None if bias is None else bias.float().cpu().numpy(), out_bf16=out_bf16)


@pytest.fixture(params=["1", "2"], ids=["one-cta-tiles", "cta-pair-tiles"])
def variant(request, monkeypatch):
    """Run a test once per GEMM kernel family (the library reads the variable on every call)."""
    monkeypatch.setenv("ANIMA_MX_GEMM_VARIANT", request.param)
    return request.param


def _gemm_case(M, N, K, seed, bias=False, out_dtype=BF16):
    ops, lib = _ops()
    x = _acts(M, K, seed).cuda()
    w = _acts(N, K, seed + 1, std=0.02, outliers=False).cuda()
    xa, _ = ops.mx_quantize(x, rowwise=True, layout=0)
    wb, _ = ops.mx_quantize(w, rowwise=True, layout=0)
    b = (torch.randn(N, generator=torch.Generator().manual_seed(seed + 2)) * 0.5).to(BF16).cuda() if bias else None
    c = ops.mx_gemm(ops.mx_retile(xa), ops.mx_retile(wb), bias=b, out_dtype=out_dtype)
    torch.cuda.synchronize()
    lib.check_status_word(c.device)
    want = _oracle_product(xa, wb, b, out_bf16=out_dtype == BF16)
    np.testing.assert_allclose(c.float().cpu().numpy(), want, rtol=RTOL, atol=ATOL)
    return c, want


def test_golden_operands(golden):
    """The reference's own codes and scales in, the reference's dequantise+matmul product out."""
    ops, lib = _ops()
    g = golden("gemm")
    def op(c, s):
        return ops.mx_retile(ops.MXOperand(torch.from_numpy(g[c]).cuda(), torch.from_numpy(g[s]).cuda(), 0))
    y = ops.mx_gemm(op("x_codes", "x_scales"), op("w_codes", "w_scales"))
    gx = ops.mx_gemm(op("g_codes", "g_scales"), op("wT_codes", "wT_scales"))
    lib.check_status_word(y.device)
    np.testing.assert_allclose(y.float().cpu().numpy(), OQ.bf16_bits_to_f32(g["y"]), rtol=RTOL, atol=ATOL)
    np.testing.assert_allclose(gx.float().cpu().numpy(), OQ.bf16_bits_to_f32(g["gx"]), rtol=RTOL, atol=ATOL)


@pytest.mark.parametrize("M,N,K", [
    (128, 128, 128),     # one tile, one K-block, narrow-N kernel
    (128, 256, 128),     # one tile of the wide kernel
    (128, 256, 512),     # ring wraps once
    (256, 512, 1024),    # several tiles per CTA are not needed yet: 4 tiles
    (384, 128, 2048),    # narrow kernel, long K (ring wraps 4x)
    (1024, 2048, 256),   # 64 tiles
])
def test_tile_aligned_shapes(M, N, K, variant):
    _gemm_case(M, N, K, seed=M + N + K)


@pytest.mark.parametrize("M,N,K", [
    (100, 72, 96),       # every dimension ragged (K % 32 == 0, N % 8 == 0)
    (130, 264, 160),     # one row / 8 columns past a tile edge, K tail of 32
    (1, 8, 32),          # smallest legal problem
    (257, 384, 416),     # N = 1.5 wide tiles: second scale chunk of the last tile is clamped
    (4096, 2048, 1024),  # cross-attn k/v shape (8 x 512 text tokens)
])
def test_ragged_shapes(M, N, K, variant):
    _gemm_case(M, N, K, seed=M * 3 + N)


def test_more_tiles_than_sms_exercises_both_accumulator_buffers(variant):
    # 320 (one CTA) / 160 (pair) tiles on 148 CTAs / 74 pairs: every CTA runs >= 2 tiles
    _gemm_case(20480, 512, 256, seed=11)
    _gemm_case(40960, 512, 128, seed=13)
    _gemm_case(20480, 128, 384, seed=12)


@pytest.mark.parametrize("M,N,K", [
    (128, 256, 32768),   # T-LoKr dB shape class: one tile, 256 K-blocks
    (256, 128, 16384),   # dA shape class: two tiles
    (128, 1024, 8192),   # four wide tiles
    (1024, 128, 8192),   # eight narrow tiles
    (100, 72, 4128),     # ragged tile, K tail of 32
])
@pytest.mark.parametrize("out_dtype", [BF16, torch.float32])
def test_split_k_matches_oracle_and_single_pass(M, N, K, out_dtype):
    """Small outputs with a long contraction are split over K into fp32 partial tiles summed in a fixed
    order: same oracle tolerance, agreement with the unsplit kernel, bit-identical on repetition."""
    ops, lib = _ops()
    assert lib.load().anima_mx_gemm_workspace_bytes(M, N, K) > 0
    x = _acts(M, K, M + K).cuda()
    w = _acts(N, K, N + K, std=0.02, outliers=False).cuda()
    bias = (torch.randn(N, generator=torch.Generator().manual_seed(3)) * 0.5).to(BF16).cuda()
    xa, _ = ops.mx_quantize(x, rowwise=True, layout=0)
    wb, _ = ops.mx_quantize(w, rowwise=True, layout=0)
    a, b = ops.mx_retile(xa), ops.mx_retile(wb)
    c = ops.mx_gemm(a, b, bias=bias, out_dtype=out_dtype)
    again = ops.mx_gemm(a, b, bias=bias, out_dtype=out_dtype)
    single = ops.mx_gemm(a, b, bias=bias, out_dtype=out_dtype, split_k=False)
    torch.cuda.synchronize()
    lib.check_status_word(c.device)
    want = _oracle_product(xa, wb, bias, out_bf16=out_dtype == BF16)
    np.testing.assert_allclose(c.float().cpu().numpy(), want, rtol=RTOL, atol=ATOL)
    assert torch.equal(c, again)
    torch.testing.assert_close(c.float(), single.float(), rtol=1e-2 if out_dtype == BF16 else 1e-4, atol=1e-3)


@pytest.mark.parametrize("width", ["192", "256"])
@pytest.mark.parametrize("M,N,K,bias,out_dtype", [
    (512, 384, 256, True, BF16),            # one tile column at 256 (128 of it outside N), two at 192
    (1024, 1152, 512, False, BF16),         # 4 x 256 + a narrow column / 6 x 192
    (264, 2112, 1024, True, BF16),          # 8 x 256 + 64 valid columns in the narrow one; ragged M
    (19200, 512, 640, False, BF16),         # 150 tiles at 256, 225 at 192: three rounds on 74 pairs, both buffers reused
    (2048, 2048, 16384, False, torch.float32),   # long contraction, fp32 chunks through the single staging buffer
    (1536, 768, 8192, True, torch.float32),      # fewer tiles than pairs: every tile split along K, partial tiles
])
def test_pair_kernel_at_both_tile_widths(M, N, K, bias, out_dtype, width, monkeypatch):
    """The CTA-pair kernel picks 256-wide tiles (overlapped accumulator buffers) from K = 4096 up and 192-wide
    ones below; both forms must serve every shape."""
    monkeypatch.setenv("ANIMA_MX_GEMM_VARIANT", "2")
    monkeypatch.setenv("ANIMA_MX_GEMM_BN", width)
    _gemm_case(M, N, K, seed=41, bias=bias, out_dtype=out_dtype)


@pytest.mark.parametrize("M,N,K", [(256, 512, 256), (200, 136, 96), (2048, 256, 128), (128, 256, 8192)])
def test_alpha_and_residual_epilogue(M, N, K, variant):
    """C = alpha * A.B^T + bias + residual, also written over the residual buffer itself."""
    ops, lib = _ops()
    x = _acts(M, K, M + 1).cuda()
    w = _acts(N, K, N + 2, std=0.02, outliers=False).cuda()
    g = torch.Generator().manual_seed(M + N + K)
    bias = (torch.randn(N, generator=g) * 0.5).to(BF16).cuda()
    res = torch.randn(M, N, generator=g).to(BF16).cuda()
    xa, _ = ops.mx_quantize(x, rowwise=True, layout=0)
    wb, _ = ops.mx_quantize(w, rowwise=True, layout=0)
    a, b = ops.mx_retile(xa), ops.mx_retile(wb)
    alpha = 0.375
    want = alpha * _oracle_product(xa, wb, None, out_bf16=False) + bias.float().cpu().numpy() + res.float().cpu().numpy()
    c = ops.mx_gemm(a, b, bias=bias, residual=res, alpha=alpha)
    c32 = ops.mx_gemm(a, b, bias=bias, residual=res, alpha=alpha, out_dtype=torch.float32)
    inplace = res.clone()
    ops.mx_gemm(a, b, bias=bias, residual=inplace, alpha=alpha, out=inplace)
    torch.cuda.synchronize()
    lib.check_status_word(c.device)
    np.testing.assert_allclose(c.float().cpu().numpy(), want, rtol=RTOL, atol=ATOL)
    np.testing.assert_allclose(c32.cpu().numpy(), want, rtol=1e-3, atol=2e-3)
    # in place the CTA-pair kernel lets its stores add the (bf16-rounded) tile to C: one more rounding
    np.testing.assert_allclose(inplace.float().cpu().numpy(), want, rtol=RTOL, atol=ATOL)


def test_split_k_is_not_used_for_large_outputs_or_short_contractions():
    _, lib = _ops()
    f = lib.load().anima_mx_gemm_workspace_bytes
    assert f(32768, 2048, 2048) == 0 and f(128, 128, 2048) == 0 and f(32768, 128, 32768) == 0


def test_bias_and_fp32_output(variant):
    _gemm_case(256, 512, 256, seed=5, bias=True)
    _gemm_case(256, 512, 256, seed=6, bias=True, out_dtype=torch.float32)
    _gemm_case(200, 136, 96, seed=7, out_dtype=torch.float32)


def test_scale_bytes_are_applied_per_block(variant):
    """Doubling one operand's scale byte for a single (row-tile, K-block) changes exactly the rows
    of that block's contribution: checks the shared->tensor-memory scale path and the sf_id
    selection of each of the four K sub-blocks."""
    ops, lib = _ops()
    M, N, K = 256, 256, 256
    x = _acts(M, K, 1, outliers=False).cuda()
    w = _acts(N, K, 2, std=0.02, outliers=False).cuda()
    xa, _ = ops.mx_quantize(x, rowwise=True, layout=0)
    wb, _ = ops.mx_quantize(w, rowwise=True, layout=0)
    for kb in range(K // 32):
        for who in ("a", "b"):
            xs, ws = xa.scales.clone(), wb.scales.clone()
            (xs if who == "a" else ws)[5:40, kb] += 1
            (xs if who == "a" else ws)[130:250, kb] += 2
            a2 = ops.MXOperand(xa.codes, xs, 0)
            b2 = ops.MXOperand(wb.codes, ws, 0)
            c = ops.mx_gemm(ops.mx_retile(a2), ops.mx_retile(b2), out_dtype=torch.float32)
            want = _oracle_product(a2, b2, out_bf16=False)
            np.testing.assert_allclose(c.cpu().numpy(), want, rtol=1e-3, atol=1e-3)
    lib.check_status_word(x.device)


def _rel_max(ref, got):
    return float((ref.float() - got.float()).abs().max() / (ref.float().abs().max() + 1e-9))


@pytest.mark.parametrize("D_in,D_out", [(2048, 2048), (1024, 2048), (2048, 8192), (8192, 2048)])
def test_reference_acceptance_fwd_dgrad_wgrad(D_in, D_out):
    """The reference's sanity shapes (tests/sanity_mxfp8_triton.py:86-90) at BS = 4096 rows: forward,
    dgrad and wgrad through the quantiser + GEMM vs bf16 matmuls, rel_max < 0.10; and the frozen
    linear autograd op with the reference's signature."""
    ops, lib = _ops()
    from anima_trainer_sm120_b200 import mxfp8_gemm as mg
    torch.manual_seed(0)
    BS = 4096
    x = torch.randn(BS, D_in, device="cuda", dtype=BF16)
    W = (torch.randn(D_out, D_in, device="cuda") / D_in ** 0.5).to(BF16)
    gy = torch.randn(BS, D_out, device="cuda", dtype=BF16)
    xr, xc = ops.mx_quantize(x, rowwise=True, colwise=True)
    wr, wc = ops.mx_quantize(W, rowwise=True, colwise=True)
    gr, gc = ops.mx_quantize(gy, rowwise=True, colwise=True)
    y = ops.mx_gemm(xr, wr)                 # x . W^T
    dx = ops.mx_gemm(gr, wc)                # gy . W      (contraction over D_out)
    dw = ops.mx_gemm(gc, xc)                # gy^T . x    (contraction over the rows)
    lib.check_status_word(x.device)
    assert _rel_max(x @ W.t(), y) < 0.10
    assert _rel_max(gy @ W, dx) < 0.10
    assert _rel_max(gy.t() @ x, dw) < 0.10
    # autograd op, reference signature (mxfp8_gemm.py:342-419)
    W_fwd, W_bwd = mg.quantize_weight_for_lhs(W), mg.quantize_weight_for_dgrad(W)
    assert W_bwd.data.shape == W.shape and W_bwd.scales.shape == (D_in, D_out // 32)
    xk = x.clone().requires_grad_(True)
    yk = mg.mxfp8_frozen_linear_triton(xk, W_fwd, W_bwd, None)
    yk.float().pow(2).mean().backward()
    xr_ = x.clone().requires_grad_(True)
    yr = torch.nn.functional.linear(xr_, W)
    yr.float().pow(2).mean().backward()
    assert _rel_max(yr, yk) < 0.10 and _rel_max(xr_.grad, xk.grad) < 0.10
    assert torch.equal(yk, y)


def test_reference_call_pattern_mxfp8_matmul():
    """mxfp8_matmul with the stride arguments of both reference call sites (:375-380, :409-414)."""
    ops, _ = _ops()
    from anima_trainer_sm120_b200 import mxfp8_gemm as mg
    x = _acts(256, 512, 3).cuda()
    W = _acts(384, 512, 4, std=0.02, outliers=False).cuda()
    gy = _acts(256, 384, 5, outliers=False).cuda()
    xb, W_fwd, W_bwd, gb = mg.quantize_rowwise(x), mg.quantize_weight_for_lhs(W), mg.quantize_weight_for_dgrad(W), mg.quantize_rowwise(gy)
    y = mg.mxfp8_matmul(xb, W_fwd.data, W_fwd.scales, M=256, N=384, K=512,
                        B_stride_k=W_fwd.data.stride(1), B_stride_n=W_fwd.data.stride(0))
    gx = mg.mxfp8_matmul(gb, W_bwd.data, W_bwd.scales, M=256, N=512, K=384,
                         B_stride_k=W_bwd.data.stride(0), B_stride_n=W_bwd.data.stride(1))
    want_y = OQ.matmul(xb.data.cpu().numpy(), xb.scales.cpu().numpy(), W_fwd.data.cpu().numpy(), W_fwd.scales.cpu().numpy())
    np.testing.assert_allclose(y.float().cpu().numpy(), want_y, rtol=RTOL, atol=ATOL)
    wT = W_bwd.data.t().contiguous()
    want_gx = OQ.matmul(gb.data.cpu().numpy(), gb.scales.cpu().numpy(), wT.cpu().numpy(), W_bwd.scales.cpu().numpy())
    np.testing.assert_allclose(gx.float().cpu().numpy(), want_gx, rtol=RTOL, atol=ATOL)
    with pytest.raises(NotImplementedError):
        mg.mxfp8_matmul(xb, W_fwd.data, W_fwd.scales, M=256, N=384, K=512, B_stride_k=512, B_stride_n=1)
    deq = mg.dequantize_rowwise(xb, tuple(x.shape))
    assert _rel_max(x, deq) < 0.10


def test_full_size_config2_properties():
    """Config 2, (N, K) = (8192, 2048) at M = 32768: three disjoint output tiles against the oracle
    on identical codes, the wgrad GEMM against its transposed formulation, and exact zero rows for
    zero activations."""
    ops, lib = _ops()
    M, N, K = 32768, 8192, 2048
    x = _acts(M, K, 42).cuda()
    x[777] = 0
    w = _acts(N, K, 43, std=0.02, outliers=False).cuda()
    xa, _ = ops.mx_quantize(x, rowwise=True, layout=0)
    wb, _ = ops.mx_quantize(w, rowwise=True, layout=0)
    c = ops.mx_gemm(ops.mx_retile(xa), ops.mx_retile(wb))
    lib.check_status_word(c.device)
    assert not bool(c[777].any())
    for r0, c0 in [(0, 0), (32768 - 128, 8192 - 256), (12345 // 128 * 128, 4096)]:
        a = ops.MXOperand(xa.codes[r0:r0 + 128], xa.scales[r0:r0 + 128], 0)
        b = ops.MXOperand(wb.codes[c0:c0 + 256], wb.scales[c0:c0 + 256], 0)
        np.testing.assert_allclose(c[r0:r0 + 128, c0:c0 + 256].float().cpu().numpy(), _oracle_product(a, b),
                                   rtol=RTOL, atol=ATOL)
    # wgrad: dW = gy^T x over 32768 rows; (gy^T x)^T == x^T gy with the operands swapped
    gy = _acts(M, 2048, 44, outliers=False).cuda()
    _, gc = ops.mx_quantize(gy, rowwise=False, colwise=True)
    _, xc = ops.mx_quantize(x, rowwise=False, colwise=True)
    dw = ops.mx_gemm(gc, xc, out_dtype=torch.float32)
    dw_t = ops.mx_gemm(xc, gc, out_dtype=torch.float32)
    lib.check_status_word(c.device)
    # the same products summed in a different association (a tile of one may be K-split where the other's is
    # not): equal up to fp32 rounding of sums of 32768 terms
    torch.testing.assert_close(dw, dw_t.t(), rtol=1e-4, atol=2e-5 * float(dw.abs().max()))
    assert _rel_max(gy.float().t() @ x.float(), dw) < 0.10


@pytest.mark.parametrize("M,N,K", [(512, 768, 1024), (4096, 2048, 2048)])
def test_agrees_with_the_vendor_library_mxfp8_gemm(M, N, K):
    """Independent check on the GPU: cuBLASLt's block-scaled MXFP8 GEMM (torch._scaled_mm) consumes the very
    same code and TILED scale buffers (its swizzled layout is the 128 x 4 tiled layout) and must give the same
    product up to fp32 accumulation order. Skipped where the installed torch / cuBLASLt rejects the call."""
    ops, lib = _ops()
    from anima_trainer_sm120_b200.kernel_bench import cublaslt_mxfp8
    x = _acts(M, K, 21).cuda()
    w = _acts(N, K, 22, std=0.02, outliers=False).cuda()
    a, _ = ops.mx_quantize(x, rowwise=True)
    b, _ = ops.mx_quantize(w, rowwise=True)
    try:
        want = cublaslt_mxfp8(a, b)()
    except Exception as e:  # noqa: BLE001
        pytest.skip(f"torch._scaled_mm MXFP8 unavailable: {str(e)[:120]}")
    got = ops.mx_gemm(a, b)
    torch.cuda.synchronize()
    lib.check_status_word(got.device)
    torch.testing.assert_close(got.float(), want.float(), rtol=RTOL, atol=ATOL)
    assert float((got.float() - want.float()).abs().max()) <= 0.0625 * float(want.float().abs().max()) / 8


def _planes_from_rows(t: torch.Tensor) -> torch.Tensor:
    """[items, 8, r] -> the plane order [8 * items, r] (row i of item t at i * items + t)."""
    return t.transpose(0, 1).reshape(-1, t.shape[-1]).contiguous()


@pytest.mark.parametrize("M,N,K", [
    (256, 2048, 256),     # blocks of 256 columns against 192-wide tiles: runs of 192, 64|128, 128|64, 192 ... and a narrow tile
    (384, 1024, 128),     # blocks of 128: a tile touches two or three blocks; the last row tile is half empty
    (1024, 512, 512),     # blocks of 64
    (512, 512, 16384),    # fewer tiles than CTA pairs and a long contraction: every tile is K-split, the delta rides the last range
    (4096, 2048, 1024),   # cross-attention k / v on the text tokens
])
@pytest.mark.parametrize("width", ["192", "256"])
def test_low_rank_delta_as_extra_k_blocks(M, N, K, width, monkeypatch):
    """anima_mx_gemm_delta: C = A.B^T + bias + sum_r planes[i*M + m, r] * d[p, r] for column i * N/8 + p, against
    the oracle on identical codes; the planes come from the quantising mix, checked against its plain row form.
    Run at both tile widths of the CTA-pair kernel (the runs of a tile's columns inside one block differ)."""
    monkeypatch.setenv("ANIMA_MX_GEMM_BN", width)
    ops, lib = _ops()
    from oracle import tlokr as OT
    g = torch.Generator().manual_seed(M + N + K)
    x = _acts(M, K, 31).cuda()
    w = _acts(N, K, 32, std=0.02, outliers=False).cuda()
    bias = (torch.randn(N, generator=g) * 0.3).to(BF16).cuda()
    blk = N // 8
    batch = 2
    hidden = torch.randn(batch, M // batch, 8, 128, generator=g).to(BF16).cuda()
    cmat = (torch.randn(8, 8, generator=g) * 0.4).to(BF16).cuda()
    mask = OT.rank_mask(torch.rand(batch, generator=g), max_rank=128, min_rank=64, dtype=BF16).cuda()
    d = (torch.randn(blk, 128, generator=g) * 0.05).to(BF16).cuda()
    xa, _ = ops.mx_quantize(x, rowwise=True, layout=0)
    wb, _ = ops.mx_quantize(w, rowwise=True, layout=0)
    dq, _ = ops.mx_quantize(d, rowwise=True, layout=0)
    planes, col = ops.tlokr_rank_mix_quant_planes(hidden, cmat, mask, False, colwise=True)
    # the planes hold the codes of the plain row form, reordered; the column form is unchanged
    row, col2, _ = ops.tlokr_rank_mix_quant(hidden, cmat, mask, False, rowwise=True, colwise=True)
    assert torch.equal(planes.codes, _planes_from_rows(row.codes.view(M, 8, 128)))
    assert torch.equal(col.codes, col2.codes) and torch.equal(col.scales, col2.scales)
    mixed = ops.tlokr_rank_mix(hidden, cmat, mask, False)                     # bf16 [batch, n, 8, 128]
    pl_plain, _ = ops.mx_quantize(_planes_from_rows(mixed.view(M, 8, 128)), rowwise=True, layout=0)
    assert torch.equal(pl_plain.codes, planes.codes)
    assert torch.equal(ops.mx_retile(pl_plain).scales, planes.scales)
    c = ops.mx_gemm_delta(ops.mx_retile(xa), ops.mx_retile(wb), planes, ops.mx_retile(dq), bias=bias)
    again = ops.mx_gemm_delta(ops.mx_retile(xa), ops.mx_retile(wb), planes, ops.mx_retile(dq), bias=bias)
    torch.cuda.synchronize()
    lib.check_status_word(c.device)
    assert torch.equal(c, again)
    base = _oracle_product(xa, wb, bias, out_bf16=False)
    delta = _oracle_product(pl_plain, dq, out_bf16=False).reshape(8, M, blk).transpose(1, 0, 2).reshape(M, N)
    want = base + delta
    got = c.float().cpu().numpy()
    bound = ATOL + RTOL * (np.abs(base) + np.abs(delta))
    assert (np.abs(got - want) <= bound).all(), float(np.abs(got - want).max())
    assert float(np.abs(delta).max()) > 0.05 * float(np.abs(base).max())      # the delta is not a rounding-level term


def test_delta_gemm_rejects_shapes_it_cannot_tile():
    ops, _ = _ops()
    assert not ops.can_fold_delta(128, 2048) and not ops.can_fold_delta(200, 2048) and not ops.can_fold_delta(256, 1032)
    assert ops.can_fold_delta(32768, 8192) and ops.can_fold_delta(4096, 1024)
