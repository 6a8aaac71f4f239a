"""Thin tensor-level wrappers, one per entry point of ``libanima_b200.so``.

Each wrapper validates dtypes, allocates the outputs with ``torch.empty`` (the
library itself never allocates), passes raw pointers plus the current CUDA
stream, and raises on a negative status. Nothing here computes on the host.
"""
from __future__ import annotations

from typing import NamedTuple

import torch

from . import _lib
from ._lib import SCALES_PLAIN, SCALES_TILED, check, ptr

BF16 = torch.bfloat16


def _bf16_2d(x: torch.Tensor, name: str) -> torch.Tensor:
    if x.dtype != BF16:
        raise TypeError(f"{name} must be bfloat16, got {x.dtype}")
    if x.dim() != 2:
        raise ValueError(f"{name} must be 2-D, got shape {tuple(x.shape)}")
    return x


class MXOperand(NamedTuple):
    """One K-major MXFP8 GEMM operand: e4m3 codes ``[rows, k]`` and its e8m0 scales."""

    codes: torch.Tensor   # uint8 [rows, k]
    scales: torch.Tensor  # uint8, PLAIN [rows, k/32] or TILED (flat, see anima_b200.h)
    layout: int           # SCALES_PLAIN | SCALES_TILED

    @property
    def rows(self) -> int:
        return self.codes.shape[0]

    @property
    def k(self) -> int:
        return self.codes.shape[1]


def scales_bytes(rows: int, k: int, layout: int) -> int:
    return check(_lib.load().anima_mx_scales_bytes(rows, k, layout))


def _alloc_scales(rows: int, k: int, layout: int, device) -> torch.Tensor:
    if layout == SCALES_PLAIN:
        return torch.empty((rows, k // 32), dtype=torch.uint8, device=device)
    return torch.empty(scales_bytes(rows, k, layout), dtype=torch.uint8, device=device)


def _quantize_call(entry: str, x: torch.Tensor, extra: tuple, rowwise: bool, colwise: bool, layout: int,
                   after_ld: tuple = ()) -> tuple[MXOperand | None, MXOperand | None]:
    dev = _lib.require_cuda(x)
    rows, cols = x.shape
    if rowwise and cols % 32:
        raise ValueError(f"rowwise quantisation needs cols % 32 == 0, got {cols}")
    if colwise and rows % 32:
        raise ValueError(f"columnwise quantisation needs rows % 32 == 0, got {rows}")
    row_op = col_op = None
    if rowwise:
        row_op = MXOperand(torch.empty((rows, cols), dtype=torch.uint8, device=dev),
                           _alloc_scales(rows, cols, layout, dev), layout)
    if colwise:
        col_op = MXOperand(torch.empty((cols, rows), dtype=torch.uint8, device=dev),
                           _alloc_scales(cols, rows, layout, dev), layout)
    if rows == 0 or cols == 0:   # empty tensors have no storage to point at
        return row_op, col_op
    with torch.cuda.device(dev):
        check(getattr(_lib.load(), entry)(
            ptr(x), *extra, rows, cols, x.stride(0) if rows > 1 else cols, *after_ld,
            ptr(row_op.codes) if row_op else None, ptr(row_op.scales) if row_op else None,
            ptr(col_op.codes) if col_op else None, ptr(col_op.scales) if col_op else None,
            layout, _lib.stream_ptr(dev)))
    return row_op, col_op


def mx_quantize(
    x: torch.Tensor, *, rowwise: bool = True, colwise: bool = False, layout: int = SCALES_TILED
) -> tuple[MXOperand | None, MXOperand | None]:
    """Quantise bf16 ``x [rows, cols]`` (last-dim stride 1) from one read.

    Returns ``(row_op, col_op)``: ``row_op`` is x quantised along its columns
    (``[rows, cols]``), ``col_op`` is x quantised along its rows and stored
    transposed (``[cols, rows]``) — i.e. ``quantize_rowwise(x.t().contiguous())``.
    """
    _bf16_2d(x, "x")
    if x.stride(1) != 1 and x.shape[1] > 1:
        x = x.contiguous()
    return _quantize_call("anima_mx_quantize", x, (), rowwise, colwise, layout)


def mx_quantize_gelu(
    h: torch.Tensor, grad_act: torch.Tensor | None = None, *, rowwise: bool = True, colwise: bool = False,
    layout: int = SCALES_TILED, act_out: torch.Tensor | None = None,
) -> tuple[MXOperand | None, MXOperand | None]:
    """MXFP8 forms of ``gelu(h)`` (``grad_act`` None) or of ``grad_act * gelu'(h)``, from one read of the bf16
    pre-activation ``h [rows, cols]``; the activation / its gradient is not written as a bf16 tensor unless
    ``act_out`` (bf16, contiguous, h's shape) is given to receive it."""
    _bf16_2d(h, "h")
    h = h.contiguous()
    if grad_act is not None:
        _bf16_2d(grad_act, "grad_act")
        if grad_act.shape != h.shape:
            raise ValueError(f"grad_act {tuple(grad_act.shape)} does not match h {tuple(h.shape)}")
        grad_act = grad_act.contiguous()
        _lib.require_cuda(h, grad_act)
    if act_out is not None:
        _lib.require_cuda(h, act_out)
        if act_out.dtype != BF16 or act_out.shape != h.shape or not act_out.is_contiguous():
            raise ValueError("act_out must be contiguous bfloat16 of h's shape")
    return _quantize_call("anima_mx_quantize_gelu", h, (ptr(grad_act),), rowwise, colwise, layout,
                          after_ld=(ptr(act_out),))


def mx_dequantize(op: MXOperand) -> torch.Tensor:
    dev = _lib.require_cuda(op.codes, op.scales)
    out = torch.empty(op.codes.shape, dtype=BF16, device=dev)
    with torch.cuda.device(dev):
        check(_lib.load().anima_mx_dequantize(ptr(op.codes), ptr(op.scales), op.rows, op.k, op.layout,
                                              ptr(out), _lib.stream_ptr(dev)))
    return out


def mx_retile(op: MXOperand) -> MXOperand:
    """PLAIN-scaled operand -> TILED-scaled operand (codes are shared, not copied)."""
    if op.layout == SCALES_TILED:
        return op
    dev = _lib.require_cuda(op.codes, op.scales)
    tiled = _alloc_scales(op.rows, op.k, SCALES_TILED, dev)
    with torch.cuda.device(dev):
        check(_lib.load().anima_mx_scales_retile(ptr(op.scales.contiguous()), op.rows, op.k, ptr(tiled),
                                                 _lib.stream_ptr(dev)))
    return MXOperand(op.codes, tiled, SCALES_TILED)


def mx_regroup(op: MXOperand, rows: int, k: int) -> MXOperand:
    """The same row-wise codes viewed as ``[rows, k]`` (``rows * k`` unchanged, ``k % 32 == 0``), with TILED scales
    re-tiled for that shape. The code buffer is shared, not copied."""
    if op.layout != SCALES_TILED:
        raise ValueError("mx_regroup needs TILED scales")
    if rows * k != op.rows * op.k or k % 32:
        raise ValueError(f"cannot view [{op.rows}, {op.k}] as [{rows}, {k}]")
    dev = _lib.require_cuda(op.codes, op.scales)
    scales = _alloc_scales(rows, k, SCALES_TILED, dev)
    if rows:
        with torch.cuda.device(dev):
            check(_lib.load().anima_mx_scales_regroup(ptr(op.scales), op.rows, op.k, ptr(scales), rows, k,
                                                      _lib.stream_ptr(dev)))
    return MXOperand(op.codes.view(rows, k), scales, SCALES_TILED)


def mx_gemm(a: MXOperand, b: MXOperand, *, bias: torch.Tensor | None = None,
            out_dtype: torch.dtype = BF16, out: torch.Tensor | None = None, split_k: bool = True,
            residual: torch.Tensor | None = None, alpha: float = 1.0) -> torch.Tensor:
    """``C[M,N] = alpha * A[M,K] . B[N,K]^T (+ bias) (+ residual)`` on the tcgen05 block-scaled tensor path.
    ``residual`` is bf16 [M, N] and may be ``out`` itself. Small outputs with a long contraction are split over K
    through a scratch buffer unless ``split_k`` is False."""
    dev = _lib.require_cuda(a.codes, a.scales, b.codes, b.scales, bias)
    if a.layout != SCALES_TILED or b.layout != SCALES_TILED:
        raise ValueError("mx_gemm needs TILED scales; convert with mx_retile()")
    if a.k != b.k:
        raise ValueError(f"contraction sizes differ: A has K={a.k}, B has K={b.k}")
    if not (a.codes.is_contiguous() and b.codes.is_contiguous()):
        raise ValueError("mx_gemm operands must be contiguous (K-major)")
    if out_dtype not in (BF16, torch.float32):
        raise TypeError("out_dtype must be bfloat16 or float32")
    if bias is not None and (bias.dtype != BF16 or bias.numel() != b.rows or not bias.is_contiguous()):
        raise ValueError("bias must be contiguous bfloat16 of length N")
    M, N, K = a.rows, b.rows, a.k
    if residual is not None:
        _lib.require_cuda(a.codes, residual)
        if residual.dtype != BF16 or residual.shape != (M, N) or residual.stride(1) != 1:
            raise ValueError("residual must be bfloat16 [M, N] with unit column stride")
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=dev)
    elif out.shape != (M, N) or out.dtype != out_dtype or out.stride(1) != 1:
        raise ValueError("out has the wrong shape, dtype or layout")
    lib = _lib.load()
    ws_bytes = check(lib.anima_mx_gemm_workspace_bytes(M, N, K)) if split_k else 0
    ws = _lib.workspace(ws_bytes, dev, "gemm_splitk") if ws_bytes else None
    with torch.cuda.device(dev):
        check(lib.anima_mx_gemm_ex(
            ptr(a.codes), ptr(a.scales), ptr(b.codes), ptr(b.scales), ptr(out), M, N, K, out.stride(0),
            ptr(bias), ptr(residual), residual.stride(0) if residual is not None else 0, float(alpha),
            1 if out_dtype == torch.float32 else 0, ptr(ws), ws.numel() if ws is not None else 0,
            ptr(_lib.status_word(dev)), _lib.stream_ptr(dev)))
    return out


def can_fold_delta(M: int, N: int) -> bool:
    """Shapes for which a T-LoKr delta can enter the base GEMM as extra K-blocks (:func:`mx_gemm_delta`)."""
    return M > 128 and N > 128 and M % 128 == 0 and N % 8 == 0 and (N // 8) % 64 == 0


def mx_gemm_delta(a: MXOperand, b: MXOperand, planes: MXOperand, d: MXOperand, *, bias: torch.Tensor | None = None,
                  out: torch.Tensor | None = None) -> torch.Tensor:
    """``C[m, i * N/8 + p] = (A . B^T)[m, i * N/8 + p] + planes[i * M + m, :] . d[p, :] (+ bias)`` as ONE GEMM: the
    low-rank delta of a T-LoKr linear enters as extra K-blocks of the base product. ``planes`` is the
    ``[8 * M, 128]`` operand written by :func:`tlokr_rank_mix_quant_planes`, ``d`` the ``[N / 8, 128]`` factor
    (with any scalar already folded in). bf16 output, rounded once."""
    dev = _lib.require_cuda(a.codes, a.scales, b.codes, b.scales, planes.codes, planes.scales, d.codes, d.scales, bias)
    if any(op.layout != SCALES_TILED for op in (a, b, planes, d)):
        raise ValueError("mx_gemm_delta needs TILED scales")
    M, N, K = a.rows, b.rows, a.k
    if a.k != b.k:
        raise ValueError(f"contraction sizes differ: A has K={a.k}, B has K={b.k}")
    if not can_fold_delta(M, N):
        raise ValueError(f"mx_gemm_delta cannot take M={M}, N={N}")
    if planes.codes.shape != (8 * M, 128) or d.codes.shape != (N // 8, 128):
        raise ValueError(f"delta operands must be [8 * M, 128] and [N / 8, 128], got {tuple(planes.codes.shape)} "
                         f"and {tuple(d.codes.shape)}")
    if not all(t.is_contiguous() for t in (a.codes, b.codes, planes.codes, d.codes)):
        raise ValueError("mx_gemm_delta operands must be contiguous (K-major)")
    if bias is not None and (bias.dtype != BF16 or bias.numel() != N or not bias.is_contiguous()):
        raise ValueError("bias must be contiguous bfloat16 of length N")
    if out is None:
        out = torch.empty((M, N), dtype=BF16, device=dev)
    elif out.shape != (M, N) or out.dtype != BF16 or out.stride(1) != 1:
        raise ValueError("out has the wrong shape, dtype or layout")
    lib = _lib.load()
    ws_bytes = check(lib.anima_mx_gemm_workspace_bytes(M, N, K))
    ws = _lib.workspace(ws_bytes, dev, "gemm_splitk") if ws_bytes else None
    with torch.cuda.device(dev):
        check(lib.anima_mx_gemm_delta(
            ptr(a.codes), ptr(a.scales), ptr(b.codes), ptr(b.scales), ptr(out), M, N, K, out.stride(0), ptr(bias), 0,
            ptr(planes.codes), ptr(planes.scales), ptr(d.codes), ptr(d.scales), ptr(ws),
            ws.numel() if ws is not None else 0, ptr(_lib.status_word(dev)), _lib.stream_ptr(dev)))
    return out


def _factor_flag(w1: torch.Tensor, w2: torch.Tensor) -> int:
    if w1.dtype != w2.dtype or w1.dtype not in (BF16, torch.float32):
        raise TypeError("LoKr factors must both be bfloat16 or both float32")
    return 1 if w1.dtype == torch.float32 else 0


def lokr_merge_quantize(
    w: torch.Tensor, w1: torch.Tensor, w2: torch.Tensor, alpha: float, *, want_merged: bool = True,
    rowwise: bool = False, colwise: bool = False, layout: int = SCALES_TILED,
) -> tuple[torch.Tensor | None, MXOperand | None, MXOperand | None]:
    """``merged = W + alpha * kron(w1, w2)`` and/or its MXFP8 forms, from one read of W."""
    _bf16_2d(w, "W")
    dev = _lib.require_cuda(w, w1, w2)
    w, w1, w2 = w.contiguous(), w1.contiguous(), w2.contiguous()
    N, K = w.shape
    up, uq = w1.shape
    if w2.shape != (N // up, K // uq) or N % up or K % uq:
        raise ValueError(f"kron({tuple(w1.shape)}, {tuple(w2.shape)}) does not match W {tuple(w.shape)}")
    merged = torch.empty_like(w) if want_merged else None
    row_op = col_op = None
    if rowwise:
        row_op = MXOperand(torch.empty((N, K), dtype=torch.uint8, device=dev),
                           _alloc_scales(N, K, layout, dev), layout)
    if colwise:
        col_op = MXOperand(torch.empty((K, N), dtype=torch.uint8, device=dev),
                           _alloc_scales(K, N, layout, dev), layout)
    with torch.cuda.device(dev):
        check(_lib.load().anima_lokr_merge_quantize(
            ptr(w), ptr(w1), ptr(w2), _factor_flag(w1, w2), float(alpha), N, K, up, uq, ptr(merged),
            ptr(row_op.codes) if row_op else None, ptr(row_op.scales) if row_op else None,
            ptr(col_op.codes) if col_op else None, ptr(col_op.scales) if col_op else None,
            layout, _lib.stream_ptr(dev)))
    return merged, row_op, col_op


def lokr_kron_backward(dw: torch.Tensor, w1: torch.Tensor, w2: torch.Tensor, alpha: float
                       ) -> tuple[torch.Tensor, torch.Tensor]:
    """fp32 ``(dw1, dw2)`` from ``dW`` (bf16 or fp32) of the merged weight."""
    dev = _lib.require_cuda(dw, w1, w2)
    if dw.dtype not in (BF16, torch.float32) or dw.dim() != 2:
        raise TypeError("dW must be a 2-D bfloat16 or float32 tensor")
    dw, w1, w2 = dw.contiguous(), w1.contiguous(), w2.contiguous()
    N, K = dw.shape
    up, uq = w1.shape
    lib = _lib.load()
    nbytes = check(lib.anima_lokr_kron_backward_workspace_bytes(N, K, up, uq))
    ws = _lib.workspace(nbytes, dev, "kron")
    dw1 = torch.empty((up, uq), dtype=torch.float32, device=dev)
    dw2 = torch.empty((N // up, K // uq), dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        check(lib.anima_lokr_kron_backward(
            ptr(dw), 1 if dw.dtype == torch.float32 else 0, ptr(w1), ptr(w2), _factor_flag(w1, w2),
            float(alpha), N, K, up, uq, ptr(dw1), ptr(dw2), ptr(ws), ws.numel(), _lib.stream_ptr(dev)))
    return dw1, dw2


def can_emit_row_codes(rows: int, d: int) -> bool:
    """Shapes for which the AdaLN forward kernels can also write the row-wise MXFP8 operand of their output."""
    return rows > 0 and rows % 128 == 0 and d % 128 == 0 and d <= 4096


def _row_operand(rows: int, d: int, dev) -> MXOperand:
    return MXOperand(torch.empty((rows, d), dtype=torch.uint8, device=dev),
                     torch.empty(scales_bytes(rows, d, SCALES_TILED), dtype=torch.uint8, device=dev), SCALES_TILED)


def adaln_fwd(x: torch.Tensor, scale: torch.Tensor, shift: torch.Tensor, eps: float, hw: int, *, quant: bool = False):
    """x ``[rows, d]``, scale/shift ``[rows/hw, d]`` (bf16, contiguous) -> (y, mean, rstd); with ``quant`` also
    the row-wise MXFP8 operand of y (tiled scales), bit-identical to ``mx_quantize(y)``, from the same pass."""
    dev = _lib.require_cuda(x, scale, shift)
    rows, d = x.shape
    y = torch.empty_like(x)
    mean = torch.empty(rows, dtype=torch.float32, device=dev)
    rstd = torch.empty(rows, dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        if quant:
            op = _row_operand(rows, d, dev)
            check(_lib.load().anima_adaln_fwd_quant(ptr(x), ptr(scale), ptr(shift), float(eps), rows, hw, d, ptr(y),
                                                    ptr(mean), ptr(rstd), ptr(op.codes), ptr(op.scales), op.layout,
                                                    _lib.stream_ptr(dev)))
            return y, mean, rstd, op
        check(_lib.load().anima_adaln_fwd(ptr(x), ptr(scale), ptr(shift), float(eps), rows, hw, d, ptr(y),
                                          ptr(mean), ptr(rstd), _lib.stream_ptr(dev)))
    return y, mean, rstd


def gated_add_adaln_fwd(x: torch.Tensor, gate: torch.Tensor, sub: torch.Tensor, scale: torch.Tensor,
                        shift: torch.Tensor, eps: float, hw: int, *, quant: bool = False):
    """``x_new = x + gate * sub`` and ``y = AdaLN(x_new)`` in one pass -> (x_new, y, mean, rstd); with ``quant``
    also the row-wise MXFP8 operand of y."""
    dev = _lib.require_cuda(x, gate, sub, scale, shift)
    rows, d = x.shape
    x_new, y = torch.empty_like(x), torch.empty_like(x)
    mean = torch.empty(rows, dtype=torch.float32, device=dev)
    rstd = torch.empty(rows, dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        if quant:
            op = _row_operand(rows, d, dev)
            check(_lib.load().anima_gated_add_adaln_fwd_quant(
                ptr(x), ptr(gate), ptr(sub), ptr(scale), ptr(shift), float(eps), rows, hw, d, ptr(x_new), ptr(y),
                ptr(mean), ptr(rstd), ptr(op.codes), ptr(op.scales), op.layout, _lib.stream_ptr(dev)))
            return x_new, y, mean, rstd, op
        check(_lib.load().anima_gated_add_adaln_fwd(ptr(x), ptr(gate), ptr(sub), ptr(scale), ptr(shift), float(eps),
                                                    rows, hw, d, ptr(x_new), ptr(y), ptr(mean), ptr(rstd),
                                                    _lib.stream_ptr(dev)))
    return x_new, y, mean, rstd


def gated_add_adaln_bwd(d_y: torch.Tensor, d_xnew: torch.Tensor, x_new: torch.Tensor, scale: torch.Tensor,
                        mean: torch.Tensor, rstd: torch.Tensor, sub: torch.Tensor, gate: torch.Tensor, hw: int):
    """Backward of :func:`gated_add_adaln_fwd` in one pass -> (dx, dsub, dscale, dshift, dgate)."""
    dev = _lib.require_cuda(d_y, d_xnew, x_new, scale, mean, rstd, sub, gate)
    rows, d = x_new.shape
    bt = rows // hw if hw else 0
    dx, dsub = torch.empty_like(x_new), torch.empty_like(x_new)
    dscale, dshift, dgate = (torch.empty((bt, d), dtype=BF16, device=dev) for _ in range(3))
    if rows == 0:
        return dx, dsub, dscale, dshift, dgate
    lib = _lib.load()
    nbytes = check(lib.anima_gated_add_adaln_bwd_workspace_bytes(rows, hw, d))
    ws = _lib.workspace(nbytes, dev, "gated_adaln_bwd")
    with torch.cuda.device(dev):
        check(lib.anima_gated_add_adaln_bwd(ptr(d_y), ptr(d_xnew), ptr(x_new), ptr(scale), ptr(mean), ptr(rstd),
                                            ptr(sub), ptr(gate), rows, hw, d, ptr(dx), ptr(dsub), ptr(dscale),
                                            ptr(dshift), ptr(dgate), ptr(ws), ws.numel(), _lib.stream_ptr(dev)))
    return dx, dsub, dscale, dshift, dgate


def adaln_bwd(dy: torch.Tensor, x: torch.Tensor, scale: torch.Tensor, mean: torch.Tensor,
              rstd: torch.Tensor, hw: int) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    dev = _lib.require_cuda(dy, x, scale, mean, rstd)
    rows, d = x.shape
    lib = _lib.load()
    nbytes = check(lib.anima_adaln_bwd_workspace_bytes(rows, hw, d))
    ws = _lib.workspace(nbytes, dev, "adaln")
    dx = torch.empty_like(x)
    dscale = torch.empty_like(scale)
    dshift = torch.empty_like(scale)
    with torch.cuda.device(dev):
        check(lib.anima_adaln_bwd(ptr(dy), ptr(x), ptr(scale), ptr(mean), ptr(rstd), rows, hw, d, ptr(dx),
                                  ptr(dscale), ptr(dshift), ptr(ws), ws.numel(), _lib.stream_ptr(dev)))
    return dx, dscale, dshift


def gated_add_fwd(x: torch.Tensor, gate: torch.Tensor, y: torch.Tensor, hw: int) -> torch.Tensor:
    dev = _lib.require_cuda(x, gate, y)
    rows, d = x.shape
    out = torch.empty_like(x)
    with torch.cuda.device(dev):
        check(_lib.load().anima_gated_add_fwd(ptr(x), ptr(gate), ptr(y), rows, hw, d, ptr(out),
                                              _lib.stream_ptr(dev)))
    return out


def gated_add_bwd(dout: torch.Tensor, y: torch.Tensor, gate: torch.Tensor, hw: int
                  ) -> tuple[torch.Tensor, torch.Tensor]:
    dev = _lib.require_cuda(dout, y, gate)
    rows, d = y.shape
    lib = _lib.load()
    nbytes = check(lib.anima_gated_add_bwd_workspace_bytes(rows, hw, d))
    ws = _lib.workspace(nbytes, dev, "gated")
    dy = torch.empty_like(y)
    dgate = torch.empty_like(gate)
    with torch.cuda.device(dev):
        check(lib.anima_gated_add_bwd(ptr(dout), ptr(y), ptr(gate), rows, hw, d, ptr(dy), ptr(dgate),
                                      ptr(ws), ws.numel(), _lib.stream_ptr(dev)))
    return dy, dgate


def tlokr_rank_mix(hidden: torch.Tensor, c: torch.Tensor, mask: torch.Tensor | None, transpose: bool
                   ) -> torch.Tensor:
    dev = _lib.require_cuda(hidden, c, mask)
    batch, n, _, rank = hidden.shape
    out = torch.empty_like(hidden)
    with torch.cuda.device(dev):
        check(_lib.load().anima_tlokr_rank_mix(ptr(hidden), ptr(c), ptr(mask), batch, n, rank,
                                               1 if transpose else 0, ptr(out), _lib.stream_ptr(dev)))
    return out


def can_quantise_rank_mix(batch: int, n: int, rank: int) -> bool:
    """Shapes for which the mix kernel can write the MXFP8 operands of its output itself."""
    return rank in (128, 256, 512) and batch * n > 0 and (batch * n) % 16 == 0


def tlokr_rank_mix_quant(hidden: torch.Tensor, c: torch.Tensor, mask: torch.Tensor | None, transpose: bool, *,
                         rowwise: bool = True, colwise: bool = False, want_bf16: bool = False
                         ) -> tuple[MXOperand | None, MXOperand | None, torch.Tensor | None]:
    """The 8x8 mix of ``hidden [batch, n, 8, rank]`` leaving as the MXFP8 operands of the mixed tensor viewed as
    ``[batch * n * 8, rank]`` (row form, and / or column form stored ``[rank, batch * n * 8]``), bit-identical to
    ``mx_quantize(tlokr_rank_mix(...))``; the bf16 tensor is written only with ``want_bf16``."""
    dev = _lib.require_cuda(hidden, c, mask)
    batch, n, _, rank = hidden.shape
    R = batch * n * 8
    row = col = out = None
    if rowwise:
        row = MXOperand(torch.empty((R, rank), dtype=torch.uint8, device=dev),
                        torch.empty(scales_bytes(R, rank, SCALES_TILED), dtype=torch.uint8, device=dev), SCALES_TILED)
    if colwise:
        col = MXOperand(torch.empty((rank, R), dtype=torch.uint8, device=dev),
                        torch.empty(scales_bytes(rank, R, SCALES_TILED), dtype=torch.uint8, device=dev), SCALES_TILED)
    if want_bf16:
        out = torch.empty_like(hidden)
    with torch.cuda.device(dev):
        check(_lib.load().anima_tlokr_rank_mix_quant(
            ptr(hidden), ptr(c), ptr(mask), batch, n, rank, 1 if transpose else 0, ptr(out),
            ptr(row.codes) if row else None, ptr(row.scales) if row else None,
            ptr(col.codes) if col else None, ptr(col.scales) if col else None, _lib.stream_ptr(dev)))
    return row, col, out


def can_mix_to_planes(batch: int, n: int, rank: int) -> bool:
    """Shapes for which the quantising mix can write its row form as eight planes (``rank`` is one K-block)."""
    return rank == 128 and batch * n > 0 and (batch * n) % 128 == 0


def tlokr_rank_mix_quant_planes(hidden: torch.Tensor, c: torch.Tensor, mask: torch.Tensor | None, transpose: bool, *,
                                colwise: bool = False) -> tuple[MXOperand, MXOperand | None]:
    """The 8x8 mix of ``hidden [batch, n, 8, rank]`` leaving as the MXFP8 row form laid out as eight planes
    (row ``i`` of item ``t`` at row ``i * items + t`` of a ``[8 * items, rank]`` operand, which
    :func:`mx_gemm_delta` consumes), and optionally the usual transposed column form ``[rank, items * 8]``."""
    dev = _lib.require_cuda(hidden, c, mask)
    batch, n, _, rank = hidden.shape
    R = batch * n * 8
    planes = MXOperand(torch.empty((R, rank), dtype=torch.uint8, device=dev),
                       torch.empty(scales_bytes(R, rank, SCALES_TILED), dtype=torch.uint8, device=dev), SCALES_TILED)
    col = None
    if colwise:
        col = MXOperand(torch.empty((rank, R), dtype=torch.uint8, device=dev),
                        torch.empty(scales_bytes(rank, R, SCALES_TILED), dtype=torch.uint8, device=dev), SCALES_TILED)
    with torch.cuda.device(dev):
        check(_lib.load().anima_tlokr_rank_mix_quant_planes(
            ptr(hidden), ptr(c), ptr(mask), batch, n, rank, 1 if transpose else 0, ptr(planes.codes),
            ptr(planes.scales), ptr(col.codes) if col else None, ptr(col.scales) if col else None,
            _lib.stream_ptr(dev)))
    return planes, col


def tlokr_hidden_mix_planes(g: MXOperand, f: MXOperand, c: torch.Tensor, mask: torch.Tensor | None, batch: int,
                            transpose: bool = False, *, want_hidden: bool = False
                            ) -> tuple[MXOperand, torch.Tensor | None]:
    """``hidden = g . f^T`` (``g [batch * n * 8, k]``, ``f [128, k]``), the 8x8 mix, the mask and the MXFP8
    quantisation of the mixed tensor in ONE kernel; returns the eight-plane operand (as
    :func:`tlokr_rank_mix_quant_planes`) and, with ``want_hidden``, the bf16 hidden tensor ``[batch, n, 8, 128]``,
    which otherwise never leaves the SM. Bit-identical to ``mx_gemm`` followed by the quantising mix."""
    dev = _lib.require_cuda(g.codes, g.scales, f.codes, f.scales, c, mask)
    if g.layout != SCALES_TILED or f.layout != SCALES_TILED:
        raise ValueError("tlokr_hidden_mix_planes needs TILED scales")
    R, k = g.rows, g.k
    if f.codes.shape != (128, k):
        raise ValueError(f"the factor operand must be [128, {k}], got {tuple(f.codes.shape)}")
    if R % (8 * batch) or not can_mix_to_planes(batch, R // (8 * batch), 128):
        raise ValueError(f"cannot mix {R} grouped rows of {batch} samples into planes")
    if c.dtype != BF16 or c.shape != (8, 8) or not c.is_contiguous():
        raise ValueError("c must be contiguous bfloat16 [8, 8]")
    if mask is not None and (mask.dtype != BF16 or mask.shape != (batch, 128) or not mask.is_contiguous()):
        raise ValueError("mask must be contiguous bfloat16 [batch, 128]")
    n = R // (8 * batch)
    planes = MXOperand(torch.empty((R, 128), dtype=torch.uint8, device=dev),
                       torch.empty(scales_bytes(R, 128, SCALES_TILED), dtype=torch.uint8, device=dev), SCALES_TILED)
    hidden = torch.empty((batch, n, 8, 128), dtype=BF16, device=dev) if want_hidden else None
    with torch.cuda.device(dev):
        check(_lib.load().anima_tlokr_hidden_mix_planes(
            ptr(g.codes), ptr(g.scales), ptr(f.codes), ptr(f.scales), ptr(c), ptr(mask), batch, n, k,
            1 if transpose else 0, ptr(hidden), ptr(planes.codes), ptr(planes.scales), ptr(_lib.status_word(dev)),
            _lib.stream_ptr(dev)))
    return planes, hidden


def tlokr_rank_mix_wgrad(grad_mixed: torch.Tensor, hidden: torch.Tensor, mask: torch.Tensor | None
                         ) -> torch.Tensor:
    dev = _lib.require_cuda(grad_mixed, hidden, mask)
    batch, n, _, rank = hidden.shape
    lib = _lib.load()
    nbytes = check(lib.anima_tlokr_rank_mix_wgrad_workspace_bytes(batch, n, rank))
    ws = _lib.workspace(nbytes, dev, "mixwgrad")
    dc = torch.empty((8, 8), dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        check(lib.anima_tlokr_rank_mix_wgrad(ptr(grad_mixed), ptr(hidden), ptr(mask), batch, n, rank, ptr(dc),
                                             ptr(ws), ws.numel(), _lib.stream_ptr(dev)))
    return dc


def rmsnorm_rope_fwd(x: torch.Tensor, weight: torch.Tensor, cos: torch.Tensor | None, sin: torch.Tensor | None,
                     eps: float) -> tuple[torch.Tensor, torch.Tensor]:
    """x bf16 (..., tokens-major, heads, 128) contiguous; weight fp32 [128]; cos / sin fp32 [seq_len, 128] or None.
    Returns (out bf16 like x, rstd fp32 [tokens * heads])."""
    dev = _lib.require_cuda(x, weight, cos, sin)
    heads, d = x.shape[-2], x.shape[-1]
    tokens = x.numel() // (heads * d) if x.numel() else 0
    out = torch.empty_like(x)
    rstd = torch.empty(tokens * heads, dtype=torch.float32, device=dev)
    if tokens == 0:
        return out, rstd
    seq = cos.shape[0] if cos is not None else 1
    with torch.cuda.device(dev):
        check(_lib.load().anima_rmsnorm_rope_fwd(ptr(x), ptr(weight), ptr(cos), ptr(sin), float(eps), tokens, heads, d,
                                                 seq, ptr(out), ptr(rstd), _lib.stream_ptr(dev)))
    return out, rstd


def rmsnorm_rope_bwd(dout: torch.Tensor, x: torch.Tensor, weight: torch.Tensor, cos: torch.Tensor | None,
                     sin: torch.Tensor | None, rstd: torch.Tensor) -> torch.Tensor:
    dev = _lib.require_cuda(dout, x, weight, cos, sin, rstd)
    heads, d = x.shape[-2], x.shape[-1]
    tokens = x.numel() // (heads * d) if x.numel() else 0
    dx = torch.empty_like(x)
    if tokens == 0:
        return dx
    seq = cos.shape[0] if cos is not None else 1
    with torch.cuda.device(dev):
        check(_lib.load().anima_rmsnorm_rope_bwd(ptr(dout), ptr(x), ptr(weight), ptr(cos), ptr(sin), ptr(rstd), tokens,
                                                 heads, d, seq, ptr(dx), _lib.stream_ptr(dev)))
    return dx
