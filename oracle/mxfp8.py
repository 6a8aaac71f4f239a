"""Oracle: MXFP8 quantise / dequantise / block-scaled matmul (numpy).

Follows anima-trainer ``src/anima_trainer/mxfp8_gemm.py``:
quantiser math :83-91 and :111-147, column-wise form :201-222, inverse :225-232,
GEMM semantics :267-271 and :299-312.
"""
from __future__ import annotations

import numpy as np

FP8_E4M3_MAX = np.float32(448.0)   # mxfp8_gemm.py:45
AMAX_FLOOR = np.float32(1e-30)     # mxfp8_gemm.py:114


# ----------------------------------------------------------------------------- bf16 helpers
def bf16_bits_to_f32(bits: np.ndarray) -> np.ndarray:
    return (bits.astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even fp32 -> bf16 bit pattern (NaN kept quiet)."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    rounded = ((u + np.uint32(0x7FFF) + ((u >> 16) & np.uint32(1))) >> 16).astype(np.uint16)
    return np.where(np.isnan(x), np.uint16(0x7FC0), rounded)


def round_to_bf16(x: np.ndarray) -> np.ndarray:
    return bf16_bits_to_f32(f32_to_bf16_bits(x))


# ----------------------------------------------------------------------------- e4m3
def e4m3_encode(y: np.ndarray) -> np.ndarray:
    """fp32 -> e4m3fn code, round-to-nearest-even, saturating to +-448 (0x7E); NaN -> 0x7F.
    This is the conversion `y.to(tl.float8e4nv)` performs on NVIDIA hardware
    (cvt.rn.satfinite.e4m3x2.f32), mxfp8_gemm.py:129-130."""
    y = np.asarray(y, dtype=np.float32)
    a = np.abs(y).astype(np.float64)
    finite = np.isfinite(a)
    a_safe = np.where(finite, a, 0.0)
    _, ex = np.frexp(a_safe)                       # a = m * 2^ex, m in [0.5, 1)
    e = np.where(a_safe == 0, -6, np.maximum(ex - 1, -6))   # binade exponent, clamped at the subnormal one
    q = np.rint(a_safe / np.ldexp(1.0, e - 3))     # mantissa in eighths, ties to even
    code = ((e + 7) * 8 + (q.astype(np.int64) - 8))
    code = np.clip(code, 0, 0x7E)                  # carry past 448 saturates
    code = np.where(np.isinf(a), 0x7E, code)
    code = np.where(np.isnan(y), 0x7F, code)
    sign = (np.signbit(y).astype(np.int64) << 7)
    return (code | sign).astype(np.uint8)


def e4m3_decode(code: np.ndarray) -> np.ndarray:
    code = np.asarray(code, dtype=np.uint8)
    s = np.where(code & 0x80, -1.0, 1.0)
    e = ((code >> 3) & 0xF).astype(np.int32)
    m = (code & 0x7).astype(np.float64)
    mag = np.where(e == 0, m / 8.0 * 2.0 ** -6, (1.0 + m / 8.0) * np.exp2((e - 7).astype(np.float64)))
    mag = np.where((code & 0x7F) == 0x7F, np.nan, mag)
    return (s * mag).astype(np.float32)


# ----------------------------------------------------------------------------- exponent rule
def exponent_reference_fp32(amax: np.ndarray) -> np.ndarray:
    """The reference's literal fp32 expression, mxfp8_gemm.py:118-120:
    ceil(log2(amax) - log2(448)) clamped to [-127, 127]."""
    amax = np.asarray(amax, dtype=np.float32)
    with np.errstate(over="ignore"):
        e = np.ceil(np.log2(amax) - np.log2(FP8_E4M3_MAX))
    return np.clip(e, -127.0, 127.0).astype(np.int32)


def exponent_exact(amax: np.ndarray) -> np.ndarray:
    """The same quantity in exact arithmetic: amax = m * 2^E (1 <= m < 2), 448 = 1.75 * 2^8
    => ceil(log2(amax/448)) = E - 8 + (m > 1.75). Equals exponent_reference_fp32 for every
    bf16-representable amax with E < 64 (beyond that fp32 rounding of log2 flips m == 1.75)."""
    amax = np.ascontiguousarray(amax, dtype=np.float32)
    u = amax.view(np.uint32)
    E = (u >> 23).astype(np.int32) - 127
    mant = u & np.uint32(0x7FFFFF)
    e = E - 8 + (mant > 0x600000).astype(np.int32)
    e = np.where(E == 128, 127, e)
    return np.clip(e, -127, 127).astype(np.int32)


# ----------------------------------------------------------------------------- quantiser
def quantize_rowwise(x: np.ndarray, *, exact_rule: bool = True) -> tuple[np.ndarray, np.ndarray]:
    """x fp32 (values of a bf16 tensor) [R, K], K % 32 == 0 -> (codes u8 [R,K], scales u8 [R,K/32]).
    mxfp8_gemm.py:111-147: amax over 32, floor 1e-30, e = ceil(log2(amax/448)) clamped,
    code = e4m3(x / 2^e), scale byte = e + 127."""
    x = np.asarray(x, dtype=np.float32)
    R, K = x.shape
    assert K % 32 == 0
    g = x.reshape(R, K // 32, 32)
    amax = np.maximum(np.max(np.abs(g), axis=2), AMAX_FLOOR)
    e = exponent_exact(amax) if exact_rule else exponent_reference_fp32(amax)
    scale = np.ldexp(np.float32(1.0), e).astype(np.float32)     # 2^e; 2^-127 is subnormal
    with np.errstate(over="ignore", invalid="ignore"):
        y = g / scale[..., None]
    return e4m3_encode(y).reshape(R, K), (e + 127).astype(np.uint8)


def quantize_colwise_T(x: np.ndarray, **kw) -> tuple[np.ndarray, np.ndarray]:
    """Blocks of 32 along the ROWS of x [R, C], stored transposed: codes [C, R], scales
    [C, R/32] — i.e. quantize_rowwise(x.T). mxfp8_gemm.py:217-218 (the reference then
    transposes the codes back, :221; the scales stay (C, R//32), :222)."""
    return quantize_rowwise(np.ascontiguousarray(np.asarray(x, dtype=np.float32).T), **kw)


def dequantize_rowwise(codes: np.ndarray, scales: np.ndarray) -> np.ndarray:
    """fp32 values code * 2^(byte-127) (mxfp8_gemm.py:225-232 before its bf16 cast)."""
    R, K = codes.shape
    v = e4m3_decode(codes).reshape(R, K // 32, 32)
    s = np.ldexp(np.float32(1.0), scales.astype(np.int32) - 127).astype(np.float32)
    return (v * s[..., None]).reshape(R, K)


def scales_to_tiled(scales: np.ndarray) -> np.ndarray:
    """PLAIN [rows, kb] -> flat TILED layout of include/anima_b200.h (padding bytes 0)."""
    rows, kb = scales.shape
    rt, kt = -(-rows // 128), -(-kb // 4)
    padded = np.zeros((rt * 128, kt * 4), dtype=np.uint8)
    padded[:rows, :kb] = scales
    # [rt, 4(q), 32(r32), kt, 4(j)] -> chunk (rt, kt), inside: r32*16 + q*4 + j
    t = padded.reshape(rt, 4, 32, kt, 4).transpose(0, 3, 2, 1, 4)
    return np.ascontiguousarray(t).reshape(-1)


def matmul(a_codes, a_scales, b_codes, b_scales, bias=None, *, out_bf16=True) -> np.ndarray:
    """C[M,N] = dequant(A)[M,K] @ dequant(B)[N,K]^T, accumulated in float64, (+ bias), rounded
    to bf16. Semantics of mxfp8_gemm.py:267-271, :299-312 (fp32 accumulate -> bf16)."""
    a = dequantize_rowwise(a_codes, a_scales).astype(np.float64)
    b = dequantize_rowwise(b_codes, b_scales).astype(np.float64)
    c = a @ b.T
    if bias is not None:
        c = c + np.asarray(bias, dtype=np.float64)[None, :]
    c = c.astype(np.float32)
    return round_to_bf16(c) if out_bf16 else c
