"""The CPU oracle against golden vectors computed by anima-trainer's own code
(tests/golden/make_golden.py: its Triton kernels under the Triton CPU interpreter and its
CPU-capable torch paths). This is what pins the oracle the GPU parity tests rely on."""
from __future__ import annotations

import numpy as np
import torch

from conftest import bf16_from_bits, bits_from_bf16
from oracle import adaln as OA
from oracle import mxfp8 as OQ
from oracle import tlokr as OT


def _interpreter_cast_is_trustworthy(x, scales):
    """Mask of elements where the Triton CPU interpreter's emulated fp32 -> e4m3 cast agrees with
    the hardware conversion the reference relies on (cvt.rn.satfinite: round to nearest EVEN,
    saturating; mxfp8_gemm.py:87, :129-130). The emulation rounds ties away from zero, drops the
    exponent carry when the mantissa rounds up to 2.0 and truncates subnormals; those elements
    are pinned by the torch float8_e4m3fn cast instead (test_e4m3_encode_matches_torch_cast)."""
    R, K = x.shape
    e = scales.astype(np.int32) - 127
    y = np.abs(x.reshape(R, K // 32, 32).astype(np.float64) / np.ldexp(1.0, e)[..., None]).reshape(R, K)
    _, ex = np.frexp(y)
    eb = np.where(y == 0, -6, np.maximum(ex - 1, -6))
    q = y / np.ldexp(1.0, eb - 3)
    tie = (q - np.floor(q)) == 0.5
    carry = np.rint(q) >= 16
    subnormal = (y < 2.0 ** -6) & (y > 0)
    return ~(tie | carry | subnormal)


def test_quantiser_codes_and_scales_bit_exact(golden):
    g = golden("quantiser")
    x = OQ.bf16_bits_to_f32(g["x"])
    for exact in (True, False):
        codes, scales = OQ.quantize_rowwise(x, exact_rule=exact)
        assert np.array_equal(scales, g["scales"]), f"scale bytes differ (exact_rule={exact})"
        ok = _interpreter_cast_is_trustworthy(x, scales)
        assert ok.mean() > 0.85
        assert np.array_equal(codes[ok], g["codes"][ok]), f"codes differ (exact_rule={exact})"
    # planted cases: all-zero block -> byte 19; amax 1.75 -> 2^-8 (byte 119) and code 0x7E
    assert g["scales"][0, 0] == 19 and not g["codes"][0, :32].any()
    assert g["scales"][1, 0] == 119 and g["codes"][1, 0] == 0x7E


def test_e4m3_encode_matches_torch_cast():
    rng = np.random.default_rng(0)
    y = np.concatenate([rng.normal(0, 100, 200000), rng.normal(0, 1, 200000), rng.normal(0, 0.01, 200000),
                        np.arange(-512, 512) * 0.5, np.arange(0, 64) * 2.0 ** -10,
                        [448, 449, 463.9, 464, 465, 480, 1e9, -1e9, 0.0, -0.0]]).astype(np.float32)
    want = torch.from_numpy(y).clamp(-448, 448).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    assert np.array_equal(OQ.e4m3_encode(y), want)
    allc = np.arange(256, dtype=np.uint8)
    keep = (allc & 0x7F) != 0x7F
    assert np.array_equal(OQ.e4m3_encode(OQ.e4m3_decode(allc))[keep], allc[keep])


def test_quantiser_weight_forms(golden):
    g = golden("quantiser")
    w = OQ.bf16_bits_to_f32(g["w"])
    codes, scales = OQ.quantize_rowwise(w)
    ok = _interpreter_cast_is_trustworthy(w, scales)
    assert np.array_equal(scales, g["lhs_scales"]) and np.array_equal(codes[ok], g["lhs_codes"][ok])
    codes_t, scales_c = OQ.quantize_colwise_T(w)
    ok_t = _interpreter_cast_is_trustworthy(np.ascontiguousarray(w.T), scales_c)
    # the reference hands back the codes in W's own (N, K) orientation, scales as (K, N//32)
    assert np.array_equal(scales_c, g["dgrad_scales"])
    assert np.array_equal(codes_t[ok_t], np.ascontiguousarray(g["dgrad_codes"].T)[ok_t])


def test_dequantise_matches_reference(golden):
    g = golden("quantiser")
    deq = OQ.round_to_bf16(OQ.dequantize_rowwise(g["codes"], g["scales"]))
    ref = OQ.bf16_bits_to_f32(g["deq"])
    assert np.array_equal(deq.view(np.uint32), ref.view(np.uint32))


def test_exponent_rules_agree_on_every_bf16_amax_below_2_pow_64():
    bits = np.arange(0x0080, 0x7F80, dtype=np.uint16)
    amax = np.maximum(OQ.bf16_bits_to_f32(bits), OQ.AMAX_FLOOR)
    a, b = OQ.exponent_reference_fp32(amax), OQ.exponent_exact(amax)
    bad = amax[a != b]
    assert bad.size == 0 or bad.min() >= 2.0 ** 64
    assert bad.size <= 8  # only mantissa 1.75 with exponent 64..71


def test_gemm_oracle_matches_reference_dequant_matmul(golden):
    """Same operands (the reference's own codes and scales) -> same product as the reference's
    dequantize_rowwise + matmul; differences are accumulation order and the final bf16 rounding."""
    g = golden("gemm")
    y = OQ.matmul(g["x_codes"], g["x_scales"], g["w_codes"], g["w_scales"])
    np.testing.assert_allclose(y, OQ.bf16_bits_to_f32(g["y"]), rtol=1e-2, atol=2e-2)
    gx = OQ.matmul(g["g_codes"], g["g_scales"], g["wT_codes"], g["wT_scales"])
    np.testing.assert_allclose(gx, OQ.bf16_bits_to_f32(g["gx"]), rtol=1e-2, atol=2e-2)
    # scale bytes of all four operands are bit-exact with the oracle quantiser
    x, w, gy = (OQ.bf16_bits_to_f32(g[k]) for k in ("x", "w", "gy"))
    assert np.array_equal(OQ.quantize_rowwise(x)[1], g["x_scales"])
    assert np.array_equal(OQ.quantize_rowwise(w)[1], g["w_scales"])
    assert np.array_equal(OQ.quantize_rowwise(gy)[1], g["g_scales"])
    assert np.array_equal(OQ.quantize_colwise_T(w)[1], g["wT_scales"])


def test_scales_tiled_layout_roundtrip():
    rng = np.random.default_rng(0)
    s = rng.integers(1, 255, size=(200, 10), dtype=np.uint8)
    t = OQ.scales_to_tiled(s)
    assert t.size == 2 * 3 * 512
    for r, j in [(0, 0), (31, 3), (32, 0), (127, 9), (128, 4), (199, 9)]:
        chunk = (r // 128) * 3 + j // 4
        off = (r % 32) * 16 + ((r % 128) // 32) * 4 + j % 4
        assert t[chunk * 512 + off] == s[r, j]


def _ulp_gap(mine: torch.Tensor, ref_bits: np.ndarray) -> int:
    """Largest distance, in bf16 steps, between two same-shaped bf16 arrays (sign-magnitude order)."""
    def key(b):
        b = b.astype(np.int32)
        return np.where(b & 0x8000, -(b & 0x7FFF), b & 0x7FFF)
    return int(np.abs(key(bits_from_bf16(mine)) - key(ref_bits)).max())


def test_adaln_oracle_matches_reference_kernels(golden):
    g = golden("adaln")
    for n in ("a", "b"):
        BT, HW, D = (int(v) for v in g[f"{n}_shape"])
        x, s, b, gate, y2, dy = (bf16_from_bits(g[f"{n}_{k}"]) for k in ("x", "s", "b", "gate", "y2", "dy"))
        y, mean, rstd = OA.adaln_fwd_fp32(x, s, b, 1e-6, HW)
        np.testing.assert_allclose(mean.numpy(), g[f"{n}_mean"], rtol=1e-5, atol=1e-6)
        np.testing.assert_allclose(rstd.numpy(), g[f"{n}_rstd"], rtol=1e-5, atol=1e-6)
        # The interpreter stores fp32 -> bf16 by truncation (hardware Triton rounds to nearest),
        # so its bf16 outputs sit at most one ulp below the correctly rounded oracle value.
        assert _ulp_gap(y.to(torch.bfloat16), g[f"{n}_y"]) <= 1
        dx, ds, db = OA.adaln_bwd_fp32(dy, x, s, torch.from_numpy(g[f"{n}_mean"]), torch.from_numpy(g[f"{n}_rstd"]), HW)
        ref_dx = bf16_from_bits(g[f"{n}_dx"]).float()
        torch.testing.assert_close(dx.to(torch.bfloat16).float(), ref_dx, rtol=1e-2, atol=2e-3)
        np.testing.assert_allclose(ds.numpy(), g[f"{n}_ds"], rtol=1e-4, atol=1e-4)
        np.testing.assert_allclose(db.numpy(), g[f"{n}_db"], rtol=1e-4, atol=1e-4)
        go = OA.gated_add_fwd_fp32(x, gate, y2, HW).to(torch.bfloat16)
        # the reference rounds gate*y to bf16 before the add (double rounding): <= 1 ulp apart
        torch.testing.assert_close(go.float(), bf16_from_bits(g[f"{n}_go"]).float(), rtol=1e-2, atol=2e-2)
        _, dg = OA.gated_add_bwd_fp32(dy, y2, gate, HW)
        np.testing.assert_allclose(dg.numpy(), g[f"{n}_dg"], rtol=1e-4, atol=1e-4)


def test_tlokr_schedule_and_mask(golden):
    g = golden("tlokr")
    for (t, a, b), want in zip(g["sched_cases"], g["sched_out"]):
        assert OT.active_rank_for_timestep(t, max_rank=int(a), min_rank=int(b)) == int(want)
    # the reference's own known answers, tests/test_tlokr.py:59-76
    assert OT.active_rank_for_timestep(1.0, max_rank=128, min_rank=64) == 64
    assert OT.active_rank_for_timestep(0.5, max_rank=128, min_rank=64) == 96
    assert OT.active_rank_for_timestep(0.0, max_rank=128, min_rank=64) == 128
    assert OT.active_rank_for_timestep(2.0, max_rank=8, min_rank=4) == 4
    assert OT.active_rank_for_timestep(-1.0, max_rank=8, min_rank=4) == 8
    m = OT.rank_mask(torch.from_numpy(g["mask_t"]), max_rank=128, min_rank=64)
    assert np.array_equal(m.numpy(), g["mask"])


def test_tlokr_rank_mix_oracle(golden):
    g = golden("tlokr")
    hidden, weight, grad, mask = (bf16_from_bits(g[f"mix_{k}"]) for k in ("hidden", "weight", "grad", "mask"))
    for tr in (False, True):
        o = OT.rank_mix_fp32(hidden, weight, mask, transpose=tr).to(torch.bfloat16)
        # reference tolerance for this op: tests/test_tlokr.py:94
        torch.testing.assert_close(o.float(), bf16_from_bits(g[f"mix_cpu_t{int(tr)}"]).float(), rtol=2e-2, atol=6.25e-2)
    o = OT.rank_mix_fp32(hidden, weight, None).to(torch.bfloat16)
    torch.testing.assert_close(o.float(), bf16_from_bits(g["mix_cpu_nomask"]).float(), rtol=2e-2, atol=6.25e-2)
    dc = OT.rank_mix_wgrad_fp64(grad, hidden, mask).float()
    np.testing.assert_allclose(dc.numpy(), g["wgrad"], rtol=1e-4, atol=1e-2)
    np.testing.assert_allclose(dc.numpy(), g["wgrad_cpu"], rtol=1e-4, atol=1e-2)


def test_tlokr_structured_delta_oracle(golden):
    g = golden("tlokr")
    x, w1, a, b, mask, probe = (torch.from_numpy(g[f"sd_{k}"]) for k in ("x", "w1", "a", "b", "mask", "probe"))
    y = OT.structured_delta_fwd(x, w1, a, b, mask)
    torch.testing.assert_close(y, torch.from_numpy(g["sd_y"]), rtol=1e-5, atol=1e-5)
    gx, gw1, ga, gb = OT.structured_delta_bwd(x, w1, a, b, mask, probe)
    for got, key in ((gx, "sd_gx"), (gw1, "sd_gw1"), (ga, "sd_ga"), (gb, "sd_gb")):
        torch.testing.assert_close(got, torch.from_numpy(g[key]), rtol=1e-4, atol=1e-4)
    # and the explicit-Kronecker statement of the same delta (tests/test_tlokr.py:137-156)
    base = torch.zeros(w1.shape[0] * a.shape[0], x.shape[-1])
    want = OT.explicit_kron_linear(x, base, None, w1, a, b, torch.from_numpy(g["sd_t"]), rank=8, min_rank=4, scale=1.0)
    torch.testing.assert_close(y, want, rtol=1e-4, atol=1e-4)
