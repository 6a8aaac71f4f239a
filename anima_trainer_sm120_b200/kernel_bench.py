"""Per-kernel throughput of ``libanima_b200.so`` at the production shapes.

    python -m anima_trainer_sm120_b200.kernel_bench [--iters 20] [--only gemm|hbm|tlokr] [--small]
                                                   [--pick TEXT] [--direct]

Every kernel is timed alone with CUDA events on the launching stream (warm-ups, then the median
over ``--iters`` replays of a CUDA graph holding 4 launches, an L2-sized buffer rewritten before
each replay; all tensor sets are larger than L2) and reported as
one JSON line: achieved HBM GB/s for the memory-bound kernels (algorithmic bytes, i.e. each
tensor read or written once) or TFLOP/s for the GEMMs (2*M*N*K), next to the measured peak of
``MEASURED_PEAKS.json`` when that file is present. ``--small`` shrinks every shape (for ncu
captures, which should hold a few GB at most and end quickly).
"""
from __future__ import annotations

import argparse
import json
from pathlib import Path

import torch

from . import _lib, ops

BF16 = torch.bfloat16
ROOT = Path(__file__).resolve().parents[1]


def _peaks() -> dict:
    p = ROOT / "MEASURED_PEAKS.json"
    return json.loads(p.read_text()) if p.exists() else {}


class Timer:
    """Median device time of one launch. The launch is captured ``reps`` times into a CUDA graph so
    that host-side launch overhead (allocation of the outputs, ctypes) cannot show up as idle time
    between the two events; every tensor set here is larger than L2, and an L2-sized buffer is
    rewritten before each replay."""

    def __init__(self, iters: int, reps: int = 4, direct: bool = False):
        self.iters, self.reps, self.direct = iters, reps, direct
        self.flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")

    def __call__(self, fn) -> float:
        if self.direct:                            # plain launches: what a profiler capture wants
            fn()
            times = []
            for _ in range(self.iters):
                self.flush.zero_()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                fn()
                e1.record()
                e1.synchronize()
                times.append(e0.elapsed_time(e1))
            times.sort()
            return times[len(times) // 2]
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for _ in range(self.reps):
                fn()
        graph.replay()
        torch.cuda.synchronize()
        times = []
        for _ in range(self.iters):
            self.flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            graph.replay()
            e1.record()
            e1.synchronize()
            times.append(e0.elapsed_time(e1) / self.reps)
        times.sort()
        return times[len(times) // 2]


def _acts(rows, cols, std=1.0):
    return (torch.randn(rows, cols, device="cuda") * std).to(BF16)


def cublaslt_mxfp8(a, b):
    """A callable running ``torch._scaled_mm`` (cuBLASLt block-scaled MXFP8) on two TILED MXFP8 operands."""
    a8 = a.codes.view(torch.float8_e4m3fn)
    b8 = b.codes.view(torch.float8_e4m3fn).t()
    sa = a.scales.view(torch.float8_e8m0fnu)
    sb = b.scales.view(torch.float8_e8m0fnu)
    return lambda: torch._scaled_mm(a8, b8, scale_a=sa, scale_b=sb, out_dtype=BF16)


class _Ctx:
    """Stand-in for an autograd context, so that the forward and the backward of an autograd node can be timed
    (and captured into a CUDA graph) as plain functions, without the autograd engine around them."""

    needs_input_grad = (True,) * 16

    def save_for_backward(self, *tensors):
        self.saved_tensors = tensors

    def mark_dirty(self, *tensors):
        pass


# The four module shapes of the 168-module T-LoKr preset (cross-attn q/o, k/v on the text tokens, mlp.layer1,
# mlp.layer2): (name, in, out, rows at M = 32768 image tokens / 4096 text tokens).
TLOKR_MODULES = [("cross q/o", 2048, 2048, 32768), ("cross k/v", 1024, 2048, 4096),
                 ("mlp.layer1", 2048, 8192, 32768), ("mlp.layer2", 8192, 2048, 32768)]


def run(iters: int, only: str | None, small: bool, pick: str | None = None, direct: bool = False,
        yardstick: bool = False, quiet: bool = False) -> list[dict]:
    _lib.load()
    torch.manual_seed(0)
    peaks = _peaks()
    hbm_peak = peaks.get("hbm_gbs")
    tf_peak = 2.0 * peaks["bf16_tflops"] if "bf16_tflops" in peaks else None  # timed alone: burst figure
    t = Timer(iters, direct=direct)
    out: list[dict] = []
    M = 4096 if small else 32768

    def wanted(name, shape):
        return pick is None or pick in f"{name} {shape}"

    def hbm(name, shape, nbytes, fn):
        if not wanted(name, shape):
            return
        ms = t(fn)
        gbs = nbytes / ms / 1e6
        out.append({"kernel": name, "shape": shape, "ms": round(ms, 4), "bound": "hbm", "achieved": round(gbs, 1),
                    "unit": "GB/s", "algorithmic_bytes": nbytes, "peak": hbm_peak,
                    "frac_of_measured": round(gbs / hbm_peak, 3) if hbm_peak else None,
                    "frac_of_nominal_8000": round(gbs / 8000.0, 3)})
        if not quiet:
            print(json.dumps(out[-1]), flush=True)

    probe = torch.zeros(8, dtype=torch.int64, device="cuda")
    sms = torch.cuda.get_device_properties(0).multi_processor_count

    def tensor(name, shape, flops, fn):
        if not wanted(name, shape):
            return
        # SM cycles / ns added up by CTA 0 of every CTA-pair GEMM launch while this entry is timed: the clock the
        # GPU holds under the kernel's own power draw (a library GEMM timed as a yardstick adds nothing)
        probe.zero_()
        _lib.check(_lib.load().anima_mx_gemm_set_clock_probe(probe.data_ptr()))
        ms = t(fn)
        _lib.check(_lib.load().anima_mx_gemm_set_clock_probe(None))
        cycles, ns, _, w_stage, w_operands, w_acc, w_epi, _ = (int(v) for v in probe.cpu().tolist())
        tf = flops / ms / 1e9
        ghz = cycles / ns if ns else None
        out.append({"kernel": name, "shape": shape, "ms": round(ms, 4), "bound": "tensor", "achieved": round(tf, 1),
                    "unit": "TFLOP/s", "algorithmic_flops": flops, "peak": tf_peak,
                    "peak_note": "2 x measured burst bf16 cuBLAS (no measured fp8 figure)",
                    "frac_of_measured": round(tf / tf_peak, 3) if tf_peak else None,
                    "frac_of_nominal_4500": round(tf / 4500.0, 3),
                    "sm_mhz_in_kernel": round(ghz * 1000.0) if ghz else None,
                    "tensor_pipe_util_at_that_clock": round(tf * 1e3 / (sms * 16384 * ghz), 3) if ghz else None})
        if cycles:   # share of CTA 0's cycles its warps spent waiting (producer: free stage; issuer: operands,
            # accumulator buffer; first epilogue warp: a finished accumulator)
            out[-1]["wait_share"] = {"producer_free_stage": round(w_stage / cycles, 3),
                                     "issuer_operands": round(w_operands / cycles, 3),
                                     "issuer_accumulator": round(w_acc / cycles, 3),
                                     "epilogue_idle": round(w_epi / cycles, 3)}
        if not quiet:
            print(json.dumps(out[-1]), flush=True)

    if only in (None, "hbm"):
        K = 2048
        x = _acts(M, K)
        n = M * K
        hbm("mx_quantize rowwise", [M, K], int(n * 3.03125), lambda: ops.mx_quantize(x, rowwise=True))
        hbm("mx_quantize row+col", [M, K], int(n * 4.0625), lambda: ops.mx_quantize(x, rowwise=True, colwise=True))
        hbm("mx_quantize colwise", [M, K], int(n * 3.03125), lambda: ops.mx_quantize(x, rowwise=False, colwise=True))
        W = _acts(8192, 2048, 0.02)
        w1 = torch.randn(8, 8, device="cuda") * 0.1
        w2 = torch.randn(1024, 256, device="cuda") * 0.02
        hbm("lokr_merge_quantize row+col", [8192, 2048], int(8192 * 2048 * 4.0625),
            lambda: ops.lokr_merge_quantize(W, w1, w2, 1.0, want_merged=False, rowwise=True, colwise=True))
        dW = torch.randn(8192, 2048, device="cuda")
        hbm("lokr_kron_backward (fp32 dW)", [8192, 2048], 8192 * 2048 * 4, lambda: ops.lokr_kron_backward(dW, w1, w2, 1.0))
        BT, D = 8, 2048
        HW = M // BT
        xa, dy, y2 = _acts(M, D), _acts(M, D), _acts(M, D)
        sc, sh, ga = _acts(BT, D, 0.1), _acts(BT, D, 0.1), _acts(BT, D, 0.1)
        _, mean, rstd = ops.adaln_fwd(xa, sc, sh, 1e-6, HW)
        hbm("adaln_fwd", [BT, HW, D], M * D * 4 + M * 8, lambda: ops.adaln_fwd(xa, sc, sh, 1e-6, HW))
        hbm("adaln_fwd + row-wise MXFP8 operand of y", [BT, HW, D], int(M * D * 5.03125) + M * 8,
            lambda: ops.adaln_fwd(xa, sc, sh, 1e-6, HW, quant=True))
        hbm("adaln_bwd (dx+dscale+dshift)", [BT, HW, D], M * D * 6 + M * 8, lambda: ops.adaln_bwd(dy, xa, sc, mean, rstd, HW))
        hbm("gated_add_fwd", [BT, HW, D], M * D * 6, lambda: ops.gated_add_fwd(xa, ga, y2, HW))
        hbm("gated_add_bwd (dy+dgate)", [BT, HW, D], M * D * 6, lambda: ops.gated_add_bwd(dy, y2, ga, HW))
        hbm("gated_add + adaln fwd (one pass)", [BT, HW, D], M * D * 8 + M * 8,
            lambda: ops.gated_add_adaln_fwd(xa, ga, y2, sc, sh, 1e-6, HW))
        hbm("gated_add + adaln fwd + row-wise MXFP8 operand of y", [BT, HW, D], int(M * D * 9.03125) + M * 8,
            lambda: ops.gated_add_adaln_fwd(xa, ga, y2, sc, sh, 1e-6, HW, quant=True))
        hbm("gated_add + adaln bwd (one pass)", [BT, HW, D], M * D * 12 + M * 8,
            lambda: ops.gated_add_adaln_bwd(dy, y2, xa, sc, mean, rstd, y2, ga, HW))
        hid = (torch.randn(8, M // 8, 8, 128, device="cuda")).to(BF16)
        gm = torch.randn_like(hid)
        c = _acts(8, 8)
        mask = (torch.rand(8, 128, device="cuda") > 0.3).to(BF16)
        hbm("tlokr_rank_mix", list(hid.shape), hid.numel() * 4, lambda: ops.tlokr_rank_mix(hid, c, mask, False))
        hbm("tlokr_rank_mix + row-wise operand (no bf16 output)", list(hid.shape), int(hid.numel() * 3.03125),
            lambda: ops.tlokr_rank_mix_quant(hid, c, mask, False, rowwise=True))
        hbm("tlokr_rank_mix + column operand (no bf16 output)", list(hid.shape), int(hid.numel() * 3.03125),
            lambda: ops.tlokr_rank_mix_quant(hid, c, mask, False, rowwise=False, colwise=True))
        hbm("tlokr_rank_mix + row and column operands (no bf16 output)", list(hid.shape), int(hid.numel() * 4.0625),
            lambda: ops.tlokr_rank_mix_quant(hid, c, mask, True, rowwise=True, colwise=True))
        hbm("tlokr_rank_mix_wgrad", list(hid.shape), hid.numel() * 4, lambda: ops.tlokr_rank_mix_wgrad(gm, hid, mask))
        hbm("tlokr_rank_mix + row form as planes and column operand", list(hid.shape), int(hid.numel() * 4.0625),
            lambda: ops.tlokr_rank_mix_quant_planes(hid, c, mask, True, colwise=True))
        # hidden = grouped . B^T, mix, mask, quantise in one kernel: reads the grouped codes, writes the planes
        xg = _acts(M * 8, 256)
        xgq, _ = ops.mx_quantize(xg, rowwise=True)
        bq, _ = ops.mx_quantize(_acts(128, 256, 0.2), rowwise=True)
        hbm("tlokr hidden GEMM + mix + quantise to planes (one kernel)", [8, M // 8, 8, 256],
            int(M * 8 * (256 * 1.03125 + 128 * 1.03125)), lambda: ops.tlokr_hidden_mix_planes(xgq, bq, c, mask, 8, False))
        hbm("mx_scales_regroup", [M, 2048], M * 2048 // 32 * 2, lambda: ops.mx_regroup(xgq, M, 2048))
        del xg, xgq
        hh, gg = _acts(M, 8192), _acts(M, 8192)
        nh = M * 8192
        hbm("mx_quantize_gelu rowwise", [M, 8192], int(nh * 3.03125), lambda: ops.mx_quantize_gelu(hh, rowwise=True))
        hbm("mx_quantize_gelu row+col", [M, 8192], int(nh * 4.0625),
            lambda: ops.mx_quantize_gelu(hh, rowwise=True, colwise=True))
        hbm("mx_quantize_gelu backward row+col", [M, 8192], int(nh * 6.0625),
            lambda: ops.mx_quantize_gelu(hh, gg, rowwise=True, colwise=True))
        del hh, gg
        L = M // BT
        q, dq = _acts(M, D).view(BT, L, 16, 128), _acts(M, D).view(BT, L, 16, 128)
        wn = torch.ones(128, device="cuda")
        ang = torch.rand(L, 128, device="cuda") * 60
        cos, sin = ang.cos(), ang.sin()
        _, rs = ops.rmsnorm_rope_fwd(q, wn, cos, sin, 1e-6)
        hbm("rmsnorm_rope_fwd", [BT, L, 16, 128], M * D * 4 + M * 16 * 4, lambda: ops.rmsnorm_rope_fwd(q, wn, cos, sin, 1e-6))
        hbm("rmsnorm_rope_bwd", [BT, L, 16, 128], M * D * 6 + M * 16 * 4, lambda: ops.rmsnorm_rope_bwd(dq, q, wn, cos, sin, rs))

    if only in (None, "tlokr"):
        # The T-LoKr delta of one module, x -> x @ kron(W1, (A * mask) @ B)^T, as the training step runs it: inside
        # the one-node quantised linear, where the mixed hidden tensor is made by one kernel and enters the base
        # GEMM as extra K-blocks. Its cost is what the linear takes beyond the base projection on the same
        # operands: forward = linear - base GEMM; backward = (input gradient + factor gradients) - base dgrad.
        # Algorithmic bytes of the delta alone: forward reads x and writes the delta, 2 B * rows * (in + out);
        # backward reads x and the incoming gradient and writes the input gradient, 2 B * rows * (2 * in + out).
        from . import tlokr
        from .fp8_quant import quantize_weight
        rank, batch = 128, 8
        for name, d_in, d_out, rows in TLOKR_MODULES:
            rows = rows // 8 if small else rows
            shape = [rows, d_in, d_out]
            if not any(wanted(f"tlokr_delta {d} {name}", shape) for d in ("fwd", "bwd")):
                continue
            x = _acts(rows, d_in)
            g = _acts(rows, d_out, 0.01)
            W_mx = quantize_weight(_acts(d_out, d_in, 0.02))
            w1 = torch.nn.Parameter(torch.randn(8, 8, device="cuda") * 0.3)
            a = torch.nn.Parameter(torch.randn(d_out // 8, rank, device="cuda") * 0.05)
            b = torch.nn.Parameter(torch.randn(rank, d_in // 8, device="cuda") * 0.05)
            mask = tlokr._TimestepState(timesteps=torch.rand(batch, device="cuda")).mask(
                max_rank=rank, min_rank=rank // 2, dtype=BF16, device=x.device)
            lead = (batch, rows // batch)
            gq, gq_col = ops.mx_quantize(x.view(rows * 8, d_in // 8), rowwise=True, colwise=True)
            x_row = ops.mx_regroup(gq, rows, d_in)
            gbq, gbq_col = ops.mx_quantize(g.view(rows * 8, d_out // 8), rowwise=True, colwise=True)
            g_row = ops.mx_regroup(gbq, rows, d_out)
            y = torch.empty(rows, d_out, dtype=BF16, device="cuda")
            gx = torch.empty(rows, d_in, dtype=BF16, device="cuda")
            _, fops = tlokr._mx_linear_fwd(x_row, gq, lead, W_mx, None, w1, a, b, mask, 0.5)
            t_lin = t(lambda: tlokr._mx_linear_fwd(x_row, gq, lead, W_mx, None, w1, a, b, mask, 0.5))
            t_base = t(lambda: ops.mx_gemm(x_row, W_mx.row, out=y))
            t_bwd = t(lambda: tlokr._mx_linear_bwd(lambda r, k: (gbq, gbq_col), lambda r, k: (gq, gq_col), lead, d_in, W_mx,
                                                   w1, a, b, mask, 0.5, fops))
            t_dgrad = t(lambda: ops.mx_gemm(g_row, W_mx.col, out=gx))
            for direction, ms, ms_base, nbytes in (("fwd", t_lin, t_base, 2 * rows * (d_in + d_out)),
                                                   ("bwd", t_bwd, t_dgrad, 2 * rows * (2 * d_in + d_out))):
                d_ms = max(ms - ms_base, 1e-6)
                gbs = nbytes / d_ms / 1e6
                out.append({"kernel": f"tlokr_delta {direction} {name}", "shape": shape, "ms": round(d_ms, 4),
                            "bound": "hbm", "achieved": round(gbs, 1), "unit": "GB/s", "algorithmic_bytes": nbytes,
                            "peak": hbm_peak, "frac_of_measured": round(gbs / hbm_peak, 3) if hbm_peak else None,
                            "frac_of_nominal_8000": round(gbs / 8000.0, 3),
                            "how": f"one-node T-LoKr linear {ms:.4f} ms - base GEMM alone {ms_base:.4f} ms, same operands"})
                if not quiet:
                    print(json.dumps(out[-1]), flush=True)
            del x, g, W_mx, gq, gq_col, gbq, gbq_col, x_row, g_row, y, gx

    if only in (None, "gemm"):
        for (N, K) in [(2048, 2048), (6144, 2048), (8192, 2048), (2048, 8192)]:
            x, w, gy = _acts(M, K), _acts(N, K, 0.02), _acts(M, N, 0.01)
            xr, xc = ops.mx_quantize(x, rowwise=True, colwise=True)
            wr, wc = ops.mx_quantize(w, rowwise=True, colwise=True)
            gr, gc = ops.mx_quantize(gy, rowwise=True, colwise=True)
            fl = 2.0 * M * N * K
            y = torch.empty(M, N, dtype=BF16, device="cuda")
            dx = torch.empty(M, K, dtype=BF16, device="cuda")
            dw = torch.empty(N, K, dtype=torch.float32, device="cuda")
            tensor("mx_gemm fwd", [M, N, K], fl, lambda: ops.mx_gemm(xr, wr, out=y))
            tensor("mx_gemm dgrad", [M, K, N], fl, lambda: ops.mx_gemm(gr, wc, out=dx))
            tensor("mx_gemm wgrad (fp32 out)", [N, K, M], fl, lambda: ops.mx_gemm(gc, xc, out_dtype=torch.float32, out=dw))
            if ops.can_fold_delta(M, N):
                # the T-LoKr linear as one GEMM: one more K-block per run of a tile's columns inside a delta block
                pl, _ = ops.mx_quantize(_acts(8 * M, 128), rowwise=True)
                dq, _ = ops.mx_quantize(_acts(N // 8, 128, 0.05), rowwise=True)
                tensor("mx_gemm_delta fwd (base + rank-128 delta)", [M, N, K], 2.0 * M * N * (K + 128),
                       lambda: ops.mx_gemm_delta(xr, wr, pl, dq, out=y))
                del pl, dq
            if yardstick:
                # the vendor library's MXFP8 GEMM on the SAME operands (its swizzled scale layout is the
                # 128 x 4 tiled layout): a measured ceiling to read the kernel against, not a code path
                try:
                    fn = cublaslt_mxfp8(xr, wr)
                    fn()
                    tensor("yardstick: cuBLASLt MXFP8 via torch._scaled_mm, fwd", [M, N, K], fl, fn)
                except Exception as e:  # noqa: BLE001 - the yardstick is optional
                    if not quiet:
                        print(json.dumps({"kernel": "yardstick: cuBLASLt MXFP8", "unavailable": str(e)[:200]}), flush=True)
            del x, w, gy, xr, xc, wr, wc, gr, gc, y, dx, dw
        # the T-LoKr factor gradients: small outputs over a contraction of rows * 8, split over K on the one-CTA kernel
        R8 = M * 8
        for (m_, n_) in [(256, 128), (128, 256), (1024, 128)]:
            aq, _ = ops.mx_quantize(_acts(m_, R8, 0.05), rowwise=True)
            bq2, _ = ops.mx_quantize(_acts(n_, R8, 0.05), rowwise=True)
            tensor("mx_gemm split-K factor gradient (fp32 out)", [m_, n_, R8], 2.0 * m_ * n_ * R8,
                   lambda: ops.mx_gemm(aq, bq2, out_dtype=torch.float32))
            del aq, bq2
        _lib.check_status_word(torch.device("cuda", torch.cuda.current_device()))
    return out


def summary(iters: int = 8) -> dict:
    """Every kernel at its production shape as one compact record per kernel (for the benchmark line):
    ``{name: {shape, ms, achieved, unit, peak, frac}}``; peaks are the measured ones (HBM copy; 2 x burst bf16
    GEMM, a kernel timed alone being in the burst regime)."""
    rows = run(iters, None, False, quiet=True, yardstick=True)   # incl. the vendor library's MXFP8 GEMM on the same operands
    out = {}
    for r in rows:
        out[f"{r['kernel']} {r['shape']}"] = {
            "ms": r["ms"], "achieved": r["achieved"], "unit": r["unit"], "bound": r["bound"], "peak": r["peak"],
            "frac": r["frac_of_measured"],
            "algorithmic": r.get("algorithmic_bytes", r.get("algorithmic_flops")),
            **({"sm_mhz_in_kernel": r["sm_mhz_in_kernel"], "tensor_pipe_util_at_that_clock":
                r["tensor_pipe_util_at_that_clock"]} if r.get("sm_mhz_in_kernel") else {})}
    return out


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--only", choices=["gemm", "hbm", "tlokr"], default=None)
    ap.add_argument("--small", action="store_true")
    ap.add_argument("--pick", default=None, help="run only entries whose 'name [shape]' contains this text")
    ap.add_argument("--direct", action="store_true", help="plain launches instead of CUDA-graph replays")
    ap.add_argument("--yardstick", action="store_true",
                    help="also time the vendor library's MXFP8 GEMM (torch._scaled_mm) on the same operands")
    a = ap.parse_args()
    run(a.iters, a.only, a.small, a.pick, a.direct, a.yardstick)
