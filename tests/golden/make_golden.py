"""Generate golden vectors from anima-trainer's OWN code (run once, where the reference
checkout is available; the .npz files it writes are committed, this script documents how).

    TRITON_INTERPRET=1 python tests/golden/make_golden.py /path/to/anima-trainer

* The reference's Triton kernels that the Triton CPU interpreter can execute (quantiser, AdaLN
  forward / dx / dscale+dshift, the gated-add dgate reduction, rank-mix wgrad) run under it, i.e.
  the reference source itself computes those vectors.
* Its torch code that runs on CPU (dequantize_rowwise, _StructuredLoKr, the timestep mask and
  schedule, the CPU branches of rank_mix / rank_mix_wgrad) is imported unmodified.
* What the interpreter cannot run (tl.dot_scaled; kernels doing bf16 arithmetic: rank mix forward,
  gated-add forward) comes from the reference's own stated equivalents: quantiser +
  dequantize_rowwise + fp32 matmul for the GEMM, the torch branch of rank_mix, the eager
  expression x + gate * y.
bf16 tensors are stored as uint16 bit patterns.
"""
from __future__ import annotations

import os
import sys
from pathlib import Path

os.environ.setdefault("TRITON_INTERPRET", "1")
if len(sys.argv) < 2:
    sys.exit("usage: make_golden.py /path/to/anima-trainer")
REF = Path(sys.argv[1])
sys.path.insert(0, str(REF / "src"))

import numpy as np  # noqa: E402
import torch  # noqa: E402

OUT = Path(__file__).resolve().parent
BF16 = torch.bfloat16


def bits(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).numpy().view(np.uint16).copy()


def quantiser_inputs() -> torch.Tensor:
    """[96, 256] bf16 with the quantiser's edge cases planted in known blocks."""
    g = torch.Generator().manual_seed(1234)
    x = torch.randn(96, 256, generator=g)
    x[:, 7] *= 50.0                                   # outlier channel (config 2 style)
    x[0, 0:32] = 0.0                                  # all-zero block -> scale byte 19
    x[1, 0:32] = 0.5; x[1, 0] = 1.75                  # amax mantissa exactly 1.75
    x[2, 0:32] = 0.25; x[2, 3] = -3.5                 # 1.75 * 2, negative
    x[3, 0:32] = 1e-3; x[3, 5] = 1.7578125            # next bf16 above 1.75
    x[4, 0:32] = 1e-3; x[4, 9] = 1.7421875            # next bf16 below 1.75
    x[5, 0:32] = torch.linspace(-500, 500, 32)        # large magnitudes
    x[6, 0:32] = 1e-20                                # tiny but above the 1e-30 floor
    x[7, 0:32] = 1e-38                                # below the floor
    x[8, 0:32] = 448.0; x[8, 1] = 449.0
    x[9, 0:32] = 3.0e38 * torch.sign(torch.randn(32, generator=g))   # near bf16 max
    x[10, 0:32] = torch.tensor([2.0 ** -k for k in range(32)])       # wide dynamic range in one block
    for e in range(-20, 20):                          # 1.75 * 2^e across exponents
        x[11 + (e + 20), 32:64] = 0.1 * 2.0 ** e
        x[11 + (e + 20), 40] = 1.75 * 2.0 ** e
    return x.to(BF16)


def gen_quantiser() -> None:
    from anima_trainer.mxfp8_gemm import (dequantize_rowwise, quantize_rowwise,
                                          quantize_weight_for_dgrad, quantize_weight_for_lhs)
    x = quantiser_inputs()
    blk = quantize_rowwise(x)
    deq = dequantize_rowwise(blk, tuple(x.shape))
    w = x[:64, :128].contiguous()
    lhs = quantize_weight_for_lhs(w)
    dg = quantize_weight_for_dgrad(w)
    np.savez_compressed(
        OUT / "quantiser.npz", x=bits(x), codes=blk.data.numpy(), scales=blk.scales.numpy(), deq=bits(deq),
        w=bits(w), lhs_codes=lhs.data.numpy(), lhs_scales=lhs.scales.numpy(),
        dgrad_codes=dg.data.numpy(), dgrad_scales=dg.scales.numpy())
    print("quantiser:", blk.data.shape, blk.scales.shape, dg.data.shape, dg.scales.shape)


def gen_gemm() -> None:
    from anima_trainer import mxfp8_gemm as ref
    g = torch.Generator().manual_seed(77)
    M, N, K = 64, 128, 256
    x = torch.randn(M, K, generator=g).to(BF16)
    x[:, 11] *= 50.0
    w = (torch.randn(N, K, generator=g) * 0.02).to(BF16)
    gy = torch.randn(M, N, generator=g).to(BF16)
    xq, wq, wq_b, gq = (ref.quantize_rowwise(x), ref.quantize_weight_for_lhs(w),
                        ref.quantize_weight_for_dgrad(w), ref.quantize_rowwise(gy))
    # The Triton interpreter cannot execute tl.dot_scaled, so the GEMM vectors come from the
    # reference's quantiser (interpreted) and its own dequantize_rowwise (mxfp8_gemm.py:225-232)
    # followed by an fp32 matmul: the "quantize+dequant+mm" reference its docstring names (:34-36).
    def deq(blk, shape):
        return ref.dequantize_rowwise(blk, shape).float()
    y = (deq(xq, (M, K)) @ deq(wq, (N, K)).t()).to(BF16)                       # fwd: x . W^T
    w_col = ref.MXFP8Block(data=wq_b.data.t().contiguous(), scales=wq_b.scales)  # (K, N) codes, (K, N//32) scales
    gx = (deq(gq, (M, N)) @ deq(w_col, (K, N)).t()).to(BF16)                   # dgrad: gy . W
    # The codes are stored too: the interpreter's emulated e4m3 cast is not the hardware's on ties,
    # mantissa carries and subnormals, so GEMM parity is pinned on these exact operands.
    np.savez_compressed(
        OUT / "gemm.npz", x=bits(x), w=bits(w), gy=bits(gy), y=bits(y), gx=bits(gx),
        x_codes=xq.data.numpy(), x_scales=xq.scales.numpy(), w_codes=wq.data.numpy(), w_scales=wq.scales.numpy(),
        g_codes=gq.data.numpy(), g_scales=gq.scales.numpy(), wT_codes=w_col.data.numpy(),
        wT_scales=w_col.scales.numpy())
    print("gemm:", y.shape, gx.shape, float(y.float().abs().max()), float(gx.float().abs().max()))


def gen_adaln() -> None:
    from anima_trainer import adaln_kernel as ref
    out = {}
    for name, (BT, HW, D) in {"a": (2, 24, 256), "b": (3, 8, 768)}.items():
        g = torch.Generator().manual_seed(5)
        N = BT * HW
        x = torch.randn(N, D, generator=g).to(BF16)
        s = (torch.randn(BT, D, generator=g) * 0.1).to(BF16)
        b = (torch.randn(BT, D, generator=g) * 0.1).to(BF16)
        gate = (torch.randn(BT, D, generator=g) * 0.1).to(BF16)
        y2 = torch.randn(N, D, generator=g).to(BF16)
        dy = torch.randn(N, D, generator=g).to(BF16)
        eps = 1e-6
        BLOCK_D = 1 << (D - 1).bit_length()
        y = torch.empty_like(x); mean = torch.empty(N); rstd = torch.empty(N)
        ref._fwd_kernel[(N,)](x, s, b, y, mean, rstd, HW, D, eps, BLOCK_D=BLOCK_D)
        dx = torch.empty_like(x)
        ref._bwd_dx_kernel[(N,)](dy, x, s, mean, rstd, dx, HW, D, BLOCK_D=BLOCK_D)
        ds = torch.zeros(BT, D); db = torch.zeros(BT, D)
        bd, bhw = min(BLOCK_D, 128), min(HW, 64)
        ref._bwd_dsdb_kernel[(BT, -(-HW // bhw), -(-D // bd))](dy, x, mean, rstd, ds, db, HW, D,
                                                               BLOCK_D=bd, BLOCK_HW=bhw)
        # _gated_add_fwd_kernel computes in bf16, which the CPU interpreter cannot represent; its
        # stated semantics (adaln_kernel.py:342-346, "out = x + gate * y") are taken in eager bf16.
        go = (x.view(BT, HW, D) + gate.view(BT, 1, D) * y2.view(BT, HW, D)).view(N, D)
        dg = torch.zeros(BT, D)
        ref._gated_add_bwd_dgate_kernel[(BT, -(-HW // bhw), -(-D // bd))](dy, y2, dg, HW, D,
                                                                          BLOCK_D=bd, BLOCK_HW=bhw)
        for k, v in dict(x=x, s=s, b=b, gate=gate, y2=y2, dy=dy, y=y, dx=dx, go=go).items():
            out[f"{name}_{k}"] = bits(v)
        for k, v in dict(mean=mean, rstd=rstd, ds=ds, db=db, dg=dg).items():
            out[f"{name}_{k}"] = v.numpy()
        out[f"{name}_shape"] = np.array([BT, HW, D])
    np.savez_compressed(OUT / "adaln.npz", **out)
    print("adaln: ok")


def gen_tlokr() -> None:
    from anima_trainer import tlokr as ref
    from anima_trainer import tlokr_kernels as rk
    out = {}
    # schedule known answers (tests/test_tlokr.py:59-76) straight from the reference function
    cases = [(1.0, 128, 64), (0.5, 128, 64), (0.0, 128, 64), (2.0, 8, 4), (-1.0, 8, 4), (0.375, 4, 2),
             (0.2, 4, 2), (0.9, 4, 2), (0.33, 128, 64), (0.999, 128, 64)]
    out["sched_cases"] = np.array(cases, dtype=np.float64)
    out["sched_out"] = np.array([ref.active_rank_for_timestep(t, max_rank=a, min_rank=b) for t, a, b in cases])
    t = torch.tensor([0.0, 0.2, 0.5, 0.9, 1.0, 1.5, -0.3, 0.731])
    st = ref._TimestepState(timesteps=t)
    out["mask_t"] = t.numpy()
    out["mask"] = st.mask(max_rank=128, min_rank=64, dtype=torch.float32, device=torch.device("cpu")).numpy()
    # rank mix: reference Triton kernels (interpreter) and its torch CPU branch
    g = torch.Generator().manual_seed(11)
    B, n, r = 2, 12, 128
    hidden = torch.randn(B, n, 8, r, generator=g).to(BF16)
    weight = torch.randn(8, 8, generator=g).to(BF16)
    grad = torch.randn(B, n, 8, r, generator=g).to(BF16)
    mask = torch.zeros(B, r, dtype=BF16); mask[0, :73] = 1; mask[1, :111] = 1
    total = B * n * r
    # _rank_mix_kernel multiplies in bf16, which the CPU interpreter cannot represent; the
    # reference's own torch branch of rank_mix (tlokr_kernels.py:140-146) gives the vectors.
    for tr in (False, True):
        out[f"mix_cpu_t{int(tr)}"] = bits(rk.rank_mix(hidden, weight, mask, transpose=tr))
    out["mix_cpu_nomask"] = bits(rk.rank_mix(hidden, weight, None))
    dc = torch.zeros(8, 8)
    rk._rank_mix_wgrad_kernel[(64, -(-total // 1024))](grad, hidden, mask, dc, n_per_batch=n, rank=r,
                                                       reduce_size=total, HAS_MASK=True, BLOCK=1024)
    out["wgrad"] = dc.numpy()
    out["wgrad_cpu"] = rk.rank_mix_wgrad(grad.float(), hidden.float(), mask.float()).numpy()
    for k, v in dict(hidden=hidden, weight=weight, grad=grad, mask=mask).items():
        out[f"mix_{k}"] = bits(v)
    # structured delta, fp32, forward + manual backward (tlokr.py:451-540), unmodified
    g = torch.Generator().manual_seed(3)
    Bs, L, up, uq, vp, vq, rk_ = 2, 5, 8, 8, 16, 8, 8
    x = torch.randn(Bs, L, uq * vq, generator=g, requires_grad=True)
    w1 = torch.randn(up, uq, generator=g, requires_grad=True)
    A = torch.randn(vp, rk_, generator=g, requires_grad=True)
    Bm = (torch.randn(rk_, vq, generator=g) * 0.2).requires_grad_(True)
    tt = torch.tensor([0.2, 0.9])
    m = ref._TimestepState(timesteps=tt).mask(max_rank=rk_, min_rank=4, dtype=torch.float32,
                                              device=torch.device("cpu"))
    probe = torch.randn(Bs, L, up * vp, generator=g)
    y = ref._StructuredLoKr.apply(x, w1, A, Bm, m)
    (y * probe).sum().backward()
    out.update(sd_x=x.detach().numpy(), sd_w1=w1.detach().numpy(), sd_a=A.detach().numpy(),
               sd_b=Bm.detach().numpy(), sd_mask=m.numpy(), sd_t=tt.numpy(), sd_probe=probe.numpy(),
               sd_y=y.detach().numpy(), sd_gx=x.grad.numpy(), sd_gw1=w1.grad.numpy(), sd_ga=A.grad.numpy(),
               sd_gb=Bm.grad.numpy())
    np.savez_compressed(OUT / "tlokr.npz", **out)
    print("tlokr: ok", out["sched_out"])


if __name__ == "__main__":
    torch.manual_seed(0)
    gen_quantiser()
    gen_gemm()
    gen_adaln()
    gen_tlokr()
