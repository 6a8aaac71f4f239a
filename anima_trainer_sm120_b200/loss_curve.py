"""50-step LoKr loss-curve parity and step timing of the Anima-shaped training step.

    python -m anima_trainer_sm120_b200.loss_curve [--steps 50] [--depth 28] [--batch 8] [--latent 128]
                                                  [--variant lokr|tlokr] [--arms bf16,mxfp8] [--lr 1e-4]
                                                  [--no-checkpoint]
    torchrun --nproc-per-node N ... -m anima_trainer_sm120_b200.loss_curve    (data parallel, NCCL)

Both arms start from the same seeded random-init stand-in DiT and adapters, see the same seeded
synthetic batch, noise and timesteps at every step and use the same AdamW optimizer; only the kernels
differ (``train_step.Trainer``). Prints one JSON line: per-step losses of each arm, the largest
per-step relative difference (criterion: <= 2 %), and steps/s of each arm (CUDA events, after 2
warm-up steps, max over ranks). Synthetic data stands in for the reference's private dataset and
AdamW for its Prodigy + ScheduleFree optimizer, neither of which is available.
"""
from __future__ import annotations

import argparse
import gc
import json
import os

import torch
import torch.distributed as dist

from .anima_dit import AnimaConfig
from .train_step import StepConfig, Trainer


def two_arm_curve(dev: torch.device, steps: int = 50, *, depth: int = 28, batch: int = 8, latent: int = 128,
                  text: int = 512, variant: str = "lokr", lr: float = 1e-4) -> dict:
    """The two-arm curve on one GPU as a compact record: largest per-step relative loss difference between the
    bf16 restatement and this library's kernels (criterion: <= 2 % at every step), the first and last losses and
    each arm's steps/s. Same seeded model, adapters, batches, noise and timesteps in both arms."""
    losses, rate = {}, {}
    for arm in ("bf16", "mxfp8"):
        gc.collect()
        torch.cuda.empty_cache()
        tr = Trainer(AnimaConfig(depth=depth), StepConfig(precision=arm, variant=variant, lr=lr), dev)
        ls, times = [], []
        for s in range(steps):
            lat, ctx, seed = tr.synthetic_batch(batch, latent, text, s)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            ls.append(tr.step(lat, ctx, seed))
            e1.record()
            e1.synchronize()
            if s >= 2:
                times.append(e0.elapsed_time(e1))
        losses[arm] = ls
        rate[arm] = 1000.0 * len(times) / sum(times) if times else None
        del tr
    gc.collect()
    torch.cuda.empty_cache()
    rel = [abs(b - m) / b for b, m in zip(losses["bf16"], losses["mxfp8"])]
    return {"steps": steps, "max_rel_diff": max(rel), "within_2pct": max(rel) <= 0.02,
            "step_of_max": rel.index(max(rel)), "first_losses": {a: l[0] for a, l in losses.items()},
            "last_losses": {a: l[-1] for a, l in losses.items()}, "steps_per_s": rate,
            "config": {"model": f"Anima-shaped stand-in DiT, {depth} blocks (random init, seed 42)", "batch": batch,
                       "latent_tokens": (latent // 2) ** 2, "text_tokens": text, "variant": variant,
                       "optimizer": "AdamW (stand-in for Prodigy + ScheduleFree, both arms)", "lr": lr,
                       "arms": "bf16 = eager restatement of the reference's bf16 mode; mxfp8 = this library",
                       "data": "synthetic"}}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--depth", type=int, default=28)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--latent", type=int, default=128, help="latent height = width (128 -> 4096 tokens)")
    ap.add_argument("--text", type=int, default=512)
    ap.add_argument("--variant", default="lokr", choices=["lokr", "tlokr"])
    ap.add_argument("--arms", default="bf16,mxfp8")
    ap.add_argument("--lr", type=float, default=1e-4)
    ap.add_argument("--no-checkpoint", action="store_true",
                    help="keep every block's activations instead of recomputing them (the reference's configuration "
                         "recomputes; 180 GB of HBM leaves room not to)")
    a = ap.parse_args()

    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    rank = dist.get_rank() if world > 1 else 0
    mcfg = AnimaConfig(depth=a.depth)
    out = {"config": {"depth": a.depth, "batch_per_gpu": a.batch, "tokens": (a.latent // 2) ** 2, "text_tokens": a.text,
                      "variant": a.variant, "n_gpus": world, "steps": a.steps, "optimizer": "AdamW (stand-in)",
                      "gradient_checkpointing": not a.no_checkpoint, "data": "synthetic"}, "losses": {}, "steps_per_s": {}}
    for arm in a.arms.split(","):
        gc.collect()                              # the previous arm's model sits in reference cycles (hooks)
        torch.cuda.empty_cache()
        torch.cuda.reset_peak_memory_stats(dev)   # peak memory is reported per arm
        tr = Trainer(mcfg, StepConfig(precision=arm, variant=a.variant, lr=a.lr,
                                       gradient_checkpointing=not a.no_checkpoint), dev)
        losses, times = [], []
        for s in range(a.steps):
            lat, ctx, seed = tr.synthetic_batch(a.batch, a.latent, a.text, s)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            losses.append(tr.step(lat, ctx, seed))
            e1.record()
            e1.synchronize()
            if s >= 2:
                times.append(e0.elapsed_time(e1))
        ms = torch.tensor([sum(times) / max(len(times), 1)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        out["losses"][arm] = losses
        out["steps_per_s"][arm] = 1000.0 / float(ms) if float(ms) > 0 else None
        out.setdefault("peak_mem_gb", {})[arm] = torch.cuda.max_memory_allocated(dev) / 2 ** 30
        del tr
        torch.cuda.empty_cache()
    if "bf16_fused" in out["losses"] and "mxfp8" in out["losses"]:
        rel = [abs(b - m) / b for b, m in zip(out["losses"]["bf16_fused"], out["losses"]["mxfp8"])]
        out["max_rel_diff_vs_bf16_fused"] = max(rel)
    if "bf16" in out["losses"] and "mxfp8" in out["losses"]:
        rel = [abs(b - m) / b for b, m in zip(out["losses"]["bf16"], out["losses"]["mxfp8"])]
        out["max_rel_diff"] = max(rel)
        out["within_2pct"] = max(rel) <= 0.02
    if rank == 0:
        print(json.dumps(out), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
