"""Per-kernel device time of one optimizer step of the Anima-shaped training step.

    python -m anima_trainer_sm120_b200.step_profile [--arm mxfp8|bf16] [--variant lokr|tlokr] [--top 30]
                                                    [--no-checkpoint]

Runs two warm-up steps, then one step under ``torch.profiler`` (CUDA activities) and prints the kernels
ranked by total device time with launch counts and shares. This is how the share of the hot-path
kernels, of the library SDPA and of the remaining eager glue in a full step is read.
"""
from __future__ import annotations

import argparse
import collections

import torch
from torch.profiler import ProfilerActivity, profile

from .anima_dit import AnimaConfig
from .train_step import StepConfig, Trainer


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--arm", default="mxfp8", choices=["mxfp8", "bf16"])
    ap.add_argument("--variant", default="lokr", choices=["lokr", "tlokr"])
    ap.add_argument("--depth", type=int, default=28)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--latent", type=int, default=128)
    ap.add_argument("--text", type=int, default=512)
    ap.add_argument("--top", type=int, default=30)
    ap.add_argument("--no-checkpoint", action="store_true")
    ap.add_argument("--gaps", type=int, default=0,
                    help="also list the N largest idle gaps between consecutive kernels (where the host fell behind)")
    a = ap.parse_args()
    dev = torch.device("cuda", 0)
    tr = Trainer(AnimaConfig(depth=a.depth), StepConfig(precision=a.arm, variant=a.variant,
                                                        gradient_checkpointing=not a.no_checkpoint), dev)
    for s in range(2):
        tr.step(*tr.synthetic_batch(a.batch, a.latent, a.text, s))
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA, ProfilerActivity.CPU]) as prof:
        tr.step(*tr.synthetic_batch(a.batch, a.latent, a.text, 2))
        torch.cuda.synchronize()
    agg: dict[str, list] = collections.defaultdict(lambda: [0, 0.0])
    for e in prof.events():
        if e.device_type == torch.autograd.DeviceType.CUDA:
            agg[e.name[:90]][0] += 1
            agg[e.name[:90]][1] += e.device_time
    total = sum(v[1] for v in agg.values())
    print(f"{a.arm} {a.variant} checkpointing={'off' if a.no_checkpoint else 'on'}: "
          f"{total / 1e3:.1f} ms of device time in {sum(v[0] for v in agg.values())} launches")
    for name, (n, us) in sorted(agg.items(), key=lambda kv: -kv[1][1])[:a.top]:
        print(f"{n:6d} {us / 1e3:9.2f} ms {100 * us / total:5.1f}%  {name}")
    if a.gaps:
        ev = sorted(((e.time_range.start, e.time_range.end, e.name) for e in prof.events()
                     if e.device_type == torch.autograd.DeviceType.CUDA), key=lambda t: t[0])
        span = ev[-1][1] - ev[0][0]
        gaps, busy_end = [], ev[0][1]
        for (st, en, name), (_, _, prev) in zip(ev[1:], ev[:-1]):
            if st > busy_end:
                gaps.append((st - busy_end, prev[:50], name[:50]))
            busy_end = max(busy_end, en)
        idle = sum(g[0] for g in gaps)
        print(f"span {span / 1e3:.1f} ms, idle {idle / 1e3:.1f} ms in {len(gaps)} gaps "
              f"({sum(1 for g in gaps if g[0] > 20)} longer than 20 us)")
        by_pair: dict[tuple, list] = collections.defaultdict(lambda: [0, 0.0])
        for us, prev, nxt in gaps:
            by_pair[(prev, nxt)][0] += 1
            by_pair[(prev, nxt)][1] += us
        for (prev, nxt), (n, us) in sorted(by_pair.items(), key=lambda kv: -kv[1][1])[:a.gaps]:
            print(f"{n:6d} {us / 1e3:8.2f} ms  after {prev}  before {nxt}")


if __name__ == "__main__":
    main()
