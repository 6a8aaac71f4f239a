"""Worker of the two-rank gloo test: one data-parallel step of the bf16 arm on a tiny model, and (on
rank 0) the hand-averaged single-process equivalent. Launched by test_modules_cpu.py via torchrun."""
import sys
from pathlib import Path

import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))

from anima_trainer_sm120_b200.anima_dit import tiny_config  # noqa: E402
from anima_trainer_sm120_b200.train_step import StepConfig, Trainer  # noqa: E402


def main(out_dir: str) -> None:
    dist.init_process_group("gloo")
    rank = dist.get_rank()
    torch.set_num_threads(2)
    cfg = StepConfig(precision="bf16", lokr_dim=8, gradient_checkpointing=True, lr=1e-2)
    mcfg = tiny_config(dim=128, heads=2, mlp_dim=256, context_dim=64, adaln_lora_dim=16, depth=2)
    tr = Trainer(mcfg, cfg, torch.device("cpu"))
    with torch.no_grad():                                   # non-zero delta so every adapter gets a gradient
        g = torch.Generator().manual_seed(5)
        for m in tr.network.unet_loras:
            m.lokr_w2.copy_(torch.randn(m.lokr_w2.shape, generator=g) * 0.05)
    start = [p.detach().clone() for p in tr.params]
    losses = tr.run(steps=1, batch=2, latent_hw=8, text_tokens=6)
    torch.save({"losses": losses, "params": [p.detach().clone() for p in tr.params]}, Path(out_dir) / f"rank{rank}.pt")
    dist.barrier()
    dist.destroy_process_group()
    if rank == 0:
        # single process: gradients of both shards averaged by hand, then the same clip + AdamW step
        ref = Trainer(mcfg, cfg, torch.device("cpu"))
        with torch.no_grad():
            for p, s in zip(ref.params, start):
                p.copy_(s)
        grads = torch.zeros_like(ref.flat_grad)
        for r in (0, 1):
            ref.rank = r
            lat, ctx, seed = ref.synthetic_batch(2, 8, 6, 0)
            ref.flat_grad.zero_()
            ref.forward_and_loss(lat, ctx, seed).backward()
            grads += ref.flat_grad
        ref.flat_grad.copy_(grads / 2)
        torch.nn.utils.clip_grad_norm_(ref.params, cfg.max_grad_norm)
        ref.opt.step()
        torch.save({"params": [p.detach().clone() for p in ref.params]}, Path(out_dir) / "single.pt")


if __name__ == "__main__":
    main(sys.argv[1])
