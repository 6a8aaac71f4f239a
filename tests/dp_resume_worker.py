"""Worker of the two-rank save / reload test (gloo, CPU, bf16 arm). Launched by test_adapter_state_cpu.py."""
import copy
import sys
from pathlib import Path

import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))

from anima_trainer_sm120_b200 import adapter_io, training_state  # noqa: E402
from anima_trainer_sm120_b200.anima_dit import tiny_config  # noqa: E402
from anima_trainer_sm120_b200.train_step import StepConfig, Trainer  # noqa: E402


def main(out_dir: str) -> None:
    dist.init_process_group("gloo")
    rank = dist.get_rank()
    torch.set_num_threads(2)
    out = Path(out_dir)
    cfg = StepConfig(precision="bf16", lokr_dim=8, gradient_checkpointing=True, lr=1e-2,
                     grad_bucket_blocks=1)
    mcfg = tiny_config(dim=128, heads=2, mlp_dim=256, context_dim=64, adaln_lora_dim=16, depth=2)
    tr = Trainer(mcfg, cfg, torch.device("cpu"))
    with torch.no_grad():
        g = torch.Generator().manual_seed(5)
        for m in tr.network.unet_loras:
            m.lokr_w2.copy_(torch.randn(m.lokr_w2.shape, generator=g) * 0.05)
    tr.run(steps=1, batch=2, latent_hw=8, text_tokens=6)
    # checkpoint: adapter file (rank 0 only), RNG payload gathered on rank 0, optimizer state (replicated)
    ckpt = out / "adapter.safetensors"
    written = tr.save(ckpt)
    if written:
        (out / f"wrote_rank{rank}").touch()
    payload = training_state.gather_rng_states()
    if rank == 0:
        torch.save(payload, out / "rng.pt")
    dist.barrier()
    opt_state = copy.deepcopy(tr.opt.state_dict())    # a snapshot: state_dict() hands out the live tensors
    # the run that continues works from the bf16-rounded adapters too, so that both arms start equal
    tr.load(ckpt)
    loss_continued = tr.run(steps=1, batch=2, latent_hw=8, text_tokens=6)
    continued = [p.detach().clone() for p in tr.params]
    # the run that resumes: fresh trainer, adapter file, optimizer state, this rank's RNG snapshot
    fresh = Trainer(mcfg, cfg, torch.device("cpu"))
    fresh.load(ckpt)
    fresh.opt.load_state_dict(opt_state)
    fresh.step_idx = 1
    payload = torch.load(out / "rng.pt", weights_only=False)
    rng = training_state.restore_rng_state(payload)
    try:
        training_state.restore_rng_state({"world_size": 1, "ranks": payload["ranks"][:1]})
        world_change = "accepted"
    except training_state.TrainingStateError as e:
        world_change = type(e).__name__
    loss_resumed = fresh.run(steps=1, batch=2, latent_hw=8, text_tokens=6)
    dist.barrier()
    writers = sorted(int(p.name[len("wrote_rank"):]) for p in out.glob("wrote_rank*"))
    torch.save({"continued": continued, "resumed": [p.detach().clone() for p in fresh.params],
                "loss_continued": loss_continued, "loss_resumed": loss_resumed, "rng": rng,
                "world_change": world_change, "writers": writers}, out / f"resume_rank{rank}.pt")
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main(sys.argv[1])
