"""Data-parallel LoKr training step on the Anima-shaped DiT: the caller of the hot path.

What anima-trainer's loop does per step (``train.py:410-457``; ``flow.py:11-36``): draw
``t = sigmoid(N(0,1))`` per sample, ``noisy = (1-t) x + t noise``, ``target = noise - x``; forward
under bf16 autocast, fp32 MSE, backward, ``clip_grad_norm_(1.0)``, optimizer step. The reference is
single-GPU; here the batch is additionally sharded over the ranks of one node and the adapter
gradients are summed with ONE all-reduce of a flat fp32 buffer between backward and the clip
(the clip needs the global gradient), then scaled by 1 / world.

Two precision arms share everything but the kernels:
  ``bf16``   the reference's bf16 mode restated — eager LayerNorm / modulation / gated add, merged
             weight ``F.linear`` for the adapters (``lokr_patch`` bf16 path). Runs on CPU too.
  ``bf16_fused``  bf16 linears with this package's AdaLN / gated-add / RMSNorm+RoPE kernels (the reference's bf16
             mode keeps its fused glue kernels too): isolates the gain of the MXFP8 linears.
  ``mxfp8``  this package's kernels behind the same module patches: fused AdaLN + gated residual,
             fused q / k RMSNorm + RoPE, merged modulation MLPs, the LoKr MLP as one node
             with GELU quantised in its producer, MXFP8 frozen linears, fused MXFP8 LoKr linears (or T-LoKr).
The optimizer is AdamW for both arms: the reference's Prodigy + ScheduleFree is not available, so
loss-curve parity is between arms, not against the reference's optimizer trajectory.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist
import torch.nn.functional as F

from . import adaln_kernel, adaln_merge, adaln_patch, lokr_patch, mlp_patch, precision, qk_norm_rope
from .anima_dit import AnimaConfig, AnimaDiT, Attention, Block, GPT2FeedForward
from .lokr import attach_lokr


def noisy_input_and_target(latents: torch.Tensor, gen: torch.Generator | None = None):
    """(noisy, target, t) for rectified flow; t = 1 is pure noise (reference ``flow.py:17-36``)."""
    B = latents.shape[0]
    t = torch.sigmoid(torch.randn(B, device=latents.device, generator=gen))
    noise = torch.randn(latents.shape, device=latents.device, generator=gen).to(latents.dtype)
    tb = t.view(B, *([1] * (latents.dim() - 1))).to(latents.dtype)
    return (1 - tb) * latents + tb * noise, noise - latents, t


@dataclass
class StepConfig:
    precision: str = "mxfp8"          # "bf16" | "bf16_fused" | "mxfp8"
    variant: str = "lokr"             # "lokr" | "tlokr"
    preset: str = "anima-cross-mlp"
    lokr_dim: int = 128
    lokr_factor: int = 8
    min_rank_ratio: float = 0.5
    lr: float = 1e-4
    gradient_checkpointing: bool = True
    max_grad_norm: float = 1.0
    seed: int = 42
    grad_bucket_blocks: int = 4       # DP: adapter gradients of this many DiT blocks travel in one all-reduce
    status_check_every: int = 1       # steps between reads of the kernels' bounded-wait status words (0 = never)
    cuda_graph: bool = False          # capture forward + backward per input shape and replay it (cuda_graphs.py)
    cuda_graph_warmup: int = 3


class Trainer:
    """Builds model + adapters for one rank and runs optimizer steps on synthetic batches."""

    def __init__(self, model_cfg: AnimaConfig, cfg: StepConfig, device: torch.device):
        if cfg.precision not in ("bf16", "bf16_fused", "mxfp8"):
            raise ValueError(f"precision must be 'bf16', 'bf16_fused' or 'mxfp8', got {cfg.precision!r}")
        self.cfg, self.model_cfg, self.device = cfg, model_cfg, device
        self.world = dist.get_world_size() if dist.is_initialized() else 1
        self.rank = dist.get_rank() if dist.is_initialized() else 0
        torch.manual_seed(cfg.seed)                      # identical base weights and adapters on every rank
        self.dit = AnimaDiT(model_cfg).to(device=device, dtype=torch.bfloat16)
        self.dit.enable_gradient_checkpointing(cfg.gradient_checkpointing)
        self.network = attach_lokr(self.dit, preset=cfg.preset, factor=cfg.lokr_factor, dim=cfg.lokr_dim,
                                   alpha=cfg.lokr_dim, variant=cfg.variant,
                                   timestep_min_rank_ratio=cfg.min_rank_ratio)
        self.tlokr = cfg.variant == "tlokr"
        if self.tlokr:
            from . import tlokr
            self._tlokr = tlokr
            # checkpoint recomputation runs on autograd's worker thread, which does not inherit the
            # ContextVar: the block wrapper re-enters the forward's timestep state there
            tlokr.install_root_timestep_hooks(self.dit)
        if cfg.precision == "mxfp8":
            if device.type != "cuda":
                raise RuntimeError("precision='mxfp8' needs a CUDA device: the kernels have no CPU path")
            from . import fp8_quant
            adaln_merge.merge_adaln_modulation(self.dit)
            adaln_patch.install(Block)
            qk_norm_rope.install(Attention)
            mlp_patch.install(GPT2FeedForward)       # takes effect for plain LoKr adapters on the quantised path
            adaln_kernel.emit_row_operand(True)      # every consumer of an AdaLN output is a quantised linear here
            wrapped = fp8_quant.collect_lokr_wrapped_linears(self.network)
            self.n_frozen_quantised = fp8_quant.quantize_frozen_linears(self.dit, skip=wrapped)
            if self.tlokr:
                fp8_quant.quantize_tlokr_base_weights(self.network)
            else:
                lokr_patch.enable_fp8(self.network)
        elif cfg.precision == "bf16_fused":
            # bf16 linears (cuBLAS, merged-weight F.linear for the adapters) with this package's AdaLN / gated-add
            # and q/k RMSNorm+RoPE kernels: the reference's bf16 mode also runs its fused glue kernels, so this arm
            # separates what the MXFP8 linears gain from what the glue kernels gain.
            if device.type != "cuda":
                raise RuntimeError("precision='bf16_fused' needs a CUDA device: the kernels have no CPU path")
            adaln_merge.merge_adaln_modulation(self.dit)
            adaln_patch.install(Block)
            qk_norm_rope.install(Attention)
            mlp_patch.uninstall(GPT2FeedForward)
            lokr_patch.disable_fp8()
            adaln_kernel.emit_row_operand(False)
        else:
            adaln_patch.uninstall(Block)
            qk_norm_rope.uninstall(Attention)
            mlp_patch.uninstall(GPT2FeedForward)
            lokr_patch.disable_fp8()
            adaln_kernel.emit_row_operand(False)
        self.dit.train()
        self.params = [p for p in self.network.parameters() if p.requires_grad]
        # flat fp32 gradient buffer; every .grad is a view into it, so the DP exchange is one call
        n = sum(p.numel() for p in self.params)
        self.flat_grad = torch.zeros(n, dtype=torch.float32, device=device)
        off = 0
        for p in self.params:
            p.grad = self.flat_grad[off:off + p.numel()].view_as(p)
            off += p.numel()
        self.opt = torch.optim.AdamW(self.params, lr=cfg.lr, betas=(0.9, 0.99), weight_decay=0.0)
        self.step_idx = 0
        self.autocast_mode = "bf16" if cfg.precision.startswith("bf16") else "mxfp8"
        self.runner = None
        if cfg.cuda_graph:
            if device.type != "cuda":
                raise RuntimeError("cuda_graph=True needs a CUDA device")
            from .cuda_graphs import CUDAGraphRunner
            self.runner = CUDAGraphRunner(self._loss_of_batch, warmup_steps=cfg.cuda_graph_warmup)
        self.last_allreduce_exposed_ms: float | None = None
        self._build_buckets()

    # ---------------------------------------------------------------- data-parallel exchange
    def _build_buckets(self) -> None:
        """Split the flat gradient into contiguous buckets of ``grad_bucket_blocks`` DiT blocks each. Backward
        retires the blocks last to first; a hook on every parameter counts its bucket down and the bucket's
        all-reduce is launched (asynchronously: the communication library runs it on its own stream, ordered
        after the kernels that produced the bucket) the moment its last gradient has been accumulated, so the
        exchange of all but the first blocks' gradients hides under the rest of backward."""
        self._buckets: list[tuple[int, int]] = []          # (start, end) offsets into flat_grad
        self._bucket_of: dict[int, int] = {}               # id(param) -> bucket index
        self._bucket_size: list[int] = []
        self._pending: list[int] = []
        self._works: list = []
        if self.world == 1:
            return
        per_bucket = max(1, int(self.cfg.grad_bucket_blocks))
        n_mod_per_block = max(1, len(self.network.unet_loras) // max(1, self.model_cfg.depth))
        params_per_module = len(self.params) // max(1, len(self.network.unet_loras))
        group = max(1, n_mod_per_block * params_per_module * per_bucket)
        off = 0
        for i in range(0, len(self.params), group):
            chunk = self.params[i:i + group]
            n = sum(p.numel() for p in chunk)
            for p in chunk:
                self._bucket_of[id(p)] = len(self._buckets)
            self._buckets.append((off, off + n))
            self._bucket_size.append(len(chunk))
            off += n
        for p in self.params:
            p.register_post_accumulate_grad_hook(self._on_grad_ready)

    def _on_grad_ready(self, p: torch.Tensor) -> None:
        if not self._pending:
            return                                         # a backward outside step(): nothing to exchange
        b = self._bucket_of[id(p)]
        self._pending[b] -= 1
        if self._pending[b] == 0:
            lo, hi = self._buckets[b]
            self._works.append(dist.all_reduce(self.flat_grad[lo:hi], async_op=True))

    def _finish_exchange(self) -> None:
        """Launch what the hooks did not (a parameter that received no gradient keeps its bucket open), wait for
        every bucket and average."""
        for b, left in enumerate(self._pending):
            if left > 0:
                lo, hi = self._buckets[b]
                self._works.append(dist.all_reduce(self.flat_grad[lo:hi], async_op=True))
        self._pending = []
        timed = self.device.type == "cuda"
        if timed:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
        for w in self._works:
            w.wait()
        self._works = []
        if timed:
            e1.record()
            self._exchange_events = (e0, e1)
        self.flat_grad.mul_(1.0 / self.world)

    # ---------------------------------------------------------------- data
    def synthetic_batch(self, batch: int, latent_hw: int, text_tokens: int, step: int):
        """Seeded per (step, rank): latents (B,16,1,h,w) ~ N(0,1), text embeddings ~ N(0,1)."""
        g = torch.Generator(device="cpu").manual_seed(1000003 * step + 7919 * self.rank + self.cfg.seed)
        c = self.model_cfg
        lat = torch.randn(batch, c.latent_channels, 1, latent_hw, latent_hw, generator=g)
        ctx = torch.randn(batch, text_tokens, c.context_dim, generator=g)
        noise_seed = int(torch.randint(0, 2 ** 31 - 1, (1,), generator=g))
        return lat.to(self.device, torch.bfloat16), ctx.to(self.device, torch.bfloat16), noise_seed

    # ---------------------------------------------------------------- one step
    def make_batch(self, latents, ctx, noise_seed: int) -> dict:
        """Noise, timesteps and targets of one step (drawn outside any captured region)."""
        g = torch.Generator(device=self.device).manual_seed(noise_seed)
        noisy, target, t = noisy_input_and_target(latents, g)
        return {"noisy": noisy, "target": target, "timesteps": t, "context": ctx}

    def _loss_of_batch(self, batch: dict) -> torch.Tensor:
        if self.tlokr:
            self._tlokr.set_timestep(batch["timesteps"])
        with precision.autocast_for(self.autocast_mode, self.device.type), precision.fp8_autocast_for(self.autocast_mode):
            pred = self.dit(batch["noisy"], batch["timesteps"], batch["context"])
        return F.mse_loss(pred.float(), batch["target"].float())

    def forward_and_loss(self, latents, ctx, noise_seed: int):
        return self._loss_of_batch(self.make_batch(latents, ctx, noise_seed))

    def step(self, latents, ctx, noise_seed: int) -> float:
        self.flat_grad.zero_()
        if self.runner is not None:
            # forward + backward as a replayed CUDA graph; no Python runs inside it, so the gradient buckets cannot be
            # launched as backward retires them: the whole buffer is exchanged after the replay
            from .cuda_graphs import make_bucket_key
            batch = self.make_batch(latents, ctx, noise_seed)
            try:
                loss = self.runner.step(make_bucket_key(batch["noisy"], batch["context"]), batch, self.params)
            finally:
                if self.tlokr:
                    self._tlokr.clear_timestep()
            if self.world > 1:
                dist.all_reduce(self.flat_grad)
                self.flat_grad.mul_(1.0 / self.world)
        else:
            if self.world > 1:
                self._pending = list(self._bucket_size)
            try:
                loss = self.forward_and_loss(latents, ctx, noise_seed)
                loss.backward()
            finally:
                if self.tlokr:
                    self._tlokr.clear_timestep()
                if self.world > 1 and not self._works and self._pending == self._bucket_size:
                    self._pending = []              # forward or backward raised before any bucket left
            if self.world > 1:                      # the only exchange of the data-parallel step
                self._finish_exchange()
        torch.nn.utils.clip_grad_norm_(self.params, self.cfg.max_grad_norm)
        self.opt.step()
        self.step_idx += 1
        value = float(loss.detach())            # synchronises: everything the step launched has run
        ev = getattr(self, "_exchange_events", None)
        if ev is not None:
            self.last_allreduce_exposed_ms = ev[0].elapsed_time(ev[1])
            self._exchange_events = None
        every = self.cfg.status_check_every
        if self.cfg.precision == "mxfp8" and every and self.step_idx % every == 0:
            self.check_kernel_status()
        return value

    def check_kernel_status(self) -> None:
        """Raise if a bounded wait inside one of the library's kernels gave up since the last check (its outputs
        are then undefined, and so are this step's loss and update). Call after a synchronisation."""
        from . import _lib
        _lib.check_status_word(self.device)
        _lib.check_quantize_status()

    # ---------------------------------------------------------------- adapter file
    def save(self, path) -> int:
        """Publish the adapter file (rank 0 writes, every rank waits; ``adapter_io.save_adapter``)."""
        from .adapter_io import save_adapter
        return save_adapter(self.network, path)

    def load(self, path) -> dict:
        """Load an adapter file on every rank (``adapter_io.load_adapter``)."""
        from .adapter_io import load_adapter
        return load_adapter(self.network, path)

    def run(self, steps: int, batch: int, latent_hw: int, text_tokens: int) -> list[float]:
        losses = []
        for s in range(steps):
            lat, ctx, seed = self.synthetic_batch(batch, latent_hw, text_tokens, self.step_idx)
            losses.append(self.step(lat, ctx, seed))
        return losses
