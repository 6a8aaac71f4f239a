"""CUDA-graph capture of one rank's forward + backward, with the call surface of anima-trainer's
``cuda_graphs.py`` (``CUDAGraphRunner`` :68-234, ``make_bucket_key`` :237-241).

What is in the graph: the DiT forward under autocast, the loss and ``loss.backward()``; the adapter gradients
accumulate into the ``.grad`` tensors the parameters already hold (views of the trainer's flat gradient buffer),
which therefore must exist before capture. What stays outside, as in the reference: drawing noise and timesteps,
the data-parallel gradient exchange, clipping and ``optimizer.step()``. One graph per ``bucket_key`` (the input
shapes), all sharing one memory pool; the first ``warmup_steps`` calls of a key run eagerly on the capture stream
(lazy per-device state of the kernels - shared-memory opt-in, lookup tables, scratch buffers, work-list cache -
settles there), the last of them is followed by the capture, and every later call copies the batch into the static
inputs and replays.

Every kernel of this library is capturable: entry points take the stream they are launched on, never allocate and
never synchronise (the two documented exceptions, the GELU table fill and the no-allocation AdaLN backward's
symbol lookup, happen on a device's first call, i.e. during warm-up). Tensor maps are encoded on the host from
buffer addresses, which a replay reuses because the buffers come from the graph's private pool.

The batch is a plain dict of tensors; every entry gets a static twin (the reference fixes the field names of its
own model, :51-65; the runner here is agnostic to them).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable

import torch


@dataclass
class _BucketGraph:
    """One captured graph, the static tensors that feed it and the loss it writes."""

    graph: torch.cuda.CUDAGraph
    inputs: dict
    loss: torch.Tensor


class CUDAGraphRunner:
    """One captured forward+backward graph per bucket key.

    >>> runner = CUDAGraphRunner(forward_and_loss_fn, warmup_steps=3)
    >>> loss = runner.step(bucket_key, batch, params)      # inside the training loop
    >>> # caller: gradient exchange, clip_grad_norm_, optimizer.step(), zeroing the gradients in place

    ``forward_and_loss_fn(batch) -> scalar loss`` is the captured region's forward; the runner calls
    ``loss.backward()``. Gradients must be zeroed IN PLACE between steps (the graph accumulates into fixed
    buffers)."""

    def __init__(self, forward_and_loss_fn: Callable[[dict], torch.Tensor], *, warmup_steps: int = 3) -> None:
        if warmup_steps < 1:
            raise ValueError("warmup_steps must be at least 1")
        self._forward = forward_and_loss_fn
        self._warmup_steps = warmup_steps
        self._pool = torch.cuda.graph_pool_handle()       # shared by all buckets' graphs
        self._capture_stream = torch.cuda.Stream()        # warm-up and capture run here (one stream for autograd)
        self._state: dict = {}

    @staticmethod
    def _warm_grads(params) -> None:
        for p in params:
            if p.grad is None:
                p.grad = torch.zeros_like(p)

    @staticmethod
    def _copy_in(bg: _BucketGraph, batch: dict) -> None:
        for k, dst in bg.inputs.items():
            dst.copy_(batch[k], non_blocking=True)

    def captured(self, bucket_key) -> bool:
        return isinstance(self._state.get(bucket_key), _BucketGraph)

    def step(self, bucket_key, batch: dict, params) -> torch.Tensor:
        """One forward+backward for ``bucket_key``; returns the detached scalar loss (on the GPU)."""
        st = self._state.get(bucket_key)
        default_stream = torch.cuda.current_stream()
        if isinstance(st, _BucketGraph):                    # captured: copy in, replay
            self._copy_in(st, batch)
            st.graph.replay()
            return st.loss
        self._capture_stream.wait_stream(default_stream)
        count = 1 if st is None else st + 1
        self._state[bucket_key] = count
        if count < self._warmup_steps:                      # eager warm-up on the capture stream
            with torch.cuda.stream(self._capture_stream):
                loss = self._forward(batch)
                loss.backward()
            default_stream.wait_stream(self._capture_stream)
            return loss.detach()
        with torch.cuda.stream(self._capture_stream):       # last eager pass, then the capture
            loss = self._forward(batch)
            loss.backward()
            self._warm_grads(params)
            bg = _BucketGraph(torch.cuda.CUDAGraph(), {k: torch.empty_like(v.detach()) for k, v in batch.items()},
                              torch.empty((), device=loss.device, dtype=torch.float32))
            self._copy_in(bg, batch)
            eager_loss = loss.detach().clone()
            del loss
            torch.cuda.current_stream().synchronize()
            # The eager pass above already accumulated this step's gradients; the capture below only records
            # work (a captured region does not execute), so the step's result is the eager one.
            override = getattr(torch.autograd.graph, "set_override_stale_capture_stream", None)
            if override is not None:
                override(True)
            try:
                with torch.cuda.graph(bg.graph, pool=self._pool):
                    static_loss = self._forward(bg.inputs)
                    bg.loss.copy_(static_loss.detach())
                    static_loss.backward()
            finally:
                if override is not None:
                    override(False)
        default_stream.wait_stream(self._capture_stream)
        self._state[bucket_key] = bg
        return eager_loss


def make_bucket_key(*tensors: torch.Tensor) -> tuple:
    """Hashable key of a captured graph: the shapes of the tensors that vary between buckets (the reference keys
    on the latent and the text-token shapes, :237-241)."""
    return tuple(tuple(t.shape) for t in tensors)
