"""The scratch-free AdaLN backward entry point, called straight through the C ABI.

``anima_adaln_bwd_noalloc`` serves callers that are not in a position to allocate device memory when
they call the library (an operator embedded in a host framework that owns all GPU memory, a service with
a memory plan fixed at start-up): its partial sums live in an array compiled into the library. It must
return exactly what ``anima_adaln_bwd`` returns with a caller workspace — the reductions are fixed-order,
so the comparison is bit for bit — on back-to-back calls that reuse the shared array, must refuse shapes
that do not fit, and must work whether it is the first thing a process runs or the last.
This file sorts last on purpose: a run that stops at the first failure has then run everything else.
"""
from __future__ import annotations

import pytest
import torch

pytestmark = pytest.mark.gpu
BF16 = torch.bfloat16


def _inputs(bt, hw, d, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    rows = bt * hw
    x = torch.randn(rows, d, generator=g, device="cuda").to(BF16)
    dy = torch.randn(rows, d, generator=g, device="cuda").to(BF16)
    scale = (torch.randn(bt, d, generator=g, device="cuda") * 0.1).to(BF16)
    shift = (torch.randn(bt, d, generator=g, device="cuda") * 0.1).to(BF16)
    return x, dy, scale, shift


def _call_noalloc(lib, dy, x, scale, mean, rstd, hw):
    rows, d = x.shape
    dx, dscale, dshift = torch.empty_like(x), torch.empty_like(scale), torch.empty_like(scale)
    rc = lib.anima_adaln_bwd_noalloc(dy.data_ptr(), x.data_ptr(), scale.data_ptr(), mean.data_ptr(), rstd.data_ptr(),
                                     rows, hw, d, dx.data_ptr(), dscale.data_ptr(), dshift.data_ptr(),
                                     torch.cuda.current_stream().cuda_stream)
    return rc, dx, dscale, dshift


def test_noalloc_entry_matches_workspace_entry_on_consecutive_calls(lib):
    from anima_trainer_sm120_b200 import ops
    # two different shapes back to back (the second reuses, and partly overwrites, the shared array),
    # then the first again: stale contents of the array must never leak into a result
    cases = [(8, 1024, 2048, 1), (3, 40, 768, 2), (8, 1024, 2048, 3)]
    for bt, hw, d, seed in cases:
        x, dy, scale, shift = _inputs(bt, hw, d, seed)
        _, mean, rstd = ops.adaln_fwd(x, scale, shift, 1e-6, hw)
        want = ops.adaln_bwd(dy, x, scale, mean, rstd, hw)           # existing entry point, caller workspace
        for _ in range(2):
            rc, dx, dscale, dshift = _call_noalloc(lib, dy, x, scale, mean, rstd, hw)
            assert rc == 0, lib.anima_last_error()
            torch.cuda.synchronize()
            assert torch.equal(dx, want[0]) and torch.equal(dscale, want[1]) and torch.equal(dshift, want[2])


def test_noalloc_entry_refuses_shapes_beyond_the_built_in_array(lib):
    need = lib.anima_adaln_bwd_workspace_bytes(64 * 4096, 4096, 4096)
    assert need > 8 << 20
    x, dy, scale, shift = _inputs(1, 8, 64, 4)          # pointers only; the size check comes first
    mean = torch.zeros(8, device="cuda")
    rc = lib.anima_adaln_bwd_noalloc(dy.data_ptr(), x.data_ptr(), scale.data_ptr(), mean.data_ptr(), mean.data_ptr(),
                                     64 * 4096, 4096, 4096, x.data_ptr(), scale.data_ptr(), scale.data_ptr(), None)
    assert rc == -7 and b"built-in array" in lib.anima_last_error()
    rc = lib.anima_adaln_bwd_noalloc(dy.data_ptr(), x.data_ptr(), scale.data_ptr(), mean.data_ptr(), mean.data_ptr(),
                                     10, 4, 64, x.data_ptr(), scale.data_ptr(), scale.data_ptr(), None)
    assert rc == -3                                       # rows not a multiple of hw
