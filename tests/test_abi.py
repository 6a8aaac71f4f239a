"""CPU-side checks of the C ABI: the library loads without a GPU, exports every symbol the
header declares, the ctypes prototypes cover them, and argument validation answers with the
documented status codes before anything touches a device."""
from __future__ import annotations

import ctypes
import re
from pathlib import Path

import pytest

from anima_trainer_sm120_b200 import _lib

HEADER = Path(__file__).resolve().parents[1] / "include" / "anima_b200.h"


def declared_functions() -> list[str]:
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(anima_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_and_library_exports_every_entry_point(lib):
    names = declared_functions()
    assert len(names) >= 19
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in anima_b200.h but not exported"
        assert n in _lib.PROTOTYPES, f"{n} has no ctypes prototype"
    assert sorted(_lib.PROTOTYPES) == names


def test_abi_version_and_sizes(lib):
    assert lib.anima_abi_version() == 1
    assert lib.anima_mx_scales_bytes(130, 160, _lib.SCALES_PLAIN) == 130 * 5
    assert lib.anima_mx_scales_bytes(130, 160, _lib.SCALES_TILED) == 2 * 2 * 512
    assert lib.anima_mx_scales_bytes(32768, 2048, _lib.SCALES_TILED) == 32768 * 64
    assert lib.anima_mx_scales_bytes(8, 33, _lib.SCALES_PLAIN) == -3
    assert lib.anima_lokr_kron_backward_workspace_bytes(8192, 2048, 8, 8) == (1024 * 32 // 128) * 64 * 4
    assert lib.anima_adaln_bwd_workspace_bytes(100, 7, 64) == -3       # rows not a multiple of hw
    assert lib.anima_tlokr_rank_mix_wgrad_workspace_bytes(2, 3, 12) == -3  # rank % 8


def test_argument_errors_are_reported_not_executed(lib):
    buf = (ctypes.c_uint8 * 4096)()
    p = ctypes.addressof(buf)
    p16 = (p + 15) & ~15
    # null input
    assert lib.anima_mx_quantize(None, 32, 32, 32, p16, p16, None, None, 0, None) == -1
    assert b"null" in lib.anima_last_error()
    # codes without scales
    assert lib.anima_mx_quantize(p16, 32, 32, 32, p16, None, None, None, 0, None) == -1
    # cols % 32 for the rowwise form
    assert lib.anima_mx_quantize(p16, 32, 40, 40, p16, p16, None, None, 0, None) == -3
    # rows % 32 for the columnwise form
    assert lib.anima_mx_quantize(p16, 40, 32, 32, None, None, p16, p16, 0, None) == -3
    # misaligned pointer
    assert lib.anima_mx_quantize(p16 + 2, 32, 32, 32, p16, p16, None, None, 0, None) == -2
    # GEMM: K % 32
    assert lib.anima_mx_gemm(p16, p16, p16, p16, p16, 128, 128, 48, 128, None, 0, None, None) == -3
    # AdaLN: rows % hw, d % 8, d too large
    assert lib.anima_adaln_fwd(p16, p16, p16, 1e-6, 10, 4, 64, p16, p16, p16, None) == -3
    assert lib.anima_adaln_fwd(p16, p16, p16, 1e-6, 8, 4, 60, p16, p16, p16, None) == -3
    assert lib.anima_adaln_fwd(p16, p16, p16, 1e-6, 8, 4, 8192, p16, p16, p16, None) == -7
    # workspace too small
    assert lib.anima_gated_add_bwd(p16, p16, p16, 8, 4, 64, p16, p16, p16, 16, None) == -6
    # kron factor larger than 8x8
    assert lib.anima_lokr_kron_backward(p16, 0, p16, p16, 0, 1.0, 256, 256, 16, 16, p16, p16, p16, 1 << 20, None) == -5
    # empty inputs are a no-op success
    assert lib.anima_mx_quantize(p16, 0, 32, 32, p16, p16, None, None, 0, None) == 0
    assert lib.anima_gated_add_fwd(p16, p16, p16, 0, 4, 64, p16, None) == 0


def test_python_wrappers_refuse_cpu_tensors():
    import torch
    from anima_trainer_sm120_b200 import adaln_kernel, mxfp8_gemm, ops, tlokr_kernels
    x = torch.zeros(32, 64, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="CUDA"):
        ops.mx_quantize(x)
    with pytest.raises(RuntimeError, match="CUDA"):
        mxfp8_gemm.quantize_rowwise(x)
    with pytest.raises(AssertionError):
        adaln_kernel.fused_adaln(x.view(1, 1, 4, 8, 64), x[:1].view(1, 1, 1, 1, 64), x[:1].view(1, 1, 1, 1, 64), 1e-6)
    with pytest.raises(RuntimeError, match="CUDA"):
        tlokr_kernels.rank_mix(torch.zeros(1, 2, 8, 16, dtype=torch.bfloat16), torch.eye(8, dtype=torch.bfloat16), None)
    with pytest.raises(AssertionError):
        mxfp8_gemm.quantize_rowwise(torch.zeros(4, 40))
