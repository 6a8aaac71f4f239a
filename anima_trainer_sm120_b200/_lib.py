"""ctypes binding of ``libanima_b200.so`` (the C ABI declared in ``include/anima_b200.h``).

The shared library is the product; this module only loads it, declares the
prototypes and turns negative status codes into exceptions. There is no CPU or
eager-PyTorch fallback: if the library is missing, or a call is made without a
usable GPU, the call raises.
"""
from __future__ import annotations

import ctypes
from ctypes import c_char_p, c_float, c_int, c_int64, c_void_p
from pathlib import Path

import torch

LIB_NAME = "libanima_b200.so"
LIB_PATH = Path(__file__).resolve().parent / LIB_NAME

SCALES_PLAIN = 0
SCALES_TILED = 1

_STATUS_EXC = {
    -1: ValueError,    # ANIMA_E_ARG
    -2: ValueError,    # ANIMA_E_ALIGN
    -3: ValueError,    # ANIMA_E_SHAPE
    -4: RuntimeError,  # ANIMA_E_CUDA
    -5: NotImplementedError,  # ANIMA_E_UNSUPPORTED
    -6: ValueError,    # ANIMA_E_WORKSPACE
    -7: ValueError,    # ANIMA_E_TOO_LARGE
}

P = c_void_p
I64 = c_int64

# name -> (restype, argtypes); mirrors include/anima_b200.h one to one.
PROTOTYPES: dict[str, tuple[object, list[object]]] = {
    "anima_abi_version": (c_int, []),
    "anima_last_error": (c_char_p, []),
    "anima_mx_quantize": (c_int, [P, I64, I64, I64, P, P, P, P, c_int, P]),
    "anima_mx_quantize_status": (c_int, []),
    "anima_mx_exponent_probe": (c_int, [P, I64, P, P, P]),
    "anima_mx_quantize_gelu": (c_int, [P, P, I64, I64, I64, P, P, P, P, P, c_int, P]),
    "anima_mx_scales_bytes": (I64, [I64, I64, c_int]),
    "anima_mx_dequantize": (c_int, [P, P, I64, I64, c_int, P, P]),
    "anima_mx_scales_retile": (c_int, [P, I64, I64, P, P]),
    "anima_mx_scales_regroup": (c_int, [P, I64, I64, P, I64, I64, P]),
    "anima_mx_gemm": (c_int, [P, P, P, P, P, I64, I64, I64, I64, P, c_int, P, P]),
    "anima_mx_gemm_workspace_bytes": (I64, [I64, I64, I64]),
    "anima_mx_gemm_ex": (c_int, [P, P, P, P, P, I64, I64, I64, I64, P, P, I64, c_float, c_int, P, I64, P, P]),
    "anima_mx_gemm_delta": (c_int, [P, P, P, P, P, I64, I64, I64, I64, P, c_int, P, P, P, P, P, I64, P, P]),
    "anima_mx_gemm_pair_plan": (c_int, [I64, I64, I64, c_int, P]),
    "anima_mx_gemm_set_clock_probe": (c_int, [P]),
    "anima_lokr_merge_quantize": (
        c_int, [P, P, P, c_int, c_float, I64, I64, I64, I64, P, P, P, P, P, c_int, P]),
    "anima_lokr_kron_backward_workspace_bytes": (I64, [I64, I64, I64, I64]),
    "anima_lokr_kron_backward": (
        c_int, [P, c_int, P, P, c_int, c_float, I64, I64, I64, I64, P, P, P, I64, P]),
    "anima_adaln_fwd": (c_int, [P, P, P, c_float, I64, I64, I64, P, P, P, P]),
    "anima_adaln_bwd_workspace_bytes": (I64, [I64, I64, I64]),
    "anima_adaln_bwd": (c_int, [P, P, P, P, P, I64, I64, I64, P, P, P, P, I64, P]),
    "anima_adaln_bwd_noalloc": (c_int, [P, P, P, P, P, I64, I64, I64, P, P, P, P]),
    "anima_gated_add_adaln_fwd": (c_int, [P, P, P, P, P, c_float, I64, I64, I64, P, P, P, P, P]),
    "anima_adaln_fwd_quant": (c_int, [P, P, P, c_float, I64, I64, I64, P, P, P, P, P, c_int, P]),
    "anima_gated_add_adaln_fwd_quant": (c_int, [P, P, P, P, P, c_float, I64, I64, I64, P, P, P, P, P, P, c_int, P]),
    "anima_gated_add_adaln_bwd_workspace_bytes": (I64, [I64, I64, I64]),
    "anima_gated_add_adaln_bwd": (c_int, [P, P, P, P, P, P, P, P, I64, I64, I64, P, P, P, P, P, P, I64, P]),
    "anima_gated_add_fwd": (c_int, [P, P, P, I64, I64, I64, P, P]),
    "anima_gated_add_bwd_workspace_bytes": (I64, [I64, I64, I64]),
    "anima_gated_add_bwd": (c_int, [P, P, P, I64, I64, I64, P, P, P, I64, P]),
    "anima_tlokr_rank_mix": (c_int, [P, P, P, I64, I64, I64, c_int, P, P]),
    "anima_tlokr_rank_mix_quant": (c_int, [P, P, P, I64, I64, I64, c_int, P, P, P, P, P, P]),
    "anima_tlokr_rank_mix_quant_planes": (c_int, [P, P, P, I64, I64, I64, c_int, P, P, P, P, P]),
    "anima_tlokr_hidden_mix_planes": (c_int, [P, P, P, P, P, P, I64, I64, I64, c_int, P, P, P, P, P]),
    "anima_tlokr_rank_mix_wgrad_workspace_bytes": (I64, [I64, I64, I64]),
    "anima_tlokr_rank_mix_wgrad": (c_int, [P, P, P, I64, I64, I64, P, P, I64, P]),
    "anima_rmsnorm_rope_fwd": (c_int, [P, P, P, P, c_float, I64, I64, I64, I64, P, P, P]),
    "anima_rmsnorm_rope_bwd": (c_int, [P, P, P, P, P, P, I64, I64, I64, I64, P, P]),
}

_lib: ctypes.CDLL | None = None


def load() -> ctypes.CDLL:
    """Load the library once and declare every prototype. Raises if it is absent."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m anima_trainer_sm120_b200.build` "
            "(there is no fallback path)"
        )
    lib = ctypes.CDLL(str(LIB_PATH))
    for name, (restype, argtypes) in PROTOTYPES.items():
        fn = getattr(lib, name)  # AttributeError if the symbol is not exported
        fn.restype = restype
        fn.argtypes = argtypes
    if lib.anima_abi_version() != 1:
        raise RuntimeError(f"{LIB_NAME}: ABI version {lib.anima_abi_version()} != 1")
    _lib = lib
    return lib


def last_error() -> str:
    msg = load().anima_last_error()
    return msg.decode("utf-8", "replace") if msg else ""


def check(status: int) -> int:
    """Raise the exception that belongs to a negative status; pass through sizes."""
    if status < 0:
        raise _STATUS_EXC.get(status, RuntimeError)(f"libanima_b200: {last_error()} (status {status})")
    return status


def ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def stream_ptr(device: torch.device | None = None) -> int:
    """The current torch CUDA stream as a cudaStream_t value."""
    return torch.cuda.current_stream(device).cuda_stream


def require_cuda(*tensors: torch.Tensor | None) -> torch.device:
    """All given tensors must live on one CUDA device; that device is made current."""
    dev = None
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise RuntimeError("anima_trainer_sm120_b200 kernels need CUDA tensors (no CPU path)")
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise RuntimeError(f"tensors on different devices: {dev} and {t.device}")
    if dev is None:
        raise RuntimeError("no tensor given")
    return dev


_workspaces: dict[tuple[int, int, str], torch.Tensor] = {}


def workspace(nbytes: int, device: torch.device, tag: str = "") -> torch.Tensor:
    """Scratch buffer (uint8, 256-byte aligned by the torch allocator), grown on demand and
    reused per (device, stream, tag) so that stream-ordered reuse is race free."""
    key = (device.index or 0, torch.cuda.current_stream(device).cuda_stream, tag)
    buf = _workspaces.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.empty(max(int(nbytes), 256), dtype=torch.uint8, device=device)
        _workspaces[key] = buf
    return buf


_status_words: dict[int, torch.Tensor] = {}


def status_word(device: torch.device) -> torch.Tensor:
    """Per-device int32 the GEMM raises if one of its bounded waits gives up."""
    idx = device.index or 0
    w = _status_words.get(idx)
    if w is None:
        w = torch.zeros(1, dtype=torch.int32, device=device)
        _status_words[idx] = w
    return w


def check_status_word(device: torch.device) -> None:
    """Synchronising check of the GEMM status word (tests and debugging)."""
    w = status_word(device)
    if int(w.item()) != 0:
        w.zero_()
        raise RuntimeError("anima_mx_gemm: a bounded wait inside the kernel timed out")


def check_quantize_status() -> None:
    """Synchronising check of the quantiser's bounded-wait flag on the current device."""
    rc = check(load().anima_mx_quantize_status())
    if rc != 0:
        raise RuntimeError("anima_mx_quantize: a bounded wait inside the copy-engine-fed kernel timed out")
