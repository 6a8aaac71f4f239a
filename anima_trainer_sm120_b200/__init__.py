"""B200-native (sm_100a) kernels for anima-trainer's quantised-linear hot path.

The product is ``libanima_b200.so`` (C ABI in ``include/anima_b200.h``); the
modules here mirror the anima-trainer operator layer on top of it:

* :mod:`.mxfp8_gemm`    quantiser + block-scaled GEMM (``mxfp8_gemm.py``)
* :mod:`.adaln_kernel`  FusedAdaLN / FusedGatedAdd (``adaln_kernel.py``)
* :mod:`.tlokr_kernels` rank_mix / rank_mix_wgrad (``tlokr_kernels.py``)
* :mod:`.ops`           one thin wrapper per C entry point
"""
from . import _lib  # noqa: F401

__all__ = ["_lib"]
