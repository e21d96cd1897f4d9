"""B200 (sm_100a) implementation of the reference's bfAintBGemm path.

The product is ``libafb.so`` (hand-written CUDA behind the C ABI of ``include/afb_capi.h``)
plus the C++ host driver in ``driver/``.  This Python package is the thin host-side binding
the tests, the benchmark and the multi-GPU launcher use; it never computes anything itself
and raises if the CUDA library is missing.
"""
from .capi import (  # noqa: F401
    AfbError,
    GemmArgs,
    Library,
    ENC_TWOS, ENC_OFFSET, LAYOUT_ROW, LAYOUT_COL, SCALE_F32, SCALE_BF16,
    VARIANT_AUTO, VARIANT_DECODE, VARIANT_PREFILL, VARIANT_NAIVE, FLAG_C_F32, FLAG_PREFILL_SMEM_B, FLAG_PREFILL_TMEM_A, FLAG_PUSH_VIA_LOCAL,
    library_path, load,
)
from .build import build_library  # noqa: F401

__all__ = [
    "AfbError", "GemmArgs", "Library", "library_path", "load", "build_library",
    "ENC_TWOS", "ENC_OFFSET", "LAYOUT_ROW", "LAYOUT_COL", "SCALE_F32", "SCALE_BF16",
    "VARIANT_AUTO", "VARIANT_DECODE", "VARIANT_PREFILL", "VARIANT_NAIVE", "FLAG_C_F32", "FLAG_PREFILL_SMEM_B", "FLAG_PREFILL_TMEM_A", "FLAG_PUSH_VIA_LOCAL",
]
