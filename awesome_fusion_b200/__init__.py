"""B200 (sm_100a) implementation of the reference's bfAintBGemm path.

The product is ``libafb.so`` (hand-written CUDA behind the C ABI of ``include/afb_capi.h``)
plus the C++ host driver in ``driver/``.  This Python package is the thin host-side binding
the tests, the benchmark and the multi-GPU launcher use; it never computes anything itself
and raises if the CUDA library is missing.
"""
from . import capi as _capi
from .capi import AfbError, FusedArgs, GemmArgs, Library, library_path, load  # noqa: F401
from .build import build_library  # noqa: F401

# every ENC_ / LAYOUT_ / SCALE_ / VARIANT_ / FLAG_ / ACT_ constant of include/afb_capi.h
_CONSTANTS = [n for n in dir(_capi) if n.split("_")[0] in ("ENC", "LAYOUT", "SCALE", "VARIANT", "FLAG", "ACT", "PACK")]
globals().update({n: getattr(_capi, n) for n in _CONSTANTS})

__all__ = ["AfbError", "FusedArgs", "GemmArgs", "Library", "library_path", "load", "build_library"] + _CONSTANTS
