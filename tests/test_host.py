"""CPU tests of the host side: the C-ABI library loads and exports every declared symbol, argument
validation and variant selection answer without a GPU, and the C++ driver + headers build."""
import ctypes
import os
import re
import subprocess

import numpy as np
import pytest

import awesome_fusion_b200 as pkg
from awesome_fusion_b200.capi import EXPORTS

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    if not os.path.exists(pkg.library_path()):
        pkg.build_library()
    return pkg.load()


def test_library_exports_every_declared_symbol(lib):
    header = open(os.path.join(ROOT, "include", "afb_capi.h")).read()
    declared = set(re.findall(r"\b(afb_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations found"
    for name in sorted(declared):
        assert hasattr(lib.lib, name), f"{name} is declared in afb_capi.h but not exported by libafb.so"
    assert declared >= set(EXPORTS)


def test_args_struct_layout_matches_reference_block():
    # the first ten fields are the reference's packed kernarg block: 4 pointers then 6 x u32 (bfAintBGemm.cc:119-133)
    A = pkg.GemmArgs
    assert [A.ptr_c.offset, A.ptr_a.offset, A.ptr_b.offset, A.ptr_scale.offset] == [0, 8, 16, 24]
    assert [A.m.offset, A.n.offset, A.k.offset, A.lda.offset, A.ldb.offset, A.ldc.offset] == [32, 36, 40, 44, 48, 52]
    assert ctypes.sizeof(A) == 104 and A.ptr_zero.offset == 88


def test_validation_without_gpu(lib):
    a = lib.make_args(0x1000, 0x1000, 0x1000, 0x1000, 4, 128, 256)
    v = ctypes.c_uint32()
    assert lib.lib.afb_gemm_resolve_variant(ctypes.byref(a), ctypes.byref(v)) == 0 and v.value == pkg.VARIANT_DECODE
    a.m = 512
    assert lib.lib.afb_gemm_resolve_variant(ctypes.byref(a), ctypes.byref(v)) == 0 and v.value == pkg.VARIANT_PREFILL
    a.b_layout = pkg.LAYOUT_ROW; a.ldb = 128       # the reference's [K,N] layout has no fast variant
    assert lib.lib.afb_gemm_resolve_variant(ctypes.byref(a), ctypes.byref(v)) == 0 and v.value == pkg.VARIANT_NAIVE
    a.variant = pkg.VARIANT_PREFILL
    assert lib.lib.afb_gemm_resolve_variant(ctypes.byref(a), ctypes.byref(v)) == -2
    bad = lib.make_args(0, 0x1000, 0x1000, 0x1000, 4, 128, 256)
    assert lib.lib.afb_gemm_resolve_variant(ctypes.byref(bad), ctypes.byref(v)) == -1
    bad = lib.make_args(0x1000, 0x1000, 0x1000, 0x1000, 4, 128, 256, bits=5)
    assert lib.lib.afb_gemm_resolve_variant(ctypes.byref(bad), ctypes.byref(v)) == -1
    bad = lib.make_args(0x1000, 0x1000, 0x1000, 0x1000, 4, 128, 256, lda=8)
    assert lib.lib.afb_gemm_resolve_variant(ctypes.byref(bad), ctypes.byref(v)) == -1
    bad = lib.make_args(0x1000, 0x1000, 0x1000, 0x1000, 4, 128, 256, group=96)
    assert lib.lib.afb_gemm_resolve_variant(ctypes.byref(bad), ctypes.byref(v)) == -1
    # pointers the kernels would load or store through as 2- or 4-byte words must be aligned to them: a status, never a GPU fault
    bad = lib.make_args(0x1000, 0x1000, 0x1000, 0x1002, 4, 128, 256)                                  # fp32 scales at a 2-byte boundary
    assert lib.lib.afb_gemm_resolve_variant(ctypes.byref(bad), ctypes.byref(v)) == -1
    bad = lib.make_args(0x1000, 0x1000, 0x1000, 0x1001, 4, 128, 256, scale_dtype=pkg.SCALE_BF16)      # bf16 scales at an odd address
    assert lib.lib.afb_gemm_resolve_variant(ctypes.byref(bad), ctypes.byref(v)) == -1
    bad = lib.make_args(0x1001, 0x1000, 0x1000, 0x1000, 4, 128, 256)                                  # bf16 C at an odd address
    assert lib.lib.afb_gemm_resolve_variant(ctypes.byref(bad), ctypes.byref(v)) == -1
    assert lib.gemm_launch_static_status(lib.make_args(0x1000, 0x1000, 0x1000, 0x1002, 4, 128, 256)) == -1
    ok = lib.make_args(0x1000, 0x1000, 0x1000, 0x1002, 4, 128, 256, scale_dtype=pkg.SCALE_BF16)       # bf16 scales at a 2-byte boundary are fine
    assert lib.lib.afb_gemm_resolve_variant(ctypes.byref(ok), ctypes.byref(v)) == 0
    # packed layout, flags and the tail of the argument block
    pk = lib.make_args(0x1000, 0x1000, 0x1000, 0x1000, 4, 128, 256, layout=pkg.LAYOUT_COL_PACKED, flags=pkg.FLAG_PDL)
    assert lib.lib.afb_gemm_resolve_variant(ctypes.byref(pk), ctypes.byref(v)) == 0 and v.value == pkg.VARIANT_DECODE
    pk.reserved2 = 1
    assert lib.lib.afb_gemm_resolve_variant(ctypes.byref(pk), ctypes.byref(v)) == -1
    g32 = lib.make_args(0x1000, 0x1000, 0x1000, 0x1000, 4, 128, 256, bits=4, group=32, scale_dtype=pkg.SCALE_BF16)   # groups of 32: the prefill kernel takes them
    assert lib.lib.afb_gemm_resolve_variant(ctypes.byref(g32), ctypes.byref(v)) == 0 and v.value == pkg.VARIANT_PREFILL
    assert lib.lib.afb_status_string(-4).decode().startswith("a bounded")


def test_missing_library_fails_loudly(tmp_path):
    with pytest.raises(pkg.AfbError):
        pkg.Library(str(tmp_path / "nope.so"))


def test_balanced_decode_partition_arithmetic():
    """The one-wave form of the decode kernel gives CTA c the units [c*U/G, (c+1)*U/G) and finds the CTA of unit u as
    ceil((u+1)*G/U) - 1 (csrc/decode.cu, kernel and pick_shape use the same two formulas).  Restated here and checked:
    the runs tile [0, U) exactly, the inverse agrees with them, and the contributors of a channel block are consecutive CTAs."""
    def start(c, U, G):
        return c * U // G

    def cta_of(u, U, G):
        return ((u + 1) * G + U - 1) // U - 1

    for cbs, ku, G in [(224, 32, 444), (896, 16, 592), (2, 16, 32), (1792, 16, 592), (63, 8, 444), (7, 64, 296), (448, 5, 444)]:
        U = cbs * ku
        G = min(G, U)
        owner = [None] * U
        for c in range(G):
            for u in range(start(c, U, G), start(c + 1, U, G)):
                assert owner[u] is None
                owner[u] = c
        assert all(o is not None for o in owner)                       # every unit has exactly one CTA
        assert all(cta_of(u, U, G) == owner[u] for u in range(U))      # the closed form finds it
        for cb in range(cbs):
            first, last = cta_of(cb * ku, U, G), cta_of(cb * ku + ku - 1, U, G)
            assert sorted(set(owner[cb * ku:(cb + 1) * ku])) == list(range(first, last + 1))


def test_automatic_exchange_choice():
    """dist.pick_exchange: the form `--exchange auto` stands for, from the shapes alone."""
    from awesome_fusion_b200 import dist
    assert dist.pick_exchange(8, "f32", 4096, 8192) == "inkernel"
    assert dist.pick_exchange(4, "f32", 4096, 8192) == "inkernel"
    assert dist.pick_exchange(2, "f32", 4096, 8192) == "push"            # measured level on 2 GPUs: the simpler form stays
    assert dist.pick_exchange(4, "f32", 4096, 8192 + 128) == "push"      # N is not a whole number of column chunks
    assert dist.pick_exchange(4, "f32", 4096 + 256, 8192) == "fused"     # rows do not split into whole tiles per owner
    assert dist.pick_exchange(8, "bf16", 4096, 8192) == "fused"          # bf16 partial sums travel only in the pull form
