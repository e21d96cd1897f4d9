"""CPU tests of the host-side mirror headers (include/bfAintBGemm/*.hpp): the re-written type_convert,
bf16_convert_rtn, mem_transfer and gemm_rrr are fed the golden vectors recorded from the reference's own
host code (tests/golden/*.npz; datatype.hpp:32-121, mem_transfer.hpp:12-32, host_ref.hpp:3-25) and must
return the same bits; the formats the reference does not have (RNE write-back, two's complement, packed
int4) are checked against the CPU oracle."""
import ctypes
import os
import subprocess

import numpy as np
import pytest

import afb_testlib as T

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLD = os.path.join(ROOT, "tests", "golden")
_f32p, _u16p, _u8p, _i8p = (ctypes.POINTER(t) for t in (ctypes.c_float, ctypes.c_uint16, ctypes.c_uint8, ctypes.c_int8))


@pytest.fixture(scope="module")
def mir(tmp_path_factory):
    out = str(tmp_path_factory.mktemp("mirror") / "libafb_mirror.so")
    subprocess.check_call(["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-ffp-contract=off", "-I" + os.path.join(ROOT, "include"),
                           "-o", out, os.path.join(ROOT, "tests", "mirror", "mirror_shim.cc")])
    L = ctypes.CDLL(out)
    sz = ctypes.c_size_t
    L.mir_f32_to_bf16_trunc.argtypes = [_f32p, _u16p, sz]
    L.mir_f32_to_bf16_rtn.argtypes = [_f32p, _u16p, sz]
    L.mir_bf16_to_f32.argtypes = [_u16p, _f32p, sz]
    L.mir_bf16_to_i8.argtypes = [_u16p, _i8p, sz]
    L.mir_i8_to_bf16.argtypes = [_i8p, _u16p, sz]
    L.mir_mem_transfer_i8.argtypes = [_f32p, _u8p, sz]
    L.mir_mem_transfer_bf16.argtypes = [_f32p, _u16p, sz]
    L.mir_mem_transfer_bf16_rne.argtypes = [_f32p, _u16p, _f32p, sz]
    L.mir_mem_transfer_int8_twos.argtypes = [_f32p, _u8p, sz]
    L.mir_mem_transfer_int4.argtypes = [_f32p, _u8p, sz, ctypes.c_int]
    L.mir_gemm_rrr.argtypes = [_f32p] * 4 + [sz] * 6
    L.mir_gemm_ref.argtypes = [_f32p] * 4 + [sz] * 6 + [ctypes.c_int, sz]
    L.mir_valid_vector_bf16.argtypes = [_f32p, _u16p, ctypes.c_int, ctypes.c_float, ctypes.c_float, ctypes.c_float]
    L.mir_matrix_space_size.argtypes = [sz, sz, sz, ctypes.c_int]
    L.mir_matrix_space_size.restype = sz
    return L


def _run(fn, src, out_dtype, src_t, dst_t, out_shape=None, *extra):
    src = np.ascontiguousarray(src)
    out = np.empty(src.shape if out_shape is None else out_shape, out_dtype)
    fn(src.ctypes.data_as(src_t), out.ctypes.data_as(dst_t), src.size, *extra)
    return out


def test_conversions_match_reference_golden(mir):
    g = np.load(os.path.join(GOLD, "conversions.npz"))
    f = g["f32_bits"].view(np.float32)
    assert np.array_equal(_run(mir.mir_f32_to_bf16_trunc, f, np.uint16, _f32p, _u16p), g["bf16_trunc"])       # datatype.hpp:45-55
    assert np.array_equal(_run(mir.mir_f32_to_bf16_rtn, f, np.uint16, _f32p, _u16p), g["bf16_rtn"])           # datatype.hpp:80-121
    assert np.array_equal(_run(mir.mir_bf16_to_f32, g["bf16_all"], np.float32, _u16p, _f32p).view(np.uint32), g["bf16_all_f32_bits"])
    assert np.array_equal(_run(mir.mir_mem_transfer_i8, g["i8_src"], np.uint8, _f32p, _u8p), g["i8_plus128"])  # mem_transfer.hpp:30
    assert np.array_equal(_run(mir.mir_mem_transfer_bf16, f, np.uint16, _f32p, _u16p), g["bf16_trunc"])       # mem_transfer.hpp:12-21


def test_int8_bf16_round_trip(mir):
    v = np.arange(-128, 128, dtype=np.int8)
    h = _run(mir.mir_i8_to_bf16, v, np.uint16, _i8p, _u16p)                # datatype.hpp:67-73: exact for every int8
    assert np.array_equal(T.np_bf16_to_f32(h), v.astype(np.float32))
    assert np.array_equal(_run(mir.mir_bf16_to_i8, h, np.int8, _u16p, _i8p), v)   # datatype.hpp:58-64


def test_added_formats_match_the_oracle(mir, oracle):
    rng = np.random.default_rng(5)
    f = rng.standard_normal(4096).astype(np.float32)
    out = np.empty(f.shape, np.uint16); master = np.empty_like(f)
    mir.mir_mem_transfer_bf16_rne(f.ctypes.data_as(_f32p), out.ctypes.data_as(_u16p), master.ctypes.data_as(_f32p), f.size)
    assert np.array_equal(out, oracle.bf16_rne(f))
    assert np.array_equal(master, T.np_bf16_to_f32(out))                   # the write-back: CPU check and GPU see the same inputs
    q8 = rng.integers(-128, 128, 1024).astype(np.float32)
    assert np.array_equal(_run(mir.mir_mem_transfer_int8_twos, q8, np.uint8, _f32p, _u8p), oracle.to_i8(q8, 0))
    assert np.array_equal(_run(mir.mir_mem_transfer_i8, q8, np.uint8, _f32p, _u8p), oracle.to_i8(q8, 1))
    q4 = rng.integers(-8, 8, 1024).astype(np.float32)
    for enc in (0, 1):
        got = _run(mir.mir_mem_transfer_int4, q4, np.uint8, _f32p, _u8p, (512,), enc)
        assert np.array_equal(got, oracle.to_i4(q4, enc))


@pytest.mark.parametrize("name", ["gemm_rrr_integer.npz", "gemm_rrr_real.npz"])
def test_gemm_rrr_matches_reference_golden(mir, name):
    g = np.load(os.path.join(GOLD, name))
    a = g["a"].astype(np.float32) if "a" in g.files else T.np_bf16_to_f32(g["a_bf16"])
    b, s = g["b"].astype(np.float32), g["scale"].astype(np.float32)
    m, k = a.shape; n = b.shape[1]
    a, b, s = (np.ascontiguousarray(x) for x in (a, b, s))
    c = np.empty((m, n), np.float32)
    mir.mir_gemm_rrr(*(x.ctypes.data_as(_f32p) for x in (c, a, b, s)), m, n, k, k, n, n)
    assert np.array_equal(c.view(np.uint32), g["c"].view(np.uint32))
    # the [N,K] form of the same check gives the same bits
    bt = np.ascontiguousarray(b.T)
    c2 = np.empty((m, n), np.float32)
    mir.mir_gemm_ref(*(x.ctypes.data_as(_f32p) for x in (c2, a, bt, s)), m, n, k, k, k, n, 1, 0)
    assert np.array_equal(c2.view(np.uint32), g["c"].view(np.uint32))


def test_gemm_ref_with_groups_matches_the_oracle(mir, oracle):
    case = T.make_case(5, 24, 256, bits=4, group=64, seed=3)
    a = T.np_bf16_to_f32(case.a); w = np.ascontiguousarray(case.q.astype(np.float32)); s = np.ascontiguousarray(case.scale_f32())
    c = np.empty((case.m, case.n), np.float32)
    mir.mir_gemm_ref(*(x.ctypes.data_as(_f32p) for x in (c, a, w, s)), case.m, case.n, case.k, case.k, case.k, case.n, 1, 64)
    assert np.array_equal(c.view(np.uint32), oracle.gemm(case).view(np.uint32))


def test_valid_vector_and_size_rule(mir, capfd):
    ref = np.array([1.0, -2.0, 0.0, 100.0] * 8, np.float32)
    good = T.np_bf16_rne(ref)
    assert mir.mir_valid_vector_bf16(ref.ctypes.data_as(_f32p), good.ctypes.data_as(_u16p), ref.size, 1e-3, 1e-2, 0.05) == 1
    bad = good.copy(); bad[1] = T.np_bf16_rne(np.array([-3.0], np.float32))[0]       # next to a NEGATIVE reference value:
    assert mir.mir_valid_vector_bf16(ref.ctypes.data_as(_f32p), bad.ctypes.data_as(_u16p), ref.size, 1e-3, 1e-2, 0.05) == 0   # validation.hpp:27 misses it
    capfd.readouterr()
    # bfAintBGemm.cc:68-76: (rows - 1) * ld + cols for Row, (cols - 1) * ld + rows for Col
    assert mir.mir_matrix_space_size(32, 512, 520, 1) == 31 * 520 + 512
    assert mir.mir_matrix_space_size(512, 128, 520, 0) == 127 * 520 + 512
