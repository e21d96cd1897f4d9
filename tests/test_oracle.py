"""CPU tests: the oracle restatement against the golden vectors recorded from the reference's own
host code, and (when oracle/_ref is present) against that code directly."""
import os

import numpy as np
import pytest

import afb_testlib as T

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def test_conversions_match_reference_golden(oracle):
    g = np.load(os.path.join(GOLD, "conversions.npz"))
    f = g["f32_bits"].view(np.float32)
    assert np.array_equal(oracle.bf16_trunc(f), g["bf16_trunc"])      # datatype.hpp:45-55
    assert np.array_equal(oracle.bf16_rne(f), g["bf16_rtn"])          # datatype.hpp:80-121, NaN/Inf/subnormal cases included
    assert np.array_equal(oracle.bf16_to_f32(g["bf16_all"]).view(np.uint32), g["bf16_all_f32_bits"])  # datatype.hpp:32-42
    assert np.array_equal(oracle.to_i8(g["i8_src"], 1), g["i8_plus128"])  # mem_transfer.hpp:30
    # the numpy helper used to prepare inputs agrees with the reference on every finite value
    finite = np.isfinite(f)
    assert np.array_equal(T.np_bf16_rne(f[finite]), g["bf16_rtn"][finite])


def test_gemm_rrr_integer_golden(oracle):
    g = np.load(os.path.join(GOLD, "gemm_rrr_integer.npz"))
    a, b, s = g["a"].astype(np.float32), g["b"].astype(np.float32), g["scale"].astype(np.float32)
    assert np.array_equal(oracle.gemm_rrr(a, b, s).view(np.uint32), g["c"].view(np.uint32))
    # the device-format oracle (bf16 A, packed int8 B in the reference's [K,N] offset-binary storage) gives the same bits
    case = T.Case(m=a.shape[0], n=b.shape[1], k=a.shape[1], bits=8, group=0, layout=0, enc=1, scale_dtype=0,
                  a=T.np_bf16_rne(a), b=oracle.to_i8(b, 1), scale=s, ldb=b.shape[1])
    assert np.array_equal(oracle.gemm(case).view(np.uint32), g["c"].view(np.uint32))


def test_gemm_rrr_real_golden(oracle):
    g = np.load(os.path.join(GOLD, "gemm_rrr_real.npz"))
    a_bf16, b, s = g["a_bf16"], g["b"], g["scale"]
    a = T.np_bf16_to_f32(a_bf16)
    assert np.array_equal(oracle.gemm_rrr(a, b.astype(np.float32), s).view(np.uint32), g["c"].view(np.uint32))
    for layout, enc in [(0, 0), (0, 1), (1, 0), (1, 1)]:
        stored = (b.astype(np.int16) + (128 if enc else 0)).astype(np.uint8) if enc else b.view(np.uint8)
        bb = np.ascontiguousarray(stored if layout == 0 else stored.T)
        case = T.Case(m=a.shape[0], n=b.shape[1], k=b.shape[0], bits=8, group=0, layout=layout, enc=enc, scale_dtype=0,
                      a=a_bf16, b=bb, scale=s, ldb=bb.shape[1])
        assert np.array_equal(oracle.gemm(case).view(np.uint32), g["c"].view(np.uint32)), (layout, enc)
        # row-parallel threads compute every element identically
        assert np.array_equal(oracle.gemm(case, threads=4).view(np.uint32), g["c"].view(np.uint32))


def test_oracle_against_reference_build(oracle):
    ref = T.load_hostref()
    if ref is None:
        pytest.skip("oracle/_ref not built (reference sources absent)")
    rng = np.random.default_rng(7)
    f = rng.integers(0, 2**32, size=20000, dtype=np.uint64).astype(np.uint32).view(np.float32)
    assert np.array_equal(oracle.bf16_trunc(f), ref.bf16_trunc(f))
    assert np.array_equal(oracle.bf16_rne(f), ref.bf16_rtn(f))
    a = rng.standard_normal((9, 200)).astype(np.float32)
    b = rng.integers(-127, 128, size=(200, 40)).astype(np.float32)
    s = rng.uniform(0.001, 0.01, 40).astype(np.float32)
    assert np.array_equal(oracle.gemm_rrr(a, b, s).view(np.uint32), ref.gemm_rrr(a, b, s).view(np.uint32))
    assert np.array_equal(ref.gemm_rrr(a, b, s, threads=3).view(np.uint32), ref.gemm_rrr(a, b, s).view(np.uint32))


@pytest.mark.parametrize("bits,group,enc", [(8, 0, 0), (8, 0, 1), (8, 128, 0), (4, 0, 0), (4, 128, 0), (4, 128, 1), (4, 64, 0)])
def test_extended_oracle_is_self_consistent(oracle, bits, group, enc):
    """int4 / group scales / [N,K]: the packed path equals gemm_rrr fed with the expanded fp32 weights."""
    case = T.make_case(5, 24, 256, bits=bits, group=group, enc=enc, seed=3)
    a = T.np_bf16_to_f32(case.a)
    s = case.scale_f32()
    w = case.q.astype(np.float32)  # [N,K]
    if group:
        # gemm_rrr has one scale per n, so fold the group scale into B and use scale = 1:
        # b*1 is exact and a*(q*s) is what the extended loop forms too
        wk = (w.reshape(case.n, -1, group) * s[:, :, None]).reshape(case.n, case.k)
        ref = oracle.gemm_rrr(a, wk.T, np.ones(case.n, np.float32))
    else:
        ref = oracle.gemm_rrr(a, w.T, s)
    got = oracle.gemm(case)
    assert np.array_equal(got.view(np.uint32), ref.view(np.uint32))
    # unpack is exact
    dq = oracle.dequant_bf16(case)
    expect = w if not group else (w.reshape(case.n, -1, group) * s[:, :, None]).reshape(case.n, case.k)
    assert np.array_equal(dq, T.np_bf16_rne(expect))


def test_int4_pack_layout(oracle):
    q = np.array([[-8, 7, -1, 0, 3, -4]], np.float32)
    assert oracle.to_i4(q, 0).tolist() == [[0x78, 0x0F, 0xC3]]   # low nibble = even k
    assert oracle.to_i4(q, 1).tolist() == [[0xF0, 0x87, 0x4B]]


def test_compare_metric(oracle):
    ref = np.array([1.0, -2.0, 0.0, 100.0], np.float32)
    pred = T.np_bf16_rne(np.array([1.0, -2.0, 0.0, 101.0], np.float32))
    mx, nrms, worst = oracle.compare(ref, pred, 1e-3)
    assert worst == 3 and abs(mx - 0.01) < 1e-6   # bf16(101) = 101
    # a wrong value next to a NEGATIVE reference is caught (the reference's signed denominator misses it, validation.hpp:27)
    pred2 = T.np_bf16_rne(np.array([1.0, -3.0, 0.0, 100.0], np.float32))
    mx2, _, w2 = oracle.compare(ref, pred2, 1e-3)
    assert w2 == 1 and mx2 == 0.5
