"""Weight pre-packing (afb_prepack): the packed bytes against the CPU restatement, bit for bit, and the GEMM on packed
weights against the GEMM on plain weights, bit for bit, for every kernel that reads them.  The reference's own [K,N]
layout (bfAintBGemm.cc:20-23,51) reaches the fast kernels through this step."""
import numpy as np
import pytest

import afb_testlib as T
import awesome_fusion_b200 as pkg
from test_gpu_parity import check_close


def test_packed_layout_in_the_oracle(oracle):
    """CPU: packing moves integers, never changes them, so the oracle reads the same GEMM out of both layouts."""
    for bits, group, layout in [(8, 0, 1), (8, 0, 0), (4, 0, 1), (4, 128, 1), (8, 64, 1)]:
        case = T.make_case(5, 24, 256, bits=bits, group=group, layout=layout, seed=13)
        packed = oracle.prepack(case)
        assert packed.layout == 2 and packed.b.shape == (case.n, case.k * bits // 8)
        assert np.array_equal(oracle.gemm(packed).view(np.uint32), oracle.gemm(case).view(np.uint32))
        plain_dq = oracle.dequant_bf16(case)
        assert np.array_equal(oracle.dequant_bf16(packed), plain_dq if layout != 0 else plain_dq.T)
    # the documented word orders
    case = T.make_case(1, 1, 8, bits=8, seed=1)
    case.b[:] = np.arange(8, dtype=np.uint8)
    assert oracle.prepack(case).b.tolist() == [[0, 2, 1, 3, 4, 6, 5, 7]]
    c4 = T.make_case(1, 1, 8, bits=4, seed=1)
    c4.b[:] = np.array([0x10, 0x32, 0x54, 0x76], np.uint8)            # nibbles k0..k7 = 0..7
    assert oracle.prepack(c4).b.tolist() == [[0x20, 0x64, 0x31, 0x75]]   # [k0,k2,k4,k6,k1,k3,k5,k7]


def _prepack_on_gpu(afb, case, out_ldb=None, in_place=False):
    out_ldb = out_ldb or case.k
    d_b = afb.to_device(case.b)
    nbytes = case.n * out_ldb * case.bits // 8
    d_o = d_b if in_place else afb.malloc(nbytes)
    if not in_place:
        afb.memset(d_o, 0, nbytes)
    args = afb.make_args(d_o, d_b, d_b, d_b, 1, case.n, case.k, ldb=case.ldb, bits=case.bits, layout=case.layout)
    afb.prepack(args, d_o, out_ldb)
    afb.device_sync()
    got = afb.to_host(d_o, (case.n, out_ldb * case.bits // 8), np.uint8)
    afb.free(d_b)
    if not in_place:
        afb.free(d_o)
    return got


@pytest.mark.gpu
@pytest.mark.parametrize("bits,layout,n,k,pad", [(8, 1, 96, 512, 0), (8, 0, 96, 512, 0), (8, 0, 70, 100, 28), (4, 1, 96, 512, 0), (8, 1, 33, 132, 60), (4, 1, 17, 264, 24)])
def test_prepack_bytes_match_the_restatement(afb, oracle, bits, layout, n, k, pad):
    case = T.make_case(1, n, k, bits=bits, layout=layout, seed=n + k)
    got = _prepack_on_gpu(afb, case, out_ldb=k + pad)
    want = oracle.prepack(case, out_ldb=k + pad).b
    assert np.array_equal(got, want)
    if layout == 1 and pad == 0:
        assert np.array_equal(_prepack_on_gpu(afb, case, in_place=True), want)


@pytest.mark.gpu
@pytest.mark.parametrize("m,variant,flags", [(1, pkg.VARIANT_DECODE, 0), (8, pkg.VARIANT_DECODE, 0), (16, pkg.VARIANT_DECODE, 0), (13, pkg.VARIANT_DECODE, pkg.FLAG_PDL),
                                             (96, pkg.VARIANT_PREFILL, pkg.FLAG_PREFILL_SMEM_B), (300, pkg.VARIANT_PREFILL, pkg.FLAG_PREFILL_TMEM_A),
                                             (7, pkg.VARIANT_NAIVE, 0)])
@pytest.mark.parametrize("bits,group", [(8, 0), (4, 0), (4, 128), (8, 128)])
def test_gemm_on_packed_weights_equals_gemm_on_plain_weights(afb, oracle, m, variant, flags, bits, group):
    case = T.make_case(m, 520, 1024, bits=bits, group=group, seed=3 * m + bits, scale_range=(0.005, 0.05))
    plain, _ = T.run_case(afb, case, variant=variant, flags=flags)
    packed_case = oracle.prepack(case)
    packed_case.b = _prepack_on_gpu(afb, case)                     # the GPU's own packing feeds the GEMM
    packed, _ = T.run_case(afb, packed_case, variant=variant, flags=flags)
    assert np.array_equal(plain, packed), "the packed GEMM differs from the plain one"
    if variant != pkg.VARIANT_NAIVE:
        ref = oracle.gemm(case, threads=4, round_w=bool(group and variant == pkg.VARIANT_PREFILL))
        check_close(oracle, ref, packed, f"packed weights, variant {variant}, int{bits} g{group}")
    assert afb.read_status()[0] == 0


@pytest.mark.gpu
@pytest.mark.parametrize("m", [4, 16, 256])
def test_reference_layout_reaches_the_fast_kernels_through_prepack(afb, oracle, m):
    """B as the reference stores it: [K,N], N contiguous, value + 128 (bfAintBGemm.cc:20-23,51; mem_transfer.hpp:30)."""
    case = T.make_case(m, 1024, 1024, layout=0, enc=1, a_dist="uniform", scale_range=(0.002, 0.02), seed=0)
    packed_case = oracle.prepack(case)
    packed_case.b = _prepack_on_gpu(afb, case)
    dc = T.DeviceCase(afb, packed_case)
    try:
        want_variant = pkg.VARIANT_DECODE if m <= 16 else pkg.VARIANT_PREFILL
        assert afb.resolve_variant(dc.args()) == want_variant
        afb.gemm_launch(dc.args()); afb.device_sync()
        got = dc.result()[0]
    finally:
        dc.close()
    check_close(oracle, oracle.gemm(case, threads=8), got, f"reference layout through prepack, M={m}")


@pytest.mark.gpu
@pytest.mark.parametrize("bits,group", [(8, 0), (4, 128)])
def test_dequant_dump_reads_packed_weights(afb, oracle, bits, group):
    case = T.make_case(1, 64, 512, bits=bits, group=group, seed=19, scale_range=(0.005, 0.05))
    packed_case = oracle.prepack(case)
    d_b, d_s = afb.to_device(packed_case.b), afb.to_device(case.scale)
    d_o = afb.malloc(case.n * case.k * 2)
    args = afb.make_args(d_o, d_b, d_b, d_s, 1, case.n, case.k, ldb=case.k, bits=bits, layout=pkg.LAYOUT_COL_PACKED,
                         scale_dtype=case.scale_dtype, group=group)
    afb.dequant_dump(args, d_o)
    afb.device_sync()
    got = afb.to_host(d_o, (case.n, case.k), np.uint16)
    for p in (d_b, d_s, d_o):
        afb.free(p)
    assert np.array_equal(got, oracle.dequant_bf16(case))
