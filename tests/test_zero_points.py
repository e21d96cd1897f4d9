"""Zero-points (asymmetric quantisation) and small scale groups: weight = decode(stored) - decode(zero), one zero-point byte
per scale entry.  This generalises the reference's fixed "stored - 128" (bf16gemm_kernel_gfx90a.s:210, mem_transfer.hpp:30)."""
import numpy as np
import pytest

import afb_testlib as T
import awesome_fusion_b200 as pkg
from test_gpu_parity import check_close


def test_zero_point_semantics_in_the_oracle(oracle):
    # the reference's own convention as a special case: offset-binary storage with zero-point byte 128 == no zero-point
    case = T.make_case(3, 16, 128, enc=1, seed=2)
    with_z = T.Case(**{**case.__dict__, "zero": np.full(16, 128, np.uint8)})
    assert np.array_equal(oracle.gemm(with_z).view(np.uint32), oracle.gemm(case).view(np.uint32))
    # general case: the GEMM on (q - z) * s, written out with numpy
    for bits, group, enc in [(8, 0, 0), (8, 64, 1), (4, 0, 0), (4, 32, 1)]:
        case = T.make_case(3, 8, 128, bits=bits, group=group, enc=enc, seed=5, zero_points=True)
        raw = case.zero.astype(np.int32)
        if bits == 8:
            z = raw - 128 if enc == 1 else raw.astype(np.uint8).view(np.int8).astype(np.int32)
        else:
            z = raw - 8 if enc == 1 else np.where(raw >= 8, raw - 16, raw)
        zfull = np.repeat(z.reshape(case.n, -1), case.k // (z.size // case.n), axis=1)
        s = case.scale_f32().reshape(case.n, -1)
        sfull = np.repeat(s, case.k // s.shape[1], axis=1).astype(np.float32)
        w = (case.q.astype(np.int32) - zfull).astype(np.float32) * sfull
        ref = oracle.gemm_rrr(T.np_bf16_to_f32(case.a), w.T, np.ones(case.n, np.float32))
        assert np.array_equal(oracle.gemm(case).view(np.uint32), ref.view(np.uint32))
        assert np.array_equal(oracle.dequant_bf16(case), T.np_bf16_rne(w if group else (case.q.astype(np.int32) - zfull).astype(np.float32)))


@pytest.mark.gpu
@pytest.mark.parametrize("bits,group,enc", [(8, 0, 0), (8, 0, 1), (8, 128, 0), (4, 0, 0), (4, 0, 1), (4, 128, 1), (4, 32, 0), (8, 64, 1)])
@pytest.mark.parametrize("flags", [0, pkg.FLAG_DUMP_DECODE_PAIRING])
def test_dequant_with_zero_points_is_bit_exact(afb, oracle, bits, group, enc, flags):
    if flags and group:
        pytest.skip("the decode kernel never scales weights: its dump is integers only")
    case = T.make_case(1, 64, 512, bits=bits, group=group, enc=enc, seed=23, zero_points=True, scale_range=(0.005, 0.05))
    d_b, d_s, d_z = afb.to_device(case.b), afb.to_device(case.scale), afb.to_device(case.zero)
    d_o = afb.malloc(case.n * case.k * 2)
    args = afb.make_args(d_o, d_b, d_b, d_s, 1, case.n, case.k, ldb=case.k, bits=bits, encoding=enc, scale_dtype=case.scale_dtype, group=group,
                         flags=flags, zero=d_z)
    afb.dequant_dump(args, d_o)
    afb.device_sync()
    got = afb.to_host(d_o, (case.n, case.k), np.uint16)
    for p in (d_b, d_s, d_z, d_o):
        afb.free(p)
    assert np.array_equal(got, oracle.dequant_bf16(case))


@pytest.mark.gpu
@pytest.mark.parametrize("bits,group", [(8, 0), (4, 0), (4, 128), (8, 128)])
def test_naive_with_zero_points_is_bit_exact_fp32(afb, oracle, bits, group):
    case = T.make_case(5, 72, 384, bits=bits, group=group, seed=6, zero_points=True)
    got, _ = T.run_case(afb, case, variant=pkg.VARIANT_NAIVE, c_f32=True)
    assert np.array_equal(got.view(np.uint32), oracle.gemm(case).view(np.uint32))


@pytest.mark.gpu
@pytest.mark.parametrize("m", [1, 8, 16])
@pytest.mark.parametrize("bits,group,enc", [(8, 0, 0), (8, 0, 1), (4, 0, 0), (4, 128, 0), (4, 128, 1), (8, 128, 0)])
def test_decode_with_zero_points(afb, oracle, m, bits, group, enc):
    case = T.make_case(m, 520, 2048, bits=bits, group=group, enc=enc, seed=m + bits, zero_points=True, scale_range=(0.005, 0.05))
    got, _ = T.run_case(afb, case, variant=pkg.VARIANT_DECODE)
    check_close(oracle, oracle.gemm(case, threads=4), got, f"decode with zero-points int{bits} g{group}")
    packed = oracle.prepack(case)
    got2, _ = T.run_case(afb, packed, variant=pkg.VARIANT_DECODE)
    assert np.array_equal(got, got2)


@pytest.mark.gpu
@pytest.mark.parametrize("m", [96, 300])
@pytest.mark.parametrize("bits,group,enc", [(8, 0, 0), (8, 0, 1), (4, 0, 1), (4, 128, 0), (8, 64, 0), (4, 32, 0), (8, 32, 1)])
def test_prefill_with_zero_points_and_small_groups(afb, oracle, m, bits, group, enc):
    case = T.make_case(m, 392, 1024, bits=bits, group=group, enc=enc, seed=m + group, zero_points=True, scale_range=(0.005, 0.05))
    got, _ = T.run_case(afb, case, variant=pkg.VARIANT_PREFILL)
    if group:
        check_close(oracle, oracle.gemm(case, threads=4, round_w=True), got, f"prefill zero-points int{bits} g{group} (rounded-weight oracle)")
        exact, _ = T.run_case(afb, case, variant=pkg.VARIANT_PREFILL, flags=pkg.FLAG_GROUP_EXACT)
        check_close(oracle, oracle.gemm(case, threads=4), exact, f"prefill zero-points int{bits} g{group}, two-term mode")
    else:
        check_close(oracle, oracle.gemm(case, threads=4), got, f"prefill zero-points int{bits}")
    assert afb.read_status()[0] == 0
    # the shared-memory form does not read zero-points: it must refuse, not ignore them
    dc = T.DeviceCase(afb, case)
    try:
        assert afb.gemm_launch_status(dc.args(variant=pkg.VARIANT_PREFILL, flags=pkg.FLAG_PREFILL_SMEM_B)) == -2
    finally:
        dc.close()


@pytest.mark.gpu
@pytest.mark.parametrize("m,bits,group", [(4, 4, 64), (16, 4, 32), (8, 8, 32), (200, 4, 32), (200, 8, 64)])
def test_small_scale_groups_without_zero_points(afb, oracle, m, bits, group):
    """Groups of 32 and 64: the decode kernel needs whole 64-byte chunks per group, so small M with such groups runs on the
    tensor-memory prefill kernel (AFB_VARIANT_AUTO picks it); the result is held to the same bounds."""
    case = T.make_case(m, 264, 1024, bits=bits, group=group, seed=77, scale_range=(0.005, 0.05))
    dc = T.DeviceCase(afb, case)
    try:
        v = afb.resolve_variant(dc.args())
        afb.gemm_launch(dc.args(flags=pkg.FLAG_GROUP_EXACT)); afb.device_sync()
        got = dc.result()[0]
    finally:
        dc.close()
    assert v in (pkg.VARIANT_DECODE, pkg.VARIANT_PREFILL)
    check_close(oracle, oracle.gemm(case, threads=4), got, f"group {group} int{bits} M={m} (variant {v})")
