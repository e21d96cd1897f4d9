"""Fused neighbours of the GEMM (afb_gemm_fused_launch): bias, SiLU, gate * up and residual in the epilogue of the prefill
kernel.  The check is the same formula in fp32 on the CPU oracle's fp32 GEMM results:
    v = gemm + bias;  plain: act(v) + residual;  gated: act(v[:, 0::2]) * v[:, 1::2] + residual;  one rounding to bf16."""
import numpy as np
import pytest

import afb_testlib as T
import awesome_fusion_b200 as pkg
from test_gpu_parity import check_close

pytestmark = pytest.mark.gpu


def silu(x):
    x = x.astype(np.float32)
    return (x / (np.float32(1) + np.exp(-x, dtype=np.float32))).astype(np.float32)


def interleave_rows(g, u):
    out = np.empty((2 * g.shape[0],) + g.shape[1:], g.dtype)
    out[0::2], out[1::2] = g, u
    return out


@pytest.mark.parametrize("m,n,k", [(300, 264, 512), (64, 136, 256), (4, 128, 1024), (1024, 512, 2048)])
@pytest.mark.parametrize("bits,group,zero_points", [(8, 0, False), (4, 128, False), (8, 0, True), (4, 0, False)])
def test_gated_silu_matches_the_fp32_formula(afb, oracle, m, n, k, bits, group, zero_points):
    gate = T.make_case(m, n, k, bits=bits, group=group, seed=101, zero_points=zero_points, scale_range=(0.002, 0.01))
    up = T.make_case(m, n, k, bits=bits, group=group, seed=102, zero_points=zero_points, scale_range=(0.002, 0.01))
    up.a = gate.a                                     # one activation matrix, two projections
    rng = np.random.default_rng(7)
    residual = T.np_bf16_rne(rng.standard_normal((m, n), dtype=np.float32))
    exact = pkg.FLAG_GROUP_EXACT if group else 0        # group scales: the two-term mode, so that the fp32 formula is the reference
    want = silu(oracle.gemm(gate, threads=8)) * oracle.gemm(up, threads=8) + T.np_bf16_to_f32(residual)

    d_a = afb.to_device(gate.a)
    d_bg, d_bu, d_sg, d_su = (afb.to_device(x) for x in (gate.b, up.b, gate.scale, up.scale))
    d_zg = afb.to_device(gate.zero) if zero_points else None
    d_zu = afb.to_device(up.zero) if zero_points else None
    row_bytes = k * bits // 8
    d_b2 = afb.malloc(2 * n * row_bytes)
    d_s2 = afb.malloc(2 * gate.scale.nbytes)
    d_z2 = afb.malloc(2 * gate.zero.nbytes) if zero_points else None
    d_res = afb.to_device(residual)
    d_c = afb.malloc(m * n * 2)
    try:
        gate_args = afb.make_args(d_c, d_a, d_bg, d_sg, m, n, k, bits=bits, group=group, scale_dtype=gate.scale_dtype, zero=d_zg)
        afb.prepack_gated(gate_args, d_bu, d_su, d_zu, d_b2, k, d_s2, d_z2)
        afb.device_sync()
        # the interleaved, packed matrix is what the restatement builds from the two cases
        both = T.Case(**{**gate.__dict__, "n": 2 * n, "b": interleave_rows(gate.b, up.b), "scale": interleave_rows(gate.scale, up.scale),
                         "zero": interleave_rows(gate.zero, up.zero) if zero_points else None})
        assert np.array_equal(afb.to_host(d_b2, (2 * n, row_bytes), np.uint8), oracle.prepack(both).b)
        assert np.array_equal(afb.to_host(d_s2, both.scale.shape, both.scale.dtype), both.scale)
        g2 = afb.make_args(d_c, d_a, d_b2, d_s2, m, 2 * n, k, ldc=n, bits=bits, group=group, scale_dtype=gate.scale_dtype,
                           layout=pkg.LAYOUT_COL_PACKED, flags=exact, zero=d_z2)
        f = afb.make_fused_args(g2, gated=True, activation=pkg.ACT_SILU, residual=d_res, ld_residual=n)
        afb.memset(d_c, 0xCD, m * n * 2)
        afb.gemm_fused_launch(f)
        afb.device_sync()
        got = afb.to_host(d_c, (m, n), np.uint16)
        assert afb.read_status()[0] == 0
    finally:
        for p in (d_a, d_bg, d_bu, d_sg, d_su, d_zg, d_zu, d_b2, d_s2, d_z2, d_res, d_c):
            if p is not None:
                afb.free(p)
    check_close(oracle, want, got, f"gated SiLU int{bits} g{group} {m}x{n}x{k}")


@pytest.mark.parametrize("act", [pkg.ACT_NONE, pkg.ACT_SILU])
def test_bias_activation_residual_without_gate(afb, oracle, act):
    case = T.make_case(200, 264, 512, seed=111)
    rng = np.random.default_rng(8)
    bias = rng.standard_normal(case.n).astype(np.float32)
    residual = T.np_bf16_rne(rng.standard_normal((case.m, case.n), dtype=np.float32))
    v = oracle.gemm(case, threads=4) + bias[None, :]
    want = (silu(v) if act == pkg.ACT_SILU else v) + T.np_bf16_to_f32(residual)
    dc = T.DeviceCase(afb, case)
    d_bias, d_res = afb.to_device(bias), afb.to_device(residual)
    try:
        f = afb.make_fused_args(dc.args(), activation=act, bias=d_bias, residual=d_res, ld_residual=case.n)
        afb.gemm_fused_launch(f); afb.device_sync()
        got = dc.result()[0]
        # no epilogue options at all: the plain GEMM, bit for bit
        afb.gemm_fused_launch(afb.make_fused_args(dc.args())); afb.device_sync()
        bare = dc.result()[0]
        afb.gemm_launch(dc.args(variant=pkg.VARIANT_PREFILL, flags=pkg.FLAG_PREFILL_TMEM_A)); afb.device_sync()
        plain = dc.result()[0]
    finally:
        dc.close(); afb.free(d_bias); afb.free(d_res)
    check_close(oracle, want, got, "bias + activation + residual")
    assert np.array_equal(bare, plain)


def test_fused_launch_refuses_what_it_cannot_do(afb):
    a = afb.make_args(0x1000, 0x1000, 0x1000, 0x1000, 64, 130, 256)
    assert afb.gemm_fused_launch_status(afb.make_fused_args(a, gated=True)) == -2 or afb.gemm_fused_launch_status(afb.make_fused_args(a, gated=True)) == -1
    a = afb.make_args(0x1000, 0x1000, 0x1000, 0x1000, 64, 131, 256)
    assert afb.gemm_fused_launch_status(afb.make_fused_args(a, gated=True)) == -1          # odd number of rows cannot be gate / up pairs
    a = afb.make_args(0x1000, 0x1000, 0x1000, 0x1000, 64, 128, 256, flags=pkg.FLAG_C_F32)
    assert afb.gemm_fused_launch_status(afb.make_fused_args(a)) == -2                      # bf16 output only
    a = afb.make_args(0x1000, 0x1000, 0x1000, 0x1000, 64, 128, 256, layout=pkg.LAYOUT_ROW, ldb=128)
    assert afb.gemm_fused_launch_status(afb.make_fused_args(a)) == -2
