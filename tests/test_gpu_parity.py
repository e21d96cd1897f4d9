"""GPU parity tests: every kernel variant, through the C ABI, against the CPU oracle on the same
seeded inputs.  Integer / byte work (unpack, dequant) must be bit-exact; bf16 outputs must be within
max relative error 1e-2 of the oracle (denominators floored at a stated fraction of the tensor RMS)."""
import os

import numpy as np
import pytest

import afb_testlib as T
import awesome_fusion_b200 as pkg

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")

TOL = 1e-2            # max relative error on bf16 outputs
FLOOR_FRAC = 0.05     # |ref| below this fraction of RMS(ref) is compared against the floor instead
# Group-scaled prefill in its default (one rounded bf16 term per weight) mode against the pure-fp32 formula, at the same floor:
# the documented exception to the 1e-2 contract (AFB_FLAG_GROUP_EXACT is the mode that meets it).
GROUPED_ONE_TERM_BOUND = 0.25    # measured: 0.11 to 0.16 of max(|ref|, 0.05 x RMS), NRMS 1.6e-3


def check_close(oracle, ref, got_bf16, what, tol=TOL, floor_frac=FLOOR_FRAC):
    floor = max(T.rms(ref) * floor_frac, 1e-30)
    mx, nrms, worst = oracle.compare(ref, got_bf16, floor)
    assert mx <= tol, f"{what}: max rel err {mx:.4g} at {worst} (ref {ref.reshape(-1)[worst]}, got " \
                      f"{T.np_bf16_to_f32(got_bf16.reshape(-1)[worst:worst + 1])[0]}), nrms {nrms:.3g}"
    return mx, nrms


# ---------------------------------------------------------------- unpack + dequant: bit-exact
@pytest.mark.parametrize("enc", [0, 1])
@pytest.mark.parametrize("layout", [0, 1])
def test_dequant_int8_all_byte_values(afb, oracle, enc, layout):
    n, k = 64, 256
    b = np.arange(n * k, dtype=np.uint32).astype(np.uint8).reshape(n, k)        # every byte value, many times
    b = np.ascontiguousarray(b if layout == 1 else b.T)
    case = T.Case(m=1, n=n, k=k, bits=8, group=0, layout=layout, enc=enc, scale_dtype=0, b=b,
                  scale=np.ones(n, np.float32), ldb=b.shape[1])
    d_b, d_s = afb.to_device(case.b), afb.to_device(case.scale)
    d_o = afb.malloc(n * k * 2)
    args = afb.make_args(d_o, d_b, d_b, d_s, 1, n, k, ldb=case.ldb, bits=8, encoding=enc, layout=layout)
    afb.dequant_dump(args, d_o)
    afb.device_sync()
    got = afb.to_host(d_o, (n, k) if layout == 1 else (k, n), np.uint16)
    for p in (d_b, d_s, d_o):
        afb.free(p)
    assert np.array_equal(got, oracle.dequant_bf16(case))


@pytest.mark.parametrize("bits,group,enc,scale_dtype", [(4, 0, 0, 0), (4, 0, 1, 0), (4, 128, 0, 1), (4, 128, 1, 1), (4, 64, 0, 1),
                                                       (8, 128, 0, 1), (8, 64, 1, 1), (4, 128, 0, 0)])
def test_dequant_groups_and_int4(afb, oracle, bits, group, enc, scale_dtype):
    case = T.make_case(1, 96, 512, bits=bits, group=group, enc=enc, scale_dtype=scale_dtype, seed=11, scale_range=(0.005, 0.05))
    d_b, d_s = afb.to_device(case.b), afb.to_device(case.scale)
    d_o = afb.malloc(case.n * case.k * 2)
    args = afb.make_args(d_o, d_b, d_b, d_s, 1, case.n, case.k, ldb=case.ldb, bits=bits, encoding=enc, layout=1,
                         scale_dtype=scale_dtype, group=group)
    afb.dequant_dump(args, d_o)
    afb.device_sync()
    got = afb.to_host(d_o, (case.n, case.k), np.uint16)
    for p in (d_b, d_s, d_o):
        afb.free(p)
    if group and scale_dtype == 0:
        # fp32 scales are first rounded to bf16 by the kernels (the dequant contract multiplies two bf16 values)
        case.scale = T.np_bf16_rne(case.scale); case.scale_dtype = 1
    assert np.array_equal(got, oracle.dequant_bf16(case))


@pytest.mark.parametrize("bits,enc", [(8, 0), (8, 1), (4, 0), (4, 1)])
def test_dequant_decode_pairing_is_bit_exact(afb, oracle, bits, enc):
    """The decode kernel unpacks with the strided pairing ({k0,k2},{k1,k3} for int8, {k0,k4}..{k3,k7} for int4).  The dump runs
    those same device routines and stores the values back in natural k order: every byte value, both encodings."""
    n, k = 64, 512
    raw = (np.arange(n * k * bits // 8, dtype=np.uint32) * 7 + 3).astype(np.uint8).reshape(n, k * bits // 8)   # every byte value, many times
    case = T.Case(m=1, n=n, k=k, bits=bits, group=0, layout=1, enc=enc, scale_dtype=0, b=raw, scale=np.ones(n, np.float32), ldb=k)
    d_b, d_s = afb.to_device(case.b), afb.to_device(case.scale)
    d_o = afb.malloc(n * k * 2)
    args = afb.make_args(d_o, d_b, d_b, d_s, 1, n, k, ldb=k, bits=bits, encoding=enc, layout=1, flags=pkg.FLAG_DUMP_DECODE_PAIRING)
    afb.dequant_dump(args, d_o)
    afb.device_sync()
    got = afb.to_host(d_o, (n, k), np.uint16)
    for p in (d_b, d_s, d_o):
        afb.free(p)
    assert np.array_equal(got, oracle.dequant_bf16(case))


# ---------------------------------------------------------------- naive variant: fp32 bit-exact with the oracle
@pytest.mark.parametrize("bits,group,layout,enc", [(8, 0, 0, 1), (8, 0, 0, 0), (8, 0, 1, 0), (8, 128, 1, 1), (4, 0, 1, 0), (4, 128, 1, 0)])
def test_naive_is_bit_exact_fp32(afb, oracle, bits, group, layout, enc):
    case = T.make_case(7, 72, 384, bits=bits, group=group, layout=layout, enc=enc, seed=5)
    got, _ = T.run_case(afb, case, variant=pkg.VARIANT_NAIVE, c_f32=True)
    assert np.array_equal(got.view(np.uint32), oracle.gemm(case).view(np.uint32))


def test_naive_matches_reference_golden(afb):
    g = np.load(os.path.join(GOLD, "gemm_rrr_real.npz"))
    b = g["b"]                                     # [K,N] int8, the reference's layout
    for enc in (0, 1):
        stored = (b.astype(np.int16) + 128).astype(np.uint8) if enc else b.view(np.uint8)
        case = T.Case(m=g["a_bf16"].shape[0], n=b.shape[1], k=b.shape[0], bits=8, group=0, layout=0, enc=enc, scale_dtype=0,
                      a=g["a_bf16"], b=np.ascontiguousarray(stored), scale=g["scale"], ldb=b.shape[1])
        got, _ = T.run_case(afb, case, variant=pkg.VARIANT_NAIVE, c_f32=True)
        assert np.array_equal(got.view(np.uint32), g["c"].view(np.uint32))


# ---------------------------------------------------------------- decode variant
DECODE_SHAPES = [(1, 128, 256), (4, 256, 1024), (8, 136, 512), (9, 128, 64), (16, 4096, 4096), (3, 1000, 2048), (16, 264, 4096 + 64)]


@pytest.mark.parametrize("m,n,k", DECODE_SHAPES)
@pytest.mark.parametrize("enc", [0, 1])
def test_decode_int8_per_channel(afb, oracle, m, n, k, enc):
    case = T.make_case(m, n, k, bits=8, enc=enc, seed=m * 131 + n)
    got, _ = T.run_case(afb, case, variant=pkg.VARIANT_DECODE)
    check_close(oracle, oracle.gemm(case, threads=8), got, f"decode int8 {m}x{n}x{k}")


@pytest.mark.parametrize("m,n,k", [(1, 128, 256), (16, 256, 2048), (5, 1000, 1024), (16, 4096, 4096)])
@pytest.mark.parametrize("bits,group,scale_dtype", [(4, 0, 0), (4, 128, 1), (8, 128, 1), (4, 256, 1), (4, 128, 0), (4, 0, 1)])
def test_decode_int4_and_groups(afb, oracle, m, n, k, bits, group, scale_dtype):
    case = T.make_case(m, n, k, bits=bits, group=group, scale_dtype=scale_dtype, seed=k + m, scale_range=(0.005, 0.05))
    got, _ = T.run_case(afb, case, variant=pkg.VARIANT_DECODE)
    check_close(oracle, oracle.gemm(case, threads=8), got, f"decode int{bits} g{group} {m}x{n}x{k}")


def test_decode_is_deterministic_and_leaves_workspace_clean(afb, oracle):
    case = T.make_case(16, 4096, 4096, seed=1)
    first, _ = T.run_case(afb, case, variant=pkg.VARIANT_DECODE)
    for _ in range(3):
        again, _ = T.run_case(afb, case, variant=pkg.VARIANT_DECODE)
        assert np.array_equal(first, again)


# ---------------------------------------------------------------- prefill variant
PREFILL_SHAPES = [(128, 256, 64), (128, 256, 512), (17, 128, 256), (256, 512, 1024), (300, 264, 320), (128, 128, 4096), (640, 1280, 2048)]


# the prefill variant has two forms; each is forced in turn so that both are covered whatever the default is
IMPLS = [pytest.param(pkg.FLAG_PREFILL_SMEM_B, id="smem-b"), pytest.param(pkg.FLAG_PREFILL_TMEM_A, id="tmem-a")]


@pytest.mark.parametrize("impl", IMPLS)
@pytest.mark.parametrize("m,n,k", PREFILL_SHAPES)
@pytest.mark.parametrize("enc", [0, 1])
def test_prefill_int8_per_channel(afb, oracle, m, n, k, enc, impl):
    case = T.make_case(m, n, k, bits=8, enc=enc, seed=n + k)
    got, _ = T.run_case(afb, case, variant=pkg.VARIANT_PREFILL, flags=impl)
    check_close(oracle, oracle.gemm(case, threads=8), got, f"prefill int8 {m}x{n}x{k}")
    assert afb.read_status()[0] == 0


@pytest.mark.parametrize("impl", IMPLS)
@pytest.mark.parametrize("m,n,k", [(128, 256, 256), (200, 520, 1024), (384, 1024, 2048)])
@pytest.mark.parametrize("bits,group,scale_dtype", [(4, 0, 0), (4, 128, 1), (8, 128, 1), (4, 64, 1), (8, 0, 1)])
def test_prefill_int4_and_groups(afb, oracle, m, n, k, bits, group, scale_dtype, impl):
    case = T.make_case(m, n, k, bits=bits, group=group, scale_dtype=scale_dtype, seed=7 * m + k, scale_range=(0.005, 0.05))
    got, _ = T.run_case(afb, case, variant=pkg.VARIANT_PREFILL, flags=impl)
    ref_exact = oracle.gemm(case, threads=8)
    if group:
        # Tensor-core operands are bf16, so by default a per-group scale is folded into the weight before the MMA:
        # w = bf16_rn(q * s) carries a relative error of up to 2^-9 per weight that the fp32 formula of host_ref.hpp:15-24
        # does not have.  Tight check against the oracle fed with the SAME rounded weights ...
        check_close(oracle, oracle.gemm(case, round_w=True, threads=8), got, f"prefill int{bits} g{group} (rounded-weight oracle)")
        # ... and the deviation from the pure-fp32 formula, at the standard floor, stated as what it is (it does not meet 1e-2):
        mx, nrms, _ = oracle.compare(ref_exact, got, T.rms(ref_exact) * FLOOR_FRAC)
        print(f"group-scaled prefill, one rounded term: max rel err {mx:.3e} at the 0.05 x RMS floor, nrms {nrms:.3e}")
        assert nrms < 3e-3 and mx < GROUPED_ONE_TERM_BOUND
        # AFB_FLAG_GROUP_EXACT feeds q * s as two bf16 terms (exact): this mode meets the 1e-2 contract against host_ref
        if impl == pkg.FLAG_PREFILL_TMEM_A:
            exact, _ = T.run_case(afb, case, variant=pkg.VARIANT_PREFILL, flags=impl | pkg.FLAG_GROUP_EXACT)
            check_close(oracle, ref_exact, exact, f"prefill int{bits} g{group} two-term mode (host_ref formula)")
    else:
        check_close(oracle, ref_exact, got, f"prefill int{bits} {m}x{n}x{k}")
    assert afb.read_status()[0] == 0


@pytest.mark.parametrize("impl", IMPLS)
def test_prefill_fp32_output_for_k_split_partials(afb, oracle, impl):
    """AFB_FLAG_C_F32: the fp32 accumulator times the scale, unrounded (what a K-split rank hands to the all-reduce)."""
    case = T.make_case(300, 264, 512, seed=44)
    got, _ = T.run_case(afb, case, variant=pkg.VARIANT_PREFILL, c_f32=True, flags=impl)
    ref = oracle.gemm(case, threads=4)
    assert np.abs(got - ref).max() <= 1e-4 * T.rms(ref)      # only the fp32 summation order differs


# ---------------------------------------------------------------- known-answer cases (exact)
@pytest.mark.parametrize("variant,m,flags", [(pkg.VARIANT_DECODE, 16, 0), (pkg.VARIANT_DECODE, 3, 0), (pkg.VARIANT_PREFILL, 160, pkg.FLAG_PREFILL_SMEM_B),
                                             (pkg.VARIANT_PREFILL, 160, pkg.FLAG_PREFILL_TMEM_A), (pkg.VARIANT_PREFILL, 300, pkg.FLAG_PREFILL_TMEM_A),
                                             (pkg.VARIANT_NAIVE, 20, 0)])
@pytest.mark.parametrize("bits", [8, 4])
def test_reference_style_integer_data_is_exact(afb, oracle, variant, m, bits, flags):
    """The reference validates on integers in {-2,-1,0,1} (random_gen.hpp:24,37,50): every product and
    partial sum is exact, so any correct kernel must reproduce the oracle exactly after bf16 rounding."""
    case = T.make_case(m, 256, 512, bits=bits, seed=2, integer_data=True)
    got, _ = T.run_case(afb, case, variant=variant, flags=flags)
    # compared as numbers: with a zero scale the kernels form (sum * 0), which may be -0 where the oracle's sum of (a * (b * 0)) is +0
    assert np.array_equal(T.np_bf16_to_f32(got), T.np_bf16_to_f32(T.np_bf16_rne(oracle.gemm(case))))


@pytest.mark.parametrize("variant,m,flags", [(pkg.VARIANT_DECODE, 8, 0), (pkg.VARIANT_PREFILL, 128, pkg.FLAG_PREFILL_SMEM_B), (pkg.VARIANT_PREFILL, 256, pkg.FLAG_PREFILL_TMEM_A)])
@pytest.mark.parametrize("bits", [8, 4])
def test_one_hot_weights_select_activation_columns(afb, variant, m, bits, flags):
    n, k = 128, 256
    case = T.make_case(m, n, k, bits=bits, seed=9)
    q = np.zeros((n, k), np.int32)
    sel = (np.arange(n) * 37) % k
    q[np.arange(n), sel] = 1
    u = q & (0xFF if bits == 8 else 0xF)
    case.b = np.ascontiguousarray(u.astype(np.uint8) if bits == 8 else (u[:, 0::2] | (u[:, 1::2] << 4)).astype(np.uint8))
    case.scale = np.ones(n, np.float32)
    got, _ = T.run_case(afb, case, variant=variant, flags=flags)
    assert np.array_equal(got, case.a[:, sel])      # scale 1, weight 1: C = selected columns of A, exactly


@pytest.mark.parametrize("variant,m,flags", [(pkg.VARIANT_DECODE, 4, 0), (pkg.VARIANT_PREFILL, 128, pkg.FLAG_PREFILL_SMEM_B), (pkg.VARIANT_PREFILL, 130, pkg.FLAG_PREFILL_TMEM_A)])
@pytest.mark.parametrize("bits,val", [(8, -128), (8, 127), (4, -8), (4, 7)])
def test_extreme_weights_sign_extension(afb, oracle, variant, m, bits, val, flags):
    case = T.make_case(m, 128, 256, bits=bits, seed=4)
    u = val & (0xFF if bits == 8 else 0xF)
    case.b[:] = u if bits == 8 else (u | (u << 4))
    case.q[:] = val
    got, _ = T.run_case(afb, case, variant=variant, flags=flags)
    check_close(oracle, oracle.gemm(case), got, f"all weights {val}")


# ---------------------------------------------------------------- memory safety (no compute-sanitizer on this pool)
@pytest.mark.parametrize("variant,m,n,k,flags", [(pkg.VARIANT_DECODE, 5, 264, 512, 0), (pkg.VARIANT_PREFILL, 130, 264, 256, pkg.FLAG_PREFILL_SMEM_B),
                                                 (pkg.VARIANT_PREFILL, 130, 264, 256, pkg.FLAG_PREFILL_TMEM_A), (pkg.VARIANT_PREFILL, 259, 136, 128, pkg.FLAG_PREFILL_TMEM_A),
                                                 (pkg.VARIANT_NAIVE, 5, 70, 64, 0)])
def test_guard_bytes_and_padding_untouched(afb, oracle, variant, m, n, k, flags):
    case = T.make_case(m, n, k, seed=6)
    ldc = n + 24
    got, raw = T.run_case(afb, case, variant=variant, ldc=ldc, guard=4096, flags=flags)
    check_close(oracle, oracle.gemm(case), got, "padded C")
    assert np.all(raw[:4096] == 0xCD) and np.all(raw[-4096:] == 0xCD)
    body = raw[4096:-4096].view(np.uint16)
    full = np.full(m * ldc, 0xCDCD, np.uint16); full[:body.size] = body
    assert np.all(full.reshape(m, ldc)[:, n:].reshape(-1)[:(m - 1) * 24] == 0xCDCD)   # the ldc padding columns


@pytest.mark.parametrize("variant,m,flags", [(pkg.VARIANT_DECODE, 7, 0), (pkg.VARIANT_DECODE, 16, 0), (pkg.VARIANT_PREFILL, 96, pkg.FLAG_PREFILL_SMEM_B),
                                             (pkg.VARIANT_PREFILL, 300, pkg.FLAG_PREFILL_TMEM_A), (pkg.VARIANT_NAIVE, 9, 0)])
@pytest.mark.parametrize("bits", [8, 4])
def test_leading_dimensions_larger_than_the_matrix(afb, oracle, variant, m, flags, bits):
    """lda / ldb / ldc as the reference driver takes them on its command line (bfAintBGemm.cc:49-58): rows padded in memory."""
    case = T.make_case(m, 264, 640, bits=bits, seed=31)
    got, _ = T.run_case(afb, case, variant=variant, flags=flags, lda=640 + 64, ldb=640 + 128, ldc=264 + 8)
    check_close(oracle, oracle.gemm(case, threads=4), got, f"padded leading dimensions, int{bits}")


@pytest.mark.parametrize("m,n,k,ldc", [(300, 264, 320, 264), (259, 136, 128, 160), (1024, 512, 512, 512)])
def test_prefill_tile_stores_equal_register_stores(afb, oracle, monkeypatch, m, n, k, ldc):
    """A plain bf16 result leaves the prefill kernel through shared memory and 32 x 32 tile stores (clipped at the edges of C);
    AFB_PREFILL_TILE_STORE=0 stores the same values from registers.  Same bits, and the padding of C stays untouched."""
    case = T.make_case(m, n, k, seed=77)
    got_tile, raw_tile = T.run_case(afb, case, variant=pkg.VARIANT_PREFILL, flags=pkg.FLAG_PREFILL_TMEM_A, ldc=ldc, guard=4096)
    monkeypatch.setenv("AFB_PREFILL_TILE_STORE", "0")
    got_reg, raw_reg = T.run_case(afb, case, variant=pkg.VARIANT_PREFILL, flags=pkg.FLAG_PREFILL_TMEM_A, ldc=ldc, guard=4096)
    assert np.array_equal(got_tile.view(np.uint16), got_reg.view(np.uint16))
    assert np.array_equal(raw_tile, raw_reg)   # guard bytes and ldc padding included
    check_close(oracle, oracle.gemm(case, threads=4), got_tile, "tile stores")
    assert afb.read_status()[0] == 0


def test_gemm_publishing_tiles_and_tile_exchange_on_one_rank(afb, oracle):
    """The tile-granular K-split exchange with a single rank: the GEMM counts its tiles, the exchange kernel waits for the
    counts, rounds the fp32 partial sums to bf16 and stores C.  (Several ranks: tests/test_dist.py on a multi-GPU box.)"""
    from awesome_fusion_b200 import dist as D
    case = T.make_case(300, 264, 512, seed=51)
    px = D.PeerExchange(afb, None, 0, 1, case.m, case.n, partial_f32=True)
    d_a, d_b, d_s = afb.to_device(case.a), afb.to_device(case.b), afb.to_device(case.scale)
    try:
        args = afb.make_args(px.partial, d_a, d_b, d_s, case.m, case.n, case.k, flags=pkg.FLAG_C_F32)
        outs = []
        for _ in range(2):
            afb.memset(px.c, 0, case.m * case.n * 2)
            px.gemm_publishing_tiles(args)
            px.allreduce_tiles()
            afb.device_sync()
            outs.append(afb.to_host(px.c, (case.m, case.n), np.uint16))
        counts = afb.to_host(px.tile_done, (px.num_tiles,), np.uint32)
        assert afb.read_status()[0] == 0
        assert np.all(counts == counts[0]) and counts[0] > 0 and counts[0] % 2 == 0      # every tile counted equally, twice
        assert np.array_equal(outs[0], outs[1])
        check_close(oracle, oracle.gemm(case, threads=4), outs[0], "tile exchange, one rank")
    finally:
        px.close()
        for p in (d_a, d_b, d_s):
            afb.free(p)


def test_unsupported_requests_return_status_not_fault(afb):
    case = T.make_case(4, 128, 256, layout=0, seed=1)
    dc = T.DeviceCase(afb, case)
    try:
        assert afb.gemm_launch_status(dc.args(variant=pkg.VARIANT_DECODE)) == -2
        assert afb.gemm_launch_status(dc.args(variant=pkg.VARIANT_PREFILL)) == -2
        a = dc.args(); a.k = 100; a.lda = 100
        assert afb.gemm_launch_status(a) in (0, -2)      # auto falls back to the naive variant
        a = dc.args(); a.ptr_a = 0
        assert afb.gemm_launch_status(a) == -1
        afb.device_sync()
    finally:
        dc.close()


@pytest.mark.parametrize("m,n,k", [(64, 256, 512), (48, 4096, 256), (300, 8192, 128)])     # the last two take the chunked, pipelined path
def test_host_pointer_entry_point(afb, oracle, m, n, k):
    case = T.make_case(m, n, k, seed=12)
    c = np.zeros((case.m, case.n), np.uint16)
    args = afb.make_args(c, case.a, case.b, case.scale, case.m, case.n, case.k, ldb=case.ldb)
    afb.gemm_host(args)
    check_close(oracle, oracle.gemm(case), c, "afb_gemm_host")


def test_host_pointer_entry_point_two_calls_in_flight(afb, oracle):
    """afb_gemm_host_async: three GEMMs queued back to back on alternating staging sets (the third reuses the first one's),
    one wait at the end; each result against the oracle."""
    cases = [T.make_case(300, 8192, 128, seed=13), T.make_case(64, 256, 512, seed=14), T.make_case(320, 4096, 256, seed=15)]
    outs = [np.zeros((c.m, c.n), np.uint16) for c in cases]
    args = [afb.make_args(o, c.a, c.b, c.scale, c.m, c.n, c.k, ldb=c.ldb) for c, o in zip(cases, outs)]
    for a in args:
        afb.gemm_host_async(a)
    afb.gemm_host_wait()
    for c, o in zip(cases, outs):
        check_close(oracle, oracle.gemm(c, threads=4), o, "afb_gemm_host_async")


@pytest.mark.gpu
@pytest.mark.parametrize("m,n,k,bits,group", [(16, 1000, 4096, 8, 0), (9, 2048, 8192, 4, 128), (16, 136, 1024, 8, 0), (12, 4104, 2048, 4, 0),
                                               (16, 520, 2048, 8, 256), (3, 776, 4096, 4, 128)])
def test_decode_balanced_form_on_ragged_shapes(afb, oracle, monkeypatch, m, n, k, bits, group):
    """The one-wave form of the decode kernel (contiguous runs of K units per CTA, channel blocks shared between CTAs and
    finished by the last to arrive) is chosen by itself only for large matrices; here it is forced on small and ragged
    ones: channel counts that are no multiple of the CTA's block, fewer units than CTAs, every CTA shape."""
    case = T.make_case(m, n, k, bits=bits, group=group, seed=81)
    ref = oracle.gemm(case, threads=4)
    monkeypatch.setenv("AFB_DECODE_BALANCED", "1")
    outs = {}
    for wr in ("1", "2", "4", "8"):
        monkeypatch.setenv("AFB_DECODE_WR", wr)
        a, _ = T.run_case(afb, case, variant=pkg.VARIANT_DECODE, guard=256)
        b, raw = T.run_case(afb, case, variant=pkg.VARIANT_DECODE, guard=256)
        assert np.array_equal(a, b), f"wr={wr}: two runs differ"
        assert np.all(raw[:256] == 0xCD) and np.all(raw[-256:] == 0xCD)
        check_close(oracle, ref, a, f"balanced decode wr={wr}")
        outs[wr] = a
    assert afb.read_status()[0] == 0
    # the split-K workspace counters are back at zero: the grid form right after it must still be correct
    monkeypatch.setenv("AFB_DECODE_BALANCED", "0")
    monkeypatch.delenv("AFB_DECODE_WR")
    c, _ = T.run_case(afb, case, variant=pkg.VARIANT_DECODE)
    check_close(oracle, ref, c, "grid form after the balanced form")


@pytest.mark.gpu
def test_exchange_wait_runs_out_and_reports_status(afb, oracle):
    """A bounded wait that nothing satisfies: the exchange kernel of a 2-rank job whose peer never signals gives up after
    wait_ms, stores nothing, reports AFB_ERR_TIMEOUT with the place it gave up, and the device stays usable."""
    import ctypes
    from awesome_fusion_b200 import dist as D
    m, n = 64, 256
    partial, peer_partial = afb.malloc(m * n * 4), afb.malloc(m * n * 4)
    c, peer_c = afb.malloc(m * n * 2), afb.malloc(m * n * 2)
    sig, peer_sig = afb.malloc(2 * D.MAX_RANKS * 4), afb.malloc(2 * D.MAX_RANKS * 4)
    try:
        for p_, nb in ((partial, m * n * 4), (peer_partial, m * n * 4), (sig, 2 * D.MAX_RANKS * 4), (peer_sig, 2 * D.MAX_RANKS * 4)):
            afb.memset(p_, 0, nb)
        afb.memset(c, 0xCD, m * n * 2)
        a = D.AllReduceArgs()
        a.partial[0], a.partial[1] = partial, peer_partial
        a.c[0], a.c[1] = c, peer_c
        a.signals[0], a.signals[1] = sig, peer_sig       # "rank 1" is a buffer nobody writes: its signal never comes
        a.rank, a.world, a.m, a.n, a.ld_partial, a.ldc, a.partial_f32 = 0, 2, m, n, n, n, 1
        a.epoch, a.wait_ms, a.reserved, a.c_multicast = 1, 20, 0, None
        f = afb.lib.afb_ksplit_allreduce_launch
        f.argtypes = [ctypes.POINTER(D.AllReduceArgs), ctypes.c_void_p]
        assert f(ctypes.byref(a), None) == 0
        st = afb.read_status()                            # synchronises
        assert st[0] == -4 and st[1] == 10 and st[2] == 0 and st[3] == 1, st      # AFB_ERR_TIMEOUT, phase-0 wait, rank 0, epoch 1
        assert np.all(afb.to_host(c, (m * n * 2,), np.uint8) == 0xCD)             # nothing was stored
        # ... and completion was not announced: every CTA runs its own clock, and one that gave up vetoes the "my block is in
        # place" signal (second half of the signal words) even if the last CTA to finish saw the peers in time
        assert np.all(afb.to_host(peer_sig, (2 * D.MAX_RANKS,), np.uint32)[D.MAX_RANKS:] == 0)
        assert np.all(afb.to_host(sig, (2 * D.MAX_RANKS,), np.uint32)[D.MAX_RANKS:] == 0)
        assert afb.read_status()[0] == 0                                          # reading cleared it
        # the context is intact: an ordinary GEMM still runs and is right
        case = T.make_case(4, 256, 512, seed=82)
        out, _ = T.run_case(afb, case)
        check_close(oracle, oracle.gemm(case, threads=2), out, "GEMM after a timed-out exchange")
    finally:
        for p_ in (partial, peer_partial, c, peer_c, sig, peer_sig):
            afb.free(p_)


@pytest.mark.gpu
@pytest.mark.parametrize("bits,group,c_f32", [(8, 0, False), (4, 128, False), (8, 0, True)])
def test_prefill_tail_tiles_split_along_k(afb, oracle, monkeypatch, bits, group, c_f32):
    """150 tiles on 148 SMs: the two tiles beyond the last full wave are each cut into stretches of K that different CTAs
    compute; the last CTA to arrive adds the stretches in order.  Checked against the oracle, for repeatability, and against
    the same GEMM with the split switched off."""
    if afb.sm_count() != 148:
        pytest.skip("the shape is chosen for 148 SMs")
    case = T.make_case(2560, 1920, 2048, bits=bits, group=group, seed=91)
    ref = oracle.gemm(case, threads=8)
    flags = pkg.FLAG_PREFILL_TMEM_A
    a, _ = T.run_case(afb, case, variant=pkg.VARIANT_PREFILL, flags=flags, c_f32=c_f32)
    b, _ = T.run_case(afb, case, variant=pkg.VARIANT_PREFILL, flags=flags, c_f32=c_f32)
    assert np.array_equal(a, b), "two runs differ"
    monkeypatch.setenv("AFB_PREFILL_SPLIT_TAIL", "0")
    whole, _ = T.run_case(afb, case, variant=pkg.VARIANT_PREFILL, flags=flags, c_f32=c_f32)
    assert afb.read_status()[0] == 0
    if c_f32:
        tol = 1e-5 * max(1.0, float(np.abs(ref).max()))
        assert np.abs(a - ref).max() <= 2e-3 * T.rms(ref) + tol and np.abs(whole - ref).max() <= 2e-3 * T.rms(ref) + tol
        assert not np.array_equal(a[:, -256:], np.zeros_like(a[:, -256:]))
    else:
        if group:   # one rounded term per weight: tight against the oracle fed with the same rounded weights
            ref = oracle.gemm(case, threads=8, round_w=True)
        check_close(oracle, ref, a, "tail split")
        check_close(oracle, ref, whole, "no tail split")
        if group:   # the two-term mode through the tail split, against the fp32 formula
            ex, _ = T.run_case(afb, case, variant=pkg.VARIANT_PREFILL, flags=flags | pkg.FLAG_GROUP_EXACT)
            check_close(oracle, oracle.gemm(case, threads=8), ex, "tail split, two-term mode")
    # the split only changes the order of the fp32 additions of the two tail tiles: everything else is bit-identical
    same = np.mean(a == whole)
    assert same > 0.97, same


@pytest.mark.gpu
@pytest.mark.parametrize("m,n,k,bits,group", [(96, 1024, 4096, 8, 0), (200, 2048, 2048, 8, 0), (128, 1024, 4096, 4, 128)])
def test_prefill_less_than_half_a_wave_of_tiles_split_along_k(afb, oracle, monkeypatch, m, n, k, bits, group):
    """At most half a wave of tiles (8 or 16 tiles on 148 SMs): every tile is cut into stretches of K for different CTAs, as the
    tiles of a short last wave are.  Checked against the oracle, for repeatability, and against the same GEMM without the cut."""
    case = T.make_case(m, n, k, bits=bits, group=group, seed=93)
    ref = oracle.gemm(case, threads=8, round_w=True) if group else oracle.gemm(case, threads=8)
    flags = pkg.FLAG_PREFILL_TMEM_A
    a, _ = T.run_case(afb, case, variant=pkg.VARIANT_PREFILL, flags=flags)
    b, _ = T.run_case(afb, case, variant=pkg.VARIANT_PREFILL, flags=flags)
    assert np.array_equal(a, b), "two runs differ"
    monkeypatch.setenv("AFB_PREFILL_SPLIT_TAIL", "0")
    whole, _ = T.run_case(afb, case, variant=pkg.VARIANT_PREFILL, flags=flags)
    assert afb.read_status()[0] == 0
    check_close(oracle, ref, a, "every tile cut along K")
    check_close(oracle, ref, whole, "tiles whole")
    # the cut changes the order of the fp32 additions: most results still round to the same bf16
    assert np.mean(a == whole) > 0.9


@pytest.mark.gpu
def test_measurement_aids_do_not_disturb_the_device(afb, oracle):
    """afb_probe_launch (empty and read-only kernels with a decode-like launch shape, with and without programmatic dependent
    launch) and afb_phase_timestamps answer with a status, and a GEMM right after them is still correct."""
    buf = afb.malloc(1 << 20)
    afb.memset(buf, 1, 1 << 20)
    for kind in (0, 1):
        for flags in (0, pkg.FLAG_PDL):
            afb.probe_launch(kind, buf, 1 << 20, 64, 52 * 1024, flags)
    afb.device_sync()
    assert afb.lib.afb_probe_launch(2, buf, 1 << 20, 64, 0, 0, None) == -1
    assert len(afb.phase_timestamps()) == 8
    afb.free(buf)
    case = T.make_case(3, 256, 512, seed=5)
    for flags in (0, pkg.FLAG_PDL):
        out, _ = T.run_case(afb, case, flags=flags)
        check_close(oracle, oracle.gemm(case), out, "GEMM after the probes")
    assert afb.read_status()[0] == 0


@pytest.mark.gpu
@pytest.mark.parametrize("m,n,k,bits,group", [(1, 4096, 4096, 8, 0), (8, 4096, 4096, 8, 0), (16, 4096, 4096, 8, 0), (16, 2048, 4096, 4, 128), (12, 1000, 2048, 8, 0),
                                               (16, 4096, 4096 + 64, 8, 0), (5, 520, 8192, 4, 0)])
def test_decode_back_to_back_with_dependent_launch(afb, oracle, m, n, k, bits, group):
    """Several decode GEMMs on rotating weight buffers queued back to back with AFB_FLAG_PDL (each may start while its
    predecessor still runs): every result against the oracle, and identical to the same launch without the flag.  The shapes
    include the small-matrix forms (8-stage ring, whole K staged in one pass)."""
    cases = [T.make_case(m, n, k, bits=bits, group=group, seed=200 + i, scale_range=(0.005, 0.05)) for i in range(3)]
    dcs = [T.DeviceCase(afb, c) for c in cases]
    try:
        for _ in range(2):
            for dc in dcs:
                afb.gemm_launch(dc.args(variant=pkg.VARIANT_DECODE, flags=pkg.FLAG_PDL))
        afb.device_sync()
        with_flag = [dc.result()[0] for dc in dcs]
        for dc in dcs:
            afb.gemm_launch(dc.args(variant=pkg.VARIANT_DECODE))
            afb.device_sync()
        plain = [dc.result()[0] for dc in dcs]
    finally:
        for dc in dcs:
            dc.close()
    for c, a, b in zip(cases, with_flag, plain):
        assert np.array_equal(a, b)
        check_close(oracle, oracle.gemm(c, threads=4), a, f"decode with dependent launch {m}x{n}x{k}")
    assert afb.read_status()[0] == 0
