"""The allocation-free decode entry point, afb_gemm_launch_static.

It exists for host programs that cannot allocate device memory when they call the library: the framework
around them has already taken the whole GPU for its pool, or they sit in a serving loop where the implicit
device synchronisation of cudaMalloc would stall every stream.  The entry point keeps its split-K scratch in a
fixed array inside libafb.so, so this test checks what such a caller relies on: the result equals that of the
regular entry point (same tolerance as the other parity tests), on two calls in a row (the second call sees the
scratch exactly as the first one left it), and oversized problems are refused rather than overrun the array.
Collected last on purpose: a run that stops at the first failure has then already run every other test."""
import numpy as np
import pytest

import afb_testlib as T
import awesome_fusion_b200 as pkg

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("m,n,k,bits,group", [(16, 4096, 4096, 8, 0), (4, 2048, 8192, 4, 128)])
def test_static_scratch_entry_matches_regular_entry(m, n, k, bits, group):
    lib = pkg.load()
    oracle = T.load_oracle()
    case = T.make_case(m, n, k, bits=bits, group=group, seed=17, scale_range=(0.005, 0.05))
    # the new entry point first, twice in a row, before the regular path (afb_init) has been touched by this test
    dc = T.DeviceCase(lib, case)
    try:
        outs = []
        for _ in range(2):
            lib.memset(dc.d_c, 0xCD, dc.c_bytes)
            assert lib.gemm_launch_static_status(dc.args()) == 0
            lib.device_sync()
            outs.append(dc.result()[0])
        lib.init(0)
        lib.memset(dc.d_c, 0xCD, dc.c_bytes)
        lib.gemm_launch(dc.args(variant=pkg.VARIANT_DECODE))
        lib.device_sync()
        regular = dc.result()[0]
    finally:
        dc.close()
    assert np.array_equal(outs[0], outs[1]), "second call differs from the first: stale scratch"
    ref = T.np_bf16_to_f32(regular)
    floor = T.rms(ref) * 0.05
    for got in outs:
        mx, _, worst = oracle.compare(ref, got, floor)
        assert mx <= 1e-2, f"static entry differs from the regular entry: {mx} at {worst}"
    # and both agree with the CPU oracle
    o = oracle.gemm(case, threads=8)
    mx, _, _ = oracle.compare(o, outs[0], T.rms(o) * 0.05)
    assert mx <= 1e-2


@pytest.mark.parametrize("env", [{"AFB_DECODE_SLICES": "2", "AFB_DECODE_WR": "8"}, {"AFB_DECODE_SLICES": "4", "AFB_DECODE_WR": "8"},
                                 {"AFB_DECODE_BALANCED": "1"}])
def test_static_scratch_at_the_capacity_edge_and_free_memory_unchanged(monkeypatch, env):
    """M * N = 524288 is the largest problem the fixed array takes: exactly two K-slices of fp32 partial sums fit.  The
    launch shape is forced to use them (two slices: fits; four slices and the balanced form with more than two sharing
    CTAs: do not fit, and the launcher must fall back to a shape that does, not overrun the array).  Around the later
    calls the device's free memory must not move: that is the property the entry point is named for."""
    import torch
    lib = pkg.load()
    m, n, k = 16, 32768, 1024
    case = T.make_case(m, n, k, seed=23)
    dc = T.DeviceCase(lib, case, guard=4096)
    try:
        for name, val in env.items():
            monkeypatch.setenv(name, val)
        lib.memset(dc.d_c_base, 0xCD, dc.c_bytes + 2 * 4096)
        assert lib.gemm_launch_static_status(dc.args()) == 0          # set-up call for this process, if none came before
        lib.device_sync()
        first, raw = dc.result()
        free_before = torch.cuda.mem_get_info(0)[0]
        assert lib.gemm_launch_static_status(dc.args()) == 0
        lib.device_sync()
        free_after = torch.cuda.mem_get_info(0)[0]
        second, raw = dc.result()
        for name in env:
            monkeypatch.delenv(name)
        lib.init(0)
        lib.gemm_launch(dc.args(variant=pkg.VARIANT_DECODE))
        lib.device_sync()
        regular = dc.result()[0]
    finally:
        dc.close()
    assert free_after == free_before, f"free device memory moved by {free_before - free_after} bytes across a call"
    assert np.array_equal(first, second)
    assert np.all(raw[:4096] == 0xCD) and np.all(raw[-4096:] == 0xCD)
    ref = T.np_bf16_to_f32(regular)
    mx, _, worst = T.load_oracle().compare(ref, first, T.rms(ref) * 0.05)
    assert mx <= 1e-2, f"static entry differs from the regular entry: {mx} at {worst}"


def test_static_scratch_entry_refuses_what_does_not_fit():
    lib = pkg.load()
    # 16 x 40960 outputs exceed the 524288-output capacity; prefill-sized M has no static variant
    a = lib.make_args(0x1000, 0x1000, 0x1000, 0x1000, 16, 40960, 4096)
    assert lib.gemm_launch_static_status(a) == -6
    a = lib.make_args(0x1000, 0x1000, 0x1000, 0x1000, 64, 1024, 4096)
    assert lib.gemm_launch_static_status(a) == -2
    a = lib.make_args(0x1000, 0, 0x1000, 0x1000, 4, 1024, 4096)
    assert lib.gemm_launch_static_status(a) == -1
