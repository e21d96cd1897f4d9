"""The C++ host driver (awesome_fusion_b200/driver/bfAintBGemm.cc): builds on CPU; on a GPU its validation mode
(the reference's `bfAintBGemm 1 ...` invocation, bfAintBGemm.cc:38-44,198-214) must print "valid"."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DRV = os.path.join(ROOT, "awesome_fusion_b200", "driver")
BIN = os.path.join(DRV, "bfAintBGemm")


def _build():
    subprocess.check_call(["make", "-C", DRV], stdout=subprocess.DEVNULL)
    assert os.path.exists(BIN)


def test_driver_builds_and_rejects_bad_options():
    _build()
    res = subprocess.run([BIN, "0", "nonsense=1"], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    assert res.returncode == 2 and "unknown option" in res.stdout


@pytest.mark.gpu
@pytest.mark.parametrize("argv,variant", [
    (["1"], "naive"),                                                        # the reference's default problem and data, its [K,N] layout
    (["1", "64", "256", "1024"], "naive"),
    (["1", "256", "1024", "1024", "b_layout=col", "enc=twos", "data=real", "seed=0"], "prefill"),   # the CPU-checkable configuration
    (["1", "256", "1024", "1024", "b_layout=col"], "prefill"),               # reference-style integer data must match to 1e-3
    (["1", "16", "4096", "4096", "b_layout=col", "enc=twos", "data=real"], "decode"),
    (["1", "4", "1024", "2048", "b_layout=col", "bits=4", "group=128", "data=real"], "decode"),
    (["1", "160", "512", "1024", "b_layout=col", "bits=4", "group=128", "data=real", "enc=twos"], "prefill"),
    (["1", "160", "512", "1024", "b_layout=col", "bits=4", "group=128", "data=real", "enc=twos", "exact=1"], "prefill"),   # two-term mode: the 1e-2 contract
    (["1", "256", "1024", "1024", "b_layout=col", "enc=twos", "data=real", "a_dist=uniform", "scale_lo=0.002", "scale_hi=0.02", "seed=0"], "prefill"),
    (["1", "33", "136", "192", "300", "136", "200"], "naive"),               # explicit leading dimensions
    (["1", "256", "1024", "1024", "prepack=1", "data=real", "a_dist=uniform", "scale_lo=0.002", "scale_hi=0.02"], "prefill"),   # the reference's own [K,N] layout, pre-packed
    (["1", "8", "1024", "2048", "prepack=1", "data=real"], "decode"),
    (["1", "16", "512", "1024", "b_layout=col", "bits=4", "group=128", "data=real", "prepack=1"], "decode"),
])
def test_driver_validation_mode(argv, variant):
    _build()
    res = subprocess.run([BIN] + argv, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=600)
    assert res.returncode == 0 and ",valid" in res.stdout, res.stdout[-2000:]
    assert f"variant: {variant}" in res.stdout, res.stdout


@pytest.mark.gpu
@pytest.mark.parametrize("split,m", [("n", 512), ("k", 512), ("k", 96)])
def test_driver_sharded_over_the_gpus_of_the_box(split, m):
    """`gpus=G split=n|k`: the single-process multi-GPU path (afb_dist_*), validated against the host reference."""
    import torch
    count = torch.cuda.device_count()
    if count < 2:
        pytest.skip("needs two GPUs in the box")
    g = 8 if count >= 8 else 4 if count >= 4 else 2
    _build()
    m = m if m < 256 else 256 * g
    res = subprocess.run([BIN, "1", str(m), "1024", str(1024 * g), "b_layout=col", "enc=twos", "data=real", f"gpus={g}", f"split={split}"],
                         stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=600, env=dict(os.environ, NCCL_NVLS_ENABLE="0"))
    assert res.returncode == 0 and ",valid" in res.stdout, res.stdout[-2000:]
    assert f"sharded over {g} GPUs ({split}-split)" in res.stdout


def test_dist_partition_arithmetic_in_the_library():
    """afb_dist_split_range (no GPU needed) agrees with the Python launcher's split_range on every rank."""
    import ctypes
    import awesome_fusion_b200 as pkg
    from awesome_fusion_b200 import dist as D
    lib = pkg.load()
    f = lib.lib.afb_dist_split_range
    f.argtypes = [ctypes.c_uint32] * 4 + [ctypes.POINTER(ctypes.c_uint32)] * 2
    for total, world, mult in [(28672, 8, 64), (8192, 8, 8), (4096, 3, 64), (640, 3, 64), (1024, 1, 128), (24, 5, 8)]:
        for r in range(world):
            lo, hi = ctypes.c_uint32(), ctypes.c_uint32()
            assert f(total, world, r, mult, ctypes.byref(lo), ctypes.byref(hi)) == 0
            assert (lo.value, hi.value) == D.split_range(total, world, r, mult)
    lo, hi = ctypes.c_uint32(), ctypes.c_uint32()
    assert f(100, 4, 0, 64, ctypes.byref(lo), ctypes.byref(hi)) == -1
