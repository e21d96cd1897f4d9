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
])
def test_driver_validation_mode(argv, variant):
    _build()
    res = subprocess.run([BIN] + argv, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=600)
    assert res.returncode == 0 and ",valid" in res.stdout, res.stdout[-2000:]
    assert f"variant: {variant}" in res.stdout, res.stdout
