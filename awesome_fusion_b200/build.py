"""In-tree build of libafb.so with nvcc for sm_100a (works without a GPU: nvcc cross-compiles)."""
import os
import subprocess

_HERE = os.path.dirname(os.path.abspath(__file__))


def build_library(verbose: bool = False, ptxas_verbose: bool = False) -> str:
    """Runs ``make`` in ``csrc/`` and returns the path of the built ``libafb.so``."""
    cmd = ["make", "-C", os.path.join(_HERE, "csrc"), "-j8"]
    if ptxas_verbose:
        cmd.append("PTXAS_V=-Xptxas -v")
    res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if verbose or res.returncode != 0:
        print(res.stdout)
    if res.returncode != 0:
        raise RuntimeError("building libafb.so failed (see output above)")
    out = os.path.join(_HERE, "libafb.so")
    if not os.path.exists(out):
        raise RuntimeError("make succeeded but libafb.so is missing")
    return out
