"""Multi-process tests of the sharded path.  CPU: two gloo ranks exercise the partition arithmetic against the
oracle.  GPU (needs >= 2 GPUs in the box): two nccl ranks run the CUDA kernels and the peer-memory exchange."""
import os
import socket
import subprocess
import sys

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))


def _free_port():
    s = socket.socket(); s.bind(("127.0.0.1", 0)); p = s.getsockname()[1]; s.close()
    return p


def _launch(mode, world, timeout):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
           "--master-port", str(_free_port()), os.path.join(HERE, "dist_worker.py"), mode]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", OMP_NUM_THREADS="2")
    return subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=timeout, env=env)


def test_partition_functions():
    from awesome_fusion_b200 import dist as D
    for total, world, mult in [(28672, 8, 64), (8192, 8, 8), (4096, 3, 64), (1024, 1, 128)]:
        rngs = [D.split_range(total, world, r, mult) for r in range(world)]
        assert rngs[0][0] == 0 and rngs[-1][1] == total
        assert all(a[1] == b[0] for a, b in zip(rngs, rngs[1:]))
        assert all((hi - lo) % mult == 0 for lo, hi in rngs)
        assert max(hi - lo for lo, hi in rngs) - min(hi - lo for lo, hi in rngs) <= mult
    with pytest.raises(ValueError):
        D.split_range(100, 4, 0, 64)
    assert D.k_shard(8192, 2, 1, bits=4, group=128) == (4096, 8192)


def test_sharding_on_two_cpu_ranks():
    res = _launch("cpu", 2, 300)
    assert res.returncode == 0 and "DIST-OK cpu" in res.stdout, res.stdout[-3000:]


@pytest.mark.gpu
def test_sharding_on_two_gpus():
    """All the GPUs of the box (2, 4 or 8): at 8 the default exchange path differs (forwarding warps, rotated push order,
    multicast broadcast), so the widest world the box offers is the one to check."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs in the box")
    count = torch.cuda.device_count()
    world = 8 if count >= 8 else 4 if count >= 4 else 2
    res = _launch("gpu", world, 900)
    assert res.returncode == 0 and "DIST-OK gpu" in res.stdout, res.stdout[-4000:]
    print("\n".join(l for l in res.stdout.splitlines() if "max rel err" in l))


def test_push_staging_layout_matches_exchange_addressing():
    """The GEMM epilogue of rank s stores row i of its partial sum into rank o's staging buffer float[world][m/world][n] at
    slot s, row i - o*m/world (o = i // (m/world)); the exchange kernel on rank o reads partial[q] + i*n for its rows i.
    With the offsets of push_slot_offset both must address the same element."""
    import numpy as np
    from awesome_fusion_b200 import dist as D
    world, m, n = 4, 16, 8
    rows = m // world
    rng = np.random.default_rng(5)
    partials = [rng.standard_normal((m, n)).astype(np.float32) for _ in range(world)]
    stage = [np.zeros(world * rows * n, dtype=np.float32) for _ in range(world)]
    for s_rank in range(world):          # what afb_gemm_launch_push does, element by element
        for i in range(m):
            o = i // rows
            stage[o][(s_rank * rows + (i - o * rows)) * n:(s_rank * rows + (i - o * rows)) * n + n] = partials[s_rank][i]
    for o in range(world):               # what afb_ksplit_allreduce_launch reads with the offsets of allreduce_pushed()
        for i in range(o * rows, (o + 1) * rows):
            acc = np.zeros(n, dtype=np.float32)
            for q in range(world):
                off = D.push_slot_offset(q, o, world, m, n)
                assert off % 4 == 0
                first = off // 4 + i * n
                assert 0 <= first and first + n <= stage[o].size
                acc += stage[o][first:first + n]
            want = np.zeros(n, dtype=np.float32)
            for q in range(world):
                want += partials[q][i]
            assert np.array_equal(acc, want)


def test_struct_layouts_match_the_library():
    """The ctypes mirrors of the four argument blocks have the sizes the library was compiled with (no GPU needed)."""
    import ctypes
    import awesome_fusion_b200 as pkg
    from awesome_fusion_b200 import dist as D
    lib = pkg.load()
    sizes = (ctypes.c_uint32 * 4)()
    assert lib.lib.afb_abi_sizes(sizes) == 0
    assert list(sizes) == [ctypes.sizeof(pkg.GemmArgs), ctypes.sizeof(D.AllReduceArgs), ctypes.sizeof(D.TileAllReduceArgs), ctypes.sizeof(pkg.FusedArgs)]
