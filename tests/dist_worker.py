"""Rank program of the multi-process tests (launched by torch.distributed.run).

mode cpu: gloo ranks on CPU.  Every rank computes its shard of the column-parallel and row-parallel GEMMs
          with the CPU oracle, using the partition functions of awesome_fusion_b200.dist; shards are combined
          with gloo collectives and compared with the unsplit oracle.  No GPU, no CUDA library calls.
mode gpu: nccl ranks, one per GPU.  The same check with the CUDA kernels: N-split shards must concatenate to the
          single-GPU result bit for bit, and the K-split exchange (fused peer-memory kernel and the NCCL path)
          must match the oracle within tolerance, bit-identically on every rank, over several steps.
Prints "DIST-OK <mode>" on rank 0 when everything held.
"""
import os
import sys

import numpy as np
import torch
import torch.distributed as tdist

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
sys.path.insert(0, os.path.dirname(HERE))
import afb_testlib as T  # noqa: E402
from awesome_fusion_b200 import dist as D  # noqa: E402


def sub_case(case, n_rng=None, k_rng=None):
    d = dict(case.__dict__)
    if n_rng:
        lo, hi = n_rng
        d.update(n=hi - lo, b=np.ascontiguousarray(case.b[lo:hi]), scale=np.ascontiguousarray(case.scale[lo:hi]), q=case.q[lo:hi])
    if k_rng:
        lo, hi = k_rng
        d.update(k=hi - lo, a=np.ascontiguousarray(case.a[:, lo:hi]), b=np.ascontiguousarray(case.b[:, lo:hi]), q=case.q[:, lo:hi], ldb=hi - lo)
    return T.Case(**d)


def main():
    mode = sys.argv[1]
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    oracle = T.load_oracle()
    case = T.make_case(96, 512, 1024, seed=21)            # identical on every rank (same seed)
    ref = oracle.gemm(case, threads=2)
    if mode == "cpu":
        tdist.init_process_group("gloo")
        # column-parallel: shards concatenate exactly
        n_lo, n_hi = D.column_shard(case.n, world, rank)
        part = torch.from_numpy(oracle.gemm(sub_case(case, n_rng=(n_lo, n_hi))))
        sizes = [D.column_shard(case.n, world, r) for r in range(world)]
        assert sizes[0][0] == 0 and sizes[-1][1] == case.n and all(sizes[i][1] == sizes[i + 1][0] for i in range(world - 1))
        parts = [torch.empty((case.m, hi - lo)) for lo, hi in sizes]
        tdist.all_gather(parts, part)
        assert np.array_equal(torch.cat(parts, dim=1).numpy().view(np.uint32), ref.view(np.uint32)), "N-split concat != unsplit"
        # row-parallel: partial sums add up to the unsplit result (fp32 order differs: tolerance, not bits)
        k_lo, k_hi = D.k_shard(case.k, world, rank)
        ks = [D.k_shard(case.k, world, r) for r in range(world)]
        assert ks[0][0] == 0 and ks[-1][1] == case.k and all((hi - lo) % 64 == 0 for lo, hi in ks)
        partial = torch.from_numpy(oracle.gemm(sub_case(case, k_rng=(k_lo, k_hi))))
        tdist.all_reduce(partial)
        err = np.abs(partial.numpy() - ref).max() / T.rms(ref)
        assert err < 1e-5, err
        # ragged splits keep whole units
        assert D.split_range(28672, 8, 3, 64) == (3 * 3584, 4 * 3584)
        assert [D.split_range(640, 3, r, 64) for r in range(3)] == [(0, 256), (256, 448), (448, 640)]
        tdist.barrier()
        if rank == 0:
            print("DIST-OK cpu")
        return

    # ---- gpu ----
    import awesome_fusion_b200 as pkg
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    tdist.init_process_group("nccl", device_id=torch.device("cuda", local))
    lib = pkg.load(); lib.init(local)
    stream = torch.cuda.current_stream().cuda_stream
    m, n, k = 256, 1024, 4096
    case = T.make_case(m, n, k, seed=33)
    ref = oracle.gemm(case, threads=4)
    # column-parallel shards vs the single-GPU run of the same kernels
    whole, _ = T.run_case(lib, case)
    n_lo, n_hi = D.column_shard(n, world, rank)
    mine, _ = T.run_case(lib, sub_case(case, n_rng=(n_lo, n_hi)))
    assert np.array_equal(mine, whole[:, n_lo:n_hi]), "column shard differs from the unsplit run"
    # row-parallel: fused and NCCL exchanges
    k_lo, k_hi = D.k_shard(k, world, rank)
    shard = sub_case(case, k_rng=(k_lo, k_hi))
    d_a, d_b, d_s = lib.to_device(shard.a), lib.to_device(shard.b), lib.to_device(shard.scale)
    first_f32 = None
    for partial, multicast in (("f32", True), ("f32", False), ("bf16", True)):
        # multicast=True: C in symmetric memory, result rows broadcast by multimem.st where the box offers it (else plain stores)
        px = D.PeerExchange(lib, tdist, rank, world, m, n, partial_f32=(partial == "f32"), multicast=multicast)
        assert multicast or px.c_multicast is None
        assert px.ok, getattr(px, "error", "peer exchange setup failed")
        args = lib.make_args(px.partial, d_a, d_b, d_s, m, n, shard.k, flags=pkg.FLAG_C_F32 if partial == "f32" else 0)
        outs = []
        for step in range(3):
            lib.memset(px.c, 0, m * n * 2)
            tdist.barrier(); torch.cuda.synchronize()
            lib.gemm_launch(args, stream)
            px.allreduce(stream)
            torch.cuda.synchronize()
            outs.append(lib.to_host(px.c, (m, n), np.uint16))
        st = lib.read_status()
        assert st[0] == 0, f"device status {st}"
        assert all(np.array_equal(outs[0], o) for o in outs[1:]), "fused exchange is not repeatable"
        # fp32 partial sums: the usual bound.  bf16 partial sums are each rounded to 2^-9 of their OWN magnitude, which can
        # exceed the magnitude of the total where the partial sums cancel: bounded against max(|ref|, RMS) instead.
        mx, nrms, _ = oracle.compare(ref, outs[0], T.rms(ref) * (0.05 if partial == "f32" else 1.0))
        # the optional bf16 exchange trades accuracy for half the NVLink bytes: measured 1.5e-2 of max(|ref|, RMS), NRMS 1.7e-3
        assert mx <= (1e-2 if partial == "f32" else 2e-2) and nrms < 3e-3, f"fused {partial}: max rel err {mx}, nrms {nrms}"
        # every rank holds the same bits
        t = torch.from_numpy(outs[0].astype(np.int32)).cuda()
        lo, hi = t.clone(), t.clone()
        tdist.all_reduce(lo, op=tdist.ReduceOp.MIN); tdist.all_reduce(hi, op=tdist.ReduceOp.MAX)
        assert torch.equal(lo, hi), "ranks disagree on the all-reduced result"
        if partial == "f32":
            if first_f32 is None:
                first_f32 = outs[0]
            assert np.array_equal(first_f32, outs[0]), "multicast and plain broadcast disagree"
        if rank == 0:
            print(f"fused {partial} (multicast address: {'yes' if px.c_multicast else 'no'}): max rel err {mx:.3e} nrms {nrms:.3e}", flush=True)
        px.close()
    # tile-granular form: GEMM publishing tiles + exchange kernel on a second stream (needs M > 128: same shape, M = 256)
    px = D.PeerExchange(lib, tdist, rank, world, m, n, partial_f32=True)
    assert px.ok
    args = lib.make_args(px.partial, d_a, d_b, d_s, m, n, shard.k, flags=pkg.FLAG_C_F32)
    side = torch.cuda.Stream()
    outs = []
    for step in range(3):
        lib.memset(px.c, 0, m * n * 2)
        tdist.barrier(); torch.cuda.synchronize()
        if step == 2:
            # the exchange kernel may also reach the GPU FIRST (here: launched on an idle GPU, the GEMM follows): it must
            # let the GEMM in beside it and then see its tiles
            with torch.cuda.stream(side):
                px.allreduce_tiles(side.cuda_stream)
            px.gemm_publishing_tiles(args, stream)
        else:
            px.gemm_publishing_tiles(args, stream)
            with torch.cuda.stream(side):
                px.allreduce_tiles(side.cuda_stream)
        torch.cuda.synchronize()
        outs.append(lib.to_host(px.c, (m, n), np.uint16))
    st = lib.read_status()
    assert st[0] == 0, f"device status {st}"
    assert all(np.array_equal(outs[0], o) for o in outs[1:]), "tile-granular exchange is not repeatable"
    mx, nrms, _ = oracle.compare(ref, outs[0], T.rms(ref) * 0.05)
    assert mx <= 1e-2, f"tile-granular exchange: max rel err {mx}"
    if rank == 0:
        print(f"tile-granular: max rel err {mx:.3e} nrms {nrms:.3e}", flush=True)
    px.close()
    # reduce-scatter in the GEMM epilogue (peer stores) + local sum and broadcast: the same bits as GEMM + fused exchange
    mp = 256 * world
    case_p = T.make_case(mp, n, k, seed=34)
    ref_p = oracle.gemm(case_p, threads=4)
    shard_p = sub_case(case_p, k_rng=(k_lo, k_hi))
    p_a, p_b, p_s = lib.to_device(shard_p.a), lib.to_device(shard_p.b), lib.to_device(shard_p.scale)
    px = D.PeerExchange(lib, tdist, rank, world, mp, n, partial_f32=True)
    assert px.ok and px.push_supported()
    args = lib.make_args(px.partial, p_a, p_b, p_s, mp, n, shard_p.k, flags=pkg.FLAG_C_F32)
    scratch = lib.malloc(mp * n * 4)   # forward mode: the epilogue stores here, two extra warps per CTA copy the tiles out
    args_fwd = lib.make_args(scratch, p_a, p_b, p_s, mp, n, shard_p.k, flags=pkg.FLAG_C_F32 | pkg.FLAG_PUSH_VIA_LOCAL)
    outs = []
    for step in range(6):
        lib.memset(px.c, 0, mp * n * 2)
        tdist.barrier(); torch.cuda.synchronize()
        if step == 0:
            lib.gemm_launch(args, stream)
            px.allreduce(stream)
        else:
            px.gemm_pushing(args if step < 4 else args_fwd, stream)
            px.allreduce_pushed(stream)
        torch.cuda.synchronize()
        outs.append(lib.to_host(px.c, (mp, n), np.uint16))
    st = lib.read_status()
    assert st[0] == 0, f"device status {st}"
    assert all(np.array_equal(outs[0], o) for o in outs[1:]), "epilogue reduce-scatter differs from GEMM + fused exchange"
    mx, nrms, _ = oracle.compare(ref_p, outs[1], T.rms(ref_p) * 0.05)
    assert mx <= 1e-2, f"epilogue reduce-scatter: max rel err {mx}"
    if rank == 0:
        print(f"push: max rel err {mx:.3e} nrms {nrms:.3e}", flush=True)
    px.close()
    for p in (p_a, p_b, p_s, scratch):
        lib.free(p)
    # pipelined form: the pushing GEMM in column-chunk order + the chunk-by-chunk local sum and broadcast on a second stream;
    # identical bits to GEMM + fused exchange, with and without the multicast broadcast, also when the exchange kernel is launched first
    for multicast in (True, False):
        px = D.PeerExchange(lib, tdist, rank, world, mp, n, partial_f32=True, multicast=multicast)
        assert px.ok and px.pipelined_supported(4)
        p_a, p_b, p_s = lib.to_device(shard_p.a), lib.to_device(shard_p.b), lib.to_device(shard_p.scale)
        args = lib.make_args(px.partial, p_a, p_b, p_s, mp, n, shard_p.k, flags=pkg.FLAG_C_F32)
        side = torch.cuda.Stream()
        outs_p = []
        for step in range(4):
            lib.memset(px.c, 0, mp * n * 2)
            tdist.barrier(); torch.cuda.synchronize()
            if step == 3:
                with torch.cuda.stream(side):
                    px.sub_launches = getattr(px, "sub_launches", 0) + 1      # the exchange kernel reaches the GPU first: it waits for counts the GEMM has yet to make
                    px.allreduce_pipelined(4, side.cuda_stream)
                    px.sub_launches -= 1
                px.gemm_pushing_pipelined(args, 4, stream)
            else:
                px.gemm_pushing_pipelined(args, 4, stream)
                with torch.cuda.stream(side):
                    px.allreduce_pipelined(4, side.cuda_stream)
            torch.cuda.synchronize()
            outs_p.append(lib.to_host(px.c, (mp, n), np.uint16))
        st = lib.read_status()
        assert st[0] == 0, f"device status {st}"
        assert all(np.array_equal(outs[0], o) for o in outs_p), "pipelined exchange differs from GEMM + fused exchange"
        if rank == 0:
            print(f"pipelined (multicast address: {'yes' if px.c_multicast else 'no'}): bit-identical to the fused exchange", flush=True)
        # the same in ONE launch: the sum and broadcast done by two extra warps of every GEMM CTA
        outs_x = []
        for step in range(3):
            lib.memset(px.c, 0, mp * n * 2)
            tdist.barrier(); torch.cuda.synchronize()
            px.gemm_pushing_exchange(args, 4, stream)
            torch.cuda.synchronize()
            outs_x.append(lib.to_host(px.c, (mp, n), np.uint16))
        st = lib.read_status()
        assert st[0] == 0, f"device status {st}"
        assert all(np.array_equal(outs[0], o) for o in outs_x), "in-kernel exchange differs from GEMM + fused exchange"
        if rank == 0:
            print(f"in-kernel exchange (multicast address: {'yes' if px.c_multicast else 'no'}): bit-identical to the fused exchange", flush=True)
        px.close()
        for p in (p_a, p_b, p_s):
            lib.free(p)
    # NCCL comparison path
    p32 = torch.empty((m, n), device="cuda", dtype=torch.float32)
    c16 = torch.empty((m, n), device="cuda", dtype=torch.bfloat16)
    args = lib.make_args(p32, d_a, d_b, d_s, m, n, shard.k, flags=pkg.FLAG_C_F32)
    lib.gemm_launch(args, stream)
    tdist.all_reduce(p32)
    D.cast_f32_to_bf16(lib, c16.data_ptr(), p32.data_ptr(), m, n, stream)
    torch.cuda.synchronize()
    got = c16.view(torch.int16).cpu().numpy().view(np.uint16)
    mx, _, _ = oracle.compare(ref, got, T.rms(ref) * 0.05)
    assert mx <= 1e-2, f"nccl path: {mx}"
    for p in (d_a, d_b, d_s):
        lib.free(p)
    # the benchmark's own step object with its default exchange for this world size (at 8 ranks: forwarding warps, rotated
    # push order, multicast broadcast), on a reduced shape, checked by the benchmark's own parity routine
    import bench
    mlp = D.ShardedMLP(lib, torch, rank=rank, world=world, exchange="auto", m=256 * world, up=(256 * world, 1024), down=(1024, 512 * world), seed=5)
    for _ in range(3):
        mlp.step(stream)
    torch.cuda.synchronize()
    par = bench.parity_check(mlp, torch, world, rank)
    st = lib.read_status()
    assert st[0] == 0, f"device status {st}"
    assert par["ok"], par
    if rank == 0:
        print(f"sharded step ({mlp.exchange_name}): max rel err {par['max_rel']:.3e} nrms {par['nrms']:.3e}", flush=True)
    tdist.barrier(); torch.cuda.synchronize()
    mlp.close()
    tdist.barrier()
    if rank == 0:
        print("DIST-OK gpu")
    tdist.destroy_process_group()


if __name__ == "__main__":
    main()
