#!/usr/bin/env python
"""Benchmark of the bfAintBGemm path: bf16 x int GEMM TFLOP/s (and HBM GB/s for the decode cases).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload NAME]

Headline workload ("sharded-mlp", every N): the two 70B-class layers of the sharded configuration,
one step = one column-parallel up-projection (M=4096, N=28672 split over the GPUs, K=8192) followed by
one row-parallel down-projection (M=4096, N=8192, K=28672 split over the GPUs) whose partial sums are
combined across the GPUs.  int8 weights, per-channel fp32 scales, bf16 activations and outputs.
At N=1 both GEMMs run whole on one GPU (strong scaling: total work is fixed as N grows).
At N=1 the same run also measures the single-GPU configurations (decode, prefill, group-wise int4)
and reports them under "cases"; --workload picks one of them as the only thing to run (used for
profiling).  One JSON line is printed by rank 0.

Launch for N>1:  python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1
                 --master-port P bench.py --gpus N --steps K --warmup W
"""
import argparse
import json
import os
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "bf16 x int GEMM throughput (2*M*N*K / time)"
NOMINAL = {"hbm_gbs": 8000.0, "bf16_tflops": 2250.0}
# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the up-projection kernel on one GPU, from an ncu capture of
# that kernel on that shape (a profiler figure cannot be taken inside a timed run): 615.8 MB + 227.4 MB
UP_PROJ_DRAM_BYTES = 615775744 + 227428608
# same for the decode kernel, int8 M=16 at 4096 x 4096
DECODE_M16_DRAM_BYTES = 16964096
PARITY_ROWS = [0, 255, 256, 1000, 2047, 2048, 3583, 4095]   # activation rows of both GEMMs checked against the CPU oracle after the timed region
FALLBACK = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        d["_source"] = "measured"
        return d
    d = dict(FALLBACK)
    d["_source"] = "fallback"
    return d


# ----------------------------------------------------------------------------------------
# algorithmic work (the reference's own formulas, bfAintBGemm.cc:187-188, plus the scale term; units 1e12 / 1e9)
# ----------------------------------------------------------------------------------------
def gemm_flops(m, n, k):
    return 2.0 * m * n * k


def gemm_bytes(m, n, k, bits, group):
    scale_bytes = 2 * n * (k // group) if group else 4 * n
    return 2 * m * k + n * k * bits // 8 + scale_bytes + 2 * m * n


# ----------------------------------------------------------------------------------------
# clocks during the timed region
# ----------------------------------------------------------------------------------------
class ClockSampler:
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.out = open(self.path, "w")
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.gpu), f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-lms", "25"], stdout=self.out, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        res = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return res
        time.sleep(0.15)
        self.proc.terminate()   # the exact process started above
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.out.close()
        sm, mx, reasons = [], [], set()
        for line in open(self.path):
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        os.unlink(self.path)
        if sm:
            sm.sort()
            res.update(sm_mhz=sm[len(sm) // 2], sm_max_mhz=max(mx), reasons=sorted(reasons), samples=len(sm))
        return res


# ----------------------------------------------------------------------------------------
# device-resident problem instances (torch owns the memory; the kernels are ours, through the C ABI)
# ----------------------------------------------------------------------------------------
class Gemm:
    """One GEMM with synthetic inputs of the benchmark distributions, `copies` distinct weight buffers to rotate over.
    packed: the weights go through afb_prepack first (offline step, outside any timed region)."""

    def __init__(self, lib, torch, m, n, k, *, bits=8, group=0, seed=0, copies=1, variant=0, lda=None, c_f32=False, a=None, packed=False, flags=0):
        import awesome_fusion_b200 as pkg
        self.lib, self.m, self.n, self.k, self.bits, self.group = lib, m, n, k, bits, group
        dev = torch.device("cuda", torch.cuda.current_device())
        g = torch.Generator(device=dev); g.manual_seed(seed)
        self.a = a if a is not None else torch.randn((m, k), generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16)
        self.b, self.s, self.args = [], [], []
        self.c = torch.empty((m, n), device=dev, dtype=torch.float32 if c_f32 else torch.bfloat16)
        for _ in range(copies):
            if bits == 8:
                b = torch.randint(-127, 128, (n, k), generator=g, device=dev, dtype=torch.int8)
            else:
                q = torch.randint(-8, 8, (n, k), generator=g, device=dev, dtype=torch.int8)
                b = ((q[:, 0::2] & 0xF) | (q[:, 1::2] << 4)).to(torch.uint8).contiguous()
                del q
            if group:
                s = (torch.rand((n, k // group), generator=g, device=dev) * 0.045 + 0.005).to(torch.bfloat16)
            else:
                s = torch.rand((n,), generator=g, device=dev) * 0.009 + 0.001
            layout = pkg.LAYOUT_COL
            if packed:
                lib.prepack(lib.make_args(self.c, self.a, b, s, m, n, k, bits=bits), b, k)   # in place
                layout = pkg.LAYOUT_COL_PACKED
            self.b.append(b); self.s.append(s)
            self.args.append(lib.make_args(self.c, self.a, b, s, m, n, k, lda=lda or self.a.stride(0), bits=bits, group=group, layout=layout,
                                           scale_dtype=pkg.SCALE_BF16 if group else pkg.SCALE_F32, variant=variant,
                                           flags=flags | (pkg.FLAG_C_F32 if c_f32 else 0)))
        torch.cuda.synchronize()
        self.flops = gemm_flops(m, n, k)
        self.bytes = gemm_bytes(m, n, k, bits, group)
        self.i = 0

    def launch(self, stream):
        self.lib.gemm_launch(self.args[self.i], stream)
        self.i = (self.i + 1) % len(self.args)


def time_launches(torch, fn, steps, warmup):
    """ms per call of fn(), CUDA events on torch's current stream (the stream fn launches on)."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps


def time_decode_graph(lib, torch, op, copies, steps, warmup):
    """A decode launch lasts a few microseconds, less than the host needs to issue it: one CUDA graph holds one launch per
    rotated weight buffer, so that the events time the device and not the launch loop.  Returns ms per launch."""
    stream = torch.cuda.current_stream().cuda_stream
    for _ in range(max(3, warmup)):
        op.launch(stream)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        cs = torch.cuda.current_stream().cuda_stream
        for _ in range(copies):
            op.launch(cs)
    ms = time_launches(torch, graph.replay, steps, warmup) / copies
    del graph
    return ms


def single_case(lib, torch, name, m, n, k, bits, group, peaks, steps, warmup):
    """One single-GPU configuration: kernel-only timing with the weights rotated over more than L2's worth of buffers.
    Decode shapes are timed three ways, all through afb_gemm_launch: the weights as given; the same with AFB_FLAG_PDL (the
    launches of the graph overlap: each kernel streams its weights while its predecessor finishes -- legal because weights are
    constants); and with the weights pre-packed by afb_prepack as well.  The case's own figures are those of the last mode."""
    import awesome_fusion_b200 as pkg
    stream = torch.cuda.current_stream().cuda_stream
    wbytes = n * k * bits // 8
    copies = max(1, min(24, -(-400_000_000 // wbytes)))   # >= 400 MB of distinct weights (L2 is 126 MB)
    op = Gemm(lib, torch, m, n, k, bits=bits, group=group, seed=1, copies=copies)
    variant = {pkg.VARIANT_DECODE: "decode", pkg.VARIANT_PREFILL: "prefill", pkg.VARIANT_NAIVE: "naive"}[lib.resolve_variant(op.args[0])]
    timing = "events around back-to-back launches"
    modes = None
    if variant == "decode" and not os.environ.get("AFB_BENCH_NO_GRAPH"):
        timing = f"CUDA-graph replay, {copies} launches per graph"
        modes = {"weights as given": time_decode_graph(lib, torch, op, copies, steps, warmup) * 1e3}
        for label, packed in (("programmatic dependent launch", False), ("pre-packed weights + programmatic dependent launch", True)):
            del op
            torch.cuda.empty_cache()
            op = Gemm(lib, torch, m, n, k, bits=bits, group=group, seed=1, copies=copies, packed=packed, flags=pkg.FLAG_PDL)
            try:
                modes[label] = time_decode_graph(lib, torch, op, copies, steps, warmup) * 1e3
            except Exception as e:  # noqa: BLE001  (a driver that cannot capture programmatic edges)
                modes[label] = None
                timing += f"; {label}: not captured ({type(e).__name__})"
        best = [v for v in modes.values() if v]
        ms = (modes["pre-packed weights + programmatic dependent launch"] or min(best)) / 1e3
        modes = {k_: (round(v, 2) if v else None) for k_, v in modes.items()}
    else:
        ms = time_launches(torch, lambda: op.launch(stream), steps, warmup)
    tf, gb = op.flops / ms / 1e9, op.bytes / ms / 1e6
    ai = op.flops / op.bytes
    bound = "hbm" if ai < peaks["bf16_tflops"] * 1e3 / peaks["hbm_gbs"] else "tensor"
    res = {"name": name, "variant": variant, "m": m, "n": n, "k": k, "bits": bits, "group": group, "us": round(ms * 1e3, 2),
           "tflops": round(tf, 2), "gbs": round(gb, 1), "bound": bound, "weight_buffers_rotated": copies, "timing": timing,
           "frac_of_measured": round(gb / peaks["hbm_gbs"] if bound == "hbm" else tf / peaks["bf16_tflops"], 4),
           "frac_of_nominal": round(gb / NOMINAL["hbm_gbs"] if bound == "hbm" else tf / NOMINAL["bf16_tflops"], 4)}
    if modes:
        res["us_by_mode"] = modes
    del op
    torch.cuda.empty_cache()
    return res


def decode_floor(lib, torch, steps, warmup):
    """How long a launch of the decode kernel's shape takes when it does nothing, and when it only reads 16.8 MB (the weights of
    the 4096 x 4096 int8 configuration) -- both as back-to-back launches in a CUDA graph over 24 rotated buffers, without and with
    programmatic dependent launch.  These are the floors next to which the 4096 x 4096 decode figures have to be read."""
    import awesome_fusion_b200 as pkg
    n = k = 4096
    copies = 24
    bufs = [torch.randint(-127, 128, (n, k), device="cuda", dtype=torch.int8) for _ in range(copies)]
    out = {}
    for kind, kname in ((0, "empty kernel"), (1, "read-only kernel, 16.8 MB")):
        for ctas, smem in ((256, 52 * 1024), (256, 84 * 1024), (592, 52 * 1024)):
            for flags, fname in ((0, "plain"), (pkg.FLAG_PDL, "programmatic dependent launch")):
                def launch_all(stream):
                    for b in bufs:
                        lib.probe_launch(kind, b, n * k, ctas, smem, flags, stream)
                launch_all(torch.cuda.current_stream().cuda_stream)
                torch.cuda.synchronize()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    launch_all(torch.cuda.current_stream().cuda_stream)
                us = time_launches(torch, g.replay, steps, warmup) / copies * 1e3
                out[f"{kname}, {ctas} CTAs x {smem // 1024} KiB, {fname}"] = round(us, 2)
                del g
    return out


SINGLE_CASES = {
    "decode-m1": (1, 4096, 4096, 8, 0), "decode-m4": (4, 4096, 4096, 8, 0), "decode-m16": (16, 4096, 4096, 8, 0),
    "prefill": (2048, 11008, 4096, 8, 0),
    "int8-m1": (1, 28672, 8192, 8, 0), "int8-m16": (16, 28672, 8192, 8, 0),
    "int4-m1": (1, 28672, 8192, 4, 128), "int4-m16": (16, 28672, 8192, 4, 128), "int4-m128": (128, 28672, 8192, 4, 128),
    "int4-m4096": (4096, 28672, 8192, 4, 128),
    "cpu-checkable": (256, 1024, 1024, 8, 0),
}


# ----------------------------------------------------------------------------------------
# CPU arm: the reference's own gemm_rrr (host_ref.hpp) compiled into oracle/_ref, else the oracle port
# ----------------------------------------------------------------------------------------
class CpuArm:
    """The reference's CPU GEMM (oracle/_ref when it was built from the reference's own headers, else the oracle port) on a bounded
    sample of the headline workload: `rows` rows of C of the up-projection (N=28672, K=8192, all of N and K), one row-range per
    host thread.  The weights are made once; the first run calibrates how many rows fit the time a step may take."""

    def __init__(self):
        import numpy as np
        sys.path.insert(0, os.path.join(ROOT, "tests"))
        import afb_testlib as T
        self.np, self.T = np, T
        self.cores = os.cpu_count() or 1
        self.n, self.k = 28672, 8192
        self.rng = np.random.default_rng(0)
        self.ref = T.load_hostref()
        self.kind = "reference" if self.ref is not None else "port"
        # first guess: about 0.1 GFLOP/s per thread for the reference loop (B is read with stride N), 1.5 for the port
        self.per_thread_gflops = 0.1 if self.ref is not None else 1.5
        if self.ref is not None:
            self.b = self.rng.integers(-127, 128, size=(self.k, self.n), dtype=np.int8).astype(np.float32)
            self.s = self.rng.uniform(0.001, 0.01, self.n).astype(np.float32)
        else:
            self.orc = T.load_oracle()

    def run(self, seconds_target):
        """One sample of about seconds_target seconds.  Returns (tflops, info, seconds)."""
        np, n, k = self.np, self.n, self.k
        rows_per_thread = max(1, int(seconds_target * self.per_thread_gflops * 1e9 / (2.0 * n * k)))
        rows = rows_per_thread * self.cores
        if self.ref is not None:
            a = self.rng.standard_normal((rows, k), dtype=np.float32)
            fn = lambda: self.ref.gemm_rrr(a, self.b, self.s, threads=self.cores)
        else:
            case = self.T.make_case(rows, n, k, seed=0)
            fn = lambda: self.orc.gemm(case, threads=self.cores)
        t0 = time.perf_counter()
        fn()
        dt = time.perf_counter() - t0
        self.per_thread_gflops = 2.0 * rows_per_thread * n * k / dt / 1e9   # the measured rate sizes the next sample
        info = {"kind": self.kind, "cores": self.cores, "seconds": round(dt, 2),
                "sample": f"{rows} of 4096 rows of C of the up-projection (M x 28672 x 8192, int8 per-channel), all N and K, "
                          f"{rows_per_thread} row(s) per host thread; the down-projection has the same FLOPs"}
        return 2.0 * rows * n * k / dt / 1e12, info, dt


def cpu_arm(seconds_target=12.0):
    """One bounded sample for the `cpu_baseline` object of the main line: a short calibration run, then the sample."""
    arm = CpuArm()
    arm.run(1.0)
    return arm.run(seconds_target)


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    steps, warm = max(1, args.steps), max(0, args.warmup)
    # each step is one bounded sample; the whole run (warm-up included) is held to about two minutes of CPU work
    per = max(1.0, min(12.0, 120.0 / (steps + warm)))
    arm = CpuArm()
    arm.run(1.0)   # calibration of the sample size on this host
    for _ in range(warm):
        arm.run(per)
    vals, total = [], 0.0
    info = None
    for _ in range(steps):
        v, info, dt = arm.run(per)
        vals.append(v); total += dt
    v = sum(vals) / len(vals)
    line = {"impl": "reference", "metric": METRIC, "value": v, "unit": "TFLOP/s", "n_gpus": args.gpus, "steps": steps, "warmup": warm,
            "ms_per_step": total / steps * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16xint8->fp32",
            "data": "synthetic", "config": headline_config(args.gpus),
            "cpu_baseline": {"value": v, "unit": "TFLOP/s", "cores": info["cores"], "kind": info["kind"], "sample": info["sample"]},
            "e2e": {"value": v, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, "gpu_launches": 0}
    print(json.dumps(line))
    return 0


def parity_check(mlp, torch, world, rank):
    """After the timed region: PARITY_ROWS of the up-projection (this rank's channels) and of the down-projection (the
    complete sum, as this rank holds it after the exchange) against the CPU oracle on the same inputs.  For the K-split
    GEMM every rank computes the oracle's fp32 partial rows of its own K range and the ranks add them up.
    Returns the worst figures over the ranks.  The oracle is only the checker here: nothing timed runs through it."""
    import numpy as np
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import afb_testlib as T
    oracle = T.load_oracle()
    rows = [r for r in PARITY_ROWS if r < mlp.m]
    threads = max(1, (os.cpu_count() or 1) // max(1, world))

    def to_u16(t):
        return t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)

    def case_of(a, b, s):
        n, k = b.shape
        return T.Case(m=len(rows), n=n, k=k, bits=8, group=0, layout=int(mlp.layout), enc=0, scale_dtype=0, a=to_u16(a[rows]),
                      b=b.cpu().numpy().view(np.uint8), scale=s.cpu().numpy().astype(np.float32), ldb=k)

    worst, worst_nrms = 0.0, 0.0
    # column-parallel up-projection: this rank's channels
    ref = oracle.gemm(case_of(mlp.a_up, mlp.b_up, mlp.s_up), threads=threads)
    mx, nrms, _ = oracle.compare(ref, to_u16(mlp.c_up[rows]), T.rms(ref) * 0.05)
    worst, worst_nrms = max(worst, mx), max(worst_nrms, nrms)
    # row-parallel down-projection: oracle partial sums of this rank's K range, added over the ranks
    part = torch.from_numpy(oracle.gemm(case_of(mlp.a_down, mlp.b_down, mlp.s_down), threads=threads)).cuda()
    if world > 1:
        import torch.distributed as tdist
        tdist.all_reduce(part)
    ref = part.cpu().numpy()
    got = mlp.result_down()[rows].contiguous().view(torch.int16).numpy().view(np.uint16)
    mx, nrms, _ = oracle.compare(ref, got, T.rms(ref) * 0.05)
    worst, worst_nrms = max(worst, mx), max(worst_nrms, nrms)
    t = torch.tensor([worst, worst_nrms], device="cuda", dtype=torch.float64)
    if world > 1:
        tdist.all_reduce(t, op=tdist.ReduceOp.MAX)
    worst, worst_nrms = t[0].item(), t[1].item()
    return {"rows": rows, "gemms": ["up (each rank's channels)", "down (complete sum on every rank)"], "max_rel": worst, "nrms": worst_nrms,
            "tolerance": 1e-2, "floor": "0.05 x RMS(ref)", "checked_on_ranks": world, "ok": bool(worst <= 1e-2)}


def headline_config(n_gpus):
    return {"workload": "sharded-mlp: column-parallel up-proj 4096 x 28672 x 8192 + row-parallel down-proj 4096 x 8192 x 28672, "
                        "int8 weights [N,K], per-channel fp32 scales, bf16 in/out, fp32 accumulate",
            "m": 4096, "up": [28672, 8192], "down": [8192, 28672], "parallelism": f"tp{n_gpus} (N-split up, K-split down)",
            "l2": "inputs larger than L2 (weights 235 MB per GEMM)", "flops_per_step": 2 * gemm_flops(4096, 28672, 8192)}


# ----------------------------------------------------------------------------------------
# our arm
# ----------------------------------------------------------------------------------------
def run_ours(args):
    import torch
    import awesome_fusion_b200 as pkg
    from awesome_fusion_b200 import dist as afb_dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch N>1 with torch.distributed.run (see the docstring)")
    torch.cuda.set_device(local)
    lib = pkg.load()          # raises when libafb.so is missing: no fallback
    lib.init(local)
    peaks = measured_peaks()
    stream = torch.cuda.current_stream().cuda_stream
    steps, warm = args.steps, max(3, args.warmup)

    if args.workload == "decode-floor":
        print(json.dumps({"workload": "decode-floor", "us_per_launch": decode_floor(lib, torch, steps, warm), "status": lib.read_status()}))
        return 0
    if args.workload != "sharded-mlp":
        m, n, k, bits, group = SINGLE_CASES[args.workload]
        res = single_case(lib, torch, args.workload, m, n, k, bits, group, peaks, steps, warm)
        print(json.dumps({"workload": args.workload, **res, "status": lib.read_status()}))
        return 0

    if world > 1:
        import torch.distributed as tdist
        tdist.init_process_group("nccl", device_id=torch.device("cuda", local))
    mlp = afb_dist.ShardedMLP(lib, torch, rank=rank, world=world, exchange=args.exchange)

    def barrier():
        if world > 1:
            tdist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local)

    def timed_run(sample_clocks):
        """warm-up, then `steps` steps between events; returns (ms per step, up ms, down ms, launches), max over the ranks"""
        for _ in range(warm):
            mlp.step(stream)
        barrier()
        launches0 = lib.launch_count()
        if sample_clocks and rank == 0:
            sampler.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        kev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
        e0.record()
        for i in range(steps):
            mlp.step(stream, events=kev[i])
        e1.record()
        barrier()
        clk = sampler.stop() if (sample_clocks and rank == 0) else None
        t = torch.tensor([e0.elapsed_time(e1) / steps, sum(a.elapsed_time(b) for a, b, _ in kev) / steps,
                          sum(b.elapsed_time(c) for _, b, c in kev) / steps, float(lib.launch_count() - launches0)], device="cuda", dtype=torch.float64)
        if world > 1:
            tmax = t.clone(); tdist.all_reduce(tmax, op=tdist.ReduceOp.MAX)
            tsum = t.clone(); tdist.all_reduce(tsum, op=tdist.ReduceOp.SUM)
            return tmax[0].item(), tmax[1].item(), tmax[2].item(), int(tsum[3].item()), clk
        return t[0].item(), t[1].item(), t[2].item(), int(t[3].item()), clk

    ms, up_ms, down_ms, launches, clocks = timed_run(True)      # down_ms includes the exchange at N > 1
    status = lib.read_status()
    total_flops = mlp.flops_per_step_global
    value = total_flops / ms / 1e9

    # e2e: the same step through the host-pointer entry point (pinned host inputs, H2D and D2H inside the timed region)
    e2e = mlp.e2e(steps=min(steps, 10), warmup=2)
    if world > 1:
        t2 = torch.tensor([e2e["ms"]], device="cuda", dtype=torch.float64)
        tdist.all_reduce(t2, op=tdist.ReduceOp.MAX)
        e2e["ms"] = t2.item()
    e2e_obj = {"value": total_flops / e2e["ms"] / 1e9, "unit": "TFLOP/s", "h2d_bytes_per_step": e2e["h2d"] * world,
               "d2h_bytes_per_step": e2e["d2h"] * world, "ms_per_step": e2e["ms"], "api": e2e["api"]}

    phases = None
    if world > 1 and os.environ.get("AFB_PHASE_TIMESTAMPS"):
        # last step's device-side stamps (ns of each GPU's own timer; only differences on one GPU mean anything)
        ts = lib.phase_timestamps()
        mine = {"gemm_us": (ts[1] - ts[0]) / 1e3, "gemm_end_to_exchange_start_us": (ts[2] - ts[1]) / 1e3, "wait_for_all_gemms_us": (ts[3] - ts[2]) / 1e3,
                "sum_and_broadcast_us": (ts[4] - ts[3]) / 1e3, "wait_for_all_blocks_us": (ts[5] - ts[4]) / 1e3, "total_us": (ts[5] - ts[0]) / 1e3} if ts[0] and ts[5] else None
        phases = [None] * world
        tdist.all_gather_object(phases, mine)
    parity = parity_check(mlp, torch, world, rank)
    # the same step on pre-packed weights (afb_prepack is an offline step: not inside any timed region), with its own parity check
    mlp.prepack_weights()
    pk_ms, pk_up_ms, pk_down_ms, _, _ = timed_run(False)
    pk_parity = parity_check(mlp, torch, world, rank)
    parity["prepacked_run"] = {"max_rel": pk_parity["max_rel"], "nrms": pk_parity["nrms"], "ok": pk_parity["ok"]}
    parity["ok"] = bool(parity["ok"] and pk_parity["ok"])
    shutdown(mlp, world, torch)
    if rank != 0:
        return 0 if parity["ok"] else 1
    # roofline of the dominant kernel (the prefill kernel of the up-projection: no exchange inside its events)
    up_flops = gemm_flops(mlp.m, mlp.up_n_local, mlp.up_k)
    achieved = up_flops / up_ms / 1e9
    roofline = {"kernel": "prefill_ts_kernel<8,false,256> (up-projection shard)", "bound": "tensor", "achieved": achieved,
                "peak": peaks["bf16_tflops"], "unit": "TFLOP/s", "frac": achieved / peaks["bf16_tflops"],
                "peak_source": f"{peaks['_source']} cuBLAS bf16 burst", "frac_of_sustained": achieved / peaks.get("bf16_tflops_sustained", peaks["bf16_tflops"]),
                "frac_of_nominal": achieved / NOMINAL["bf16_tflops"], "avg_launch_ms": up_ms,
                "traffic": UP_PROJ_DRAM_BYTES if world == 1 else None, "traffic_source": "ncu capture of this kernel on this shape" if world == 1 else None,
                "algorithmic_bytes": gemm_bytes(mlp.m, mlp.up_n_local, mlp.up_k, 8, 0)}
    line = {"metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": steps, "warmup": warm, "ms_per_step": ms,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16xint8->fp32", "data": "synthetic",
            "config": headline_config(world), "exchange": mlp.exchange_name, "clocks": clocks, "e2e": e2e_obj, "gpu_launches": launches,
            "roofline": roofline, "per_gemm_ms": {"up": up_ms, "down_incl_exchange": down_ms}, "device_status": status, "parity": parity,
            "prepacked_weights": {"value": total_flops / pk_ms / 1e9, "unit": "TFLOP/s", "ms_per_step": pk_ms,
                                  "per_gemm_ms": {"up": pk_up_ms, "down_incl_exchange": pk_down_ms},
                                  "note": "same step after afb_prepack (offline re-ordering of the same integers); `value` is measured on the weights as given"}}
    if phases:
        line["down_projection_phases_per_rank"] = phases
    if world == 1:
        cases = []
        if not args.no_cases:
            for name in ("decode-m1", "decode-m4", "decode-m16", "int8-m1", "int8-m16", "prefill", "int4-m1", "int4-m16", "int4-m128", "int4-m4096"):
                m, n, k, bits, group = SINGLE_CASES[name]
                cases.append(single_case(lib, torch, name, m, n, k, bits, group, peaks, 50 if m <= 128 else 10, 5))
            line["cases"] = cases
            d16 = next(c for c in cases if c["name"] == "decode-m16")
            line["roofline_decode"] = {"kernel": "decode_kernel<8,2,false>", "bound": "hbm", "achieved": d16["gbs"], "peak": peaks["hbm_gbs"],
                                       "unit": "GB/s", "frac": d16["gbs"] / peaks["hbm_gbs"], "peak_source": f"{peaks['_source']} copy bandwidth",
                                       "traffic": DECODE_M16_DRAM_BYTES, "traffic_source": "ncu capture of this kernel on this shape"}
        if not args.no_cpu:
            v, info, _ = cpu_arm()
            line["cpu_baseline"] = {"value": v, "unit": "TFLOP/s", "cores": info["cores"], "kind": info["kind"], "sample": info["sample"]}
    print(json.dumps(line))
    return 0 if parity["ok"] and status[0] == 0 else 1


def shutdown(mlp, world, torch):
    """Orderly end of a multi-process run: all exchanges done, peer mappings released, then the process group."""
    if world == 1:
        return
    import torch.distributed as tdist
    tdist.barrier()
    torch.cuda.synchronize()
    mlp.close()
    tdist.barrier()
    tdist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="sharded-mlp", choices=["sharded-mlp", "decode-floor"] + sorted(SINGLE_CASES))
    ap.add_argument("--exchange", default="auto", choices=["auto", "push", "pipelined", "inkernel", "overlap", "fused", "nccl"])
    ap.add_argument("--no-cases", action="store_true", help="skip the single-GPU case sweep")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference_arm(args)
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
