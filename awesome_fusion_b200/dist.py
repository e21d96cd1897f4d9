"""Sharding of the GEMM across the GPUs of one box: one process per GPU (torch.distributed for the
rendezvous and, on the comparison path, NCCL).

* column-parallel (N-split): rank r owns B[r*N/p:(r+1)*N/p, :], the matching scales and C[:, same];
  A is replicated.  Independent units, no collective.
* row-parallel (K-split): rank r owns A[:, K_r] and B[:, K_r]; per-channel scales do not depend on k,
  so every rank applies them to its own partial sum, and the partial sums are added across ranks:
    - "fused": afb_ksplit_allreduce_launch, one kernel per GPU over NVLink peer memory (buffers shared
      between the processes with CUDA IPC handles);
    - "nccl":  fp32 partial sums, torch.distributed.all_reduce, then afb_cast_f32_to_bf16.

The partition arithmetic (`split_range`, `column_shard`, `k_shard`) is plain Python so that it can be
tested on CPU ranks.
"""
import ctypes
import os

MAX_RANKS = 8


def split_range(total, world, rank, multiple=1):
    """[lo, hi) of `total` owned by `rank`: equal shares of whole `multiple`-sized units, remainder to the first ranks."""
    if total % multiple:
        raise ValueError(f"{total} is not a multiple of {multiple}")
    units = total // multiple
    base, rem = divmod(units, world)
    lo = rank * base + min(rank, rem)
    hi = lo + base + (1 if rank < rem else 0)
    return lo * multiple, hi * multiple


def column_shard(n, world, rank):
    """Output channels of a column-parallel GEMM owned by `rank` (multiples of 8: 16-byte rows of bf16 C)."""
    return split_range(n, world, rank, 8)


def k_shard(k, world, rank, bits=8, group=0):
    """K range of a row-parallel GEMM owned by `rank`: whole 64-wide K steps (128 for 4-bit), whole scale groups."""
    mult = 64 if bits == 8 else 128
    if group:
        mult = max(mult, group)
    return split_range(k, world, rank, mult)


class AllReduceArgs(ctypes.Structure):
    """``afb_allreduce_args`` of include/afb_capi.h."""
    _fields_ = [("partial", ctypes.c_void_p * MAX_RANKS), ("c", ctypes.c_void_p * MAX_RANKS), ("signals", ctypes.c_void_p * MAX_RANKS),
                ("rank", ctypes.c_uint32), ("world", ctypes.c_uint32), ("m", ctypes.c_uint32), ("n", ctypes.c_uint32),
                ("ld_partial", ctypes.c_uint32), ("ldc", ctypes.c_uint32), ("partial_f32", ctypes.c_uint32), ("epoch", ctypes.c_uint32),
                ("wait_ms", ctypes.c_uint32), ("reserved", ctypes.c_uint32), ("c_multicast", ctypes.c_void_p)]


class TileAllReduceArgs(ctypes.Structure):
    """``afb_tile_allreduce_args`` of include/afb_capi.h."""
    _fields_ = [("base", AllReduceArgs), ("tile_done", ctypes.c_void_p * MAX_RANKS), ("tile_epoch", ctypes.c_uint32), ("reserved", ctypes.c_uint32)]


class SubAllReduceArgs(ctypes.Structure):
    """``afb_sub_allreduce_args`` of include/afb_capi.h."""
    _fields_ = [("base", AllReduceArgs), ("counters", ctypes.c_void_p), ("sub_blocks", ctypes.c_uint32), ("launches", ctypes.c_uint32),
                ("reserved", ctypes.c_uint32)]


def push_slot_offset(q, rank, world, m, n):
    """Byte offset, from the start of rank `rank`'s staging buffer float[world][m / world][n], of the address that the exchange
    kernel must be given as partial[q] so that its absolute-row indexing (rows rank*m/world .. of an [m, n] matrix) lands in slot q."""
    rows = m // world
    return (q * rows - rank * rows) * n * 4


class PeerExchange:
    """Buffers of the fused K-split all-reduce, shared between the ranks of one box by CUDA IPC.

    Each rank allocates (through the C ABI, so the allocation is a whole cudaMalloc block) its partial-sum
    buffer, its result buffer C and its signal words, exports the three handles, and maps every peer's."""

    def __init__(self, lib, torch_dist, rank, world, m, n, partial_f32=True, wait_ms=2000, multicast=None):
        self.lib, self.rank, self.world, self.m, self.n = lib, rank, world, m, n
        if multicast is None:
            multicast = os.environ.get("AFB_EXCHANGE_MULTICAST", "1") != "0"
        self.c_multicast = None   # NVSwitch multicast address of C, when torch's symmetric memory provides one
        self._symm = None
        self.partial_f32 = partial_f32
        self.wait_ms = wait_ms
        self.epoch = 0        # exchanges issued (orders the signal words)
        self.tile_epoch = 0   # tile-publishing GEMMs issued (orders the per-tile counters)
        pbytes = m * n * (4 if partial_f32 else 2)
        self.partial = lib.malloc(pbytes)
        self.c = None
        if world > 1 and multicast:
            self._symmetric_c(torch_dist, m * n * 2)
        if self.c is None:
            self.c = lib.malloc(m * n * 2)
        self.signals = lib.malloc(2 * MAX_RANKS * 4)
        lib.memset(self.signals, 0, 2 * MAX_RANKS * 4)
        # per-tile completion counters of the tile-granular form (fp32 partial sums only)
        tm, tn, nt, arr = (ctypes.c_uint32() for _ in range(4))
        lib.check(lib.lib.afb_ksplit_tile_info(m, n, ctypes.byref(tm), ctypes.byref(tn), ctypes.byref(nt), ctypes.byref(arr)), "afb_ksplit_tile_info")
        self.num_tiles = nt.value
        self.tile_done = lib.malloc(self.num_tiles * 4)
        lib.memset(self.tile_done, 0, self.num_tiles * 4)
        lib.device_sync()
        self._imported = []
        self.partials, self.cs, self.sigs, self.tds = [None] * world, [None] * world, [None] * world, [None] * world
        self.ok = True
        if world == 1:
            self.partials[0], self.cs[0], self.sigs[0], self.tds[0] = self.partial, self.c, self.signals, self.tile_done
            return
        # No rank may raise between the collectives below (the others would wait for it for ever):
        # failures are recorded, exchanged, and every rank reaches the same verdict.
        try:
            mine = (lib.ipc_export(self.partial), None if self._symm else lib.ipc_export(self.c), lib.ipc_export(self.signals),
                    lib.ipc_export(self.tile_done))
        except Exception as e:  # noqa: BLE001
            mine, self.error = None, str(e)
        everyone = [None] * world
        torch_dist.all_gather_object(everyone, mine)
        if any(h is None for h in everyone):
            self.ok = False
        else:
            try:
                for q, handles in enumerate(everyone):
                    if q == rank:
                        self.partials[q], self.cs[q], self.sigs[q], self.tds[q] = self.partial, self.c, self.signals, self.tile_done
                    else:
                        ptrs = []
                        for h in handles:
                            if h is None:   # C lives in symmetric memory: mapped by its rendezvous
                                ptrs.append(int(self._symm[1].buffer_ptrs[q]))
                                continue
                            ptrs.append(lib.ipc_import(h))
                            self._imported.append(ptrs[-1])
                        self.partials[q], self.cs[q], self.sigs[q], self.tds[q] = ptrs
            except Exception as e:  # noqa: BLE001
                self.ok, self.error = False, str(e)
        verdicts = [None] * world
        torch_dist.all_gather_object(verdicts, self.ok)
        self.ok = all(verdicts)

    def _symmetric_c(self, torch_dist, nbytes):
        """Allocates C in torch's symmetric memory so that the NVSwitch can replicate the result rows (multimem.st).
        Every step is agreed on by all ranks before the next collective one; on any failure C falls back to a plain buffer."""
        import torch
        t = None
        try:
            import torch.distributed._symmetric_memory as symm
            t = symm.empty(nbytes // 2, dtype=torch.bfloat16, device=torch.device("cuda", torch.cuda.current_device()))
        except Exception:  # noqa: BLE001
            t = None
        oks = [None] * self.world
        torch_dist.all_gather_object(oks, t is not None)
        if not all(oks):
            return
        hdl, mc = None, 0
        try:
            hdl = symm.rendezvous(t, torch_dist.group.WORLD)
            mc = int(hdl.multicast_ptr or 0)
        except Exception:  # noqa: BLE001
            hdl, mc = None, 0
        torch_dist.all_gather_object(oks, hdl is not None and mc != 0)
        if not all(oks):
            return
        self._symm = (t, hdl)
        self.c = int(t.data_ptr())
        self.c_multicast = mc

    def args(self):
        a = AllReduceArgs()
        for q in range(self.world):
            a.partial[q], a.c[q], a.signals[q] = self.partials[q], self.cs[q], self.sigs[q]
        a.rank, a.world, a.m, a.n = self.rank, self.world, self.m, self.n
        a.ld_partial, a.ldc, a.partial_f32 = self.n, self.n, 1 if self.partial_f32 else 0
        a.wait_ms, a.reserved = self.wait_ms, 0
        a.c_multicast = self.c_multicast
        return a

    def allreduce(self, stream=None):
        self.epoch += 1
        a = self.args()
        a.epoch = self.epoch
        self.lib.lib.afb_ksplit_allreduce_launch.argtypes = [ctypes.POINTER(AllReduceArgs), ctypes.c_void_p]
        self.lib.check(self.lib.lib.afb_ksplit_allreduce_launch(ctypes.byref(a), stream), "afb_ksplit_allreduce_launch")

    def push_supported(self):
        return self.partial_f32 and self.m % (256 * self.world) == 0

    def gemm_pushing(self, args, stream=None):
        """The K-split GEMM with the reduce-scatter in its epilogue: each tile of fp32 partial sums is stored into the
        partial-sum buffer of the rank owning those rows (read there as float[world][m / world][n], slot = this rank)."""
        from .capi import GemmArgs
        f = self.lib.lib.afb_gemm_launch_push
        f.argtypes = [ctypes.POINTER(GemmArgs), ctypes.POINTER(ctypes.c_void_p), ctypes.c_uint32, ctypes.c_uint32, ctypes.c_void_p]
        stage = (ctypes.c_void_p * MAX_RANKS)(*[self.partials[q] for q in range(self.world)])
        self.lib.check(f(ctypes.byref(args), stage, self.world, self.rank, stream), "afb_gemm_launch_push")

    def allreduce_pushed(self, stream=None):
        """Finishes gemm_pushing(): waits for every rank's GEMM, sums this rank's rows from its LOCAL slots in rank order,
        rounds once and broadcasts the bf16 rows."""
        self.epoch += 1
        a = self.args()
        a.epoch = self.epoch
        for q in range(self.world):   # slot q, addressed by absolute row as the kernel does
            a.partial[q] = self.partial + push_slot_offset(q, self.rank, self.world, self.m, self.n)
        self.lib.lib.afb_ksplit_allreduce_launch.argtypes = [ctypes.POINTER(AllReduceArgs), ctypes.c_void_p]
        self.lib.check(self.lib.lib.afb_ksplit_allreduce_launch(ctypes.byref(a), stream), "afb_ksplit_allreduce_launch")

    def pipelined_supported(self, sub_blocks):
        return self.push_supported() and self.n % (128 * sub_blocks) == 0 and sub_blocks <= self.num_tiles

    def gemm_pushing_pipelined(self, args, sub_blocks, stream=None):
        """The pushing GEMM in column-chunk order, counting finished tiles at their owners (the per-tile counter buffers of
        this object serve as the per-chunk counters: one form per object)."""
        from .capi import GemmArgs
        f = self.lib.lib.afb_gemm_launch_push_pipelined
        f.argtypes = [ctypes.POINTER(GemmArgs), ctypes.POINTER(ctypes.c_void_p), ctypes.POINTER(ctypes.c_void_p), ctypes.c_uint32, ctypes.c_uint32,
                      ctypes.c_uint32, ctypes.c_void_p]
        stage = (ctypes.c_void_p * MAX_RANKS)(*[self.partials[q] for q in range(self.world)])
        cnt = (ctypes.c_void_p * MAX_RANKS)(*[self.tds[q] for q in range(self.world)])
        self.lib.check(f(ctypes.byref(args), stage, cnt, self.world, self.rank, sub_blocks, stream), "afb_gemm_launch_push_pipelined")
        self.sub_launches = getattr(self, "sub_launches", 0) + 1

    def allreduce_pipelined(self, sub_blocks, stream=None):
        """Chunk-by-chunk sum of the local slots + broadcast; launch it on another stream than gemm_pushing_pipelined()."""
        self.epoch += 1
        sa = SubAllReduceArgs()
        sa.base = self.args()
        sa.base.epoch = self.epoch
        for q in range(self.world):
            sa.base.partial[q] = self.partial + push_slot_offset(q, self.rank, self.world, self.m, self.n)
        sa.counters, sa.sub_blocks, sa.launches, sa.reserved = self.tile_done, sub_blocks, self.sub_launches, 0
        f = self.lib.lib.afb_ksplit_sub_allreduce_launch
        f.argtypes = [ctypes.POINTER(SubAllReduceArgs), ctypes.c_void_p]
        self.lib.check(f(ctypes.byref(sa), stream), "afb_ksplit_sub_allreduce_launch")

    def gemm_pushing_exchange(self, args, sub_blocks, stream=None):
        """Both halves of the pipelined form in one launch: the pushing GEMM in column-chunk order, with two extra warps per CTA that
        sum each finished chunk of this rank's rows from the local slots and broadcast it.  C is complete when the launch is."""
        from .capi import GemmArgs
        self.epoch += 1
        self.sub_launches = getattr(self, "sub_launches", 0) + 1
        sa = SubAllReduceArgs()
        sa.base = self.args()
        sa.base.epoch = self.epoch
        for q in range(self.world):
            sa.base.partial[q] = self.partial + push_slot_offset(q, self.rank, self.world, self.m, self.n)
        sa.counters, sa.sub_blocks, sa.launches, sa.reserved = self.tile_done, sub_blocks, self.sub_launches, 0
        f = self.lib.lib.afb_gemm_launch_push_exchange
        f.argtypes = [ctypes.POINTER(GemmArgs), ctypes.POINTER(ctypes.c_void_p), ctypes.POINTER(ctypes.c_void_p), ctypes.c_uint32, ctypes.c_uint32,
                      ctypes.c_uint32, ctypes.POINTER(SubAllReduceArgs), ctypes.c_void_p]
        stage = (ctypes.c_void_p * MAX_RANKS)(*[self.partials[q] for q in range(self.world)])
        cnt = (ctypes.c_void_p * MAX_RANKS)(*[self.tds[q] for q in range(self.world)])
        self.lib.check(f(ctypes.byref(args), stage, cnt, self.world, self.rank, sub_blocks, ctypes.byref(sa), stream), "afb_gemm_launch_push_exchange")

    def gemm_publishing_tiles(self, args, stream=None):
        """The K-split GEMM into this rank's partial-sum buffer, counting finished tiles for allreduce_tiles()."""
        f = self.lib.lib.afb_gemm_launch_tiles
        from .capi import GemmArgs
        f.argtypes = [ctypes.POINTER(GemmArgs), ctypes.c_void_p, ctypes.c_void_p]
        self.lib.check(f(ctypes.byref(args), self.tile_done, stream), "afb_gemm_launch_tiles")
        self.tile_epoch += 1

    def allreduce_tiles(self, stream=None):
        """Tile-granular exchange; launch it AFTER gemm_publishing_tiles() of the same step, on another stream."""
        assert self.partial_f32
        self.epoch += 1
        ta = TileAllReduceArgs()
        ta.base = self.args()
        ta.base.epoch = self.epoch
        ta.tile_epoch, ta.reserved = self.tile_epoch, 0
        for q in range(self.world):
            ta.tile_done[q] = self.tds[q]
        f = self.lib.lib.afb_ksplit_tile_allreduce_launch
        f.argtypes = [ctypes.POINTER(TileAllReduceArgs), ctypes.c_void_p]
        self.lib.check(f(ctypes.byref(ta), stream), "afb_ksplit_tile_allreduce_launch")

    def close(self):
        self.lib.device_sync()
        for p in self._imported:
            self.lib.ipc_release(p)
        for p in (self.partial, None if self._symm else self.c, self.signals, self.tile_done):
            if p is not None:
                self.lib.free(p)
        self._symm = None


def cast_f32_to_bf16(lib, dst, src, rows, cols, stream=None):
    f = lib.lib.afb_cast_f32_to_bf16
    f.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_uint32, ctypes.c_uint32, ctypes.c_uint32, ctypes.c_uint32, ctypes.c_void_p]
    lib.check(f(dst, src, rows, cols, cols, cols, stream), "afb_cast_f32_to_bf16")


def pick_exchange(world, partial, m, down_n, sub_blocks=8):
    """The exchange form `auto` stands for.  Measured: the reduce-scatter in the GEMM epilogue ("push") beats the exchange kernel after
    the GEMM ("fused"), which beats the tile-granular exchange next to the GEMM (whose own NVLink traffic slows the GEMM by as much as
    the overlap saves); with the sum and broadcast done chunk by chunk by two extra warps of every GEMM CTA ("inkernel") the tail
    after the GEMM goes too: 0.584 against 0.607 ms per step on 8 GPUs, 0.897 against 0.924 on 4, 0.9225 against 0.930 ms for the
    down-projection on 2 (kept on push there).  Both need fp32 partial sums and M a multiple of 256 * world; the in-kernel form also
    N a multiple of 128 * sub_blocks."""
    if partial != "f32" or m % (256 * world) != 0:
        return "fused"
    if world >= 4 and down_n % (128 * sub_blocks) == 0:
        return "inkernel"
    return "push"


class ShardedMLP:
    """The sharded benchmark step: column-parallel up-projection + row-parallel down-projection (int8, per-channel).

    exchange: "push" (reduce-scatter in the GEMM epilogue over peer stores, then a local sum + broadcast kernel) |
              "overlap" (tile-granular exchange next to the GEMM) | "fused" (one exchange kernel after the GEMM) | "nccl" |
              "auto" (fused when the box shares memory between the processes, else nccl).
    partial:  "f32" (exact, ordered sum) | "bf16" (half the NVLink bytes; each partial rounded once)."""

    def __init__(self, lib, torch, rank=0, world=1, exchange="auto", partial="f32", m=4096, up=(28672, 8192), down=(8192, 28672), seed=0):
        import awesome_fusion_b200 as pkg
        self.lib, self.torch, self.rank, self.world, self.m = lib, torch, rank, world, m
        self.pkg = pkg
        dev = torch.device("cuda", torch.cuda.current_device())
        up_n, up_k = up
        down_n, down_k = down
        n_lo, n_hi = column_shard(up_n, world, rank)
        k_lo, k_hi = k_shard(down_k, world, rank)
        self.up_n_local, self.up_k = n_hi - n_lo, up_k
        self.down_n, self.down_k_local = down_n, k_hi - k_lo
        g = torch.Generator(device=dev); g.manual_seed(seed)            # replicated tensors: the same seed on every rank
        gr = torch.Generator(device=dev); gr.manual_seed(seed + 1 + rank)  # rank-local tensors: seed + 1 + rank
        self.a_up = torch.randn((m, up_k), generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16)
        self.b_up = torch.randint(-127, 128, (self.up_n_local, up_k), generator=gr, device=dev, dtype=torch.int8)
        self.s_up = torch.rand((self.up_n_local,), generator=gr, device=dev) * 0.009 + 0.001
        self.c_up = torch.empty((m, self.up_n_local), device=dev, dtype=torch.bfloat16)
        self.a_down = torch.randn((m, self.down_k_local), generator=gr, device=dev, dtype=torch.float32).to(torch.bfloat16)
        self.b_down = torch.randint(-127, 128, (down_n, self.down_k_local), generator=gr, device=dev, dtype=torch.int8)
        self.s_down = torch.rand((down_n,), generator=g, device=dev) * 0.009 + 0.001   # scales are per output channel: replicated
        self.flops_per_step_global = 2.0 * m * up_n * up_k + 2.0 * m * down_n * down_k
        self.layout = pkg.LAYOUT_COL
        self.args_up = lib.make_args(self.c_up, self.a_up, self.b_up, self.s_up, m, self.up_n_local, up_k)
        self.px = None
        if world == 1:
            self.exchange_name = "none (1 GPU)"
            self.c_down = torch.empty((m, down_n), device=dev, dtype=torch.bfloat16)
            self.args_down = lib.make_args(self.c_down, self.a_down, self.b_down, self.s_down, m, down_n, self.down_k_local)
            return
        import torch.distributed as tdist
        self.tdist = tdist
        mode = exchange
        # column chunks of the pipelined forms: 8 (measured on 2 GPUs: 1.03 ms for the down-projection against 1.14 with 2 chunks,
        # whose last chunk leaves half of the sum and broadcast for after the GEMM); AFB_SUB_BLOCKS overrides
        self.sub_blocks = int(os.environ.get("AFB_SUB_BLOCKS", "8"))
        if mode == "auto":
            mode = pick_exchange(world, partial, m, down_n, self.sub_blocks)
        self.overlap = mode == "overlap"
        self.push = mode == "push"
        self.pipelined = mode == "pipelined"
        self.inkernel = mode == "inkernel"
        if mode == "pipelined":
            if partial != "f32" or m % (256 * world) != 0 or down_n % (128 * self.sub_blocks) != 0:
                raise pkg.AfbError(-4, "the pipelined exchange needs fp32 partial sums, M a multiple of 256 * world and N of 128 * sub-blocks", "")
            mode = "fused"
            self.side = torch.cuda.Stream()
        if mode == "inkernel":
            if partial != "f32" or m % (256 * world) != 0 or down_n % (128 * self.sub_blocks) != 0:
                raise pkg.AfbError(-4, "the in-kernel exchange needs fp32 partial sums, M a multiple of 256 * world and N of 128 * sub-blocks", "")
            mode = "fused"
        if mode == "overlap":
            mode = "fused"
            self.side = torch.cuda.Stream()
        if mode == "push":
            if partial != "f32" or m % (256 * world) != 0:
                raise pkg.AfbError(-4, "the push exchange needs fp32 partial sums and M a multiple of 256 * world", "")
            mode = "fused"
        if mode == "fused":
            self.px = PeerExchange(lib, tdist, rank, world, m, down_n, partial_f32=(partial == "f32"))
            if not self.px.ok:
                why = getattr(self.px, "error", "a peer could not share its memory")
                self.px.close(); self.px = None
                self.overlap = False
                self.push = False
                self.pipelined = False
                self.inkernel = False
                if exchange in ("fused", "overlap", "push", "pipelined", "inkernel"):
                    raise pkg.AfbError(-3, "peer-memory exchange unavailable", why)
                if rank == 0:
                    print(f"peer memory unavailable ({why}); using the NCCL exchange", flush=True)
                mode = "nccl"
        if mode == "fused":
            self.exchange_name = (f"reduce-scatter in the GEMM epilogue in {self.sub_blocks} column chunks (peer stores of fp32 tiles), each chunk summed from local slots and broadcast by two extra warps of every GEMM CTA (one launch)" if self.inkernel
                                  else f"reduce-scatter in the GEMM epilogue in {self.sub_blocks} column chunks (peer stores of fp32 tiles), each chunk summed from local slots and broadcast next to the GEMM" if self.pipelined
                                  else f"tile-granular peer-memory all-reduce overlapped with the GEMM ({partial} partial sums)" if self.overlap
                                  else "reduce-scatter in the GEMM epilogue (peer stores of fp32 tiles) + local sum and bf16 broadcast" if self.push
                                  else f"fused peer-memory all-reduce after the GEMM ({partial} partial sums)")
            if self.px.c_multicast and not self.overlap:
                self.exchange_name += "; result rows broadcast by multimem.st through the NVSwitch"
            flags = 0 if partial == "bf16" else pkg.FLAG_C_F32
            c_down = self.px.partial
            # measured: forwarding warps win on 8 GPUs (0.618 vs 0.632 ms per step) and lose on 2 (1.72 vs 1.69)
            if self.push and os.environ.get("AFB_PUSH_FORWARD", "1" if world >= 8 else "0") != "0":
                # the epilogue stores each tile locally; two extra warps per CTA forward it to its owner during the next tile
                self.scratch32 = torch.empty((m, down_n), device=dev, dtype=torch.float32)
                c_down = self.scratch32
                flags |= pkg.FLAG_PUSH_VIA_LOCAL
                self.exchange_name += "; tiles forwarded by dedicated warps"
            self.args_down = lib.make_args(c_down, self.a_down, self.b_down, self.s_down, m, down_n, self.down_k_local, flags=flags)
        else:
            self.exchange_name = "nccl all-reduce of fp32 partial sums + cast"
            self.partial32 = torch.empty((m, down_n), device=dev, dtype=torch.float32)
            self.c_down = torch.empty((m, down_n), device=dev, dtype=torch.bfloat16)
            self.args_down = lib.make_args(self.partial32, self.a_down, self.b_down, self.s_down, m, down_n, self.down_k_local,
                                           flags=pkg.FLAG_C_F32)

    def prepack_weights(self):
        """Offline step: re-orders both weight shards in place into the pre-packed layout (afb_prepack) and points the GEMMs at them."""
        lib, pkg = self.lib, self.pkg
        if self.layout == pkg.LAYOUT_COL_PACKED:
            return
        for args, b in ((self.args_up, self.b_up), (self.args_down, self.b_down)):
            lib.prepack(args, b, args.ldb)
            args.b_layout = pkg.LAYOUT_COL_PACKED
        self.layout = pkg.LAYOUT_COL_PACKED
        self.torch.cuda.synchronize()

    def step(self, stream, events=None):
        lib = self.lib
        if events:
            events[0].record()
        lib.gemm_launch(self.args_up, stream)
        if events:
            events[1].record()
        if self.world > 1 and self.px is not None and self.overlap:
            torch = self.torch
            before = torch.cuda.current_stream().record_event()
            self.px.gemm_publishing_tiles(self.args_down, stream)
            with torch.cuda.stream(self.side):      # launched after the GEMM, runs next to it
                self.side.wait_event(before)        # no point in polling while the previous GEMM still runs
                self.px.allreduce_tiles(self.side.cuda_stream)
                done = self.side.record_event()
            torch.cuda.current_stream().wait_event(done)   # the step ends when C is complete on this rank
            if events:
                events[2].record()
            return
        if self.world > 1 and self.px is not None and self.inkernel:
            self.px.gemm_pushing_exchange(self.args_down, self.sub_blocks, stream)
            if events:
                events[2].record()
            return
        if self.world > 1 and self.px is not None and self.pipelined:
            torch = self.torch
            before = torch.cuda.current_stream().record_event()
            self.px.gemm_pushing_pipelined(self.args_down, self.sub_blocks, stream)
            with torch.cuda.stream(self.side):      # runs next to the GEMM: chunk c is summed and broadcast while chunk c + 1 is computed
                self.side.wait_event(before)
                self.px.allreduce_pipelined(self.sub_blocks, self.side.cuda_stream)
                done = self.side.record_event()
            torch.cuda.current_stream().wait_event(done)
            if events:
                events[2].record()
            return
        if self.world > 1 and self.px is not None and self.push:
            self.px.gemm_pushing(self.args_down, stream)
            self.px.allreduce_pushed(stream)
            if events:
                events[2].record()
            return
        lib.gemm_launch(self.args_down, stream)
        if self.world > 1:
            if self.px is not None:
                self.px.allreduce(stream)
            else:
                self.tdist.all_reduce(self.partial32)
                cast_f32_to_bf16(lib, self.c_down.data_ptr(), self.partial32.data_ptr(), self.m, self.down_n, stream)
        if events:
            events[2].record()

    def close(self):
        """Unmaps the peers' buffers and frees this rank's.  Collective in effect: every rank calls it between steps, with
        none of its kernels in flight, before the process group is destroyed."""
        self.torch.cuda.synchronize()
        if self.px is not None:
            self.px.close()
            self.px = None

    def result_down(self):
        """bf16 result of the down-projection as a torch tensor on the host (tests)."""
        torch = self.torch
        if self.px is not None:
            import numpy as np
            arr = self.lib.to_host(self.px.c, (self.m, self.down_n), np.uint16)
            return torch.from_numpy(arr.view(np.int16)).view(torch.bfloat16)
        return self.c_down.cpu()

    def e2e(self, steps=5, warmup=2):
        """The same step end to end from HOST buffers: pinned host inputs, host-to-device copies, the GEMMs, (at N > 1) the
        exchange of the row-parallel partial sums, and the device-to-host copy of both results, all inside the timed region.
        One GPU: through afb_gemm_host.  Several GPUs: afb_gemm_host has no exchange, so each rank copies its shards in
        through the C ABI (afb_memcpy_h2d), runs the sharded step with the exchange, and copies its up-projection shard and
        the complete down-projection result back (afb_memcpy_d2h)."""
        torch, lib = self.torch, self.lib
        import time
        host = {}
        for name in ("a_up", "b_up", "s_up", "a_down", "b_down", "s_down"):
            host[name] = getattr(self, name).cpu().pin_memory()
        c_up = torch.empty((self.m, self.up_n_local), dtype=torch.bfloat16).pin_memory()
        c_down = torch.empty((self.m, self.down_n), dtype=torch.bfloat16).pin_memory()
        h2d = sum(host[k].numel() * host[k].element_size() for k in host)
        d2h = c_up.numel() * 2 + c_down.numel() * 2
        if self.world == 1:
            a1 = lib.make_args(c_up, host["a_up"], host["b_up"], host["s_up"], self.m, self.up_n_local, self.up_k)
            a2 = lib.make_args(c_down, host["a_down"], host["b_down"], host["s_down"], self.m, self.down_n, self.down_k_local)
            api = "afb_gemm_host_async x2 + afb_gemm_host_wait (C ABI, pinned host buffers)"

            def one():   # the second GEMM's copy-in overlaps the first one's GEMM and copy-out
                lib.gemm_host_async(a1)
                lib.gemm_host_async(a2)
                lib.gemm_host_wait()
        else:
            stream = torch.cuda.current_stream().cuda_stream
            c_down_dev = self.px.c if self.px is not None else self.c_down.data_ptr()
            api = "afb_memcpy_h2d + sharded GEMMs + exchange + afb_memcpy_d2h (C ABI, pinned host buffers)"

            def one():
                for name in host:
                    lib.h2d(getattr(self, name).data_ptr(), host[name].data_ptr(), host[name].numel() * host[name].element_size())
                self.step(stream)
                torch.cuda.current_stream().synchronize()
                lib.d2h(c_up.data_ptr(), self.c_up.data_ptr(), c_up.numel() * 2)
                lib.d2h(c_down.data_ptr(), c_down_dev, c_down.numel() * 2)
        for _ in range(warmup):
            one()
        torch.cuda.synchronize()
        if self.world > 1:
            self.tdist.barrier()
        t0 = time.perf_counter()
        for _ in range(steps):
            one()
        torch.cuda.synchronize()
        ms = (time.perf_counter() - t0) / steps * 1e3
        return {"ms": ms, "h2d": h2d, "d2h": d2h, "api": api}
