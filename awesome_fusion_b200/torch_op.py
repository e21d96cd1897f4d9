"""PyTorch operator over the C ABI: ``torch.ops.afb.bf16_aintb_gemm``.

The reference has no framework binding (its driver ``bfAintBGemm/bfAintBGemm.cc:36-217`` is a stand-alone
executable); this is the thin layer an inference stack would call instead.  It computes nothing itself: the
tensors' device pointers go into ``afb_gemm_args`` and ``afb_gemm_launch`` runs on torch's current stream, so
the call is stream-ordered with the surrounding torch work and can be captured into a CUDA graph
(``DecodeGraph`` does that for the launch-bound small-M case).  There is no CPU path: a CPU tensor raises.

    out = torch.ops.afb.bf16_aintb_gemm(a, b, scale, bits, group_size, offset_binary, flags=0)

    a      bf16 [M, K], contiguous
    b      int8 [N, K] (bits = 8) or uint8 [N, K / 2] (bits = 4, low nibble = even k), contiguous
    scale  fp32 or bf16; [N] (group_size = 0) or [N, K / group_size]
    flags  AFB_FLAG_* bits passed through to afb_gemm_args.flags (e.g. FLAG_PDL for back-to-back decode GEMMs on constant
           weights, FLAG_GROUP_EXACT for the two-term group-scale mode); default 0
    out    bf16 [M, N]
"""
import torch

from .capi import ENC_OFFSET, ENC_TWOS, FLAG_PDL, SCALE_BF16, SCALE_F32, AfbError, load

_LIB_NAME = "afb::bf16_aintb_gemm"


def _check(a, b, scale, bits, group_size):
    if bits not in (4, 8):
        raise ValueError("bits must be 4 or 8")
    if a.dtype != torch.bfloat16 or a.dim() != 2:
        raise ValueError("a must be a bf16 [M, K] tensor")
    if b.dim() != 2 or b.dtype not in (torch.int8, torch.uint8):
        raise ValueError("b must be an int8 / uint8 [N, K * bits / 8] tensor")
    k = a.shape[1]
    if b.shape[1] * (8 // bits) != k:
        raise ValueError(f"b holds {b.shape[1] * (8 // bits)} weights per channel, a has K = {k}")
    n = b.shape[0]
    if scale.dtype not in (torch.float32, torch.bfloat16):
        raise ValueError("scale must be fp32 or bf16")
    if group_size == 0:
        if scale.numel() != n:
            raise ValueError("per-channel scale must have N elements")
    elif group_size < 0 or k % group_size or scale.numel() != n * (k // group_size):
        raise ValueError("per-group scale must be [N, K / group_size]")
    return a.shape[0], n, k


@torch.library.custom_op(_LIB_NAME, mutates_args=(), device_types="cuda")
def bf16_aintb_gemm(a: torch.Tensor, b: torch.Tensor, scale: torch.Tensor, bits: int, group_size: int,
                    offset_binary: bool, flags: int = 0) -> torch.Tensor:
    m, n, k = _check(a, b, scale, bits, group_size)
    if not (a.is_contiguous() and b.is_contiguous() and scale.is_contiguous()):
        raise ValueError("a, b and scale must be contiguous")
    lib = load()
    dev = a.device.index if a.device.index is not None else torch.cuda.current_device()
    with torch.cuda.device(dev):
        lib.init(dev)
        out = torch.empty((m, n), device=a.device, dtype=torch.bfloat16)
        args = lib.make_args(out, a, b, scale, m, n, k, bits=bits, group=group_size,
                             encoding=ENC_OFFSET if offset_binary else ENC_TWOS,
                             scale_dtype=SCALE_BF16 if scale.dtype == torch.bfloat16 else SCALE_F32, flags=flags)
        lib.gemm_launch(args, torch.cuda.current_stream().cuda_stream)
    return out


@bf16_aintb_gemm.register_fake
def _(a, b, scale, bits, group_size, offset_binary, flags=0):
    m, n, _ = _check(a, b, scale, bits, group_size)
    return a.new_empty((m, n), dtype=torch.bfloat16)


class DecodeGraph:
    """One small-M GEMM captured in a CUDA graph: ``replay()`` costs one graph launch instead of a Python call into the
    library per GEMM (a decode GEMM runs for microseconds, less than the host needs to issue it).  The input tensors are
    the graph's fixed buffers: copy new activations into ``self.a`` and read ``self.out`` after ``replay()``."""

    def __init__(self, a, b, scale, bits=8, group_size=0, offset_binary=False, weights_constant=False):
        """weights_constant: promise that b and scale are not written while the graph is in use; the GEMM is then launched with
        programmatic dependent launch (FLAG_PDL) and overlaps the kernel before it in the graph's stream."""
        if a.shape[0] > 16:
            raise AfbError(-4, "DecodeGraph is for M <= 16", "")
        self.a, self.b, self.scale = a, b, scale
        flags = FLAG_PDL if weights_constant else 0
        stream = torch.cuda.Stream()
        stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(stream):   # the first call of a kernel sets its attributes: do it outside the capture
            torch.ops.afb.bf16_aintb_gemm(a, b, scale, bits, group_size, offset_binary, flags)
        torch.cuda.current_stream().wait_stream(stream)
        torch.cuda.synchronize()
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.out = torch.ops.afb.bf16_aintb_gemm(a, b, scale, bits, group_size, offset_binary, flags)

    def replay(self):
        self.graph.replay()
        return self.out
