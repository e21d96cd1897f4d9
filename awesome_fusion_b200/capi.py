"""ctypes binding of ``include/afb_capi.h``: one Python method per exported C function.

Buffers are raw device pointers (ints) allocated through the library, or any object with a
``data_ptr()`` method / ``ctypes.data`` attribute.  Nothing here computes: a missing or
unloadable ``libafb.so`` raises ``AfbError`` (there is no CPU or PyTorch fallback).
"""
import ctypes
import os

import numpy as np

ENC_TWOS, ENC_OFFSET = 0, 1
LAYOUT_ROW, LAYOUT_COL, LAYOUT_COL_PACKED = 0, 1, 2
SCALE_F32, SCALE_BF16 = 0, 1
VARIANT_AUTO, VARIANT_DECODE, VARIANT_PREFILL, VARIANT_NAIVE = 0, 1, 2, 3
FLAG_C_F32 = 1
FLAG_PREFILL_SMEM_B = 2
FLAG_PREFILL_TMEM_A = 4
FLAG_PUSH_VIA_LOCAL = 8
FLAG_DUMP_DECODE_PAIRING = 16
FLAG_GROUP_EXACT = 32
FLAG_PDL = 64
ACT_NONE, ACT_SILU = 0, 1
IPC_HANDLE_BYTES = 64

_HERE = os.path.dirname(os.path.abspath(__file__))

# every symbol include/afb_capi.h declares; tests check the built library exports all of them
EXPORTS = [
    "afb_init", "afb_finalize", "afb_device_count", "afb_sm_count", "afb_malloc", "afb_free", "afb_malloc_host",
    "afb_free_host", "afb_memcpy_h2d", "afb_memcpy_d2h", "afb_memcpy_d2d", "afb_memset", "afb_event_create",
    "afb_event_record", "afb_event_sync", "afb_event_elapsed_ms", "afb_event_destroy", "afb_stream_create",
    "afb_stream_sync", "afb_stream_destroy", "afb_device_sync", "afb_gemm_launch", "afb_gemm_resolve_variant",
    "afb_gemm_host", "afb_gemm_host_async", "afb_gemm_host_wait", "afb_gemm_launch_static", "afb_prepack", "afb_prepack_gated", "afb_gemm_fused_launch", "afb_dequant_dump", "afb_read_status", "afb_ipc_export", "afb_ipc_import", "afb_ipc_release",
    "afb_ksplit_allreduce_launch", "afb_cast_f32_to_bf16", "afb_ksplit_tile_info", "afb_gemm_launch_tiles", "afb_ksplit_tile_allreduce_launch", "afb_gemm_launch_push", "afb_abi_sizes",
    "afb_dist_init", "afb_dist_world", "afb_dist_stream", "afb_dist_gemm_launch", "afb_dist_sync", "afb_dist_finalize", "afb_dist_split_range",
    "afb_ksplit_sub_info", "afb_gemm_launch_push_pipelined", "afb_ksplit_sub_allreduce_launch", "afb_gemm_launch_push_exchange", "afb_probe_launch", "afb_phase_timestamps", "afb_status_string", "afb_last_cuda_error", "afb_last_cuda_error_string", "afb_launch_count", "afb_version",
]


class AfbError(RuntimeError):
    def __init__(self, status, what, detail=""):
        self.status = status
        super().__init__(f"{what}: status {status}{(' (' + detail + ')') if detail else ''}")


class GemmArgs(ctypes.Structure):
    """``afb_gemm_args``: the reference's kernarg block (bfAintBGemm.cc:119-133) plus mode fields."""
    _fields_ = [
        ("ptr_c", ctypes.c_void_p), ("ptr_a", ctypes.c_void_p), ("ptr_b", ctypes.c_void_p), ("ptr_scale", ctypes.c_void_p),
        ("m", ctypes.c_uint32), ("n", ctypes.c_uint32), ("k", ctypes.c_uint32),
        ("lda", ctypes.c_uint32), ("ldb", ctypes.c_uint32), ("ldc", ctypes.c_uint32),
        ("b_bits", ctypes.c_uint32), ("b_encoding", ctypes.c_uint32), ("b_layout", ctypes.c_uint32),
        ("scale_dtype", ctypes.c_uint32), ("group_size", ctypes.c_uint32), ("variant", ctypes.c_uint32),
        ("flags", ctypes.c_uint32), ("reserved", ctypes.c_uint32),
        ("ptr_zero", ctypes.c_void_p), ("reserved2", ctypes.c_uint64),
    ]


class FusedArgs(ctypes.Structure):
    """``afb_fused_args``: a GEMM plus its fused epilogue (bias, activation, gate * up, residual)."""
    _fields_ = [("gemm", GemmArgs), ("gated", ctypes.c_uint32), ("activation", ctypes.c_uint32), ("ptr_bias", ctypes.c_void_p),
                ("ptr_residual", ctypes.c_void_p), ("ld_residual", ctypes.c_uint32), ("reserved", ctypes.c_uint32)]


def library_path() -> str:
    return os.environ.get("AFB_LIBRARY", os.path.join(_HERE, "libafb.so"))


def _ptr(x):
    if x is None:
        return None
    if isinstance(x, int):
        return x
    if hasattr(x, "data_ptr"):
        return x.data_ptr()
    if isinstance(x, np.ndarray):
        return x.ctypes.data
    raise TypeError(f"cannot take a pointer of {type(x)}")


class Library:
    """Loaded ``libafb.so``.  Methods raise ``AfbError`` on any non-zero status."""

    def __init__(self, path=None):
        path = path or library_path()
        if not os.path.exists(path):
            raise AfbError(-5, "libafb.so not found", f"{path}; build it with awesome_fusion_b200.build_library()")
        self.path = path
        self.lib = ctypes.CDLL(path)
        L = self.lib
        vp, sz, i32 = ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int
        L.afb_init.argtypes = [i32]
        L.afb_device_count.argtypes = [ctypes.POINTER(i32)]
        L.afb_sm_count.argtypes = [ctypes.POINTER(i32)]
        L.afb_malloc.argtypes = [ctypes.POINTER(vp), sz]
        L.afb_free.argtypes = [vp]
        L.afb_malloc_host.argtypes = [ctypes.POINTER(vp), sz]
        L.afb_free_host.argtypes = [vp]
        for f in (L.afb_memcpy_h2d, L.afb_memcpy_d2h, L.afb_memcpy_d2d):
            f.argtypes = [vp, vp, sz]
        L.afb_memset.argtypes = [vp, i32, sz]
        L.afb_event_create.argtypes = [ctypes.POINTER(vp)]
        L.afb_event_record.argtypes = [vp, vp]
        L.afb_event_sync.argtypes = [vp]
        L.afb_event_elapsed_ms.argtypes = [ctypes.POINTER(ctypes.c_float), vp, vp]
        L.afb_event_destroy.argtypes = [vp]
        L.afb_stream_create.argtypes = [ctypes.POINTER(vp)]
        L.afb_stream_sync.argtypes = [vp]
        L.afb_stream_destroy.argtypes = [vp]
        L.afb_gemm_launch.argtypes = [ctypes.POINTER(GemmArgs), vp]
        L.afb_gemm_resolve_variant.argtypes = [ctypes.POINTER(GemmArgs), ctypes.POINTER(ctypes.c_uint32)]
        L.afb_gemm_host.argtypes = [ctypes.POINTER(GemmArgs), vp]
        L.afb_gemm_host_async.argtypes = [ctypes.POINTER(GemmArgs), vp]
        L.afb_gemm_host_wait.argtypes = [vp]
        L.afb_gemm_launch_static.argtypes = [ctypes.POINTER(GemmArgs), vp]
        L.afb_dequant_dump.argtypes = [ctypes.POINTER(GemmArgs), vp, vp]
        L.afb_prepack.argtypes = [ctypes.POINTER(GemmArgs), vp, ctypes.c_uint32, vp]
        L.afb_prepack_gated.argtypes = [ctypes.POINTER(GemmArgs), vp, vp, vp, vp, ctypes.c_uint32, vp, vp, vp]
        L.afb_gemm_fused_launch.argtypes = [ctypes.POINTER(FusedArgs), vp]
        L.afb_read_status.argtypes = [ctypes.POINTER(ctypes.c_int32)]
        L.afb_ipc_export.argtypes = [vp, ctypes.c_char_p]
        L.afb_ipc_import.argtypes = [ctypes.c_char_p, ctypes.POINTER(vp)]
        L.afb_ipc_release.argtypes = [vp]
        L.afb_status_string.argtypes = [i32]
        L.afb_status_string.restype = ctypes.c_char_p
        L.afb_last_cuda_error_string.restype = ctypes.c_char_p
        L.afb_launch_count.restype = ctypes.c_ulonglong
        L.afb_version.restype = ctypes.c_char_p

    # ---- helpers -------------------------------------------------------------
    def check(self, status, what):
        if status != 0:
            detail = self.lib.afb_status_string(status).decode()
            if status == -3:
                detail += ": " + self.lib.afb_last_cuda_error_string().decode()
            raise AfbError(status, what, detail)

    # ---- device / memory -------------------------------------------------------
    def init(self, device=0):
        self.check(self.lib.afb_init(device), "afb_init")

    def finalize(self):
        self.check(self.lib.afb_finalize(), "afb_finalize")

    def device_count(self):
        c = ctypes.c_int(0)
        self.check(self.lib.afb_device_count(ctypes.byref(c)), "afb_device_count")
        return c.value

    def sm_count(self):
        c = ctypes.c_int(0)
        self.check(self.lib.afb_sm_count(ctypes.byref(c)), "afb_sm_count")
        return c.value

    def malloc(self, nbytes):
        p = ctypes.c_void_p()
        self.check(self.lib.afb_malloc(ctypes.byref(p), nbytes), "afb_malloc")
        return p.value

    def free(self, ptr):
        self.check(self.lib.afb_free(ptr), "afb_free")

    def malloc_host(self, nbytes):
        p = ctypes.c_void_p()
        self.check(self.lib.afb_malloc_host(ctypes.byref(p), nbytes), "afb_malloc_host")
        return p.value

    def free_host(self, ptr):
        self.check(self.lib.afb_free_host(ptr), "afb_free_host")

    def h2d(self, dst, src, nbytes=None):
        if nbytes is None:
            nbytes = src.nbytes
        self.check(self.lib.afb_memcpy_h2d(_ptr(dst), _ptr(src), nbytes), "afb_memcpy_h2d")

    def d2h(self, dst, src, nbytes=None):
        if nbytes is None:
            nbytes = dst.nbytes
        self.check(self.lib.afb_memcpy_d2h(_ptr(dst), _ptr(src), nbytes), "afb_memcpy_d2h")

    def d2d(self, dst, src, nbytes):
        self.check(self.lib.afb_memcpy_d2d(_ptr(dst), _ptr(src), nbytes), "afb_memcpy_d2d")

    def memset(self, dst, value, nbytes):
        self.check(self.lib.afb_memset(_ptr(dst), value, nbytes), "afb_memset")

    def to_device(self, arr):
        """Allocates a device buffer, copies a contiguous numpy array into it, returns the pointer."""
        arr = np.ascontiguousarray(arr)
        p = self.malloc(max(arr.nbytes, 1))
        if arr.nbytes:
            self.h2d(p, arr)
        return p

    def to_host(self, ptr, shape, dtype):
        out = np.empty(shape, dtype=dtype)
        if out.nbytes:
            self.d2h(out, ptr)
        return out

    # ---- events / streams --------------------------------------------------------
    def event_create(self):
        p = ctypes.c_void_p()
        self.check(self.lib.afb_event_create(ctypes.byref(p)), "afb_event_create")
        return p.value

    def event_record(self, ev, stream=None):
        self.check(self.lib.afb_event_record(ev, stream), "afb_event_record")

    def event_sync(self, ev):
        self.check(self.lib.afb_event_sync(ev), "afb_event_sync")

    def event_elapsed_ms(self, start, stop):
        ms = ctypes.c_float(0)
        self.check(self.lib.afb_event_elapsed_ms(ctypes.byref(ms), start, stop), "afb_event_elapsed_ms")
        return ms.value

    def event_destroy(self, ev):
        self.check(self.lib.afb_event_destroy(ev), "afb_event_destroy")

    def stream_create(self):
        p = ctypes.c_void_p()
        self.check(self.lib.afb_stream_create(ctypes.byref(p)), "afb_stream_create")
        return p.value

    def stream_sync(self, s):
        self.check(self.lib.afb_stream_sync(s), "afb_stream_sync")

    def stream_destroy(self, s):
        self.check(self.lib.afb_stream_destroy(s), "afb_stream_destroy")

    def device_sync(self):
        self.check(self.lib.afb_device_sync(), "afb_device_sync")

    # ---- the hot path ------------------------------------------------------------
    @staticmethod
    def make_args(c, a, b, scale, m, n, k, *, lda=None, ldb=None, ldc=None, bits=8, encoding=ENC_TWOS,
                  layout=LAYOUT_COL, scale_dtype=SCALE_F32, group=0, variant=VARIANT_AUTO, flags=0, zero=None):
        args = GemmArgs()
        args.ptr_c, args.ptr_a, args.ptr_b, args.ptr_scale = _ptr(c), _ptr(a), _ptr(b), _ptr(scale)
        args.m, args.n, args.k = m, n, k
        args.lda = k if lda is None else lda
        args.ldb = (n if layout == LAYOUT_ROW else k) if ldb is None else ldb
        args.ldc = n if ldc is None else ldc
        args.b_bits, args.b_encoding, args.b_layout = bits, encoding, layout
        args.scale_dtype, args.group_size, args.variant, args.flags, args.reserved = scale_dtype, group, variant, flags, 0
        args.ptr_zero, args.reserved2 = _ptr(zero), 0
        return args

    def gemm_launch_status(self, args, stream=None):
        return self.lib.afb_gemm_launch(ctypes.byref(args), stream)

    def gemm_launch(self, args, stream=None):
        self.check(self.lib.afb_gemm_launch(ctypes.byref(args), stream), "afb_gemm_launch")

    def gemm_launch_static_status(self, args, stream=None):
        """afb_gemm_launch_static: the decode GEMM with library-resident scratch (allocates nothing, needs no init)."""
        return self.lib.afb_gemm_launch_static(ctypes.byref(args), stream)

    def gemm_host(self, args, stream=None):
        self.check(self.lib.afb_gemm_host(ctypes.byref(args), stream), "afb_gemm_host")

    def gemm_host_async(self, args, stream=None):
        self.check(self.lib.afb_gemm_host_async(ctypes.byref(args), stream), "afb_gemm_host_async")

    def gemm_host_wait(self, stream=None):
        self.check(self.lib.afb_gemm_host_wait(stream), "afb_gemm_host_wait")

    def resolve_variant(self, args):
        v = ctypes.c_uint32(0)
        self.check(self.lib.afb_gemm_resolve_variant(ctypes.byref(args), ctypes.byref(v)), "afb_gemm_resolve_variant")
        return v.value

    def prepack(self, args, out_b, out_ldb, stream=None):
        """afb_prepack: B of `args` ([K,N] or [N,K]) -> the pre-packed [N,K] layout in `out_b`."""
        self.check(self.lib.afb_prepack(ctypes.byref(args), _ptr(out_b), out_ldb, stream), "afb_prepack")

    def prepack_gated(self, gate_args, b_up, scale_up, zero_up, out_b, out_ldb, out_scale, out_zero=None, stream=None):
        """afb_prepack_gated: gate / up projections -> one row-interleaved, pre-packed B with interleaved scales (and zero-points)."""
        self.check(self.lib.afb_prepack_gated(ctypes.byref(gate_args), _ptr(b_up), _ptr(scale_up), _ptr(zero_up), _ptr(out_b), out_ldb,
                                              _ptr(out_scale), _ptr(out_zero), stream), "afb_prepack_gated")

    @staticmethod
    def make_fused_args(gemm_args, *, gated=False, activation=ACT_NONE, bias=None, residual=None, ld_residual=0):
        f = FusedArgs()
        f.gemm = gemm_args
        f.gated, f.activation = int(gated), activation
        f.ptr_bias, f.ptr_residual, f.ld_residual, f.reserved = _ptr(bias), _ptr(residual), ld_residual, 0
        return f

    def gemm_fused_launch_status(self, fused_args, stream=None):
        return self.lib.afb_gemm_fused_launch(ctypes.byref(fused_args), stream)

    def gemm_fused_launch(self, fused_args, stream=None):
        self.check(self.lib.afb_gemm_fused_launch(ctypes.byref(fused_args), stream), "afb_gemm_fused_launch")

    def dequant_dump(self, args, out, stream=None):
        self.check(self.lib.afb_dequant_dump(ctypes.byref(args), _ptr(out), stream), "afb_dequant_dump")

    def read_status(self):
        out = (ctypes.c_int32 * 4)()
        self.check(self.lib.afb_read_status(out), "afb_read_status")
        return list(out)

    def probe_launch(self, kind, src, nbytes, ctas, smem_bytes, flags=0, stream=None):
        """afb_probe_launch: an empty (kind 0) or read-only (kind 1) kernel with a decode-like launch shape."""
        f = self.lib.afb_probe_launch
        f.argtypes = [ctypes.c_uint32, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_uint32, ctypes.c_uint32, ctypes.c_uint32, ctypes.c_void_p]
        self.check(f(kind, _ptr(src), nbytes, ctas, smem_bytes, flags, stream), "afb_probe_launch")

    def phase_timestamps(self):
        """afb_phase_timestamps: ns stamps of the last row-parallel GEMM + exchange on this device (all zero unless AFB_PHASE_TIMESTAMPS is set)."""
        out = (ctypes.c_ulonglong * 8)()
        self.check(self.lib.afb_phase_timestamps(out), "afb_phase_timestamps")
        return list(out)

    def launch_count(self):
        return int(self.lib.afb_launch_count())

    def version(self):
        return self.lib.afb_version().decode()

    # ---- peer memory -------------------------------------------------------------
    def ipc_export(self, ptr):
        buf = ctypes.create_string_buffer(IPC_HANDLE_BYTES)
        self.check(self.lib.afb_ipc_export(ptr, buf), "afb_ipc_export")
        return buf.raw

    def ipc_import(self, handle):
        p = ctypes.c_void_p()
        self.check(self.lib.afb_ipc_import(handle, ctypes.byref(p)), "afb_ipc_import")
        return p.value

    def ipc_release(self, ptr):
        self.check(self.lib.afb_ipc_release(ptr), "afb_ipc_release")


_LIB = None


def load(path=None) -> Library:
    """Process-wide ``Library`` (loads ``libafb.so`` on first use; raises ``AfbError`` if absent)."""
    global _LIB
    if _LIB is None or (path and _LIB.path != path):
        _LIB = Library(path)
    return _LIB
