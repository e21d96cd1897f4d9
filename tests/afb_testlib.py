"""Shared helpers of the test-suite: the CPU oracle (ctypes), seeded input generators that follow the
distributions of the benchmark configurations, and the comparison metric.  Test infrastructure only."""
import ctypes
import os
import subprocess

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ORACLE_DIR = os.path.join(ROOT, "oracle")

_u16p = ctypes.POINTER(ctypes.c_uint16)
_u8p = ctypes.POINTER(ctypes.c_uint8)
_f32p = ctypes.POINTER(ctypes.c_float)


def _p(arr, typ):
    return arr.ctypes.data_as(typ)


class Oracle:
    def __init__(self, path):
        self.lib = ctypes.CDLL(path)
        L = self.lib
        u32, sz, vp, i = ctypes.c_uint32, ctypes.c_size_t, ctypes.c_void_p, ctypes.c_int
        L.afb_oracle_f32_to_bf16_trunc.argtypes = [_f32p, _u16p, sz]
        L.afb_oracle_f32_to_bf16_rne.argtypes = [_f32p, _u16p, sz]
        L.afb_oracle_bf16_to_f32.argtypes = [_u16p, _f32p, sz]
        L.afb_oracle_f32_to_i8.argtypes = [_f32p, _u8p, sz, u32]
        L.afb_oracle_f32_to_i4.argtypes = [_f32p, _u8p, sz, u32]
        L.afb_oracle_dequant_bf16.argtypes = [_u16p, _u8p, vp, u32, u32, u32, u32, u32, u32, u32, u32, vp]
        L.afb_oracle_gemm.argtypes = [_f32p, _u16p, _u8p, vp] + [u32] * 11 + [i, i, vp]
        L.afb_oracle_prepack.argtypes = [_u8p, _u8p] + [u32] * 6
        L.afb_oracle_gemm_rrr.argtypes = [_f32p, _f32p, _f32p, _f32p] + [sz] * 6
        L.afb_oracle_compare.argtypes = [_f32p, _u16p, sz, ctypes.c_float, ctypes.POINTER(ctypes.c_double),
                                         ctypes.POINTER(ctypes.c_double), ctypes.POINTER(sz)]

    def bf16_trunc(self, x):
        x = np.ascontiguousarray(x, np.float32)
        out = np.empty(x.shape, np.uint16)
        self.lib.afb_oracle_f32_to_bf16_trunc(_p(x, _f32p), _p(out, _u16p), x.size)
        return out

    def bf16_rne(self, x):
        x = np.ascontiguousarray(x, np.float32)
        out = np.empty(x.shape, np.uint16)
        self.lib.afb_oracle_f32_to_bf16_rne(_p(x, _f32p), _p(out, _u16p), x.size)
        return out

    def bf16_to_f32(self, x):
        x = np.ascontiguousarray(x, np.uint16)
        out = np.empty(x.shape, np.float32)
        self.lib.afb_oracle_bf16_to_f32(_p(x, _u16p), _p(out, _f32p), x.size)
        return out

    def to_i8(self, x, enc):
        x = np.ascontiguousarray(x, np.float32)
        out = np.empty(x.shape, np.uint8)
        self.lib.afb_oracle_f32_to_i8(_p(x, _f32p), _p(out, _u8p), x.size, enc)
        return out

    def to_i4(self, x, enc):
        x = np.ascontiguousarray(x, np.float32)
        assert x.shape[-1] % 2 == 0
        out = np.empty(x.shape[:-1] + (x.shape[-1] // 2,), np.uint8)
        self.lib.afb_oracle_f32_to_i4(_p(x, _f32p), _p(out, _u8p), x.size, enc)
        return out

    def dequant_bf16(self, case):
        c = case
        shape = (c.n, c.k) if c.layout != 0 else (c.k, c.n)
        out = np.empty(shape, np.uint16)
        self.lib.afb_oracle_dequant_bf16(_p(out, _u16p), _p(c.b, _u8p), c.scale.ctypes.data, c.n, c.k, c.ldb, c.bits, c.enc,
                                         c.layout, c.scale_dtype, c.group, self._zero_ptr(c))
        return out

    @staticmethod
    def _zero_ptr(case):
        z = getattr(case, "zero", None)
        return None if z is None else z.ctypes.data

    def prepack(self, case, out_ldb=None):
        """The Case with B pre-packed (layout 2), by the CPU restatement of afb_prepack."""
        c = case
        out_ldb = out_ldb or c.k
        out = np.zeros((c.n, out_ldb * c.bits // 8), np.uint8)
        self.lib.afb_oracle_prepack(_p(out, _u8p), _p(c.b, _u8p), c.n, c.k, c.ldb, out_ldb, c.bits, c.layout)
        return Case(**{**c.__dict__, "b": out, "layout": 2, "ldb": out_ldb})

    def gemm(self, case, round_w=False, threads=1, rows=None):
        """fp32 C of the oracle; ``rows`` restricts to a list of activation rows (used at full sizes)."""
        c = case
        a = c.a if rows is None else np.ascontiguousarray(c.a[rows])
        m = a.shape[0]
        out = np.empty((m, c.n), np.float32)
        self.lib.afb_oracle_gemm(_p(out, _f32p), _p(a, _u16p), _p(c.b, _u8p), c.scale.ctypes.data, m, c.n, c.k, c.k, c.ldb,
                                 c.n, c.bits, c.enc, c.layout, c.scale_dtype, c.group, int(round_w), threads, self._zero_ptr(c))
        return out

    def gemm_rrr(self, a, b, scale):
        a = np.ascontiguousarray(a, np.float32); b = np.ascontiguousarray(b, np.float32)
        scale = np.ascontiguousarray(scale, np.float32)
        m, k = a.shape; n = b.shape[1]
        out = np.empty((m, n), np.float32)
        self.lib.afb_oracle_gemm_rrr(_p(out, _f32p), _p(a, _f32p), _p(b, _f32p), _p(scale, _f32p), m, n, k, k, n, n)
        return out

    def compare(self, ref, pred_bf16, floor_abs):
        ref = np.ascontiguousarray(ref, np.float32); pred = np.ascontiguousarray(pred_bf16, np.uint16)
        assert ref.size == pred.size
        mx, nr, w = ctypes.c_double(), ctypes.c_double(), ctypes.c_size_t()
        self.lib.afb_oracle_compare(_p(ref, _f32p), _p(pred, _u16p), ref.size, floor_abs, ctypes.byref(mx), ctypes.byref(nr),
                                    ctypes.byref(w))
        return mx.value, nr.value, w.value


def load_oracle():
    path = os.path.join(ORACLE_DIR, "libafb_oracle.so")
    if not os.path.exists(path):
        subprocess.check_call(["make", "-C", ORACLE_DIR, "libafb_oracle.so"])
    return Oracle(path)


class HostRef:
    """The reference's own host code (oracle/_ref/libafb_hostref.so, built from the reference sources)."""

    def __init__(self, path):
        self.lib = ctypes.CDLL(path)
        sz = ctypes.c_size_t
        self.lib.ref_gemm_rrr.argtypes = [_f32p, _f32p, _f32p, _f32p] + [sz] * 6
        self.lib.ref_gemm_rrr_mt.argtypes = [_f32p, _f32p, _f32p, _f32p] + [sz] * 6 + [ctypes.c_int]
        self.lib.ref_f32_to_bf16_trunc.argtypes = [_f32p, _u16p, sz]
        self.lib.ref_f32_to_bf16_rtn.argtypes = [_f32p, _u16p, sz]
        self.lib.ref_bf16_to_f32.argtypes = [_u16p, _f32p, sz]
        self.lib.ref_mem_transfer_i8.argtypes = [_f32p, _u8p, sz]
        self.lib.ref_mem_transfer_bf16.argtypes = [_f32p, _u16p, sz]

    def gemm_rrr(self, a, b, scale, threads=1):
        a = np.ascontiguousarray(a, np.float32); b = np.ascontiguousarray(b, np.float32)
        scale = np.ascontiguousarray(scale, np.float32)
        m, k = a.shape; n = b.shape[1]
        out = np.empty((m, n), np.float32)
        self.lib.ref_gemm_rrr_mt(_p(out, _f32p), _p(a, _f32p), _p(b, _f32p), _p(scale, _f32p), m, n, k, k, n, n, threads)
        return out

    def _conv(self, fn, x, it, ot, ity, oty):
        x = np.ascontiguousarray(x, it)
        out = np.empty(x.shape, ot)
        fn(_p(x, ity), _p(out, oty), x.size)
        return out

    def bf16_trunc(self, x): return self._conv(self.lib.ref_f32_to_bf16_trunc, x, np.float32, np.uint16, _f32p, _u16p)
    def bf16_rtn(self, x): return self._conv(self.lib.ref_f32_to_bf16_rtn, x, np.float32, np.uint16, _f32p, _u16p)
    def bf16_to_f32(self, x): return self._conv(self.lib.ref_bf16_to_f32, x, np.uint16, np.float32, _u16p, _f32p)
    def mem_transfer_i8(self, x): return self._conv(self.lib.ref_mem_transfer_i8, x, np.float32, np.uint8, _f32p, _u8p)
    def mem_transfer_bf16(self, x): return self._conv(self.lib.ref_mem_transfer_bf16, x, np.float32, np.uint16, _f32p, _u16p)


def load_hostref():
    path = os.path.join(ORACLE_DIR, "_ref", "libafb_hostref.so")
    return HostRef(path) if os.path.exists(path) else None


# --------------------------------------------------------------------------------------
# inputs
# --------------------------------------------------------------------------------------
def np_bf16_rne(x):
    """fp32 -> bf16 bits, round to nearest even (finite inputs)."""
    u = np.ascontiguousarray(x, np.float32).view(np.uint32).astype(np.uint64)
    u = u + 0x7FFF + ((u >> 16) & 1)
    return (u >> 16).astype(np.uint16)


def np_bf16_to_f32(h):
    return (np.ascontiguousarray(h, np.uint16).astype(np.uint32) << 16).view(np.float32)


class Case:
    """One problem instance in device formats (numpy arrays) plus its mode fields."""

    def __init__(self, **kw):
        self.__dict__.update(kw)

    def scale_f32(self):
        return np_bf16_to_f32(self.scale) if self.scale_dtype == 1 else self.scale


def make_case(m, n, k, *, bits=8, group=0, layout=1, enc=0, scale_dtype=None, seed=0, a_dist="normal",
              scale_range=(0.001, 0.01), integer_data=False, qmax=None, zero_points=False):
    """Seeded inputs with the distributions the benchmark configurations name: A ~ N(0,1) (or
    uniform[-1,1]) rounded to bf16; B integers uniform in [-127,127] (int8) or [-8,7] (int4);
    scales uniform in ``scale_range``.  ``integer_data`` reproduces the reference's own test data
    (every value an integer in {-2,-1,0,1}, random_gen.hpp:24,37,50), for which results are exact."""
    rng = np.random.default_rng(seed)
    if scale_dtype is None:
        scale_dtype = 1 if group else 0
    if integer_data:
        a32 = rng.integers(-2, 2, size=(m, k)).astype(np.float32)
        q = rng.integers(-2, 2, size=(n, k), dtype=np.int8)
    else:
        a32 = (rng.standard_normal((m, k), dtype=np.float32) if a_dist == "normal" else rng.uniform(-1, 1, (m, k)).astype(np.float32))
        lim = qmax if qmax is not None else (127 if bits == 8 else None)
        q = rng.integers(-lim, lim + 1, size=(n, k), dtype=np.int8) if lim is not None else rng.integers(-8, 8, size=(n, k), dtype=np.int8)
    a = np_bf16_rne(a32)
    ngroups = k // group if group else 1
    if integer_data:
        s32 = rng.integers(-2, 2, size=(n, ngroups)).astype(np.float32)
    else:
        s32 = rng.uniform(scale_range[0], scale_range[1], size=(n, ngroups)).astype(np.float32)
    if not group:
        s32 = s32.reshape(n)
    scale = np_bf16_rne(s32) if scale_dtype == 1 else s32
    if bits == 8:
        b = q.view(np.uint8) ^ np.uint8(0x80 if enc == 1 else 0)   # value + 128 == two's complement with the top bit flipped
        if layout == 0:
            b = np.ascontiguousarray(b.T)  # [K,N]
        ldb = k if layout == 1 else n
    else:
        assert layout == 1
        u = (q.view(np.uint8) ^ np.uint8(0x8 if enc == 1 else 0)) & np.uint8(0xF)
        b = u[:, 0::2] | (u[:, 1::2] << np.uint8(4))
        ldb = k
    zero = None
    if zero_points:   # one byte per scale entry, in the weights' own encoding: any int8 value / any nibble
        zv = rng.integers(-128, 128, size=(n, ngroups)) if bits == 8 else rng.integers(-8, 8, size=(n, ngroups))
        zero = (zv.astype(np.int8).view(np.uint8) ^ np.uint8((0x80 if bits == 8 else 0x8) if enc == 1 else 0)) & np.uint8(0xFF if bits == 8 else 0xF)
        zero = np.ascontiguousarray(zero.reshape(n, ngroups) if group else zero.reshape(n))
    return Case(m=m, n=n, k=k, bits=bits, group=group, layout=layout, enc=enc, scale_dtype=scale_dtype, a=a, b=np.ascontiguousarray(b),
                scale=np.ascontiguousarray(scale), q=q, ldb=ldb, seed=seed, zero=zero)


# --------------------------------------------------------------------------------------
# running a case through the C ABI
# --------------------------------------------------------------------------------------
class DeviceCase:
    """Device copies of a Case; frees them on close()."""

    def __init__(self, lib, case, c_f32=False, ldc=None, guard=0, lda=None, ldb=None):
        self.lib, self.case = lib, case
        self.ldc = ldc or case.n
        self.lda = lda or case.k
        self.ldb = ldb or case.ldb
        self.c_elt = 4 if c_f32 else 2
        self.guard = guard
        self.c_bytes = ((case.m - 1) * self.ldc + case.n) * self.c_elt
        a_host, b_host = case.a, case.b
        if self.lda != case.k:                       # rows of A padded to lda elements (padding filled with a recognisable pattern)
            a_host = np.full((case.m, self.lda), 0x7FC0, np.uint16); a_host[:, :case.k] = case.a
        if self.ldb != case.ldb:                     # rows of B padded to ldb elements (bytes for int8, nibbles for int4)
            row_bytes = self.ldb * case.bits // 8
            b_host = np.full((case.b.shape[0], row_bytes), 0x55, np.uint8); b_host[:, :case.b.shape[1]] = case.b
        self.d_a = lib.to_device(a_host)
        self.d_b = lib.to_device(b_host)
        self.d_s = lib.to_device(case.scale)
        self.d_z = lib.to_device(case.zero) if getattr(case, "zero", None) is not None else None
        self.d_c_base = lib.malloc(self.c_bytes + 2 * guard)
        lib.memset(self.d_c_base, 0xCD, self.c_bytes + 2 * guard)
        self.d_c = self.d_c_base + guard

    def args(self, variant=0, flags=0):
        c = self.case
        return self.lib.make_args(self.d_c, self.d_a, self.d_b, self.d_s, c.m, c.n, c.k, lda=self.lda, ldb=self.ldb, ldc=self.ldc, bits=c.bits,
                                  encoding=c.enc, layout=c.layout, scale_dtype=c.scale_dtype, group=c.group, variant=variant,
                                  flags=flags, zero=self.d_z)

    def result(self):
        """C as a [M, N] array (bf16 bits or fp32) and the raw buffer including guards."""
        raw = self.lib.to_host(self.d_c_base, (self.c_bytes + 2 * self.guard,), np.uint8)
        body = raw[self.guard:self.guard + self.c_bytes]
        dt = np.float32 if self.c_elt == 4 else np.uint16
        flat = body.view(dt)
        c = self.case
        full = np.zeros((c.m, self.ldc), dt)
        full.reshape(-1)[:flat.size] = flat
        return full[:, :c.n].copy(), raw

    def close(self):
        for p in (self.d_a, self.d_b, self.d_s, self.d_c_base, self.d_z):
            if p is not None:
                self.lib.free(p)


def run_case(lib, case, variant=0, c_f32=False, ldc=None, guard=0, flags=0, lda=None, ldb=None):
    dc = DeviceCase(lib, case, c_f32=c_f32, ldc=ldc, guard=guard, lda=lda, ldb=ldb)
    try:
        lib.gemm_launch(dc.args(variant=variant, flags=flags | (1 if c_f32 else 0)))
        lib.device_sync()
        out, raw = dc.result()
    finally:
        dc.close()
    return out, raw


def rms(x):
    return float(np.sqrt(np.mean(np.square(x.astype(np.float64)))))
