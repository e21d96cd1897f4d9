"""Generates tests/golden/*.npz from the reference's OWN host code.

Run in a checkout where the reference sources are present:
    make -C oracle REF=<reference checkout>/bfAintBGemm     # builds oracle/_ref/libafb_hostref.so from the reference's headers
    python tests/golden/make_golden.py
The reference has no test vectors of its own (its only check is the opt-in comparison of
bfAintBGemm.cc:198-214 on time-seeded data), so these files record what its host functions
return on fixed seeded inputs: gemm_rrr (host_ref.hpp:3-25), type_convert / bf16_convert_rtn
(datatype.hpp:32-121) and mem_transfer (mem_transfer.hpp:12-32).  Inputs are stored with the
outputs so that the tests need neither the reference nor this script.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
import afb_testlib as T  # noqa: E402


def main():
    ref = T.load_hostref()
    if ref is None:
        raise SystemExit("oracle/_ref/libafb_hostref.so is missing: run `make -C oracle` next to the reference sources")

    # ---- conversions: specials, ties, subnormals, NaN payloads, plus seeded random bits ----
    specials = np.array([0x00000000, 0x80000000, 0x3F800000, 0xBF800000, 0x3F808000, 0x3F818000, 0x3F807FFF, 0x3F808001,
                         0x7F7FFFFF, 0xFF7FFFFF, 0x7F800000, 0xFF800000, 0x7FC00000, 0x7F800001, 0x7F80FFFF, 0xFFC12345,
                         0x00000001, 0x00008000, 0x0000FFFF, 0x007FFFFF, 0x00800000, 0x7F7F8000, 0x3EFFFFFF, 0x4B000080,
                         0x43000000, 0xC3000000, 0x42FE0000, 0x3B03126F], dtype=np.uint32)
    rng = np.random.default_rng(1234)
    bits = np.concatenate([specials, rng.integers(0, 2**32, size=4096, dtype=np.uint64).astype(np.uint32)])
    f = bits.view(np.float32)
    np.savez_compressed(os.path.join(HERE, "conversions.npz"), f32_bits=bits, bf16_trunc=ref.bf16_trunc(f), bf16_rtn=ref.bf16_rtn(f),
                        bf16_all=np.arange(65536, dtype=np.uint16)[::37].copy(),
                        bf16_all_f32_bits=ref.bf16_to_f32(np.arange(65536, dtype=np.uint16)[::37].copy()).view(np.uint32),
                        i8_src=np.arange(-128, 128, dtype=np.float32), i8_plus128=ref.mem_transfer_i8(np.arange(-128, 128, dtype=np.float32)))

    # ---- gemm_rrr, reference-style data: every value an integer in {-2,-1,0,1} (random_gen.hpp:24,37,50),
    #      default problem m=32 n=128 k=512 (bfAintBGemm.cc:39-41) ----
    rng = np.random.default_rng(0)
    m, n, k = 32, 128, 512
    a = rng.integers(-2, 2, size=(m, k)).astype(np.float32)
    b = rng.integers(-2, 2, size=(k, n)).astype(np.float32)
    s = rng.integers(-2, 2, size=(n,)).astype(np.float32)
    np.savez_compressed(os.path.join(HERE, "gemm_rrr_integer.npz"), a=a.astype(np.int8), b=b.astype(np.int8), scale=s.astype(np.int8),
                        c=ref.gemm_rrr(a, b, s))

    # ---- gemm_rrr, real-valued data with the distributions of the CPU-checkable configuration:
    #      A uniform[-1,1] already rounded to bf16, B integers in [-127,127], scale uniform[0.002,0.02] ----
    rng = np.random.default_rng(0)
    m, n, k = 24, 96, 320
    a = T.np_bf16_to_f32(T.np_bf16_rne(rng.uniform(-1, 1, (m, k)).astype(np.float32)))
    b = rng.integers(-127, 128, size=(k, n)).astype(np.float32)
    s = rng.uniform(0.002, 0.02, size=(n,)).astype(np.float32)
    np.savez_compressed(os.path.join(HERE, "gemm_rrr_real.npz"), a_bf16=T.np_bf16_rne(a), b=b.astype(np.int8), scale=s,
                        c=ref.gemm_rrr(a, b, s))
    for fn in sorted(os.listdir(HERE)):
        if fn.endswith(".npz"):
            print(fn, os.path.getsize(os.path.join(HERE, fn)), "bytes")


if __name__ == "__main__":
    main()
