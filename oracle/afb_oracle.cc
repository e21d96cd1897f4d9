// TEST INFRASTRUCTURE ONLY.  CPU restatement of the reference's algorithm for the
// bfAintBGemm path.  Nothing in the product (libafb.so, the driver, the Python package)
// links, imports or calls this file; it is used by tests/, by __graft_entry__.smoke() and
// by bench.py's cpu_baseline / --impl reference legs, as the checker and the timed CPU arm.
//
// What it follows in the reference (paths inside the reference project):
//   * GEMM loop and formula ........ bfAintBGemm/host_ref.hpp:15-24
//         acc(fp32) += a[m,k] * (b[k,n] * scale[n]), k ascending, no fused multiply-add
//   * bf16 <-> fp32, truncation .... bfAintBGemm/datatype.hpp:32-55
//   * fp32 -> bf16 nearest-even .... bfAintBGemm/datatype.hpp:80-121 (incl. NaN handling)
//   * int8 storage = value + 128 ... bfAintBGemm/mem_transfer.hpp:30
//   * dequant = exact int, * scale . bfAintBGemm/bf16gemm_kernel_gfx90a.s:18-35, :204-210
//   * buffer size rule ............. bfAintBGemm/bfAintBGemm.cc:68-76
// Pinned against the reference itself: tests/golden/*.npz hold outputs of the reference's
// own gemm_rrr / type_convert / bf16_convert_rtn compiled unchanged (oracle/ref_wrap.cc),
// and tests/test_oracle.py checks this restatement against them bit for bit.
// Extensions with no counterpart in the reference (int4, per-group scales, [N,K] layout,
// two's-complement storage) keep the same loop order and formula; for those, parity is
// pinned by this restatement only.
//
// Build: g++ -O2 -std=c++17 -fPIC -shared -ffp-contract=off (see oracle/Makefile).
#include <cstddef>
#include <cstdint>
#include <cstring>
#include <thread>
#include <vector>

namespace {

inline float bf16_to_f32(uint16_t h) {
    uint32_t u = (uint32_t)h << 16;
    float f;
    std::memcpy(&f, &u, 4);
    return f;
}
inline uint16_t f32_to_bf16_trunc(float f) {  // datatype.hpp:45-55
    uint32_t u;
    std::memcpy(&u, &f, 4);
    return (uint16_t)(u >> 16);
}
inline uint16_t f32_to_bf16_rne(float f) {  // datatype.hpp:80-121
    uint32_t u;
    std::memcpy(&u, &f, 4);
    if ((~u & 0x7f800000u) != 0) {
        u += 0x7fffu + ((u >> 16) & 1u);  // finite: round to nearest, ties to even
    } else if ((u & 0xffffu) != 0) {
        u |= 0x10000u;  // NaN whose payload sits in the low half: keep it a NaN
    }
    return (uint16_t)(u >> 16);
}

struct Args {
    uint32_t m, n, k, lda, ldb, ldc;
    uint32_t bits, enc, layout, scale_dtype, group;
    const uint8_t* zero = nullptr;   // optional zero-points: one byte per scale entry, in the weights' encoding
};

// Position of weight k inside its 32-bit word in the pre-packed [N,K] layout (layout 2): the GPU kernels' cheap unpack
// takes bytes (0,2),(1,3) / nibbles (0,4),(1,5),(2,6),(3,7) of a word as pairs, so consecutive k sit at those places:
//   int8: word bytes   = [k0,k2,k1,k3]           int4: word nibbles = [k0,k2,k4,k6,k1,k3,k5,k7]
inline uint32_t packed_pos(uint32_t bits, uint32_t k) {
    if (bits == 8) { const uint32_t i = k & 3u; return (k & ~3u) | ((i >> 1) | ((i & 1u) << 1)); }
    const uint32_t i = k & 7u;
    return (k & ~7u) | ((i >> 1) | ((i & 1u) << 2));
}

inline int decode8(uint8_t u, uint32_t enc) { return enc == 1 ? (int)u - 128 : (int)(int8_t)u; }
inline int decode4(int nib, uint32_t enc) { return enc == 1 ? nib - 8 : (nib >= 8 ? nib - 16 : nib); }
// Integer value of weight (n, k), exact.  layout 0: [K,N]; 1: [N,K]; 2: [N,K] pre-packed.
// With zero-points the value is decode(stored) - decode(zero): the fixed "stored - 128" of the reference
// (mem_transfer.hpp:30, bf16gemm_kernel_gfx90a.s:210) with the 128 replaced by a per-channel / per-group byte.
inline int weight_q(const uint8_t* b, const Args& a, uint32_t n, uint32_t k) {
    const uint32_t kk = a.layout == 2 ? packed_pos(a.bits, k) : k;
    int z = 0;
    if (a.zero) {
        const uint8_t zb = a.zero[a.group ? (size_t)n * (a.k / a.group) + k / a.group : n];
        z = a.bits == 8 ? decode8(zb, a.enc) : decode4(zb & 0xF, a.enc);
    }
    if (a.bits == 8) {
        const size_t idx = a.layout != 0 ? (size_t)n * a.ldb + kk : (size_t)k * a.ldb + n;
        return decode8(b[idx], a.enc) - z;
    }
    const uint8_t byte = b[(size_t)n * (a.ldb / 2) + kk / 2];
    const int nib = (kk & 1) ? (byte >> 4) : (byte & 0xF);
    return decode4(nib, a.enc) - z;
}
inline float scale_at(const void* s, const Args& a, uint32_t n, uint32_t k) {
    const size_t idx = a.group ? (size_t)n * (a.k / a.group) + k / a.group : n;
    return a.scale_dtype == 1 ? bf16_to_f32(((const uint16_t*)s)[idx]) : ((const float*)s)[idx];
}

// rows [m_begin, m_end) of C.  round_w: feed bf16_rn(q * scale) instead of the fp32 product
// (what a tensor-core kernel with per-group scales must do, since its operands are bf16).
void gemm_rows(float* c, const uint16_t* a_bf16, const uint8_t* b, const void* scale, const Args& a, uint32_t m_begin,
               uint32_t m_end, int round_w) {
    std::vector<float> wcol(a.k);
    for (uint32_t n = 0; n < a.n; ++n) {
        for (uint32_t k = 0; k < a.k; ++k) {  // b * scale, exactly as host_ref.hpp:20 forms it
            float w = (float)weight_q(b, a, n, k) * scale_at(scale, a, n, k);
            if (round_w) w = bf16_to_f32(f32_to_bf16_rne(w));
            wcol[k] = w;
        }
        for (uint32_t m = m_begin; m < m_end; ++m) {
            const uint16_t* arow = a_bf16 + (size_t)m * a.lda;
            float acc = 0.f;
            for (uint32_t k = 0; k < a.k; ++k) acc += bf16_to_f32(arow[k]) * wcol[k];
            c[(size_t)m * a.ldc + n] = acc;
        }
    }
}

}  // namespace

extern "C" {

void afb_oracle_f32_to_bf16_trunc(const float* src, uint16_t* dst, size_t n) {
    for (size_t i = 0; i < n; ++i) dst[i] = f32_to_bf16_trunc(src[i]);
}
void afb_oracle_f32_to_bf16_rne(const float* src, uint16_t* dst, size_t n) {
    for (size_t i = 0; i < n; ++i) dst[i] = f32_to_bf16_rne(src[i]);
}
void afb_oracle_bf16_to_f32(const uint16_t* src, float* dst, size_t n) {
    for (size_t i = 0; i < n; ++i) dst[i] = bf16_to_f32(src[i]);
}
// fp32 master -> stored int8 (mem_transfer.hpp:23-32): C++ float->int8 conversion, then + 128 when offset-binary.
void afb_oracle_f32_to_i8(const float* src, uint8_t* dst, size_t n, uint32_t enc) {
    for (size_t i = 0; i < n; ++i) dst[i] = (uint8_t)((int8_t)src[i] + (enc == 1 ? 128 : 0));
}
// fp32 master (integers in [-8,7]) -> packed nibbles, two per byte, low nibble = even index.
void afb_oracle_f32_to_i4(const float* src, uint8_t* dst, size_t n, uint32_t enc) {
    for (size_t i = 0; i < n; i += 2) {
        const int q0 = (int)src[i], q1 = i + 1 < n ? (int)src[i + 1] : 0;
        const uint8_t n0 = (uint8_t)((enc == 1 ? q0 + 8 : q0) & 0xF), n1 = (uint8_t)((enc == 1 ? q1 + 8 : q1) & 0xF);
        dst[i / 2] = (uint8_t)(n0 | (n1 << 4));
    }
}

// Dequantised weights as bf16 in B's own logical shape ([N,K] ld=K for layout 1, [K,N] ld=N for layout 0):
// group == 0: the exact integer; else bf16_rne(float(q) * float(scale)).
void afb_oracle_dequant_bf16(uint16_t* out, const uint8_t* b, const void* scale, uint32_t n, uint32_t k, uint32_t ldb,
                             uint32_t bits, uint32_t enc, uint32_t layout, uint32_t scale_dtype, uint32_t group, const uint8_t* zero) {
    Args a{0, n, k, 0, ldb, 0, bits, enc, layout, scale_dtype, group, zero};
    for (uint32_t in = 0; in < n; ++in)
        for (uint32_t ik = 0; ik < k; ++ik) {
            float w = (float)weight_q(b, a, in, ik);
            if (group) w = w * scale_at(scale, a, in, ik);
            const size_t o = layout != 0 ? (size_t)in * k + ik : (size_t)ik * n + in;
            out[o] = f32_to_bf16_rne(w);
        }
}

// Weight pre-packing, restated: B in layout 0 ([K,N], int8) or 1 ([N,K]) -> layout 2 ([N,K], pitch out_ldb elements), the
// stored integers unchanged, only moved (the host-side format step this extends is mem_transfer.hpp:12-32).
void afb_oracle_prepack(uint8_t* out, const uint8_t* b, uint32_t n, uint32_t k, uint32_t ldb, uint32_t out_ldb, uint32_t bits, uint32_t layout) {
    for (uint32_t in = 0; in < n; ++in)
        for (uint32_t ik = 0; ik < k; ++ik) {
            const uint32_t kk = packed_pos(bits, ik);
            if (bits == 8) {
                out[(size_t)in * out_ldb + kk] = layout == 0 ? b[(size_t)ik * ldb + in] : b[(size_t)in * ldb + ik];
            } else {
                const uint8_t src = b[(size_t)in * (ldb / 2) + ik / 2];
                const uint8_t nib = (ik & 1) ? (src >> 4) : (src & 0xF);
                uint8_t& dst = out[(size_t)in * (out_ldb / 2) + kk / 2];
                dst = (kk & 1) ? (uint8_t)((dst & 0x0F) | (nib << 4)) : (uint8_t)((dst & 0xF0) | nib);
            }
        }
}

// The GEMM on device-format inputs.  C is fp32 [M,N] (ldc).  threads <= 1: the scalar loop;
// otherwise rows of C are split over `threads` host threads, each element computed identically.
void afb_oracle_gemm(float* c, const uint16_t* a_bf16, const uint8_t* b, const void* scale, uint32_t m, uint32_t n,
                     uint32_t k, uint32_t lda, uint32_t ldb, uint32_t ldc, uint32_t bits, uint32_t enc, uint32_t layout,
                     uint32_t scale_dtype, uint32_t group, int round_w, int threads, const uint8_t* zero) {
    Args a{m, n, k, lda, ldb, ldc, bits, enc, layout, scale_dtype, group, zero};
    if (threads <= 1) { gemm_rows(c, a_bf16, b, scale, a, 0, m, round_w); return; }
    if ((uint32_t)threads > m) threads = (int)m;
    std::vector<std::thread> pool;
    for (int t = 0; t < threads; ++t) {
        const uint32_t lo = (uint32_t)((uint64_t)m * t / threads), hi = (uint32_t)((uint64_t)m * (t + 1) / threads);
        pool.emplace_back([=, &a] { gemm_rows(c, a_bf16, b, scale, a, lo, hi, round_w); });
    }
    for (auto& th : pool) th.join();
}

// The reference's own signature on fp32 masters (host_ref.hpp:3-25): B is [K,N], scale per n.
void afb_oracle_gemm_rrr(float* c, const float* a, const float* b, const float* scale, size_t m, size_t n, size_t k,
                         size_t lda, size_t ldb, size_t ldc) {
    for (size_t im = 0; im < m; ++im)
        for (size_t in = 0; in < n; ++in) {
            const float s = scale[in];
            float acc = 0.f;
            for (size_t ik = 0; ik < k; ++ik) acc += a[im * lda + ik] * (b[ik * ldb + in] * s);
            c[im * ldc + in] = acc;
        }
}

// Validation metric used by the tests: max |r - p| / max(|r|, floor) and the NRMS of validation.hpp:7-46
// (sqrt(sum d^2 / sum 2 r^2)).  The reference divides by the signed r (validation.hpp:27); that quirk is not kept.
void afb_oracle_compare(const float* ref, const uint16_t* pred_bf16, size_t count, float floor_abs, double* max_rel,
                        double* nrms, size_t* worst) {
    double s0 = 0, s1 = 0, mx = 0;
    size_t wi = 0;
    for (size_t i = 0; i < count; ++i) {
        const double r = ref[i], p = bf16_to_f32(pred_bf16[i]);
        const double d = r - p;
        s0 += d * d;
        s1 += 2.0 * r * r;
        const double den = (r < 0 ? -r : r) > floor_abs ? (r < 0 ? -r : r) : floor_abs;
        const double rel = (d < 0 ? -d : d) / den;
        if (!(rel <= mx)) { mx = rel; wi = i; }  // NaN propagates to the result
    }
    *max_rel = mx;
    *nrms = s1 > 0 ? __builtin_sqrt(s0 / s1) : (s0 > 0 ? 1e30 : 0);
    *worst = wi;
}

}  // extern "C"
