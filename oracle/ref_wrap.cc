// TEST INFRASTRUCTURE ONLY.  Exposes the reference's OWN host code for the bfAintBGemm path
// through a C ABI, compiled from the reference's sources where they lie (never copied):
//   gemm_rrr .................. bfAintBGemm/host_ref.hpp:3-25
//   type_convert<> ............ bfAintBGemm/datatype.hpp:32-73
//   bf16_convert_rtn<> ........ bfAintBGemm/datatype.hpp:80-121
//   mem_transfer<> ............ bfAintBGemm/mem_transfer.hpp:12-32
// Built by oracle/Makefile into oracle/_ref/libafb_hostref.so with -I<reference>/bfAintBGemm and
// -Ioracle/ref_shim (stand-ins for the two HIP headers the reference includes).
// Used to (1) generate tests/golden/*.npz, (2) validate oracle/afb_oracle.cc, (3) serve as
// bench.py's CPU arm ("kind": "reference").
#include <cmath>
#include <cstddef>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <ctime>
#include <ostream>
#include <thread>
#include <type_traits>
#include <vector>

#include "datatype.hpp"
#include "host_ref.hpp"
#include "mem_transfer.hpp"
#include "gemm_tensor_layout.hpp"
#include "validation.hpp"

extern "C" {

void ref_gemm_rrr(float* c, const float* a, const float* b, const float* scale, size_t m, size_t n, size_t k, size_t lda,
                  size_t ldb, size_t ldc) {
    gemm_rrr(c, a, b, scale, m, n, k, lda, ldb, ldc);
}
// The same function over disjoint row ranges of C on `threads` host threads (each element is still
// computed by the reference's loop, so results are bit-identical to the single-thread call).
void ref_gemm_rrr_mt(float* c, const float* a, const float* b, const float* scale, size_t m, size_t n, size_t k, size_t lda,
                     size_t ldb, size_t ldc, int threads) {
    if (threads <= 1) { gemm_rrr(c, a, b, scale, m, n, k, lda, ldb, ldc); return; }
    if ((size_t)threads > m) threads = (int)m;
    std::vector<std::thread> pool;
    for (int t = 0; t < threads; ++t) {
        const size_t lo = m * t / threads, hi = m * (t + 1) / threads;
        pool.emplace_back([=] { gemm_rrr(c + lo * ldc, a + lo * lda, b, scale, hi - lo, n, k, lda, ldb, ldc); });
    }
    for (auto& th : pool) th.join();
}
void ref_f32_to_bf16_trunc(const float* src, uint16_t* dst, size_t n) {
    for (size_t i = 0; i < n; ++i) dst[i] = type_convert<bfloat16, float>(src[i]);
}
void ref_f32_to_bf16_rtn(const float* src, uint16_t* dst, size_t n) {
    for (size_t i = 0; i < n; ++i) dst[i] = bf16_convert_rtn<bfloat16, float>(src[i]);
}
void ref_bf16_to_f32(const uint16_t* src, float* dst, size_t n) {
    for (size_t i = 0; i < n; ++i) dst[i] = type_convert<float, bfloat16>(src[i]);
}
// mem_transfer<int8_t,float,...>: fp32 master -> stored byte (value + 128)
void ref_mem_transfer_i8(const float* src, uint8_t* dst, size_t n) {
    SimpleHostMem s(n * sizeof(float)), d(n);
    float* ps = (float*)s.GetBuffer();
    for (size_t i = 0; i < n; ++i) ps[i] = src[i];
    mem_transfer<int8_t, float, SimpleHostMem, SimpleHostMem>(d, s, n);
    const uint8_t* pd = (const uint8_t*)d.GetBuffer();
    for (size_t i = 0; i < n; ++i) dst[i] = pd[i];
}
void ref_mem_transfer_bf16(const float* src, uint16_t* dst, size_t n) {
    SimpleHostMem s(n * sizeof(float)), d(n * 2);
    float* ps = (float*)s.GetBuffer();
    for (size_t i = 0; i < n; ++i) ps[i] = src[i];
    mem_transfer<bfloat16, float, SimpleHostMem, SimpleHostMem>(d, s, n);
    const uint16_t* pd = (const uint16_t*)d.GetBuffer();
    for (size_t i = 0; i < n; ++i) dst[i] = pd[i];
}
// valid_vector<bfloat16> (validation.hpp:7-46); prints as the reference does.
int ref_valid_vector_bf16(const float* ref, const uint16_t* pred, int n, float nrms) {
    return valid_vector<bfloat16>(ref, pred, n, nrms) ? 1 : 0;
}

}  // extern "C"
