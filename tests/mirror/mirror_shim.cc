// TEST INFRASTRUCTURE ONLY.  Exposes the host-side mirror headers (include/bfAintBGemm/*.hpp, the
// re-written counterparts of the reference's bfAintBGemm/datatype.hpp, mem_transfer.hpp, host_ref.hpp
// and validation.hpp) through a C ABI so that the Python tests can feed them the golden vectors that
// were recorded from the reference's own host code.  Built on the fly by tests/test_mirror_headers.py.
#include <cstddef>
#include <cstdint>
#include <cstring>

#include "bfAintBGemm/datatype.hpp"
#include "bfAintBGemm/gemm_tensor_layout.hpp"
#include "bfAintBGemm/host_ref.hpp"
#include "bfAintBGemm/mem_transfer.hpp"
#include "bfAintBGemm/validation.hpp"

namespace {
template <typename F>
void through_host_mem(const void* src, size_t src_bytes, void* dst, size_t dst_bytes, F&& f) {
    SimpleHostMem s(src_bytes), d(dst_bytes);
    std::memcpy(s.GetBuffer(), src, src_bytes);
    f(d, s);
    std::memcpy(dst, d.GetBuffer(), dst_bytes);
}
}  // namespace

extern "C" {

void mir_f32_to_bf16_trunc(const float* src, uint16_t* dst, size_t n) {
    for (size_t i = 0; i < n; ++i) dst[i] = type_convert<bfloat16, float>(src[i]);
}
void mir_f32_to_bf16_rtn(const float* src, uint16_t* dst, size_t n) {
    for (size_t i = 0; i < n; ++i) dst[i] = bf16_convert_rtn<bfloat16, float>(src[i]);
}
void mir_bf16_to_f32(const uint16_t* src, float* dst, size_t n) {
    for (size_t i = 0; i < n; ++i) dst[i] = type_convert<float, bfloat16>(src[i]);
}
void mir_bf16_to_i8(const uint16_t* src, int8_t* dst, size_t n) {
    for (size_t i = 0; i < n; ++i) dst[i] = type_convert<int8_t, bfloat16>(src[i]);
}
void mir_i8_to_bf16(const int8_t* src, uint16_t* dst, size_t n) {
    for (size_t i = 0; i < n; ++i) dst[i] = type_convert<bfloat16, int8_t>(src[i]);
}
// mem_transfer<int8_t, float, ...>: fp32 master -> stored byte (value + 128)
void mir_mem_transfer_i8(const float* src, uint8_t* dst, size_t n) {
    through_host_mem(src, n * 4, dst, n, [n](SimpleHostMem& d, SimpleHostMem& s) { mem_transfer<int8_t, float, SimpleHostMem, SimpleHostMem>(d, s, n); });
}
// mem_transfer<bfloat16, float, ...>: truncation
void mir_mem_transfer_bf16(const float* src, uint16_t* dst, size_t n) {
    through_host_mem(src, n * 4, dst, n * 2, [n](SimpleHostMem& d, SimpleHostMem& s) { mem_transfer<bfloat16, float, SimpleHostMem, SimpleHostMem>(d, s, n); });
}
// round-to-nearest-even variant; master_out receives the fp32 master after the write-back
void mir_mem_transfer_bf16_rne(const float* src, uint16_t* dst, float* master_out, size_t n) {
    SimpleHostMem s(n * 4), d(n * 2);
    std::memcpy(s.GetBuffer(), src, n * 4);
    mem_transfer_bf16_rne(d, s, n, true);
    std::memcpy(dst, d.GetBuffer(), n * 2);
    std::memcpy(master_out, s.GetBuffer(), n * 4);
}
void mir_mem_transfer_int8_twos(const float* src, uint8_t* dst, size_t n) {
    through_host_mem(src, n * 4, dst, n, [n](SimpleHostMem& d, SimpleHostMem& s) { mem_transfer_int8_twos(d, s, n); });
}
void mir_mem_transfer_int4(const float* src, uint8_t* dst, size_t n, int offset_binary) {
    through_host_mem(src, n * 4, dst, (n + 1) / 2, [n, offset_binary](SimpleHostMem& d, SimpleHostMem& s) { mem_transfer_int4(d, s, n, offset_binary != 0); });
}
void mir_gemm_rrr(float* c, const float* a, const float* b, const float* scale, size_t m, size_t n, size_t k, size_t lda, size_t ldb, size_t ldc) {
    gemm_rrr(c, a, b, scale, m, n, k, lda, ldb, ldc);
}
void mir_gemm_ref(float* c, const float* a, const float* b, const float* scale, size_t m, size_t n, size_t k, size_t lda, size_t ldb, size_t ldc,
                  int b_col_major, size_t group) {
    gemm_ref(c, a, b, scale, m, n, k, lda, ldb, ldc, b_col_major != 0, group);
}
int mir_valid_vector_bf16(const float* ref, const uint16_t* pred, int n, float nrms, float rel_tol, float floor_frac) {
    return valid_vector<bfloat16>(ref, pred, n, nrms, rel_tol, floor_frac) ? 1 : 0;
}
// the size rule of the driver (bfAintBGemm.cc:68-76) as the mirror states it
size_t mir_matrix_space_size(size_t rows, size_t cols, size_t ld, int row_major) {
    return row_major ? gemm_layout::matrix_space_size(rows, cols, ld, gemm_layout::gemm::RowMajor{})
                     : gemm_layout::matrix_space_size(rows, cols, ld, gemm_layout::gemm::ColumnMajor{});
}

}  // extern "C"
