// CPU check of the host driver's validation mode (interface of the reference's bfAintBGemm/host_ref.hpp:3-25).
// gemm_rrr keeps the reference's signature and arithmetic: fp32, acc += a * (b * scale[n]), k ascending, B stored
// [K,N].  gemm_ref covers what the reference has no check for: B stored [N,K] and one scale per group of k.
// This is the driver's checker, used only when the user asks for validation; it is never a compute path.
#pragma once
#include <cstddef>

// b_col_major: false -> b[k*ldb + n] ([K,N]); true -> b[n*ldb + k] ([N,K]).
// group == 0: scale[n]; else scale[n * (k/group) + kk/group].
static inline void gemm_ref(float* ptr_c, const float* __restrict__ ptr_a, const float* __restrict__ ptr_b,
                            const float* __restrict__ ptr_scale, std::size_t m, std::size_t n, std::size_t k, std::size_t lda,
                            std::size_t ldb, std::size_t ldc, bool b_col_major, std::size_t group) {
    const std::size_t groups = group ? k / group : 0;
    for (std::size_t row = 0; row < m; ++row) {
        const float* a = ptr_a + row * lda;
        for (std::size_t col = 0; col < n; ++col) {
            float sum = 0.f;
            for (std::size_t kk = 0; kk < k; ++kk) {
                const float w = b_col_major ? ptr_b[col * ldb + kk] : ptr_b[kk * ldb + col];
                const float s = group ? ptr_scale[col * groups + kk / group] : ptr_scale[col];
                sum += a[kk] * (w * s);
            }
            ptr_c[row * ldc + col] = sum;
        }
    }
}

static inline void gemm_rrr(float* ptr_c, const float* __restrict__ ptr_a, const float* __restrict__ ptr_b,
                            const float* __restrict__ ptr_scale, std::size_t m, std::size_t n, std::size_t k, std::size_t lda,
                            std::size_t ldb, std::size_t ldc) {
    gemm_ref(ptr_c, ptr_a, ptr_b, ptr_scale, m, n, k, lda, ldb, ldc, false, 0);
}
