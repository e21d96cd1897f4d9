// Layout tags of the GEMM operands (interface of the reference's bfAintBGemm/gemm_tensor_layout.hpp:5-28).
// A K x N matrix B tagged RowMajor is stored [K,N] with N contiguous (the reference's own choice,
// bfAintBGemm.cc:20-23); tagged ColumnMajor it is stored [N,K] with K contiguous, the layout the fast kernels read.
#pragma once
#include <ostream>
#include <type_traits>

namespace gemm_layout {

struct BaseTensorLayout {};

namespace gemm {
struct RowMajor : BaseTensorLayout { static constexpr const char* name = "RowMajor"; };
struct ColumnMajor : BaseTensorLayout { static constexpr const char* name = "ColumnMajor"; };
}  // namespace gemm

template <typename Layout, std::enable_if_t<std::is_base_of_v<BaseTensorLayout, Layout>, int> = 0>
std::ostream& operator<<(std::ostream& os, const Layout&) { return os << Layout::name; }

// Elements a rows x cols matrix with leading dimension ld occupies (the size rule of bfAintBGemm.cc:68-76).
template <typename Layout>
constexpr std::size_t matrix_space_size(std::size_t rows, std::size_t cols, std::size_t ld, Layout) {
    if constexpr (std::is_same_v<Layout, gemm::RowMajor>) return (rows - 1) * ld + cols;
    else return (cols - 1) * ld + rows;
}

}  // namespace gemm_layout
