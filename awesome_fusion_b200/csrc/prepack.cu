// Weight pre-packing: the offline step before the GEMM (the reference's counterpart is the host-side format conversion
// mem_transfer<int8_t, float> of bfAintBGemm/mem_transfer.hpp:23-32, called once at bfAintBGemm.cc:96-97).
//
// Output layout AFB_LAYOUT_COL_PACKED: [N,K], K contiguous, same pitch rules as AFB_LAYOUT_COL; the stored integers are
// unchanged, only moved inside every 32-bit word to the places the kernels' cheap unpack reads as pairs:
//     int8: word bytes   [k0,k2,k1,k3]             int4: word nibbles [k0,k2,k4,k6,k1,k3,k5,k7]
// so that the unpack (dequant.cuh: bytes (0,2),(1,3) / nibbles (0,4),(1,5),(2,6),(3,7)) yields CONSECUTIVE k pairs and the
// activations can be used exactly as they lie in memory.  Input may be [N,K] (int8 or int4) or the reference's own
// [K,N] (int8), which is transposed on the way: that is how the reference's layout reaches the fast kernels.
#include "afb_internal.h"
#include "dequant.cuh"

namespace afb {
namespace {

__device__ __forceinline__ uint32_t pack_word8(uint32_t w) { return prmt(w, 0u, 0x3120u); }   // [b0,b2,b1,b3]
__device__ __forceinline__ uint32_t pack_word4(uint32_t w) {
    uint32_t e = w & 0x0f0f0f0fu, o = (w >> 4) & 0x0f0f0f0fu;     // even / odd nibbles, one per byte
    e = (e | (e >> 4)) & 0x00ff00ffu; e = (e | (e >> 8)) & 0xffffu;   // n0,n2,n4,n6 in 16 bits
    o = (o | (o >> 4)) & 0x00ff00ffu; o = (o | (o >> 8)) & 0xffffu;
    // wanted: nibble i of the output = weight perm[i], perm = [0,2,4,6,1,3,5,7]
    return e | (o << 16);
}

// [N,K] -> packed [N,K]: one 32-bit word per thread step
__global__ void __launch_bounds__(256) prepack_col_kernel(const uint8_t* __restrict__ in, uint8_t* __restrict__ out, uint32_t n, uint32_t row_bytes,
                                                          uint32_t in_pitch, uint32_t out_pitch, uint32_t bits) {
    const uint32_t words = row_bytes / 4;
    const size_t total = (size_t)n * words;
    for (size_t id = blockIdx.x * (size_t)blockDim.x + threadIdx.x; id < total; id += (size_t)gridDim.x * blockDim.x) {
        const uint32_t r = (uint32_t)(id / words), wi = (uint32_t)(id % words);
        const uint32_t w = *reinterpret_cast<const uint32_t*>(in + (size_t)r * in_pitch + wi * 4);
        *reinterpret_cast<uint32_t*>(out + (size_t)r * out_pitch + wi * 4) = bits == 8 ? pack_word8(w) : pack_word4(w);
    }
}

// [K,N] int8 -> packed [N,K]: a 32 (k) x 32 (n) tile through shared memory, so that both sides are coalesced
__global__ void __launch_bounds__(256) prepack_row_kernel(const uint8_t* __restrict__ in, uint8_t* __restrict__ out, uint32_t n, uint32_t k,
                                                          uint32_t in_pitch, uint32_t out_pitch) {
    __shared__ uint8_t tile[32][33];
    const uint32_t n0 = blockIdx.x * 32, k0 = blockIdx.y * 32;
    const uint32_t tx = threadIdx.x & 31, ty = threadIdx.x >> 5;   // 32 x 8
    for (uint32_t r = ty; r < 32; r += 8)
        tile[r][tx] = (k0 + r < k && n0 + tx < n) ? in[(size_t)(k0 + r) * in_pitch + n0 + tx] : (uint8_t)0;
    __syncthreads();
    // 32 channels x 8 words of 4 k
    const uint32_t ch = threadIdx.x >> 3, wi = threadIdx.x & 7;
    if (n0 + ch < n && k0 + wi * 4 < k) {
        const uint32_t w = (uint32_t)tile[wi * 4][ch] | ((uint32_t)tile[wi * 4 + 1][ch] << 8) | ((uint32_t)tile[wi * 4 + 2][ch] << 16) |
                           ((uint32_t)tile[wi * 4 + 3][ch] << 24);
        *reinterpret_cast<uint32_t*>(out + (size_t)(n0 + ch) * out_pitch + k0 + wi * 4) = pack_word8(w);
    }
}

// rows of two equally shaped byte matrices interleaved: dst row 2i = g row i, dst row 2i+1 = u row i
__global__ void __launch_bounds__(256) interleave_rows_kernel(const uint8_t* __restrict__ g, const uint8_t* __restrict__ u, uint8_t* __restrict__ dst,
                                                              uint32_t rows, uint32_t row_bytes) {
    const size_t total = (size_t)rows * row_bytes;
    for (size_t id = blockIdx.x * (size_t)blockDim.x + threadIdx.x; id < total; id += (size_t)gridDim.x * blockDim.x) {
        const size_t r = id / row_bytes, c = id % row_bytes;
        dst[(2 * r) * row_bytes + c] = g[id];
        dst[(2 * r + 1) * row_bytes + c] = u[id];
    }
}

}  // namespace
}  // namespace afb

using namespace afb;

extern "C" int afb_prepack(const afb_gemm_args* a, void* out_b, uint32_t out_ldb, void* stream) {
    if (!a || !a->ptr_b || !out_b || a->n == 0 || a->k == 0) return AFB_ERR_BAD_ARG;
    if (a->b_bits != 8 && a->b_bits != 4) return AFB_ERR_BAD_ARG;
    if (a->b_layout != AFB_LAYOUT_ROW && a->b_layout != AFB_LAYOUT_COL) return AFB_ERR_BAD_ARG;   // already packed input is refused
    if (a->b_bits == 4 && a->b_layout != AFB_LAYOUT_COL) return AFB_ERR_UNSUPPORTED;
    if (out_ldb < a->k || (a->b_layout == AFB_LAYOUT_COL ? a->ldb < a->k : a->ldb < a->n)) return AFB_ERR_BAD_ARG;
    const uint32_t per_word = a->b_bits == 8 ? 4u : 8u;
    if (a->k % per_word) return AFB_ERR_UNSUPPORTED;                      // whole 32-bit words of weights per row
    const uint32_t out_pitch = out_ldb * a->b_bits / 8, row_bytes = a->k * a->b_bits / 8;
    if (out_pitch % 4 || (uintptr_t)out_b % 4) return AFB_ERR_BAD_ARG;
    if ((const void*)a->ptr_b == (const void*)out_b && a->b_layout == AFB_LAYOUT_ROW) return AFB_ERR_BAD_ARG;   // the transpose cannot run in place
    if (!current_ctx()) return AFB_ERR_NOT_INIT;
    cudaStream_t s = (cudaStream_t)stream;
    if (a->b_layout == AFB_LAYOUT_COL) {
        const uint32_t in_pitch = a->ldb * a->b_bits / 8;
        if (in_pitch % 4 || (uintptr_t)a->ptr_b % 4) return AFB_ERR_BAD_ARG;
        prepack_col_kernel<<<592, 256, 0, s>>>(reinterpret_cast<const uint8_t*>(a->ptr_b), reinterpret_cast<uint8_t*>(out_b), a->n, row_bytes,
                                               in_pitch, out_pitch, a->b_bits);
    } else {
        dim3 grid((a->n + 31) / 32, (a->k + 31) / 32);
        if (grid.y > 65535) return AFB_ERR_UNSUPPORTED;
        prepack_row_kernel<<<grid, 256, 0, s>>>(reinterpret_cast<const uint8_t*>(a->ptr_b), reinterpret_cast<uint8_t*>(out_b), a->n, a->k, a->ldb, out_pitch);
    }
    count_launch();
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? AFB_OK : cuda_fail(e);
}

extern "C" int afb_prepack_gated(const afb_gemm_args* gate, const void* b_up, const void* scale_up, const void* zero_up, void* out_b,
                                 uint32_t out_ldb, void* out_scale, void* out_zero, void* stream) {
    if (!gate || !gate->ptr_b || !gate->ptr_scale || !b_up || !scale_up || !out_b || !out_scale || gate->n == 0 || gate->k == 0) return AFB_ERR_BAD_ARG;
    if (gate->b_bits != 8 && gate->b_bits != 4) return AFB_ERR_BAD_ARG;
    if (gate->b_layout != AFB_LAYOUT_COL) return AFB_ERR_UNSUPPORTED;
    if ((gate->ptr_zero != nullptr) != (zero_up != nullptr) || (gate->ptr_zero && !out_zero)) return AFB_ERR_BAD_ARG;
    if (gate->group_size && gate->k % gate->group_size) return AFB_ERR_BAD_ARG;
    const uint32_t per_word = gate->b_bits == 8 ? 4u : 8u;
    if (gate->k % per_word || out_ldb < gate->k || gate->ldb < gate->k) return AFB_ERR_BAD_ARG;
    const uint32_t out_pitch = out_ldb * gate->b_bits / 8, in_pitch = gate->ldb * gate->b_bits / 8, row_bytes = gate->k * gate->b_bits / 8;
    if (out_pitch % 4 || in_pitch % 4 || (uintptr_t)out_b % 4 || (uintptr_t)gate->ptr_b % 4 || (uintptr_t)b_up % 4) return AFB_ERR_BAD_ARG;
    if (!current_ctx()) return AFB_ERR_NOT_INIT;
    cudaStream_t s = (cudaStream_t)stream;
    uint8_t* ob = reinterpret_cast<uint8_t*>(out_b);
    // the packing kernel with a doubled output pitch writes every other row: gate rows at 2i, up rows at 2i + 1
    prepack_col_kernel<<<592, 256, 0, s>>>(reinterpret_cast<const uint8_t*>(gate->ptr_b), ob, gate->n, row_bytes, in_pitch, 2 * out_pitch, gate->b_bits);
    prepack_col_kernel<<<592, 256, 0, s>>>(reinterpret_cast<const uint8_t*>(b_up), ob + out_pitch, gate->n, row_bytes, in_pitch, 2 * out_pitch, gate->b_bits);
    const uint32_t groups = gate->group_size ? gate->k / gate->group_size : 1;
    const uint32_t sbytes = groups * (gate->scale_dtype == AFB_SCALE_BF16 ? 2u : 4u);
    interleave_rows_kernel<<<148, 256, 0, s>>>(reinterpret_cast<const uint8_t*>(gate->ptr_scale), reinterpret_cast<const uint8_t*>(scale_up),
                                               reinterpret_cast<uint8_t*>(out_scale), gate->n, sbytes);
    unsigned launches = 3;
    if (gate->ptr_zero) {
        interleave_rows_kernel<<<148, 256, 0, s>>>(reinterpret_cast<const uint8_t*>(gate->ptr_zero), reinterpret_cast<const uint8_t*>(zero_up),
                                                   reinterpret_cast<uint8_t*>(out_zero), gate->n, groups);
        ++launches;
    }
    count_launch(launches);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? AFB_OK : cuda_fail(e);
}
