// Naive variant: one thread per C element, fp32, the loop of the reference's CPU check
// (host_ref.hpp:15-24: acc += a * (b * scale), k ascending, no fused multiply-add), for
// every layout / bit-width / encoding / scale mode the argument block can express.
// It is the GPU-side cross-check for the fast variants at sizes the CPU cannot finish,
// and the variant AFB_VARIANT_AUTO falls back to for B in the reference's [K,N] layout.
//
// Also here: the dequant-dump kernel, which writes the weights exactly as the fast
// kernels hand them to the tensor cores (it calls the same device functions).
#include "afb_internal.h"
#include "dequant.cuh"

namespace afb {

__device__ __forceinline__ float bf16_bits_to_f32(uint16_t h) { return __uint_as_float((uint32_t)h << 16); }

// Scalar decode of weight (n, k) -> integer value as float.
__device__ __forceinline__ float load_q(const uint8_t* __restrict__ b, uint32_t n, uint32_t k, uint32_t ldb,
                                        uint32_t bits, uint32_t enc, uint32_t layout) {
    if (layout == AFB_LAYOUT_COL_PACKED) k = packed_pos(bits, k);
    if (bits == 8) {
        const size_t idx = layout != AFB_LAYOUT_ROW ? (size_t)n * ldb + k : (size_t)k * ldb + n;
        const uint8_t u = b[idx];
        const int v = enc == AFB_ENC_OFFSET_BINARY ? (int)u - 128 : (int)(int8_t)u;
        return (float)v;
    }
    // 4-bit, [N,K] only: two per byte along K, low nibble = even k
    const size_t byte = (size_t)n * (ldb >> 1) + (k >> 1);
    const uint32_t nib = (b[byte] >> ((k & 1u) * 4u)) & 0xFu;
    const int v = enc == AFB_ENC_OFFSET_BINARY ? (int)nib - 8 : (int)((nib ^ 8u)) - 8;
    return (float)v;
}

// decoded zero-point (a byte in the weights' own encoding)
__device__ __forceinline__ float decode_zero(uint8_t z, uint32_t bits, uint32_t enc) {
    if (bits == 8) return (float)(enc == AFB_ENC_OFFSET_BINARY ? (int)z - 128 : (int)(int8_t)z);
    const uint32_t nib = z & 0xFu;
    return (float)(enc == AFB_ENC_OFFSET_BINARY ? (int)nib - 8 : (int)(nib ^ 8u) - 8);
}

__device__ __forceinline__ float load_scale(const void* __restrict__ s, size_t idx, uint32_t dtype) {
    return dtype == AFB_SCALE_BF16 ? bf16_bits_to_f32(reinterpret_cast<const uint16_t*>(s)[idx])
                                   : reinterpret_cast<const float*>(s)[idx];
}

__global__ void __launch_bounds__(256) naive_gemm_kernel(afb_gemm_args a) {
    const uint32_t n = blockIdx.x * 32 + (threadIdx.x & 31);
    const uint32_t m = blockIdx.y * 8 + (threadIdx.x >> 5);
    if (m >= a.m || n >= a.n) return;
    const uint16_t* __restrict__ pa = reinterpret_cast<const uint16_t*>(a.ptr_a) + (size_t)m * a.lda;
    const uint8_t* __restrict__ pb = reinterpret_cast<const uint8_t*>(a.ptr_b);
    const uint32_t groups = a.group_size ? a.k / a.group_size : 0;
    const uint8_t* __restrict__ pz = reinterpret_cast<const uint8_t*>(a.ptr_zero);
    float scale = a.group_size ? 0.f : load_scale(a.ptr_scale, n, a.scale_dtype);
    float zero = (pz && !a.group_size) ? decode_zero(pz[n], a.b_bits, a.b_encoding) : 0.f;
    float acc = 0.f;
    for (uint32_t k = 0; k < a.k; ++k) {
        if (a.group_size && (k % a.group_size) == 0) {
            scale = load_scale(a.ptr_scale, (size_t)n * groups + k / a.group_size, a.scale_dtype);
            if (pz) zero = decode_zero(pz[(size_t)n * groups + k / a.group_size], a.b_bits, a.b_encoding);
        }
        const float q = load_q(pb, n, k, a.ldb, a.b_bits, a.b_encoding, a.b_layout) - zero;
        const float w = __fmul_rn(q, scale);
        acc = __fadd_rn(acc, __fmul_rn(bf16_bits_to_f32(pa[k]), w));
    }
    if (a.flags & AFB_FLAG_C_F32)
        reinterpret_cast<float*>(a.ptr_c)[(size_t)m * a.ldc + n] = acc;
    else
        reinterpret_cast<__nv_bfloat16*>(a.ptr_c)[(size_t)m * a.ldc + n] = __float2bfloat16_rn(acc);
}

// ---------------------------------------------------------------------------------
// Launch-floor probes (measurement aid for the decode shapes, whose kernels last a few microseconds): a kernel with the decode
// kernel's launch shape that does nothing, and one that only reads `bytes` of weights with the decode kernel's access pattern
// (16 bytes per lane, 8 rows x 64 bytes per warp instruction) and keeps a checksum so that the loads cannot be dropped.
// ---------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) probe_kernel(const uint4* __restrict__ src, size_t vecs, uint32_t* __restrict__ sink, uint32_t kind) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if (kind == 0) { asm volatile("griddepcontrol.wait;" ::: "memory"); return; }
    uint32_t acc = 0;
    const size_t per_cta = (vecs + gridDim.x - 1) / gridDim.x, begin = blockIdx.x * per_cta, end = min(vecs, begin + per_cta);
    for (size_t i = begin + threadIdx.x; i < end; i += 4 * 256) {   // four independent 16-byte loads in flight per thread
        uint4 v[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) v[j] = i + j * 256 < end ? __ldcs(src + i + j * 256) : make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int j = 0; j < 4; ++j) acc ^= v[j].x ^ v[j].y ^ v[j].z ^ v[j].w;
    }
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (acc == 0x9E3779B9u) sink[blockIdx.x & 1023] = acc;   // practically never true: keeps the loads alive
}

int launch_probe(uint32_t kind, const void* src, size_t bytes, uint32_t ctas, uint32_t smem_bytes, bool pdl, uint32_t* sink, cudaStream_t s) {
    static DeviceOnce attr_set;
    int dev = 0;
    cudaGetDevice(&dev);
    if (!attr_set.done(dev)) {
        cudaError_t e = cudaFuncSetAttribute(probe_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e != cudaSuccess) return cuda_fail(e);
        attr_set.mark(dev);
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(ctas); cfg.blockDim = dim3(256); cfg.dynamicSmemBytes = smem_bytes; cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = pdl ? 1 : 0;
    cudaError_t e = cudaLaunchKernelEx(&cfg, probe_kernel, reinterpret_cast<const uint4*>(src), bytes / 16, sink, kind);
    count_launch();
    return e == cudaSuccess ? AFB_OK : cuda_fail(e);
}

int launch_naive(const afb_gemm_args& a, DeviceCtx*, cudaStream_t s) {
    dim3 grid((a.n + 31) / 32, (a.m + 7) / 8);
    if (grid.y > 65535) return AFB_ERR_UNSUPPORTED;
    naive_gemm_kernel<<<grid, 256, 0, s>>>(a);
    count_launch();
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? AFB_OK : cuda_fail(e);
}

// ---------------------------------------------------------------------------------
// Dequant dump: each thread converts one 16-byte piece of B with the fast-path
// routines and stores the bf16 result in B's own logical layout.
// ---------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) dequant_dump_kernel(afb_gemm_args a, uint16_t* __restrict__ out) {
    const uint8_t* __restrict__ pb = reinterpret_cast<const uint8_t*>(a.ptr_b);
    const uint32_t xormask = a.b_encoding == AFB_ENC_OFFSET_BINARY ? 0x80808080u : 0u;
    const uint32_t magic4 = a.b_encoding == AFB_ENC_OFFSET_BINARY ? 0x43004300u : 0x43084308u;
    const bool packed = a.b_layout == AFB_LAYOUT_COL_PACKED;
    if (a.b_layout != AFB_LAYOUT_ROW) {
        const uint32_t per16 = a.b_bits == 8 ? 16u : 32u;  // weights per 16-byte piece
        const uint32_t pieces_per_row = a.k / per16;
        const size_t total = (size_t)a.n * pieces_per_row;
        const uint32_t groups = a.group_size ? a.k / a.group_size : 0;
        for (size_t id = blockIdx.x * (size_t)blockDim.x + threadIdx.x; id < total; id += (size_t)gridDim.x * blockDim.x) {
            const uint32_t n = (uint32_t)(id / pieces_per_row);
            const uint32_t k0 = (uint32_t)(id % pieces_per_row) * per16;
            const size_t row_bytes = a.b_bits == 8 ? (size_t)a.ldb : (size_t)(a.ldb >> 1);
            const uint4 raw = *reinterpret_cast<const uint4*>(pb + (size_t)n * row_bytes + (a.b_bits == 8 ? k0 : (k0 >> 1)));
            const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
            const uint8_t* pz = reinterpret_cast<const uint8_t*>(a.ptr_zero);
            const uint32_t zb = pz ? pz[a.group_size ? (size_t)n * groups + k0 / a.group_size : n] : 0u;
            const bool has_zero = pz != nullptr;
            const uint32_t z8 = zero8_const(has_zero ? zb : (a.b_encoding == AFB_ENC_OFFSET_BINARY ? 128u : 0u), a.b_encoding);
            const uint32_t sub4 = has_zero ? zero4_const(zb, a.b_encoding) : 0x43084308u;
            uint32_t sc = 0;
            if (a.group_size) {
                // a 16-byte piece never straddles a group (group_size is a multiple of 32)
                const size_t si = (size_t)n * groups + k0 / a.group_size;
                uint16_t sb;
                if (a.scale_dtype == AFB_SCALE_BF16) sb = reinterpret_cast<const uint16_t*>(a.ptr_scale)[si];
                else sb = __bfloat16_as_ushort(__float2bfloat16_rn(reinterpret_cast<const float*>(a.ptr_scale)[si]));
                sc = bf16_dup(sb);
            }
            uint32_t* o = reinterpret_cast<uint32_t*>(out + (size_t)n * a.k + k0);
            if ((a.flags & AFB_FLAG_DUMP_DECODE_PAIRING) && !packed) {
                // the decode kernel's unpack: cheap pairing ({k0,k2},{k1,k3} / {k0,k4}..{k3,k7}), integers only (that kernel
                // applies group scales to fp32 partial sums, never to weights); stored back in natural k order
                uint16_t* o16 = out + (size_t)n * a.k + k0;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    if (a.b_bits == 8) {
                        uint32_t p02, p13;
                        s8x4_to_bf16_strided(w[j] ^ xormask, p02, p13);
                        if (has_zero) { p02 = bf16x2_sub(p02, z8); p13 = bf16x2_sub(p13, z8); }
                        o16[4 * j + 0] = (uint16_t)(p02 & 0xffff); o16[4 * j + 2] = (uint16_t)(p02 >> 16);
                        o16[4 * j + 1] = (uint16_t)(p13 & 0xffff); o16[4 * j + 3] = (uint16_t)(p13 >> 16);
                    } else {
                        uint32_t p[4];
                        s4x8_to_bf16_strided(w[j], magic4, p, sub4);
#pragma unroll
                        for (int i = 0; i < 4; ++i) { o16[8 * j + i] = (uint16_t)(p[i] & 0xffff); o16[8 * j + 4 + i] = (uint16_t)(p[i] >> 16); }
                    }
                }
                continue;
            }
            if (a.b_bits == 8) {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    uint32_t p01, p23;
                    s8x4_to_bf16_pairs(w[j] ^ xormask, packed, p01, p23);
                    if (has_zero) { p01 = bf16x2_sub(p01, z8); p23 = bf16x2_sub(p23, z8); }
                    if (a.group_size) { p01 = bf16x2_mul(p01, sc); p23 = bf16x2_mul(p23, sc); }
                    o[2 * j] = p01; o[2 * j + 1] = p23;
                }
            } else {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    uint32_t p[4];
                    s4x8_to_bf16_pairs(w[j], magic4, packed, p, sub4);
#pragma unroll
                    for (int i = 0; i < 4; ++i) o[4 * j + i] = a.group_size ? bf16x2_mul(p[i], sc) : p[i];
                }
            }
        }
    } else {
        // [K,N] int8: 4 consecutive n per thread, scalar stores (this layout has no fast GEMM variant;
        // the strided-pair routine is exercised here so that it is covered bit-exactly too)
        const uint32_t n4 = a.n / 4;
        const size_t total = (size_t)a.k * n4;
        for (size_t id = blockIdx.x * (size_t)blockDim.x + threadIdx.x; id < total; id += (size_t)gridDim.x * blockDim.x) {
            const uint32_t k = (uint32_t)(id / n4);
            const uint32_t n0 = (uint32_t)(id % n4) * 4;
            const uint32_t w = *reinterpret_cast<const uint32_t*>(pb + (size_t)k * a.ldb + n0) ^ xormask;
            uint32_t p02, p13;
            s8x4_to_bf16_strided(w, p02, p13);
            uint16_t v[4] = {(uint16_t)(p02 & 0xffff), (uint16_t)(p13 & 0xffff), (uint16_t)(p02 >> 16), (uint16_t)(p13 >> 16)};
#pragma unroll
            for (int i = 0; i < 4; ++i) out[(size_t)k * a.n + n0 + i] = v[i];
        }
    }
}

int launch_dequant_dump(const afb_gemm_args& a, void* out, cudaStream_t s) {
    if (a.b_layout != AFB_LAYOUT_ROW) {
        const uint32_t per16 = a.b_bits == 8 ? 16u : 32u;
        if (a.k % per16 || (a.b_bits == 8 ? a.ldb % 16 : a.ldb % 32)) return AFB_ERR_UNSUPPORTED;
        if (a.group_size && a.group_size % 32) return AFB_ERR_UNSUPPORTED;
    } else {
        if (a.b_bits != 8 || a.n % 4 || a.ldb % 4 || a.group_size || a.ptr_zero) return AFB_ERR_UNSUPPORTED;
    }
    if ((uintptr_t)a.ptr_b % 16) return AFB_ERR_BAD_ARG;
    dequant_dump_kernel<<<296, 256, 0, s>>>(a, reinterpret_cast<uint16_t*>(out));
    count_launch();
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? AFB_OK : cuda_fail(e);
}

}  // namespace afb
