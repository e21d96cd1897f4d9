// Parameter block, small PTX wrappers and the end-of-piece reduction of the decode kernel (decode.cu).
#pragma once
#include "afb_internal.h"
#include "dequant.cuh"

namespace afb {

constexpr int kThreads = 256;
constexpr int kWarps = 8;
constexpr int kStageBytes = 1024;              // 2 channels x 32 lanes x 16 bytes
constexpr int kRedFloats = kWarps * 16 * 17;   // cross-warp reduction buffer, [warp][16 channels][<=16 rows + pad]; reuses the ring once the stream has ended

struct DecodeParams {
    const uint16_t* a;
    const uint8_t* b;
    const void* scale;
    const uint8_t* zero;   // optional zero-points (nullptr = none), one byte per scale entry
    uint16_t* c;
    uint32_t m, n, k, lda, ldb_bytes, ldc;
    uint32_t enc, scale_dtype, group;
    uint32_t packed;  // B is in the pre-packed order of afb_prepack: the unpack yields consecutive k, activations are staged as they lie
    uint32_t wr;      // warps along the channel dimension (1, 2, 4 or 8); WK = 8 / wr
    uint32_t kc;      // k elements per slice (multiple of the chunk)
    uint32_t pass_k;  // k elements staged per pass (m * (pass_k * 2 + 16) <= act_bytes)
    uint32_t act_bytes;  // size of the activation staging area in shared memory (chosen per launch)
    uint32_t group_shift;  // log2(group) (groups are powers of two)
    uint32_t slices;  // gridDim.y
    // balanced form (streamk = 1): the grid is one wave of CTAs; the weights are cut into units of 16*wr channels x unit_k
    // elements of K, numbered channel block major, and CTA c takes units [c*U/G, (c+1)*U/G): whole runs of K of one or more
    // channel blocks.  A channel block shared by several CTAs is finished by the last of them to arrive, in CTA order.
    uint32_t streamk, unit_k, units_per_cb, total_units;
    float* ws;        // [contributor][m][n] fp32 partial sums (K-slices, or the CTAs sharing a channel block)
    uint32_t* counters;  // one per channel block, zero on entry, zero again on exit
};

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr) : "memory");
    return v;
}
__device__ __forceinline__ uint4 ldg_act(const uint16_t* p) {
    uint4 v;
    asm volatile("ld.global.nc.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float bf16_to_f32(uint16_t h) { return __uint_as_float((uint32_t)h << 16); }
__device__ __forceinline__ float load_scale(const void* s, size_t idx, uint32_t dtype) {
    return dtype == AFB_SCALE_BF16 ? bf16_to_f32(reinterpret_cast<const uint16_t*>(s)[idx]) : reinterpret_cast<const float*>(s)[idx];
}

__device__ __forceinline__ uint32_t swz_piece(uint32_t pc) { return pc ^ (((pc >> 3) & 1u) << 1); }

// The end of a piece of work, after every warp has put its fp32 sums into s_red ([warp][16 channels][17]) and the block has
// synchronised: adds the WK warps sharing 16 channels, then either scales, rounds and stores C (one contributor) or publishes
// the sums in the workspace; the last contributor to arrive adds the published partial sums in contributor order (= ascending
// K), so the result does not depend on who that is, and puts the arrival counter back to zero.
template <bool GROUPED, typename CtaOf>
__device__ __forceinline__ void decode_finish(const DecodeParams& p, const float* s_red, uint32_t* s_last, uint32_t cb, uint32_t nblk,
                                              uint32_t wk_count, uint32_t mcols, CtaOf cta_of) {
    const uint32_t tid = threadIdx.x;
    const uint32_t rows_cta = 16 * p.wr;                // a power of two: 16, 32, 64 or 128
    const uint32_t rows_shift = 31u - (uint32_t)__clz(rows_cta);
    const uint32_t outputs = rows_cta * mcols;          // <= 2048
    uint32_t contributors = p.slices, my_slot = blockIdx.y;
    if (p.streamk) {   // the CTAs whose runs of units touch this channel block, in CTA order (= ascending K)
        const uint32_t first = cta_of(cb * p.units_per_cb), last = cta_of(cb * p.units_per_cb + p.units_per_cb - 1);
        contributors = last - first + 1; my_slot = blockIdx.x - first;
    }
    const bool single = contributors == 1;
    for (uint32_t idx = tid; idx < outputs; idx += kThreads) {
        const uint32_t mm = idx >> rows_shift, r = idx & (rows_cta - 1);   // consecutive threads -> consecutive channels
        const uint32_t nn = nblk + r;
        if (mm >= p.m || nn >= p.n) continue;
        const uint32_t w0 = (r >> 4) * wk_count;
        float sum = 0.f;
        for (uint32_t w = 0; w < wk_count; ++w) sum += s_red[((w0 + w) * 16 + (r & 15)) * 17 + mm];
        if (single) {
            if (!GROUPED) sum *= load_scale(p.scale, nn, p.scale_dtype);
            p.c[(size_t)mm * p.ldc + nn] = __bfloat16_as_ushort(__float2bfloat16_rn(sum));
        } else {
            __stcg(p.ws + ((size_t)my_slot * p.m + mm) * p.n + nn, sum);
        }
    }
    if (!single) {
        __threadfence();
        __syncthreads();
        if (tid == 0) {
            const uint32_t old = atomicAdd(p.counters + cb, 1u);
            *s_last = (old == contributors - 1) ? 1u : 0u;
        }
        __syncthreads();
        if (*s_last) {
            __threadfence();
            for (uint32_t idx = tid; idx < p.m * rows_cta; idx += kThreads) {
                const uint32_t mm = idx >> rows_shift, nn = nblk + (idx & (rows_cta - 1));
                if (nn >= p.n) continue;
                const float* src = p.ws + (size_t)mm * p.n + nn;
                const size_t slice_stride = (size_t)p.m * p.n;
                float sum = 0.f;
                for (uint32_t sl = 0; sl < contributors; sl += 8) {  // eight independent loads in flight, summed in order
                    float v[8];
#pragma unroll
                    for (int i2 = 0; i2 < 8; ++i2) v[i2] = sl + i2 < contributors ? __ldcg(src + (sl + i2) * slice_stride) : 0.f;
#pragma unroll
                    for (int i2 = 0; i2 < 8; ++i2) sum += v[i2];
                }
                if (!GROUPED) sum *= load_scale(p.scale, nn, p.scale_dtype);
                p.c[(size_t)mm * p.ldc + nn] = __bfloat16_as_ushort(__float2bfloat16_rn(sum));
            }
            if (tid == 0) p.counters[cb] = 0u;  // ready for the next launch
        }
    }
}

}  // namespace afb
