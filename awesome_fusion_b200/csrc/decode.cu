// Decode variant (M <= 16, B in [N,K] layout): the memory-bound replacement of the
// reference kernel's main loop (bf16gemm_kernel_gfx90a.s:410-489) for GEMV-like shapes.
//
// Every weight byte is read from HBM exactly once with 128-bit loads; the dominant
// stream is B (N*K*bits/8 bytes).  A CTA owns 128 output channels (16 per warp) and one
// K-slice.  Per 16-byte load a lane holds 16 (int8) or 32 (int4) consecutive-k weights of
// one channel; they are unpacked to exact bf16 in registers (dequant.cuh) and fed to
// mma.sync.m16n8k16 as the 16-row operand, the <= 16 activation rows being the 8-column
// operand.  The four lanes of a quad hold different k, so the tensor-core instruction
// performs the intra-warp split-K reduction; slices of K owned by different CTAs are
// combined through an fp32 workspace by the last CTA to arrive (fixed summation order,
// so results are run-to-run identical).
//
// Because a dot product does not care about the order of k, weights are paired in the
// order that is cheapest to unpack ({k0,k2},{k1,k3} for int8; {k0,k4}..{k3,k7} for int4)
// and the activations are permuted to match once, while they are staged in shared memory.
//
// Scales: per-channel scales multiply the fp32 sum once at the end (the reference
// multiplies every weight, .s:29-33; mathematically the same, one rounding fewer).
// Per-group scales multiply the fp32 partial sum of each group.
#include "afb_internal.h"
#include "dequant.cuh"

namespace afb {

namespace {

constexpr int kThreads = 256;
constexpr int kRowsPerCta = 128;
constexpr int kStageK = 1024;                 // activations staged per pass (k elements)
constexpr int kActRowBytes = kStageK * 2 + 16;  // +16: rows land in different bank groups
constexpr int kMaxGroupsPerStage = 8;         // group_size >= 128

struct DecodeParams {
    const uint16_t* a;
    const uint8_t* b;
    const void* scale;
    uint16_t* c;
    uint32_t m, n, k, lda, ldb_bytes, ldc;
    uint32_t enc, scale_dtype, group;
    uint32_t kc;      // k elements per slice (multiple of the chunk)
    uint32_t slices;  // gridDim.y
    float* ws;        // [slices][m][n] fp32 partial sums (slices > 1)
    uint32_t* counters;  // one per row block, zero on entry, zero again on exit
};

__device__ __forceinline__ uint4 ldg_stream(const uint8_t* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t swz_piece(uint32_t pc) { return pc ^ (((pc >> 3) & 1u) << 1); }
__device__ __forceinline__ float bf16_to_f32(uint16_t h) { return __uint_as_float((uint32_t)h << 16); }

template <int BITS, int MT, bool GROUPED>
__global__ void __launch_bounds__(kThreads, (MT == 1 ? 4 : 3)) decode_kernel(const DecodeParams p) {
    constexpr int CH = BITS == 8 ? 64 : 128;    // k per warp chunk (a quad covers 64 bytes of one row)
    constexpr int LK = CH / 4;                  // k per lane per chunk
    constexpr int PIECES = LK / 8;              // 16-byte activation pieces per lane per chunk
    constexpr int U = 4;                        // chunks in flight per warp

    __shared__ __align__(16) uint8_t s_act[MT * 8 * kActRowBytes];
    __shared__ float s_scale[GROUPED ? kRowsPerCta * kMaxGroupsPerStage : 1];
    __shared__ uint32_t s_last;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, tig = lane & 3;
    const uint32_t nblk = blockIdx.x * kRowsPerCta;
    const uint32_t row_a = nblk + warp * 16 + g, row_b = row_a + 8;
    const bool ok_a = row_a < p.n, ok_b = row_b < p.n;
    const uint8_t* pa = p.b + (size_t)(ok_a ? row_a : 0) * p.ldb_bytes + tig * 16;
    const uint8_t* pb = p.b + (size_t)(ok_b ? row_b : 0) * p.ldb_bytes + tig * 16;
    const uint32_t ks = blockIdx.y * p.kc;
    const uint32_t kend = min(p.k, ks + p.kc);
    const uint32_t xormask = (BITS == 8 && p.enc == AFB_ENC_OFFSET_BINARY) ? 0x80808080u : 0u;
    const uint32_t magic4 = p.enc == AFB_ENC_OFFSET_BINARY ? 0x43004300u : 0x43084308u;
    const uint32_t groups_per_row = GROUPED ? p.k / p.group : 0;

    float acc[MT][4];
    float accg[MT][4];  // partial sum of the current scale group (grouped mode only)
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int e = 0; e < 4; ++e) { acc[mt][e] = 0.f; accg[mt][e] = 0.f; }

    for (uint32_t kb = ks; kb < kend; kb += kStageK) {
        const uint32_t klen = min((uint32_t)kStageK, kend - kb);
        const uint32_t nchunks = klen / CH;
        const size_t kbyte0 = BITS == 8 ? kb : (kb >> 1);
        // the first weight loads of this pass go out before the activations are staged
        uint4 wa[U], wb[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            wa[u] = make_uint4(0, 0, 0, 0); wb[u] = wa[u];
            if ((uint32_t)u < nchunks) {
                if (ok_a) wa[u] = ldg_stream(pa + kbyte0 + (size_t)u * 64);
                if (ok_b) wb[u] = ldg_stream(pb + kbyte0 + (size_t)u * 64);
            }
        }
        __syncthreads();  // the previous pass has been consumed
        // ---- stage (and permute) the activations of [kb, kb+klen) ----
        const uint32_t pieces = klen >> 3;
        for (uint32_t idx = tid; idx < (uint32_t)(MT * 8) * pieces; idx += kThreads) {
            const uint32_t r = idx / pieces, pc = idx - r * pieces;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (r < p.m) v = *reinterpret_cast<const uint4*>(p.a + (size_t)r * p.lda + kb + pc * 8);
            uint4 o;
            if (BITS == 8) {  // {k0,k2},{k1,k3},{k4,k6},{k5,k7}
                o.x = prmt(v.x, v.y, 0x5410u); o.y = prmt(v.x, v.y, 0x7632u);
                o.z = prmt(v.z, v.w, 0x5410u); o.w = prmt(v.z, v.w, 0x7632u);
            } else {          // {k0,k4},{k1,k5},{k2,k6},{k3,k7}
                o.x = prmt(v.x, v.z, 0x5410u); o.y = prmt(v.x, v.z, 0x7632u);
                o.z = prmt(v.y, v.w, 0x5410u); o.w = prmt(v.y, v.w, 0x7632u);
            }
            *reinterpret_cast<uint4*>(s_act + r * kActRowBytes + swz_piece(pc) * 16) = o;
        }
        if (GROUPED) {
            const uint32_t ng = klen / p.group;  // <= kMaxGroupsPerStage
            for (uint32_t idx = tid; idx < kRowsPerCta * ng; idx += kThreads) {
                const uint32_t r = idx / ng, gi = idx - r * ng;
                float s = 0.f;
                if (nblk + r < p.n) {
                    const size_t si = (size_t)(nblk + r) * groups_per_row + kb / p.group + gi;
                    s = p.scale_dtype == AFB_SCALE_BF16 ? bf16_to_f32(reinterpret_cast<const uint16_t*>(p.scale)[si])
                                                       : reinterpret_cast<const float*>(p.scale)[si];
                }
                s_scale[r * kMaxGroupsPerStage + gi] = s;
            }
        }
        __syncthreads();

        for (uint32_t c0 = 0; c0 < nchunks; c0 += U) {
#pragma unroll
            for (int u = 0; u < U; ++u) {
                if (c0 + u < nchunks) {
                    const uint32_t kk = c0 + u;
                    const uint32_t pc0 = kk * (CH / 8) + tig * PIECES;
                    uint32_t s[MT][PIECES * 4];
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                        for (int i = 0; i < PIECES; ++i) {
                            const uint4 t = *reinterpret_cast<const uint4*>(s_act + (mt * 8 + g) * kActRowBytes + swz_piece(pc0 + i) * 16);
                            s[mt][4 * i] = t.x; s[mt][4 * i + 1] = t.y; s[mt][4 * i + 2] = t.z; s[mt][4 * i + 3] = t.w;
                        }
                    const uint32_t wav[4] = {wa[u].x, wa[u].y, wa[u].z, wa[u].w};
                    const uint32_t wbv[4] = {wb[u].x, wb[u].y, wb[u].z, wb[u].w};
                    // the registers just read are refilled with the chunk U steps ahead
                    if (kk + U < nchunks) {
                        if (ok_a) wa[u] = ldg_stream(pa + kbyte0 + (size_t)(kk + U) * 64);
                        if (ok_b) wb[u] = ldg_stream(pb + kbyte0 + (size_t)(kk + U) * 64);
                    }
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        if (BITS == 8) {
                            uint32_t a0, a1, a2, a3;
                            s8x4_to_bf16_strided(wav[j] ^ xormask, a0, a2);
                            s8x4_to_bf16_strided(wbv[j] ^ xormask, a1, a3);
#pragma unroll
                            for (int mt = 0; mt < MT; ++mt)
                                mma_bf16(GROUPED ? accg[mt] : acc[mt], a0, a1, a2, a3, s[mt][2 * j], s[mt][2 * j + 1]);
                        } else {
                            uint32_t qa[4], qb[4];
                            s4x8_to_bf16_strided(wav[j], magic4, qa);
                            s4x8_to_bf16_strided(wbv[j], magic4, qb);
#pragma unroll
                            for (int mt = 0; mt < MT; ++mt) {
                                mma_bf16(GROUPED ? accg[mt] : acc[mt], qa[0], qb[0], qa[1], qb[1], s[mt][4 * j], s[mt][4 * j + 1]);
                                mma_bf16(GROUPED ? accg[mt] : acc[mt], qa[2], qb[2], qa[3], qb[3], s[mt][4 * j + 2], s[mt][4 * j + 3]);
                            }
                        }
                    }
                    if (GROUPED) {
                        const uint32_t kdone = (kk + 1) * CH;  // k consumed in this pass
                        if (kdone % p.group == 0) {
                            const uint32_t gi = kdone / p.group - 1;
                            const float sa = s_scale[(warp * 16 + g) * kMaxGroupsPerStage + gi];
                            const float sb = s_scale[(warp * 16 + g + 8) * kMaxGroupsPerStage + gi];
#pragma unroll
                            for (int mt = 0; mt < MT; ++mt) {
                                acc[mt][0] = fmaf(sa, accg[mt][0], acc[mt][0]); acc[mt][1] = fmaf(sa, accg[mt][1], acc[mt][1]);
                                acc[mt][2] = fmaf(sb, accg[mt][2], acc[mt][2]); acc[mt][3] = fmaf(sb, accg[mt][3], acc[mt][3]);
                                accg[mt][0] = accg[mt][1] = accg[mt][2] = accg[mt][3] = 0.f;
                            }
                        }
                    }
                }
            }
        }
    }

    // ---- epilogue: acc[mt][e]: channel = e < 2 ? row_a : row_b, activation row = mt*8 + 2*tig + (e & 1)
    if (p.slices == 1) {
        float sa = 1.f, sb = 1.f;
        if (!GROUPED) {
            if (ok_a) sa = p.scale_dtype == AFB_SCALE_BF16 ? bf16_to_f32(reinterpret_cast<const uint16_t*>(p.scale)[row_a])
                                                          : reinterpret_cast<const float*>(p.scale)[row_a];
            if (ok_b) sb = p.scale_dtype == AFB_SCALE_BF16 ? bf16_to_f32(reinterpret_cast<const uint16_t*>(p.scale)[row_b])
                                                          : reinterpret_cast<const float*>(p.scale)[row_b];
        }
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const uint32_t mm = mt * 8 + 2 * tig + (e & 1);
                const uint32_t nn = e < 2 ? row_a : row_b;
                if (mm < p.m && nn < p.n)
                    p.c[(size_t)mm * p.ldc + nn] = __bfloat16_as_ushort(__float2bfloat16_rn(acc[mt][e] * (e < 2 ? sa : sb)));
            }
        return;
    }

    // several K-slices: publish this slice's partial sums, the last CTA of the row block adds them up
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const uint32_t mm = mt * 8 + 2 * tig + (e & 1);
            const uint32_t nn = e < 2 ? row_a : row_b;
            if (mm < p.m && nn < p.n) __stcg(p.ws + ((size_t)blockIdx.y * p.m + mm) * p.n + nn, acc[mt][e]);
        }
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        const uint32_t old = atomicAdd(p.counters + blockIdx.x, 1u);
        s_last = (old == p.slices - 1) ? 1u : 0u;
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    for (uint32_t idx = tid; idx < p.m * kRowsPerCta; idx += kThreads) {
        const uint32_t mm = idx / kRowsPerCta, nn = nblk + (idx % kRowsPerCta);
        if (nn >= p.n) continue;
        const float* src = p.ws + (size_t)mm * p.n + nn;
        const size_t slice_stride = (size_t)p.m * p.n;
        float sum = 0.f;
        for (uint32_t sl = 0; sl < p.slices; sl += 8) {  // eight independent loads in flight, summed in slice order
            float v[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = sl + i < p.slices ? __ldcg(src + (sl + i) * slice_stride) : 0.f;
#pragma unroll
            for (int i = 0; i < 8; ++i) sum += v[i];
        }
        if (!GROUPED)
            sum *= p.scale_dtype == AFB_SCALE_BF16 ? bf16_to_f32(reinterpret_cast<const uint16_t*>(p.scale)[nn])
                                                  : reinterpret_cast<const float*>(p.scale)[nn];
        p.c[(size_t)mm * p.ldc + nn] = __bfloat16_as_ushort(__float2bfloat16_rn(sum));
    }
    if (tid == 0) p.counters[blockIdx.x] = 0u;  // ready for the next launch
}

template <int BITS, int MT, bool GROUPED>
cudaError_t launch_one(const DecodeParams& p, dim3 grid, cudaStream_t s) {
    decode_kernel<BITS, MT, GROUPED><<<grid, kThreads, 0, s>>>(p);
    return cudaGetLastError();
}

}  // namespace

bool decode_supports(const afb_gemm_args& a) {
    if (a.m == 0 || a.m > 16) return false;
    if (a.b_layout != AFB_LAYOUT_COL) return false;
    if (a.b_bits != 8 && a.b_bits != 4) return false;
    const uint32_t ch = a.b_bits == 8 ? 64 : 128;
    if (a.k % ch) return false;
    const uint32_t ldb_bytes = a.b_bits == 8 ? a.ldb : a.ldb / 2;
    if (ldb_bytes % 16 || a.lda % 8) return false;
    if ((uintptr_t)a.ptr_a % 16 || (uintptr_t)a.ptr_b % 16) return false;
    if (a.group_size) {
        if (a.group_size % 128 || a.group_size > kStageK || kStageK % a.group_size || a.k % a.group_size) return false;
    }
    return true;
}

// Number of K-slices and slice length: enough CTAs to fill the GPU about three times over,
// slices a power-of-two fraction of K (multiple of 4 chunks and of the group).
static void pick_slices(const afb_gemm_args& a, int sm_count, size_t ws_bytes, uint32_t& slices, uint32_t& kc) {
    const uint32_t ch = a.b_bits == 8 ? 64 : 128;
    uint32_t unit = 4 * ch;
    if (a.group_size > unit) unit = a.group_size;
    const uint32_t row_blocks = (a.n + kRowsPerCta - 1) / kRowsPerCta;
    uint32_t s = 1;
    while (row_blocks * s < 3u * (uint32_t)sm_count && s < 64 && a.k / (2 * s) >= unit && (a.k % (2 * s * unit)) == 0) s *= 2;
    while (s > 1 && (size_t)s * a.m * a.n * sizeof(float) > ws_bytes) s /= 2;
    slices = s;
    kc = a.k / s;
}

int launch_decode_ws(const afb_gemm_args& a, DeviceCtx* ctx, float* ws, size_t ws_bytes, uint32_t* counters,
                     size_t counter_count, cudaStream_t s) {
    if (!decode_supports(a)) return AFB_ERR_UNSUPPORTED;
    DecodeParams p;
    p.a = reinterpret_cast<const uint16_t*>(a.ptr_a);
    p.b = reinterpret_cast<const uint8_t*>(a.ptr_b);
    p.scale = a.ptr_scale;
    p.c = reinterpret_cast<uint16_t*>(a.ptr_c);
    p.m = a.m; p.n = a.n; p.k = a.k; p.lda = a.lda; p.ldc = a.ldc;
    p.ldb_bytes = a.b_bits == 8 ? a.ldb : a.ldb / 2;
    p.enc = a.b_encoding; p.scale_dtype = a.scale_dtype; p.group = a.group_size;
    pick_slices(a, ctx->sm_count, ws_bytes, p.slices, p.kc);
    p.ws = ws; p.counters = counters;
    const uint32_t row_blocks = (a.n + kRowsPerCta - 1) / kRowsPerCta;
    if (p.slices > 1 && row_blocks > counter_count) { p.slices = 1; p.kc = a.k; }
    dim3 grid(row_blocks, p.slices);
    const bool grouped = a.group_size != 0;
    const int mt = a.m <= 8 ? 1 : 2;
    cudaError_t e;
    if (a.b_bits == 8) {
        if (mt == 1) e = grouped ? launch_one<8, 1, true>(p, grid, s) : launch_one<8, 1, false>(p, grid, s);
        else         e = grouped ? launch_one<8, 2, true>(p, grid, s) : launch_one<8, 2, false>(p, grid, s);
    } else {
        if (mt == 1) e = grouped ? launch_one<4, 1, true>(p, grid, s) : launch_one<4, 1, false>(p, grid, s);
        else         e = grouped ? launch_one<4, 2, true>(p, grid, s) : launch_one<4, 2, false>(p, grid, s);
    }
    count_launch();
    return e == cudaSuccess ? AFB_OK : cuda_fail(e);
}

int launch_decode(const afb_gemm_args& a, DeviceCtx* ctx, cudaStream_t s) {
    return launch_decode_ws(a, ctx, ctx->splitk_ws, ctx->splitk_ws_bytes, ctx->splitk_counters, ctx->splitk_counter_count, s);
}

}  // namespace afb
