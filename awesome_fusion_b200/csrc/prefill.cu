// Prefill variant (M > 16, B in [N,K] layout): the compute-bound replacement of the
// reference kernel (bf16gemm_kernel_gfx90a.s:184-636) on 5th-generation tensor cores.
//
// One persistent CTA per SM walks C tiles of 128 x BN.  Per 64-wide K step:
//   warp 0      (1 lane)  TMA: A tile [128 x 64] bf16 (128-byte swizzle) and the RAW B tile
//                         [BN x 64] int8 / int4 into a ring of stages            (reference: .s:247-286 global loads)
//   warps 6-21  (512 thr) read the raw tile, unpack to exact bf16 in registers (dequant.cuh),
//                         optionally multiply by the per-group scale, and write a K-major
//                         128-byte-swizzled bf16 tile that tcgen05.mma can consume (reference: .dequant_int8_4x1, .s:18-55)
//   warp 1      (1 lane)  tcgen05.mma kind::f16, 128 x BN x 16, fp32 accumulators in TMEM (reference: MFMA macro .s:57-94)
//   warps 2-5   (128 thr) epilogue: tcgen05.ld the finished accumulator, multiply by the
//                         per-channel scale in fp32, round to nearest-even bf16, store C   (reference: .s:594-636)
// TMEM holds two accumulators so the epilogue of tile i overlaps the main loop of tile i+1.
// All hand-offs are mbarriers; every wait is bounded and, if one gives up, the CTA drains,
// frees its TMEM, and reports AFB_ERR_TIMEOUT through the status words.
#include "afb_internal.h"
#include "dequant.cuh"
#include "ptx_sm100.cuh"

namespace afb {

namespace {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int kStagesA = 4;   // A + raw-B ring
constexpr int kStagesB = 3;   // converted-B ring
constexpr int kConvWarps = 16;   // measured against 8: 84 vs 90 us (int4 group-128, 28672 x 8192, M <= 128), 94 vs 105 us (int8): more chains in flight
constexpr int kEpiWarps = 4;
constexpr int kThreads = 32 * (2 + kEpiWarps + kConvWarps);  // 704
constexpr int kFirstConvWarp = 2 + kEpiWarps;   // warps 2 .. 2+kEpiWarps-1 are the epilogue

struct PrefillParams {
    uint16_t* c;
    const void* scale;
    uint32_t m, n, k, ldc;
    uint32_t enc, scale_dtype, group;
    uint32_t m_tiles, n_tiles;
    uint32_t c_f32;     // 1: C is fp32 (partial sums of a K-split), 0: bf16
    uint32_t packed;    // B is in the pre-packed order of afb_prepack
    int32_t* status;
};

template <int BITS, int BN>
struct SmemLayout {
    static constexpr int kRawRowBytes = BK * BITS / 8;
    static constexpr int kABytes = BM * BK * 2;            // 16 KiB
    static constexpr int kBbfBytes = BN * BK * 2;          // 32 KiB at BN = 256
    static constexpr int kRawBytes = BN * kRawRowBytes;
    static constexpr int kOffA = 0;
    static constexpr int kOffBbf = kOffA + kStagesA * kABytes;
    static constexpr int kOffRaw = kOffBbf + kStagesB * kBbfBytes;
    static constexpr int kOffBars = kOffRaw + kStagesA * kRawBytes;
    static constexpr int kNumBars = 3 * kStagesA + 2 * kStagesB + 4;
    static constexpr int kOffMisc = kOffBars + kNumBars * 8;               // tmem base, abort flag
    static constexpr int kTotal = kOffMisc + 16;
    static constexpr int kDynamic = kTotal + 1024;                         // slack for manual 1 KiB alignment
};

__device__ __forceinline__ void report_timeout(int32_t* status, int where, int a, int b) {
    if (atomicCAS(status, 0, AFB_ERR_TIMEOUT) == 0) { status[1] = where; status[2] = a; status[3] = b; }
}

// Wait that also gives up as soon as another role has flagged an abort.
__device__ __forceinline__ bool wait_or_abort(uint32_t bar, uint32_t parity, volatile uint32_t* abort_flag) {
    if (ptx::mbar_try_wait(bar, parity)) return true;
    const unsigned long long t0 = ptx::globaltimer();
    uint32_t spins = 0;
    while (!ptx::mbar_try_wait(bar, parity)) {
        if ((++spins & 0xffu) == 0) {
            if (*abort_flag) return false;
            if (ptx::globaltimer() - t0 > ptx::kWaitLimitNs) return false;
        }
    }
    return true;
}

// Eight consecutive per-channel scales starting at channel n (n % 8 == 0) as fp32.
__device__ __forceinline__ void load_scale8(const void* scale, uint32_t dtype, uint32_t n, float (&out)[8]) {
    if (dtype == AFB_SCALE_BF16) {
        const uint4 v = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(scale) + n));
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) { out[2 * i] = __uint_as_float(w[i] << 16); out[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u); }
    } else {
        const float4 lo = __ldg(reinterpret_cast<const float4*>(reinterpret_cast<const float*>(scale) + n));
        const float4 hi = __ldg(reinterpret_cast<const float4*>(reinterpret_cast<const float*>(scale) + n) + 1);
        out[0] = lo.x; out[1] = lo.y; out[2] = lo.z; out[3] = lo.w; out[4] = hi.x; out[5] = hi.y; out[6] = hi.z; out[7] = hi.w;
    }
}

template <int BITS, bool GROUPED, int BN>
__global__ void __launch_bounds__(kThreads, 1)
prefill_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b, const PrefillParams p) {
    using L = SmemLayout<BITS, BN>;
    extern __shared__ uint8_t smem_raw_base[];
    const uint32_t smem_base = (ptx::smem_u32(smem_raw_base) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw_base + (smem_base - ptx::smem_u32(smem_raw_base));

    const uint32_t bar_base = smem_base + L::kOffBars;
    auto bar_full_ab  = [&](int s) { return bar_base + 8u * s; };
    auto bar_empty_a  = [&](int s) { return bar_base + 8u * (kStagesA + s); };
    auto bar_empty_raw= [&](int s) { return bar_base + 8u * (2 * kStagesA + s); };
    auto bar_full_bf  = [&](int s) { return bar_base + 8u * (3 * kStagesA + s); };
    auto bar_empty_bf = [&](int s) { return bar_base + 8u * (3 * kStagesA + kStagesB + s); };
    auto bar_acc_full = [&](int s) { return bar_base + 8u * (3 * kStagesA + 2 * kStagesB + s); };
    auto bar_acc_empty= [&](int s) { return bar_base + 8u * (3 * kStagesA + 2 * kStagesB + 2 + s); };
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem_gen + L::kOffMisc);
    volatile uint32_t* abort_flag = tmem_slot + 1;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t num_kb = p.k / BK;
    const uint32_t num_tiles = p.m_tiles * p.n_tiles;
    constexpr uint32_t kTmemCols = 2 * BN;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStagesA; ++s) { ptx::mbar_init(bar_full_ab(s), 1); ptx::mbar_init(bar_empty_a(s), 1); ptx::mbar_init(bar_empty_raw(s), kConvWarps); }
        for (int s = 0; s < kStagesB; ++s) { ptx::mbar_init(bar_full_bf(s), kConvWarps); ptx::mbar_init(bar_empty_bf(s), 1); }
        for (int s = 0; s < 2; ++s) { ptx::mbar_init(bar_acc_full(s), 1); ptx::mbar_init(bar_acc_empty(s), kEpiWarps); }
        *abort_flag = 0;
        ptx::fence_mbar_init();
        ptx::prefetch_tmap(&tmap_a);
        ptx::prefetch_tmap(&tmap_b);
    }
    if (warp == 1) {
        ptx::tmem_alloc(ptx::smem_u32(const_cast<uint32_t*>(tmem_slot)), kTmemCols);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ======================= TMA producer =======================
        if (lane == 0) {
            uint32_t stage = 0, phase = 0;
            uint32_t issued = 0;  // bit s: stage s has a load whose completion nobody may have observed yet
            uint32_t issued_parity = 0;
            bool ok = true;
            for (uint32_t t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
                const int m0 = (int)(t % p.m_tiles) * BM;
                const int n0 = (int)(t / p.m_tiles) * BN;
                for (uint32_t kb = 0; kb < num_kb; ++kb) {
                    if (!wait_or_abort(bar_empty_a(stage), phase ^ 1u, abort_flag) ||
                        !wait_or_abort(bar_empty_raw(stage), phase ^ 1u, abort_flag)) {
                        if (!*abort_flag) { report_timeout(p.status, 1, (int)t, (int)kb); *abort_flag = 1; }
                        ok = false; break;
                    }
                    ptx::mbar_arrive_expect_tx(bar_full_ab(stage), L::kABytes + L::kRawBytes);
                    ptx::tma_load_2d(smem_base + L::kOffA + stage * L::kABytes, &tmap_a, (int)(kb * BK), m0, bar_full_ab(stage));
                    ptx::tma_load_2d(smem_base + L::kOffRaw + stage * L::kRawBytes, &tmap_b, (int)(kb * L::kRawRowBytes), n0, bar_full_ab(stage));
                    issued |= 1u << stage;
                    issued_parity = (issued_parity & ~(1u << stage)) | (phase << stage);
                    if (++stage == kStagesA) { stage = 0; phase ^= 1u; }
                }
            }
            // never leave with a bulk copy still writing this CTA's shared memory
            for (int s = 0; s < kStagesA; ++s)
                if (issued & (1u << s)) ptx::mbar_wait(bar_full_ab(s), (issued_parity >> s) & 1u);
        }
    } else if (warp == 1) {
        // ======================= MMA issuer =======================
        if (lane == 0) {
            constexpr uint32_t idesc = ptx::umma_idesc_bf16_f32(BM, BN);
            uint32_t sa = 0, pa = 0, sb = 0, pb = 0, it = 0;
            bool ok = true;
            for (uint32_t t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++it) {
                const uint32_t as = it & 1u, ap = (it >> 1) & 1u;
                if (!wait_or_abort(bar_acc_empty(as), ap ^ 1u, abort_flag)) {
                    if (!*abort_flag) { report_timeout(p.status, 2, (int)t, -1); *abort_flag = 1; }
                    break;
                }
                ptx::tc_fence_after_sync();
                const uint32_t tmem_d = tmem_base + as * BN;
                for (uint32_t kb = 0; kb < num_kb; ++kb) {
                    if (!wait_or_abort(bar_full_ab(sa), pa, abort_flag) || !wait_or_abort(bar_full_bf(sb), pb, abort_flag)) {
                        if (!*abort_flag) { report_timeout(p.status, 3, (int)t, (int)kb); *abort_flag = 1; }
                        ok = false; break;
                    }
                    ptx::tc_fence_after_sync();
                    const uint64_t da = ptx::umma_desc_kmajor_sw128(smem_base + L::kOffA + sa * L::kABytes);
                    const uint64_t db = ptx::umma_desc_kmajor_sw128(smem_base + L::kOffBbf + sb * L::kBbfBytes);
#pragma unroll
                    for (int j = 0; j < BK / 16; ++j)  // +32 bytes per 16-wide K step: +2 in the address field
                        ptx::umma_bf16(tmem_d, da + 2u * j, db + 2u * j, idesc, (kb | (uint32_t)j) ? 1u : 0u);
                    ptx::umma_commit(bar_empty_a(sa));
                    ptx::umma_commit(bar_empty_bf(sb));
                    if (++sa == kStagesA) { sa = 0; pa ^= 1u; }
                    if (++sb == kStagesB) { sb = 0; pb ^= 1u; }
                }
                if (ok) ptx::umma_commit(bar_acc_full(as));
            }
        }
    } else if (warp < kFirstConvWarp) {
        // ======================= epilogue =======================
            const uint32_t lane_group = (uint32_t)(warp & 3);    // TMEM lanes this warp may read
        uint32_t it = 0;
        for (uint32_t t = blockIdx.x; t < num_tiles; t += gridDim.x, ++it) {
            const uint32_t as = it & 1u, ap = (it >> 1) & 1u;
            const uint32_t m0 = (t % p.m_tiles) * BM, n0 = (t / p.m_tiles) * BN;
            if (!wait_or_abort(bar_acc_full(as), ap, abort_flag)) {
                if (!*abort_flag) { report_timeout(p.status, 4, (int)t, -1); *abort_flag = 1; }
                break;
            }
            ptx::tc_fence_after_sync();
            const uint32_t row = m0 + lane_group * 32 + lane;
            uint16_t* crow = p.c + (size_t)row * p.ldc + n0;
            float* crow32 = reinterpret_cast<float*>(p.c) + (size_t)row * p.ldc + n0;
#pragma unroll 1
            for (int ch = 0; ch < BN / 32; ++ch) {
                uint32_t r[32];
                ptx::tmem_ld_32x32(tmem_base + ((lane_group * 32u) << 16) + as * BN + ch * 32, r);
                ptx::tmem_ld_wait();
                if (row < p.m) {
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const uint32_t col = n0 + ch * 32 + q * 8;
                        if (col < p.n) {
                            float v[8];
#pragma unroll
                            for (int e = 0; e < 8; ++e) v[e] = __uint_as_float(r[q * 8 + e]);
                            if (!GROUPED) {
                                float sc[8];
                                load_scale8(p.scale, p.scale_dtype, col, sc);  // same address in all lanes: one broadcast
#pragma unroll
                                for (int e = 0; e < 8; ++e) v[e] *= sc[e];
                            }
                            if (p.c_f32) {
                                *reinterpret_cast<float4*>(crow32 + ch * 32 + q * 8) = make_float4(v[0], v[1], v[2], v[3]);
                                *reinterpret_cast<float4*>(crow32 + ch * 32 + q * 8 + 4) = make_float4(v[4], v[5], v[6], v[7]);
                            } else {
                                uint32_t o[4];
#pragma unroll
                                for (int e = 0; e < 4; ++e) {
                                    const __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * e], v[2 * e + 1]);
                                    o[e] = *reinterpret_cast<const uint32_t*>(&h);
                                }
                                *reinterpret_cast<uint4*>(crow + ch * 32 + q * 8) = make_uint4(o[0], o[1], o[2], o[3]);
                            }
                        }
                    }
                }
            }
            ptx::tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(bar_acc_empty(as));
        }
    } else {
        // ======================= converters =======================
        const int cid = threadIdx.x - kFirstConvWarp * 32;   // 0..511
        constexpr int kPiecesPerRow = L::kRawRowBytes / 16;   // 4 (int8) or 2 (int4)
        constexpr int kItems = (BN * kPiecesPerRow + kConvWarps * 32 - 1) / (kConvWarps * 32);   // the last item may be empty for some threads
        const uint32_t xormask = (BITS == 8 && p.enc == AFB_ENC_OFFSET_BINARY) ? 0x80808080u : 0u;
        const uint32_t magic4 = p.enc == AFB_ENC_OFFSET_BINARY ? 0x43004300u : 0x43084308u;
        const uint32_t groups_per_row = GROUPED ? p.k / p.group : 0;
        const uint32_t kb_per_group = GROUPED ? p.group / BK : 1;
        uint32_t sa = 0, pa = 0, sb = 0, pb = 0;
        bool ok = true;
        for (uint32_t t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
            const uint32_t n0 = (t / p.m_tiles) * BN;
            uint32_t sc_cur[kItems], sc_nxt[kItems];
            auto load_scale = [&](int itx, uint32_t gidx) -> uint32_t {
                const uint32_t rowi = (uint32_t)(itx * (kConvWarps * 32) + cid) / kPiecesPerRow;
                const uint32_t nn = n0 + rowi;
                if (rowi >= (uint32_t)BN || nn >= p.n || gidx >= groups_per_row) return (uint32_t)0;
                return bf16_dup(reinterpret_cast<const uint16_t*>(p.scale)[(size_t)nn * groups_per_row + gidx]);
            };
            if (GROUPED) {
#pragma unroll
                for (int itx = 0; itx < kItems; ++itx) { sc_cur[itx] = 0; sc_nxt[itx] = load_scale(itx, 0); }
            }
            for (uint32_t kb = 0; kb < num_kb; ++kb) {
                if (GROUPED && (kb % kb_per_group) == 0) {
                    const uint32_t gidx = kb / kb_per_group;
#pragma unroll
                    for (int itx = 0; itx < kItems; ++itx) { sc_cur[itx] = sc_nxt[itx]; sc_nxt[itx] = load_scale(itx, gidx + 1); }
                }
                if (!wait_or_abort(bar_full_ab(sa), pa, abort_flag) || !wait_or_abort(bar_empty_bf(sb), pb ^ 1u, abort_flag)) {
                    if (!*abort_flag) { report_timeout(p.status, 5, (int)t, (int)kb); *abort_flag = 1; }
                    ok = false; break;
                }
                const uint8_t* raw = smem_gen + L::kOffRaw + sa * L::kRawBytes;
                uint8_t* bf = smem_gen + L::kOffBbf + sb * L::kBbfBytes;
#pragma unroll
                for (int itx = 0; itx < kItems; ++itx) {
                    const uint32_t id = (uint32_t)(itx * (kConvWarps * 32) + cid);
                    if (id >= (uint32_t)(BN * kPiecesPerRow)) continue;
                    const uint32_t rowi = id / kPiecesPerRow, piece = id % kPiecesPerRow;
                    const uint4 w4 = *reinterpret_cast<const uint4*>(raw + rowi * L::kRawRowBytes + piece * 16);
                    const uint32_t w[4] = {w4.x, w4.y, w4.z, w4.w};
                    uint8_t* orow = bf + (rowi >> 3) * 1024 + (rowi & 7) * 128;
                    const uint32_t sw = rowi & 7;
                    if (BITS == 8) {
                        uint32_t o[8];
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            s8x4_to_bf16_pairs(w[j] ^ xormask, p.packed != 0, o[2 * j], o[2 * j + 1]);
                            if (GROUPED) { o[2 * j] = bf16x2_mul(o[2 * j], sc_cur[itx]); o[2 * j + 1] = bf16x2_mul(o[2 * j + 1], sc_cur[itx]); }
                        }
                        *reinterpret_cast<uint4*>(orow + (((2 * piece) ^ sw) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
                        *reinterpret_cast<uint4*>(orow + (((2 * piece + 1) ^ sw) << 4)) = make_uint4(o[4], o[5], o[6], o[7]);
                    } else {
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            uint32_t q[4];
                            s4x8_to_bf16_pairs(w[j], magic4, p.packed != 0, q);
                            if (GROUPED) {
#pragma unroll
                                for (int e = 0; e < 4; ++e) q[e] = bf16x2_mul(q[e], sc_cur[itx]);
                            }
                            *reinterpret_cast<uint4*>(orow + (((4 * piece + j) ^ sw) << 4)) = make_uint4(q[0], q[1], q[2], q[3]);
                        }
                    }
                }
                ptx::fence_proxy_async_smem();   // generic-proxy writes -> visible to the tensor core's async-proxy reads
                __syncwarp();
                if (lane == 0) { ptx::mbar_arrive(bar_full_bf(sb)); ptx::mbar_arrive(bar_empty_raw(sa)); }
                if (++sa == kStagesA) { sa = 0; pa ^= 1u; }
                if (++sb == kStagesB) { sb = 0; pb ^= 1u; }
            }
        }
    }

    // ---- teardown: every thread gets here, also after an abort ----
    ptx::tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        ptx::tc_fence_after_sync();
        ptx::tmem_dealloc(tmem_base, kTmemCols);
    }
}

int make_tmap_2d(CUtensorMap* map, CUtensorMapDataType dt, const void* base, uint64_t inner, uint64_t outer,
                 uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer, CUtensorMapSwizzle swz) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return AFB_ERR_CUDA;
    cuuint64_t dims[2] = {inner, outer};
    cuuint64_t strides[1] = {row_stride_bytes};
    cuuint32_t box[2] = {box_inner, box_outer};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? AFB_OK : AFB_ERR_CUDA;
}

template <int BITS, bool GROUPED, int BN>
int launch_cfg(const afb_gemm_args& a, DeviceCtx* ctx, cudaStream_t s) {
    using L = SmemLayout<BITS, BN>;
    static_assert(L::kDynamic <= 232448, "shared memory budget");
    CUtensorMap ta, tb;
    int rc = make_tmap_2d(&ta, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, a.ptr_a, a.k, a.m, (uint64_t)a.lda * 2, BK, BM,
                          CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
    const uint64_t row_bytes = (uint64_t)a.k * BITS / 8, ld_bytes = (uint64_t)a.ldb * BITS / 8;
    rc = make_tmap_2d(&tb, CU_TENSOR_MAP_DATA_TYPE_UINT8, a.ptr_b, row_bytes, a.n, ld_bytes, L::kRawRowBytes, BN,
                      CU_TENSOR_MAP_SWIZZLE_NONE);
    if (rc) return rc;
    PrefillParams p;
    p.c = reinterpret_cast<uint16_t*>(a.ptr_c);
    p.scale = a.ptr_scale;
    p.m = a.m; p.n = a.n; p.k = a.k; p.ldc = a.ldc;
    p.enc = a.b_encoding; p.scale_dtype = a.scale_dtype; p.group = a.group_size;
    p.m_tiles = (a.m + BM - 1) / BM;
    p.n_tiles = (a.n + BN - 1) / BN;
    p.c_f32 = (a.flags & AFB_FLAG_C_F32) ? 1u : 0u;
    p.packed = a.b_layout == AFB_LAYOUT_COL_PACKED ? 1u : 0u;
    p.status = ctx->status;
    auto kern = prefill_kernel<BITS, GROUPED, BN>;
    static DeviceOnce attr_set;  // per template instance
    if (!attr_set.done(ctx->device)) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDynamic);
        if (e != cudaSuccess) return cuda_fail(e);
        attr_set.mark(ctx->device);
    }
    const uint32_t tiles = p.m_tiles * p.n_tiles;
    const uint32_t grid = tiles < (uint32_t)ctx->sm_count ? tiles : (uint32_t)ctx->sm_count;
    kern<<<grid, kThreads, L::kDynamic, s>>>(ta, tb, p);
    count_launch();
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? AFB_OK : cuda_fail(e);
}

}  // namespace

bool prefill_supports(const afb_gemm_args& a) {
    if (a.b_layout != AFB_LAYOUT_COL && a.b_layout != AFB_LAYOUT_COL_PACKED) return false;
    if (a.b_bits != 8 && a.b_bits != 4) return false;
    if (a.m == 0 || a.n == 0 || a.k == 0) return false;
    if (a.k % BK || a.n % 8) return false;
    if (a.lda % 8 || a.ldc % 8) return false;
    const uint64_t ld_bytes = (uint64_t)a.ldb * a.b_bits / 8;
    if (ld_bytes % 16) return false;
    if ((uintptr_t)a.ptr_a % 16 || (uintptr_t)a.ptr_b % 16 || (uintptr_t)a.ptr_c % 16 || (uintptr_t)a.ptr_scale % 16) return false;
    if (a.group_size) {
        if (a.group_size % 32 || a.k % a.group_size) return false;   // the tensor-memory form converts 32 consecutive k per thread
        if (a.scale_dtype != AFB_SCALE_BF16) return false;  // the dequant contract is bf16_rn(q * bf16 scale)
    }
    return true;
}

// What only the tensor-memory form (prefill_ts.cu) covers: groups of 32 (this form converts 64-wide steps), zero-points.
bool prefill_needs_ts(const afb_gemm_args& a) { return (a.group_size && a.group_size % BK) || a.ptr_zero != nullptr; }

int launch_prefill(const afb_gemm_args& a, DeviceCtx* ctx, cudaStream_t s) {
    if (!prefill_supports(a) || prefill_needs_ts(a)) return AFB_ERR_UNSUPPORTED;
    const bool grouped = a.group_size != 0;
    // BN = 256 halves the A traffic per flop; BN = 128 wastes less on narrow N
    const bool wide = a.n > 128;
    if (a.b_bits == 8) {
        if (wide) return grouped ? launch_cfg<8, true, 256>(a, ctx, s) : launch_cfg<8, false, 256>(a, ctx, s);
        return grouped ? launch_cfg<8, true, 128>(a, ctx, s) : launch_cfg<8, false, 128>(a, ctx, s);
    }
    if (wide) return grouped ? launch_cfg<4, true, 256>(a, ctx, s) : launch_cfg<4, false, 256>(a, ctx, s);
    return grouped ? launch_cfg<4, true, 128>(a, ctx, s) : launch_cfg<4, false, 128>(a, ctx, s);
}

}  // namespace afb
