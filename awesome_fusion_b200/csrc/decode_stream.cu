// Decode variant, streaming form (M <= 16, B in [N,K] layout, plain or pre-packed): the memory-bound replacement of
// the reference kernel's main loop (bf16gemm_kernel_gfx90a.s:410-489) for GEMV-like shapes.
//
// Every weight byte is read from HBM exactly once.  A CTA has 8 warps arranged WR x WK: it owns 16*WR output channels
// and one K range; the WK warps that share 16 channels split each staged window of K into contiguous stretches.
//   * weights: each warp streams its 64-byte-per-channel chunks (16 channels x 64 bytes = 1 KiB) through a private
//     8-stage cp.async ring in shared memory; a lane reads back its own 16 bytes, so the ring needs no barrier;
//   * activations: the rows of the current K window are copied into shared memory AS THEY ARE by cp.async, into one of
//     two buffers, while the previous window is being consumed (one block-wide barrier per window, no register
//     staging); a lane reads the 16 or 32 consecutive k its weights cover;
//   * unpack to exact bf16 in registers (dequant.cuh) with the cheap pairing, mma.sync.m16n8k16 with the 16 channels as
//     the row operand and the <= 16 activation rows as the column operand.  For PRE-PACKED weights (afb_prepack) the
//     cheap pairing IS the natural k order and the activations are used as loaded; for plain weights each lane
//     re-pairs its activations with two byte permutes per four k;
//   * the first ring fill touches only the weights, which a caller may declare constant (AFB_FLAG_PDL): the kernel is
//     then launched with programmatic stream serialisation, lets its successor start at once, and waits for its
//     predecessor only before it first touches activations, workspace or C.
// Reduction across the WK warps, K-slices, the balanced one-wave form and the fixed-order cross-CTA sum are those of
// the staged form (decode.cu).
#include <cstdlib>
#include "afb_internal.h"
#include "dequant.cuh"
#include "decode_common.cuh"

namespace afb {

namespace {

constexpr int kRingS = 8;                       // cp.async stages per warp
constexpr int kRingBytesS = kWarps * kRingS * kStageBytes;   // 64 KiB
// one activation buffer: m rows x (window_k * 2 + 16) bytes.  Two buffers + the ring leave room for two CTAs per SM.
__host__ __device__ constexpr int act_buf_bytes(int mt) { return mt == 1 ? 20 * 1024 : 24 * 1024; }
__host__ __device__ constexpr int smem_bytes_s(int mt) { return kRingBytesS + 2 * act_buf_bytes(mt) + 16; }
static_assert(kRedFloats * 4 <= kRingBytesS, "the reduction buffer must fit the ring it reuses");

__device__ __forceinline__ void grid_dependents_may_start() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

template <int BITS, int MT, bool GROUPED, bool PACKED>
__global__ void __launch_bounds__(kThreads, 2) decode_stream_kernel(const DecodeParams p) {
    constexpr int CH = BITS == 8 ? 64 : 128;    // k per chunk (a quad covers 64 bytes of one channel)
    constexpr int LK = CH / 4;                  // k per lane per chunk
    constexpr int AV = LK / 8;                  // 16-byte activation vectors per lane, row and chunk
    constexpr int R = kRingS;

    extern __shared__ __align__(16) uint8_t smem[];
    float* s_red = reinterpret_cast<float*>(smem);
    uint32_t* s_last = reinterpret_cast<uint32_t*>(smem + kRingBytesS + 2 * act_buf_bytes(MT));
    const uint32_t s_act0 = (uint32_t)__cvta_generic_to_shared(smem + kRingBytesS);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, tig = lane & 3;
    const uint32_t wk_count = kWarps / p.wr;
    const uint32_t wr = warp / wk_count, wk = warp % wk_count;
    const uint32_t xormask = (BITS == 8 && p.enc == AFB_ENC_OFFSET_BINARY) ? 0x80808080u : 0u;
    const uint32_t magic4 = p.enc == AFB_ENC_OFFSET_BINARY ? 0x43004300u : 0x43084308u;
    const uint32_t groups_per_row = GROUPED ? (p.k >> p.group_shift) : 0;
    const uint32_t ring = (uint32_t)__cvta_generic_to_shared(smem) + warp * (R * kStageBytes) + lane * 16;
    const uint32_t act_row_bytes = p.pass_k * 2 + 16;   // +16: consecutive rows land in different bank groups

    grid_dependents_may_start();   // the next kernel of the stream may begin its own weight prefetch
    bool dependency_met = false;

    // Row of this lane inside a staged buffer.  Rows beyond m are never staged: such a lane reads row 0 instead, which
    // only feeds output columns (activation rows) that are never stored.
    uint32_t act_row[MT];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) act_row[mt] = ((uint32_t)(mt * 8 + g) < p.m ? mt * 8 + g : 0) * act_row_bytes;
    // 16-byte pieces of this lane inside a chunk.  int4 (16 pieces per chunk): bit 3 of the piece index flips bit 1, so that
    // the four lanes of a quad land in different bank groups; int8 (8 pieces per chunk) needs no swizzle.
    uint32_t act_off[AV];
#pragma unroll
    for (int v = 0; v < AV; ++v) act_off[v] = (BITS == 4 ? swz_piece(tig * AV + v) : (uint32_t)(tig * AV + v)) * 16;

    // ---- the pieces of work of this CTA: one (channel block, K range) in the grid form, a run of units in the balanced form
    const uint32_t u_begin = p.streamk ? (uint32_t)((uint64_t)blockIdx.x * p.total_units / gridDim.x) : 0u;
    const uint32_t u_end = p.streamk ? (uint32_t)((uint64_t)(blockIdx.x + 1) * p.total_units / gridDim.x) : 1u;
    auto cta_of = [&](uint32_t u) { return (uint32_t)((((uint64_t)u + 1) * gridDim.x + p.total_units - 1) / p.total_units) - 1u; };
    for (uint32_t u = u_begin; u < u_end;) {
    uint32_t cb, ks, kend;
    if (p.streamk) {
        cb = u / p.units_per_cb;
        const uint32_t ku0 = u - cb * p.units_per_cb, ku1 = min(p.units_per_cb, ku0 + (u_end - u));
        ks = ku0 * p.unit_k; kend = ku1 * p.unit_k;
        u += ku1 - ku0;
    } else {
        cb = blockIdx.x; ks = blockIdx.y * p.kc; kend = min(p.k, ks + p.kc);
        u = u_end;
    }
    const uint32_t nblk = cb * 16 * p.wr;
    const uint32_t row_a = nblk + wr * 16 + g, row_b = row_a + 8;
    const bool ok_a = row_a < p.n, ok_b = row_b < p.n;
    const uint8_t* pa = p.b + (size_t)(ok_a ? row_a : 0) * p.ldb_bytes + tig * 16;
    const uint8_t* pb = p.b + (size_t)(ok_b ? row_b : 0) * p.ldb_bytes + tig * 16;

    // Windows of K ("passes"): [ks + w * pass_k, ...).  Inside a window warp wk takes the contiguous chunks
    // [wk * cpw, wk * cpw + mine) with cpw = ceil(chunks of the window / WK).
    auto window_len = [&](uint32_t pk) { return min(p.pass_k, kend - pk); };
    auto my_first = [&](uint32_t plen) { const uint32_t c = plen / CH, cpw = (c + wk_count - 1) / wk_count; return min(c, wk * cpw); };
    auto my_count = [&](uint32_t plen) { const uint32_t c = plen / CH, cpw = (c + wk_count - 1) / wk_count, f = min(c, wk * cpw); return min(cpw, c - f); };

    // ---- weight stream: an issue cursor that runs up to R - 1 chunks ahead of the consumer, across window boundaries
    uint32_t iss_pk = ks, iss_left = my_count(window_len(ks));
    const uint8_t* src_a = pa + (size_t)(ks + my_first(window_len(ks)) * CH) * BITS / 8;
    const uint8_t* src_b = pb + (size_t)(ks + my_first(window_len(ks)) * CH) * BITS / 8;
    uint32_t issued = 0;
    auto issue = [&]() {   // copy this warp's next chunk (if any is left) into ring slot issued % R
        while (iss_left == 0) {
            if (kend - iss_pk <= p.pass_k) return;   // no window after this one
            iss_pk += p.pass_k;
            const uint32_t pl = window_len(iss_pk);
            iss_left = my_count(pl);
            const size_t off = (size_t)(iss_pk + my_first(pl) * CH) * BITS / 8;
            src_a = pa + off; src_b = pb + off;
        }
        const uint32_t dst = ring + (issued & (R - 1)) * kStageBytes;
        if (ok_a) cp_async16(dst, src_a);
        if (ok_b) cp_async16(dst + 512, src_b);
        src_a += 64; src_b += 64; ++issued; --iss_left;
    };
    // activation rows of window [pk, pk + plen) -> buffer `buf`, as they are (16-byte pieces, swizzled position)
    auto stage_window = [&](uint32_t pk, uint32_t plen, uint32_t buf) {
        const uint32_t pieces = plen >> 3;
        const uint32_t dst0 = s_act0 + buf * act_buf_bytes(MT);
        for (uint32_t r = tid >> 6; r < p.m; r += 4)
            for (uint32_t pc = tid & 63; pc < pieces; pc += 64)
                cp_async16(dst0 + r * act_row_bytes + (BITS == 4 ? swz_piece(pc) : pc) * 16, p.a + (size_t)r * p.lda + pk + pc * 8);
    };

    const uint16_t* sc_h = reinterpret_cast<const uint16_t*>(p.scale);
    const float* sc_f = reinterpret_cast<const float*>(p.scale);
    const size_t sc_ia = (size_t)(ok_a ? row_a : 0) * groups_per_row, sc_ib = (size_t)(ok_b ? row_b : 0) * groups_per_row;
    auto load_group_scales = [&](uint32_t k0, float& sa, float& sb) {
        const uint32_t grp = k0 >> p.group_shift;
        if (p.scale_dtype == AFB_SCALE_BF16) { sa = bf16_to_f32(sc_h[sc_ia + grp]); sb = bf16_to_f32(sc_h[sc_ib + grp]); }
        else { sa = sc_f[sc_ia + grp]; sb = sc_f[sc_ib + grp]; }
    };

    float acc[MT][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[mt][e] = 0.f;

    // the weight stream starts before anything else: these copies read only B
#pragma unroll
    for (int j = 0; j < R - 1; ++j) { issue(); cp_async_commit(); }
    if (!dependency_met) { grid_dependency_wait(); dependency_met = true; }   // from here on: activations, workspace, C
    stage_window(ks, window_len(ks), 0);
    cp_async_commit();
    cp_async_wait<0>();
    __syncthreads();

    uint32_t consumed = 0, buf = 0;
    for (uint32_t pk = ks; pk < kend; pk += p.pass_k, buf ^= 1u) {
        const uint32_t plen = window_len(pk);
        uint32_t groups_since_stage = 0;
        if (pk + p.pass_k < kend) {   // the next window travels while this one is consumed (its buffer was released by the barrier)
            stage_window(pk + p.pass_k, window_len(pk + p.pass_k), buf ^ 1u);
            cp_async_commit();
        }
        const uint32_t first = my_first(plen), mine = my_count(plen);
        uint32_t aoff = s_act0 + buf * act_buf_bytes(MT) + first * (CH * 2);
        uint32_t kcur = pk + first * CH;
        float sc_a = 0.f, sc_b = 0.f;
        for (uint32_t j = 0; j < mine; ++j, ++consumed, aoff += CH * 2, kcur += CH) {
            issue();
            cp_async_commit();
            ++groups_since_stage;
            if (GROUPED) load_group_scales(kcur, sc_a, sc_b);
            uint32_t s[MT][AV * 4];
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                for (int v = 0; v < AV; ++v) {
                    const uint4 t = lds128(aoff + act_row[mt] + act_off[v]);
                    s[mt][4 * v] = t.x; s[mt][4 * v + 1] = t.y; s[mt][4 * v + 2] = t.z; s[mt][4 * v + 3] = t.w;
                }
            if (!PACKED) {   // plain weights unpack to {k0,k2},{k1,k3} (int8) / {k0,k4},{k1,k5},{k2,k6},{k3,k7} (int4): pair the activations alike
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    if (BITS == 8) {
#pragma unroll
                        for (int q = 0; q < AV * 2; ++q) {
                            const uint32_t x = s[mt][2 * q], y = s[mt][2 * q + 1];
                            s[mt][2 * q] = prmt(x, y, 0x5410u); s[mt][2 * q + 1] = prmt(x, y, 0x7632u);
                        }
                    } else {
#pragma unroll
                        for (int q = 0; q < AV; ++q) {
                            const uint32_t x0 = s[mt][4 * q], x1 = s[mt][4 * q + 1], x2 = s[mt][4 * q + 2], x3 = s[mt][4 * q + 3];
                            s[mt][4 * q] = prmt(x0, x2, 0x5410u); s[mt][4 * q + 1] = prmt(x0, x2, 0x7632u);
                            s[mt][4 * q + 2] = prmt(x1, x3, 0x5410u); s[mt][4 * q + 3] = prmt(x1, x3, 0x7632u);
                        }
                    }
                }
            }
            cp_async_wait<R - 1>();   // this warp's chunk `consumed` has landed (each lane reads only what it copied itself)
            const uint32_t slot = ring + (consumed & (R - 1)) * kStageBytes;
            const uint4 wa4 = lds128(slot), wb4 = lds128(slot + 512);
            const uint32_t wav[4] = {wa4.x, wa4.y, wa4.z, wa4.w};
            const uint32_t wbv[4] = {wb4.x, wb4.y, wb4.z, wb4.w};
            float part[MT][4];   // grouped: the sum of this chunk alone (a chunk lies inside one scale group)
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                for (int e = 0; e < 4; ++e) part[mt][e] = 0.f;
#pragma unroll
            for (int j2 = 0; j2 < 4; ++j2) {
                if (BITS == 8) {
                    uint32_t a0, a1, a2, a3;
                    s8x4_to_bf16_strided(wav[j2] ^ xormask, a0, a2);
                    s8x4_to_bf16_strided(wbv[j2] ^ xormask, a1, a3);
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt)
                        mma_bf16(GROUPED ? part[mt] : acc[mt], a0, a1, a2, a3, s[mt][2 * j2], s[mt][2 * j2 + 1]);
                } else {
                    uint32_t qa[4], qb[4];
                    s4x8_to_bf16_strided(wav[j2], magic4, qa);
                    s4x8_to_bf16_strided(wbv[j2], magic4, qb);
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt) {
                        mma_bf16(GROUPED ? part[mt] : acc[mt], qa[0], qb[0], qa[1], qb[1], s[mt][4 * j2], s[mt][4 * j2 + 1]);
                        mma_bf16(GROUPED ? part[mt] : acc[mt], qa[2], qb[2], qa[3], qb[3], s[mt][4 * j2 + 2], s[mt][4 * j2 + 3]);
                    }
                }
            }
            if (GROUPED) {
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    acc[mt][0] = fmaf(sc_a, part[mt][0], acc[mt][0]); acc[mt][1] = fmaf(sc_a, part[mt][1], acc[mt][1]);
                    acc[mt][2] = fmaf(sc_b, part[mt][2], acc[mt][2]); acc[mt][3] = fmaf(sc_b, part[mt][3], acc[mt][3]);
                }
            }
        }
        if (pk + p.pass_k < kend) {
            // this thread's copies of the next window are older than its last R - 1 groups only if it committed that many since
            if (groups_since_stage < (uint32_t)(R - 1)) cp_async_wait<0>();
            __syncthreads();   // every thread's copies of the next window are in place; every warp is done with this one
        }
    }

    // ---- reduce the WK warps that share 16 channels.  acc[mt][e]: channel = e < 2 ? g : g + 8, activation row = mt*8 + 2*tig + (e & 1)
    constexpr int MCOLS = 8 * MT;
    cp_async_wait<0>();
    __syncthreads();   // every warp is done with its ring slots: the reduction buffer takes their place
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int e = 0; e < 4; ++e)
            s_red[(warp * 16 + (e < 2 ? g : g + 8)) * 17 + mt * 8 + 2 * tig + (e & 1)] = acc[mt][e];
    __syncthreads();
    decode_finish<GROUPED>(p, s_red, s_last, cb, nblk, wk_count, MCOLS, cta_of);
    if (u < u_end) __syncthreads();   // the next piece reuses the ring (= the reduction buffer) and the flag word
    }   // pieces of work
    if (!dependency_met) grid_dependency_wait();
}

template <int BITS, int MT, bool GROUPED, bool PACKED>
cudaError_t launch_stream_one(const DecodeParams& p, dim3 grid, bool pdl, cudaStream_t s) {
    auto kern = decode_stream_kernel<BITS, MT, GROUPED, PACKED>;
    static DeviceOnce attr_set;   // per template instance
    int dev = 0;
    cudaGetDevice(&dev);
    if (!attr_set.done(dev)) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes_s(MT));
        if (e != cudaSuccess) return e;
        attr_set.mark(dev);
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = dim3(kThreads); cfg.dynamicSmemBytes = smem_bytes_s(MT); cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, p);
}

template <int BITS, int MT, bool GROUPED, bool PACKED>
int resident_stream_one() {
    static std::atomic<int> cached[32];   // 0 = not asked yet
    int dev = 0;
    cudaGetDevice(&dev);
    int n = cached[dev & 31].load(std::memory_order_acquire);
    if (n == 0) {
        auto kern = decode_stream_kernel<BITS, MT, GROUPED, PACKED>;
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes_s(MT)) != cudaSuccess) return 0;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kern, kThreads, smem_bytes_s(MT)) != cudaSuccess) return 0;
        cached[dev & 31].store(n, std::memory_order_release);
    }
    return n;
}

template <int BITS, int MT, bool GROUPED>
cudaError_t launch_stream_packed(bool packed, const DecodeParams& p, dim3 grid, bool pdl, cudaStream_t s) {
    return packed ? launch_stream_one<BITS, MT, GROUPED, true>(p, grid, pdl, s) : launch_stream_one<BITS, MT, GROUPED, false>(p, grid, pdl, s);
}

}  // namespace

int decode_stream_act_bytes(int mt) { return act_buf_bytes(mt); }

int decode_stream_resident(uint32_t bits, int mt, bool grouped) {   // the PACKED instances have the same footprint
    if (bits == 8) {
        if (mt == 1) return grouped ? resident_stream_one<8, 1, true, false>() : resident_stream_one<8, 1, false, false>();
        return grouped ? resident_stream_one<8, 2, true, false>() : resident_stream_one<8, 2, false, false>();
    }
    if (mt == 1) return grouped ? resident_stream_one<4, 1, true, false>() : resident_stream_one<4, 1, false, false>();
    return grouped ? resident_stream_one<4, 2, true, false>() : resident_stream_one<4, 2, false, false>();
}

cudaError_t decode_stream_launch(uint32_t bits, int mt, bool grouped, bool packed, const DecodeParams& p, dim3 grid, bool pdl, cudaStream_t s) {
    if (bits == 8) {
        if (mt == 1) return grouped ? launch_stream_packed<8, 1, true>(packed, p, grid, pdl, s) : launch_stream_packed<8, 1, false>(packed, p, grid, pdl, s);
        return grouped ? launch_stream_packed<8, 2, true>(packed, p, grid, pdl, s) : launch_stream_packed<8, 2, false>(packed, p, grid, pdl, s);
    }
    if (mt == 1) return grouped ? launch_stream_packed<4, 1, true>(packed, p, grid, pdl, s) : launch_stream_packed<4, 1, false>(packed, p, grid, pdl, s);
    return grouped ? launch_stream_packed<4, 2, true>(packed, p, grid, pdl, s) : launch_stream_packed<4, 2, false>(packed, p, grid, pdl, s);
}

}  // namespace afb
