// Decode variant (M <= 16, B in [N,K] layout): the memory-bound replacement of the
// reference kernel's main loop (bf16gemm_kernel_gfx90a.s:410-489) for GEMV-like shapes.
//
// Every weight byte is read from HBM exactly once; the dominant stream is B (N*K*bits/8 bytes).
// A CTA has 8 warps arranged WR x WK: it owns 16*WR output channels and one K-slice, and the WK warps
// that share 16 channels take interleaved 64-byte chunks of K.  Each warp streams its chunks through a
// private ring in shared memory with 16-byte cp.async copies (deep memory-level parallelism without
// holding registers; the ring keeps filling across the block-wide barriers); a lane then reads back its own 16 bytes =
// 16 (int8) or 32 (int4) consecutive-k weights of one channel, unpacks them to exact bf16 in registers
// (dequant.cuh) and feeds mma.sync.m16n8k16 with the 16 channels as the row operand and the <= 16
// activation rows as the column operand.  The four lanes of a quad hold different k, so the tensor-core
// instruction performs the intra-warp split-K reduction; the WK warps are reduced through shared memory,
// and K-slices owned by different CTAs are combined through an fp32 workspace by the last CTA to arrive
// (fixed summation order, so results are run-to-run identical).
//
// Because a dot product does not care about the order of k, weights are paired in the order that is
// cheapest to unpack ({k0,k2},{k1,k3} for int8; {k0,k4}..{k3,k7} for int4); the activations of the CTA's
// K range are staged once per pass in shared memory, already permuted to match, and shared by all warps.
//
// Scales: per-channel scales multiply the fp32 sum once at the end (the reference multiplies every
// weight, .s:29-33; mathematically the same, one rounding fewer).  Per-group scales multiply the fp32
// partial sum of each chunk (a chunk never straddles a group).
#include <cstdlib>
#include "afb_internal.h"
#include "dequant.cuh"
#include "decode_common.cuh"

namespace afb {

namespace {

#ifndef AFB_DECODE_MT1_CTAS
#define AFB_DECODE_MT1_CTAS 4
#endif
#ifndef AFB_DECODE_MT2_CTAS
#define AFB_DECODE_MT2_CTAS 3
#endif
// cp.async stages per warp (RING, a power of two): 4 for large matrices (32 KiB per CTA, up to four CTAs per SM), 8 for matrices so
// small that a warp owns at most 8 chunks (64 KiB per CTA, two CTAs per SM): its whole share of the weights is then in flight
// before the kernel has to wait for anything else, which is what a launch with AFB_FLAG_PDL overlaps with its predecessor.
__host__ __device__ constexpr int ring_bytes(int ring) { return kWarps * ring * kStageBytes; }
// staged activations of one pass, m rows x (pass_k * 2 + 16) bytes: 20 KiB for m <= 8 (52 KiB per CTA: four CTAs per SM, 64 registers),
// 40 KiB for m <= 16 (72 KiB per CTA: three CTAs per SM, 80 registers)
__host__ __device__ constexpr int act_bytes(int mt) { return mt == 1 ? 20 * 1024 : 40 * 1024; }
constexpr int kOffRed = 0;
__host__ __device__ constexpr int smem_bytes(int mt, int ring) { return ring_bytes(ring) + act_bytes(mt) + 16; }
constexpr int kSmemMax = 227 * 1024;   // per CTA on sm_100
static_assert(kRedFloats * 4 <= ring_bytes(4), "the reduction buffer must fit the ring it reuses");

__device__ __forceinline__ void grid_dependents_may_start() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

__host__ __device__ constexpr int min_ctas_per_sm(int bits, int mt, bool grouped, int ring) {
    return ring == 8 ? 2 : ((bits == 4 && grouped) ? (mt == 1 ? 3 : 2) : (mt == 1 ? AFB_DECODE_MT1_CTAS : AFB_DECODE_MT2_CTAS));
}

// ZP (int8 only): zero-points cost one more packed subtraction per pair of weights; int4 zero-points ride on the constant the
// unpack subtracts anyway, so those instances take them without a switch.
template <int BITS, int MT, bool GROUPED, bool ZP, int RING>
// resident CTAs per SM the register budget is cut for: the group-scaled int4 kernels want more registers than the others (16 rows:
// about 118, 12 % faster with two CTAs and no spills than with three squeezed into 80; 8 rows: 80, 3 to 8 % faster with three
// CTAs than with four at 64); the other kernels gain nothing or lose (measured)
__global__ void __launch_bounds__(kThreads, min_ctas_per_sm(BITS, MT, GROUPED, RING))
decode_kernel(const DecodeParams p) {
    constexpr int kRing = RING;
    constexpr int kOffAct = ring_bytes(RING);
    constexpr int CH = BITS == 8 ? 64 : 128;    // k per chunk (a quad covers 64 bytes of one channel)
    constexpr int LK = CH / 4;                  // k per lane per chunk
    constexpr int AV = LK / 8;                  // 16-byte activation vectors per lane, row and chunk

    extern __shared__ __align__(16) uint8_t smem[];
    float* s_red = reinterpret_cast<float*>(smem + kOffRed);
    uint32_t* s_last = reinterpret_cast<uint32_t*>(smem + kOffAct + p.act_bytes);   // the staging area's size is chosen per launch
    const uint32_t s_act = (uint32_t)__cvta_generic_to_shared(smem + kOffAct);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, tig = lane & 3;
    const uint32_t wk_count = kWarps / p.wr;
    const uint32_t wr = warp / wk_count, wk = warp % wk_count;
    // int8: the constant of the sign half of the unpack carries the encoding (dequant.cuh), so offset-binary storage costs no instruction
    const uint32_t hi8 = p.enc == AFB_ENC_OFFSET_BINARY ? 0xC380C380u : 0xC300C300u;
    const uint32_t magic4 = p.enc == AFB_ENC_OFFSET_BINARY ? 0x43004300u : 0x43084308u;
    const uint32_t groups_per_row = GROUPED ? (p.k >> p.group_shift) : 0;
    const uint32_t ring = (uint32_t)__cvta_generic_to_shared(smem) + warp * (kRing * kStageBytes) + lane * 16;
    const uint32_t act_row_bytes = p.pass_k * 2 + 16;   // +16: consecutive rows land in different bank groups

    // Launched with AFB_FLAG_PDL this kernel may run while its predecessor on the stream is still at work.  Its successor may
    // start at once (it, too, begins with weights only); this kernel itself waits for the predecessor below, after its first
    // ring fill, before it touches activations, the workspace or C.  Without the launch attribute both are no-ops.
    grid_dependents_may_start();
    bool dependency_met = false;

    // Shared-memory address of this lane's staged activations.  Rows beyond m are never staged: such a lane reads
    // row 0 instead, which only feeds output columns (activation rows) that are never stored.
    uint32_t act_base[MT];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) act_base[mt] = s_act + ((uint32_t)(mt * 8 + g) < p.m ? mt * 8 + g : 0) * act_row_bytes;
    // piece (16-byte) offsets inside a chunk after the bank swizzle: bit 3 of the piece index flips bit 1.
    // int4: 16 pieces per chunk, so bit 3 depends on the lane only; int8: 8 pieces per chunk, bit 3 = chunk parity.
    uint32_t act_off[AV];
#pragma unroll
    for (int v = 0; v < AV; ++v) act_off[v] = (BITS == 4 ? swz_piece(tig * AV + v) : (uint32_t)(tig * AV + v)) * 16;

    // ---- the pieces of work of this CTA: one (channel block, K range) in the grid form, a run of units in the balanced form
    const uint32_t u_begin = p.streamk ? (uint32_t)((uint64_t)blockIdx.x * p.total_units / gridDim.x) : 0u;
    const uint32_t u_end = p.streamk ? (uint32_t)((uint64_t)(blockIdx.x + 1) * p.total_units / gridDim.x) : 1u;
    // CTA holding unit u of the balanced form: the largest c with c*U/G <= u
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
    const uint32_t nchunks = (kend - ks) / CH;
    const uint32_t my_chunks = nchunks > wk ? (nchunks - wk + wk_count - 1) / wk_count : 0;
    const size_t kbyte0 = BITS == 8 ? ks : (ks >> 1);

    float acc[MT][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[mt][e] = 0.f;

    // global addresses of the next chunk to copy (this warp's chunks are wk, wk + WK, ...)
    const uint8_t* src_a = pa + kbyte0 + (size_t)wk * 64;
    const uint8_t* src_b = pb + kbyte0 + (size_t)wk * 64;
    const uint32_t src_step = wk_count * 64;
    uint32_t issued = 0;
    auto issue_to = [&](uint32_t dst) {   // start the copy of this warp's next chunk into the ring slot at dst
        if (ok_a) cp_async16(dst, src_a);
        if (ok_b) cp_async16(dst + 512, src_b);
        src_a += src_step; src_b += src_step; ++issued;
    };
    auto issue = [&]() { issue_to(ring + (issued & (kRing - 1)) * kStageBytes); };   // ... into ring slot issued % kRing
    const uint16_t* sc_h = reinterpret_cast<const uint16_t*>(p.scale);
    const float* sc_f = reinterpret_cast<const float*>(p.scale);
    const size_t sc_ia = (size_t)(ok_a ? row_a : 0) * groups_per_row, sc_ib = (size_t)(ok_b ? row_b : 0) * groups_per_row;
    uint32_t sc_k = ks + wk * CH;            // k of the chunk whose scales are fetched next
    const uint32_t sc_kstep = wk_count * CH;
    // zero-points of this lane's two channels, as the packed-bf16 constants the unpack subtracts (dequant.cuh)
    uint32_t z_a = 0u, z_b = 0u;                             // int8 (ZP instances): the decoded zero
    uint32_t sub_a = 0x43084308u, sub_b = 0x43084308u;       // int4: 136 + the decoded zero
    uint32_t z_a_nxt = 0u, z_b_nxt = 0u, sub_a_nxt = 0x43084308u, sub_b_nxt = 0x43084308u;
    auto load_zeros = [&](size_t ia, size_t ib, uint32_t& za, uint32_t& zb, uint32_t& sa4, uint32_t& sb4) {
        if (BITS == 8) { if (ZP) { za = zero8_const(p.zero[ia], p.enc); zb = zero8_const(p.zero[ib], p.enc); } }
        else if (p.zero) { sa4 = zero4_const(p.zero[ia], p.enc); sb4 = zero4_const(p.zero[ib], p.enc); }
    };
    if (!GROUPED) load_zeros(ok_a ? row_a : 0, ok_b ? row_b : 0, z_a, z_b, sub_a, sub_b);
    auto load_group_scales = [&](float& sa, float& sb, uint32_t& za, uint32_t& zb, uint32_t& sa4, uint32_t& sb4) {
        const uint32_t grp = sc_k >> p.group_shift;
        if (p.scale_dtype == AFB_SCALE_BF16) { sa = bf16_to_f32(sc_h[sc_ia + grp]); sb = bf16_to_f32(sc_h[sc_ib + grp]); }
        else { sa = sc_f[sc_ia + grp]; sb = sc_f[sc_ib + grp]; }
        load_zeros(sc_ia + grp, sc_ib + grp, za, zb, sa4, sb4);
        sc_k += sc_kstep;
    };

    // the weight stream starts before anything else and keeps running across the passes below
#pragma unroll
    for (int j = 0; j < kRing - 1; ++j) {
        if ((uint32_t)j < my_chunks) issue();
        cp_async_commit();
    }
    float sc_a = 0.f, sc_b = 0.f, sc_a_nxt = 0.f, sc_b_nxt = 0.f;
    if (GROUPED && my_chunks) load_group_scales(sc_a, sc_b, z_a, z_b, sub_a, sub_b);
    if (!dependency_met) { grid_dependency_wait(); dependency_met = true; }   // so far only B, scales and zero-points were read

    uint32_t i = 0;   // chunks this warp has consumed
    for (uint32_t pk = ks; pk < kend; pk += p.pass_k) {
        const uint32_t plen = min(p.pass_k, kend - pk);
        if (pk != ks) __syncthreads();   // the previous pass has been consumed by every warp
        {   // stage the activations of [pk, pk + plen), permuted into the pairing the weights unpack to
            const uint32_t pieces = plen >> 3;
            // all 256 threads take part whatever m is: 256, 128 or 64 threads per row
            const uint32_t rsh = p.m >= 4 ? 6u : (p.m >= 2 ? 7u : 8u), per_row = 1u << rsh, rstep = 256u >> rsh;
            auto put = [&](uint32_t r, uint32_t pc, const uint4& v) {
                uint4 o;
                if (p.packed) {   // pre-packed weights unpack to consecutive k: the activations are used as they lie
                    o = v;
                } else if (BITS == 8) {  // {k0,k2},{k1,k3},{k4,k6},{k5,k7}
                    o.x = prmt(v.x, v.y, 0x5410u); o.y = prmt(v.x, v.y, 0x7632u);
                    o.z = prmt(v.z, v.w, 0x5410u); o.w = prmt(v.z, v.w, 0x7632u);
                } else {          // {k0,k4},{k1,k5},{k2,k6},{k3,k7}
                    o.x = prmt(v.x, v.z, 0x5410u); o.y = prmt(v.x, v.z, 0x7632u);
                    o.z = prmt(v.y, v.w, 0x5410u); o.w = prmt(v.y, v.w, 0x7632u);
                }
                *reinterpret_cast<uint4*>(smem + kOffAct + r * act_row_bytes + swz_piece(pc) * 16) = o;
            };
            if constexpr (min_ctas_per_sm(BITS, MT, GROUPED, RING) <= 2) {
                // The instances with 128 registers per thread send their loads out in batches (8 with the 8-stage ring, 4 with the
                // 4-stage ring), across row boundaries, before any of them is used: a pass then costs (pieces per thread / batch)
                // trips to L2, and with the whole K range staged at once those trips are most of what the kernel waits for before
                // its first tensor-core instruction (4096 x 4096, 16 rows: 9.8 us instead of 12.7; 28672 x 8192 int4 group-128,
                // 16 rows, batches of 4: 62 us instead of 68, batches of 8: 70).  The instances with tighter register budgets
                // lose 3 to 7 % with it (measured).
                constexpr int kStageBatch = RING == 8 ? 8 : 4;
                const uint32_t pc_first = tid & (per_row - 1);
                uint32_t r = tid >> rsh, pc = pc_first;
                while (r < p.m) {
                    uint4 v[kStageBatch];
                    uint32_t r2 = r, pc2 = pc;   // the second loop walks the same (row, piece) sequence again
#pragma unroll
                    for (int b = 0; b < kStageBatch; ++b) {
                        if (r < p.m && pc < pieces) v[b] = ldg_act(p.a + (size_t)r * p.lda + pk + pc * 8);
                        pc += per_row;
                        if (pc >= pieces) { pc = pc_first; r += rstep; }
                    }
#pragma unroll
                    for (int b = 0; b < kStageBatch; ++b) {
                        if (r2 < p.m && pc2 < pieces) put(r2, pc2, v[b]);
                        pc2 += per_row;
                        if (pc2 >= pieces) { pc2 = pc_first; r2 += rstep; }
                    }
                }
            } else {
                for (uint32_t r = tid >> rsh; r < p.m; r += rstep)
                    for (uint32_t pc = tid & (per_row - 1); pc < pieces; pc += per_row)
                        put(r, pc, ldg_act(p.a + (size_t)r * p.lda + pk + pc * 8));
            }
        }
        __syncthreads();

        const uint32_t chunks_in_pass = plen / CH;
        uint32_t chunk_off = wk * (CH * 2);                 // byte offset of the chunk inside a staged row
        const uint32_t chunk_step = wk_count * (CH * 2);
        // everything of a chunk after its copy has been issued: activations, weights from ring slot `slot`, unpack, tensor cores
        auto consume = [&](uint32_t slot, uint32_t coff, uint32_t par) {
            // this lane's activations of the chunk: rows g (and g + 8), k = cl*CH + tig*LK ..
            uint32_t s[MT][AV * 4];
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                for (int v = 0; v < AV; ++v) {
                    const uint4 t = lds128(act_base[mt] + coff + (act_off[v] ^ par));
                    s[mt][4 * v] = t.x; s[mt][4 * v + 1] = t.y; s[mt][4 * v + 2] = t.z; s[mt][4 * v + 3] = t.w;
                }
            cp_async_wait<kRing - 1>();   // this warp's chunk has landed (each lane reads only what it copied itself)
            const uint4 wa4 = lds128(slot), wb4 = lds128(slot + 512);
            const uint32_t wav[4] = {wa4.x, wa4.y, wa4.z, wa4.w};
            const uint32_t wbv[4] = {wb4.x, wb4.y, wb4.z, wb4.w};
            float part[MT][4];   // grouped: the sum of this chunk alone (a chunk lies inside one scale group)
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                for (int e = 0; e < 4; ++e) part[mt][e] = 0.f;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                if (BITS == 8) {
                    uint32_t a0, a1, a2, a3;
                    s8x4_enc_to_bf16_strided(wav[j], hi8, a0, a2);
                    s8x4_enc_to_bf16_strided(wbv[j], hi8, a1, a3);
                    if (ZP) { a0 = bf16x2_sub(a0, z_a); a2 = bf16x2_sub(a2, z_a); a1 = bf16x2_sub(a1, z_b); a3 = bf16x2_sub(a3, z_b); }
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt)
                        mma_bf16(GROUPED ? part[mt] : acc[mt], a0, a1, a2, a3, s[mt][2 * j], s[mt][2 * j + 1]);
                } else {
                    uint32_t qa[4], qb[4];
                    s4x8_to_bf16_strided(wav[j], magic4, qa, sub_a);
                    s4x8_to_bf16_strided(wbv[j], magic4, qb, sub_b);
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt) {
                        mma_bf16(GROUPED ? part[mt] : acc[mt], qa[0], qb[0], qa[1], qb[1], s[mt][4 * j], s[mt][4 * j + 1]);
                        mma_bf16(GROUPED ? part[mt] : acc[mt], qa[2], qb[2], qa[3], qb[3], s[mt][4 * j + 2], s[mt][4 * j + 3]);
                    }
                }
            }
            if (GROUPED) {
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    acc[mt][0] = fmaf(sc_a, part[mt][0], acc[mt][0]); acc[mt][1] = fmaf(sc_a, part[mt][1], acc[mt][1]);
                    acc[mt][2] = fmaf(sc_b, part[mt][2], acc[mt][2]); acc[mt][3] = fmaf(sc_b, part[mt][3], acc[mt][3]);
                }
                sc_a = sc_a_nxt; sc_b = sc_b_nxt;
                z_a = z_a_nxt; z_b = z_b_nxt; sub_a = sub_a_nxt; sub_b = sub_b_nxt;
            }
        };
        uint32_t cl = wk;
        while (cl < chunks_in_pass) {
            if ((i & (kRing - 1)) == 0 && cl + (kRing - 1) * wk_count < chunks_in_pass) {
                // a whole turn of the ring, unrolled: ring slots are compile-time offsets and the copy issued while chunk i + u is
                // consumed goes to slot (u - 1) mod kRing (the issue cursor runs kRing - 1 chunks ahead until the chunks run out)
                const uint32_t par0 = BITS == 8 ? ((cl & 1u) << 5) : 0u;                      // int8: odd chunks have bit 3 of the piece index set
                const uint32_t par1 = BITS == 8 ? par0 ^ ((wk_count & 1u) << 5) : 0u;          // parity of cl + wk_count
#pragma unroll
                for (int u = 0; u < kRing; ++u) {
                    if (issued < my_chunks) issue_to(ring + ((u + kRing - 1) & (kRing - 1)) * kStageBytes);
                    cp_async_commit();
                    if (GROUPED && i + 1 < my_chunks) load_group_scales(sc_a_nxt, sc_b_nxt, z_a_nxt, z_b_nxt, sub_a_nxt, sub_b_nxt);
                    consume(ring + u * kStageBytes, chunk_off, (u & 1) ? par1 : par0);
                    ++i; chunk_off += chunk_step;
                }
                cl += kRing * wk_count;
            } else {
                if (issued < my_chunks) issue();
                cp_async_commit();
                if (GROUPED && i + 1 < my_chunks) load_group_scales(sc_a_nxt, sc_b_nxt, z_a_nxt, z_b_nxt, sub_a_nxt, sub_b_nxt);
                consume(ring + (i & (kRing - 1)) * kStageBytes, chunk_off, BITS == 8 ? ((cl & 1u) << 5) : 0u);
                ++i; chunk_off += chunk_step; cl += wk_count;
            }
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

template <int BITS, int MT, bool GROUPED, bool ZP, int RING>
cudaError_t launch_one(const DecodeParams& p, dim3 grid, bool pdl, cudaStream_t s) {
    auto kern = decode_kernel<BITS, MT, GROUPED, ZP, RING>;
    static DeviceOnce attr_set;   // per template instance
    int dev = 0;
    cudaGetDevice(&dev);
    if (!attr_set.done(dev)) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemMax);
        if (e != cudaSuccess) return e;
        attr_set.mark(dev);
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = dim3(kThreads); cfg.dynamicSmemBytes = ring_bytes(RING) + p.act_bytes + 16; cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, p);
}

// CTAs of one kernel instance that fit an SM at the same time (asked once per instance and device).
template <int BITS, int MT, bool GROUPED, int RING>
int resident_one() {
    static std::atomic<int> cached[32];   // 0 = not asked yet (zero-initialised)
    int dev = 0;
    cudaGetDevice(&dev);
    int n = cached[dev & 31].load(std::memory_order_acquire);
    if (n == 0) {
        auto kern = decode_kernel<BITS, MT, GROUPED, false, RING>;
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemMax) != cudaSuccess) return 0;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kern, kThreads, smem_bytes(MT, RING)) != cudaSuccess) return 0;
        cached[dev & 31].store(n, std::memory_order_release);
    }
    return n;
}
int resident_ctas(uint32_t bits, int mt, bool grouped) {   // of the 4-stage instances (the 8-stage ones are only used when every CTA is resident anyway)
    if (bits == 8) {
        if (mt == 1) return grouped ? resident_one<8, 1, true, 4>() : resident_one<8, 1, false, 4>();
        return grouped ? resident_one<8, 2, true, 4>() : resident_one<8, 2, false, 4>();
    }
    if (mt == 1) return grouped ? resident_one<4, 1, true, 4>() : resident_one<4, 1, false, 4>();
    return grouped ? resident_one<4, 2, true, 4>() : resident_one<4, 2, false, 4>();
}

template <int BITS, int MT, bool GROUPED>
cudaError_t launch_cfg(const DecodeParams& p, dim3 grid, bool deep_ring, bool pdl, cudaStream_t s) {
    const bool zp = BITS == 8 && p.zero != nullptr;
    if (deep_ring) return zp ? launch_one<BITS, MT, GROUPED, BITS == 8, 8>(p, grid, pdl, s) : launch_one<BITS, MT, GROUPED, false, 8>(p, grid, pdl, s);
    return zp ? launch_one<BITS, MT, GROUPED, BITS == 8, 4>(p, grid, pdl, s) : launch_one<BITS, MT, GROUPED, false, 4>(p, grid, pdl, s);
}

}  // namespace

bool decode_supports(const afb_gemm_args& a) {
    if (a.m == 0 || a.m > 16) return false;
    if (a.b_layout != AFB_LAYOUT_COL && a.b_layout != AFB_LAYOUT_COL_PACKED) return false;
    if (a.b_bits != 8 && a.b_bits != 4) return false;
    const uint32_t ch = a.b_bits == 8 ? 64 : 128;
    if (a.k % ch) return false;
    const uint32_t ldb_bytes = a.b_bits == 8 ? a.ldb : a.ldb / 2;
    if (ldb_bytes % 16 || a.lda % 8) return false;
    if ((uintptr_t)a.ptr_a % 16 || (uintptr_t)a.ptr_b % 16) return false;
    if (a.group_size && (a.group_size % ch || a.k % a.group_size || (a.group_size & (a.group_size - 1)))) return false;   // power of two; a chunk never straddles a group
    return true;
}

// Shape of the launch: warps per CTA along the channels (wr), K-slices (slices) and slice length (kc).
//   * wr: activations are re-read by every column of CTAs, so more activation rows ask for more channels per CTA
//     (keeps the activation traffic through L2 below about half of the weight traffic);
//   * slices: only when the channel dimension alone cannot fill the GPU.
// act_cap: bytes of the activation staging area of this launch.
static void pick_shape(const afb_gemm_args& a, int sm_count, int ctas_per_sm, size_t ws_bytes, size_t counter_count, size_t act_cap, DecodeParams& p) {
    const uint32_t ch = a.b_bits == 8 ? 64 : 128;
    const uint32_t sms = (uint32_t)sm_count;
    const uint32_t act_bytes_per_k = 2 * a.m;                      // per k, per column of CTAs
    uint32_t wr = 1;
    while (wr < 8 && act_bytes_per_k * 2 > 16 * wr * a.b_bits / 8) wr *= 2;     // activation bytes <= half the weight bytes
    const double weight_mb = (double)a.n * a.k * a.b_bits / 8 / 1e6;
    auto ctas = [&](uint32_t w) { return (a.n + 16 * w - 1) / (16 * w); };
    while (wr < 8 && ctas(wr * 2) >= 6 * sms) wr *= 2;              // plenty of channels: larger CTAs, fewer activation re-reads
    // small matrices with 9 to 16 rows: when 16-channel CTAs alone fill the GPU, they beat wider CTAs with K-slices (no workspace
    // round trip; measured on 4096 x 4096: 10.2 vs 12.4 us at m = 9, 11.9 vs 12.6 at m = 12, equal at m = 16)
    if (weight_mb < 48.0 && a.m > 8 && ctas(1) >= sms * 3 / 2 && (size_t)a.m * (ch * kWarps * 2 + 16) <= act_cap) wr = 1;
    while (wr < 8 && (size_t)a.m * (ch * (kWarps / wr) * 2 + 16) > act_cap) wr *= 2;   // one round of the WK warps must fit the staging area
    // the balanced form (below) pays off for more than 8 activation rows on large matrices (measured: 8 to 25 % there, a loss
    // of up to 10 % for m <= 8, whose grid form needs no K-slices); it runs best with the widest CTA
    bool want_balanced = weight_mb >= 48.0 && a.m > 8;
    if (const char* e = getenv("AFB_DECODE_BALANCED")) want_balanced = atoi(e) != 0;   // tuning aid
    if (want_balanced && (size_t)a.m * (ch * 2 + 16) <= act_cap) wr = 8;
    const uint32_t want = weight_mb < 48.0 ? sms * 3 / 2 : sms * 5;   // many small CTAs even out the load of the SMs (measured)
    uint32_t s = 1;
    const uint32_t unit = a.group_size > ch ? a.group_size : ch;
    while (ctas(wr) * s < want && s < 32 && a.k % (2 * s * unit) == 0 && a.k / (2 * s) >= 4 * ch * (kWarps / wr)) s *= 2;
    while (s > 1 && ((size_t)s * a.m * a.n * sizeof(float) > ws_bytes || ctas(wr) > counter_count)) s /= 2;
    if (ctas(wr) > counter_count) s = 1;
    if (const char* e = getenv("AFB_DECODE_WR")) {       // tuning aid: force the CTA shape when it is legal
        const uint32_t v = (uint32_t)atoi(e);
        if ((v == 1 || v == 2 || v == 4 || v == 8) && (size_t)a.m * (ch * (kWarps / v) * 2 + 16) <= act_cap) wr = v;
    }
    if (const char* e = getenv("AFB_DECODE_SLICES")) {   // tuning aid: force the number of K-slices when it is legal
        const uint32_t v = (uint32_t)atoi(e);
        if (v >= 1 && v <= 64 && a.k % (v * unit) == 0 && (size_t)v * a.m * a.n * sizeof(float) <= ws_bytes && ctas(wr) <= counter_count) s = v;
    }
    p.wr = wr; p.slices = s; p.kc = a.k / s;
    // activations staged per pass: as many k as fit the staging area, in whole rounds of the WK warps
    const uint32_t round = ch * (kWarps / wr);
    uint32_t pass_max = ((uint32_t)act_cap / a.m - 16) / 2 / round * round;   // >= 512 k for m <= 16, round <= 512
    if (pass_max == 0) pass_max = round;
    const uint32_t npass = (p.kc + pass_max - 1) / pass_max;
    p.pass_k = ((p.kc + npass - 1) / npass + round - 1) / round * round;        // equal passes, whole rounds
    p.group_shift = 0;
    while (a.group_size && (1u << p.group_shift) < a.group_size) ++p.group_shift;

    // Balanced form for large weight matrices: exactly one wave of CTAs, each streaming the same number of bytes.  The grid form
    // above leaves SMs idle whenever channel blocks x slices is not a multiple of the resident CTAs (28672 channels: 448 CTAs on
    // 444 places), and it cannot be fixed by another power-of-two split.
    p.streamk = 0; p.unit_k = 0; p.units_per_cb = 0; p.total_units = 0;
    const uint32_t unit_min = a.group_size > round ? a.group_size : round;   // whole rounds of the WK warps, whole scale groups
    if (want_balanced && ctas_per_sm > 0 && a.k % unit_min == 0) {
        const uint32_t cbs = ctas(wr);
        uint32_t grid = sms * (uint32_t)ctas_per_sm;
        uint32_t unit_k = unit_min;
        while (a.k % (unit_k * 2) == 0 && (uint64_t)cbs * (a.k / (unit_k * 2)) >= 16ull * grid) unit_k *= 2;   // >= 16 units per CTA is balance enough
        const uint32_t ku = a.k / unit_k;
        const uint64_t total = (uint64_t)cbs * ku;
        if (total < grid) grid = (uint32_t)total;
        if (total < (1ull << 31)) {
            auto cta_of = [&](uint64_t u) { return (uint32_t)(((u + 1) * grid + total - 1) / total) - 1u; };   // as in the kernel
            uint32_t maxc = 1;
            for (uint32_t cb = 0; cb < cbs; ++cb) {
                const uint32_t c = cta_of((uint64_t)cb * ku + ku - 1) - cta_of((uint64_t)cb * ku) + 1;
                if (c > maxc) maxc = c;
            }
            if ((size_t)maxc * a.m * a.n * sizeof(float) <= ws_bytes && cbs <= counter_count) {
                p.streamk = 1; p.unit_k = unit_k; p.units_per_cb = ku; p.total_units = (uint32_t)total;
                p.slices = grid;          // the launcher reads the grid size from here
                p.kc = a.k;
                p.pass_k = pass_max < a.k ? pass_max : (a.k + round - 1) / round * round;
            }
        }
    }
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
    const bool grouped = a.group_size != 0;
    const int mt = a.m <= 8 ? 1 : 2;
    p.packed = a.b_layout == AFB_LAYOUT_COL_PACKED ? 1u : 0u;
    p.zero = reinterpret_cast<const uint8_t*>(a.ptr_zero);
    // Small matrices (one wave of CTAs): the whole K range of a CTA is staged at once when shared memory allows it, so that the
    // kernel pays the activations' L2 latency once instead of once per pass (16 rows x 4096 k are 128 KiB: one CTA per SM then),
    // and the ring is 8 deep when that still fits (with AFB_FLAG_PDL it fills while the preceding kernel finishes).  The CTA shape
    // is the one that fills the most CTA places of the wave; ties go to more resident warps, then to the deeper ring.
    const uint32_t sms = (uint32_t)ctx->sm_count;
    const double weight_mb = (double)a.n * a.k * a.b_bits / 8 / 1e6;
    uint32_t act = (uint32_t)act_bytes(mt);
    bool deep_ring = false;
    int forced_wr = 0;
    static const bool env_single_pass_off = [] { const char* e = getenv("AFB_DECODE_SINGLE_PASS"); return e && atoi(e) == 0; }();
    if (weight_mb < 48.0 && !env_single_pass_off && !getenv("AFB_DECODE_WR") && !getenv("AFB_DECODE_SLICES")) {
        const uint32_t chx = a.b_bits == 8 ? 64 : 128;
        double best_fill = 0.0; uint32_t best_warps = 0, best_need = 0; int best_ring = 0;
        for (uint32_t wr = 1; wr <= 8; wr *= 2) {
            const uint32_t ctas = (a.n + 16 * wr - 1) / (16 * wr), per_sm = (ctas + sms - 1) / sms;
            if (per_sm > 4) continue;
            const uint32_t round = chx * (kWarps / wr), whole_k = (a.k + round - 1) / round * round;
            const uint64_t need = (uint64_t)a.m * (whole_k * 2 + 16);   // whole K in whole rounds of the WK warps, no slices
            if (need > (uint64_t)kSmemMax) continue;
            for (int ring = 8; ring >= 4; ring -= 4) {
                if ((uint64_t)(ring_bytes(ring) + need + 16 + 1024) * per_sm > (uint64_t)kSmemMax) continue;
                const double fill = (double)ctas / ((double)per_sm * sms);
                const uint32_t warps = per_sm * kWarps;
                if (fill > best_fill + 1e-9 || (fill > best_fill - 1e-9 && (warps > best_warps || (warps == best_warps && ring > best_ring)))) {
                    best_fill = fill; best_warps = warps; best_ring = ring; forced_wr = (int)wr; best_need = (uint32_t)need;
                }
            }
        }
        if (forced_wr) { act = (best_need + 15u) & ~15u; deep_ring = best_ring == 8; }
    }
    p.act_bytes = act;
    pick_shape(a, ctx->sm_count, resident_ctas(a.b_bits, mt, grouped), ws_bytes, counter_count, act, p);
    if (forced_wr) {   // the single-pass shape: whole K per CTA, no K-slices
        p.wr = (uint32_t)forced_wr; p.slices = 1; p.kc = a.k; p.streamk = 0;
        const uint32_t chx = a.b_bits == 8 ? 64 : 128, round = chx * (kWarps / p.wr);
        p.pass_k = (a.k + round - 1) / round * round;
    }
    p.ws = ws; p.counters = counters;
    dim3 grid((a.n + 16 * p.wr - 1) / (16 * p.wr), p.slices);
    if (p.streamk) grid = dim3(p.slices, 1);
    const uint32_t ch = a.b_bits == 8 ? 64 : 128;
    const uint32_t chunks_per_warp = (p.kc / ch + (kWarps / p.wr) - 1) / (kWarps / p.wr);
    if (!forced_wr) deep_ring = !p.streamk && chunks_per_warp <= 8 && (uint64_t)grid.x * grid.y <= 2ull * (uint64_t)ctx->sm_count;
    if (const char* e = getenv("AFB_DECODE_DEEP_RING")) deep_ring = atoi(e) != 0 && !p.streamk;   // tuning aid
    if ((uint64_t)ring_bytes(deep_ring ? 8 : 4) + act + 16 > (uint64_t)kSmemMax) deep_ring = false;
    const bool pdl = (a.flags & AFB_FLAG_PDL) != 0;
    cudaError_t e;
    if (a.b_bits == 8) {
        if (mt == 1) e = grouped ? launch_cfg<8, 1, true>(p, grid, deep_ring, pdl, s) : launch_cfg<8, 1, false>(p, grid, deep_ring, pdl, s);
        else         e = grouped ? launch_cfg<8, 2, true>(p, grid, deep_ring, pdl, s) : launch_cfg<8, 2, false>(p, grid, deep_ring, pdl, s);
    } else {
        if (mt == 1) e = grouped ? launch_cfg<4, 1, true>(p, grid, deep_ring, pdl, s) : launch_cfg<4, 1, false>(p, grid, deep_ring, pdl, s);
        else         e = grouped ? launch_cfg<4, 2, true>(p, grid, deep_ring, pdl, s) : launch_cfg<4, 2, false>(p, grid, deep_ring, pdl, s);
    }
    count_launch();
    return e == cudaSuccess ? AFB_OK : cuda_fail(e);
}

int launch_decode(const afb_gemm_args& a, DeviceCtx* ctx, cudaStream_t s) {
    int rc = AFB_OK;
    const DeviceCtx::Workspace* w = workspace_for(ctx, s, &rc);
    if (!w) return rc;
    return launch_decode_ws(a, ctx, w->ws, ctx->splitk_ws_bytes, w->counters, ctx->splitk_counter_count, s);
}

}  // namespace afb
