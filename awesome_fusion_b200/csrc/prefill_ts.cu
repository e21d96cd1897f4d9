// Prefill variant, weights-in-tensor-memory form (M > 16, B in [N,K] layout).
//
// The GEMM is computed transposed, D[n, m] = sum_k W[n,k] * A[m,k]: a tile has 128 output channels as the
// 128 TMEM lanes and BMA (256 or 128) activation rows as its columns.  That lets the DEQUANTISED WEIGHTS
// be the tcgen05.mma operand that lives in tensor memory: the converter warps unpack the raw int8 / int4
// tile to exact bf16 in registers (dequant.cuh) and write it straight to TMEM with tcgen05.st, so the
// converted weights never touch shared memory, and only 128 x 64 weights are converted per 128 x BMA x 64
// block of MMA work (reference counterpart of the whole kernel: bf16gemm_kernel_gfx90a.s:184-636).
//
//   warp 0      (1 lane)  TMA: activation tile [BMA x 64] bf16 (128-byte swizzle) + raw weight tile
//                         [128 x 64] int8/int4 (64-/32-byte swizzle) into a ring of stages
//   warps 2-9   (256 thr) converters: one channel per thread (two warps per lane quarter = the two 32-wide halves of K),
//                         raw bytes -> bf16 pairs -> (x group scale) -> tcgen05.st into a ring of TMEM slots;
//                         after the last K step the same warps run the epilogue: tcgen05.ld the accumulator,
//                         multiply by the per-channel scale (one scalar per thread), round to bf16, store C
//   warp 1      (1 lane)  tcgen05.mma kind::f16, A from TMEM, B (activations) from shared memory,
//                         128 x BMA x 16, fp32 accumulator in TMEM
// One accumulator (BMA columns) + 8 weight slots (32 columns each) live in the 512 TMEM columns.
// Every wait is bounded; a wait that gives up sets the status words, all roles drain, TMEM is freed.
#include <cstdlib>
#include "afb_internal.h"
#include "dequant.cuh"
#include "ptx_sm100.cuh"
#include "sys_sync.cuh"

namespace afb {

namespace {

constexpr int BNW = 128;      // output channels per tile = TMEM lanes
constexpr int BK = 64;
constexpr int kSlotsA = 8;    // TMEM slots of converted weights (256 accumulator columns + 8 x 32 = all 512 columns)
constexpr int kWorkerWarps = 8;   // measured: 8 beats 16 (1.10 vs 1.04 PFLOP/s on 2048 x 11008 x 4096)
constexpr int kKParts = kWorkerWarps / 4;            // warps per TMEM lane quarter = parts the 64-wide K step is cut into
constexpr int kKPer = BK / kKParts;                  // k per converter thread and stage (32 or 16)
constexpr int kThreads = 32 * (2 + kWorkerWarps);   // 320
constexpr int kFwdWarps = 2;      // optional extra warps that forward finished fp32 tiles to their owner rank
constexpr int kThreadsFwd = kThreads + 32 * kFwdWarps;

struct TsParams {
    uint16_t* c;
    const void* scale;
    const uint8_t* zero;   // optional zero-points (nullptr = none): one byte per scale entry, in the weights' own encoding
    uint32_t m, n, k, ldc;
    uint32_t enc, scale_dtype, group;
    uint32_t m_tiles, n_tiles;
    uint32_t m_rot;        // row tiles are taken in rotated order, starting at this one (spreads the peers a rank pushes to)
    uint32_t group_m;      // tile order: groups of group_m row tiles; inside a group the channel tiles advance, row tile fastest
    uint32_t c_f32;
    uint32_t c_tma;        // bf16 C goes out as tile stores through shared memory (tmap_c is valid): plain GEMM, no fusion, no exchange
    uint32_t packed;       // B is in the pre-packed order of afb_prepack: the cheap unpack yields consecutive k
    uint32_t exact;        // group scales only: the weight q * s goes to the tensor cores as TWO bf16 terms, hi = bf16_rn(q * s) and
                           // lo = q * s - hi (exact: the product has at most 16 significant bits), in two TMEM slots and two MMAs
    uint32_t* tile_done;   // optional: per-tile counters, +kWorkerWarps when a tile of C has been stored (system-scope release)
    // optional (row-parallel reduce-scatter fused into the epilogue): fp32 C rows [o*push_rows, (o+1)*push_rows) go to rank o's
    // staging buffer, slot push_rank, instead of to p.c: push[o] + (push_rank * push_rows + local_row) * ldc + n
    float* push[AFB_MAX_RANKS];
    // optional: the tiles beyond the last full wave (tail_first ..) are each cut into tail_parts stretches of K, one per CTA; the
    // stretches meet as fp32 tiles in tail_ws ([tail tile][part][row][channel]) and the last CTA to arrive adds them in part order
    uint32_t tail_first, tail_tiles, tail_parts;
    float* tail_ws;
    uint32_t* tail_counters;   // one per tail tile, zero on entry, zero again on exit
    // optional fused epilogue (bf16 output only): v = acc * scale + bias[channel]; gated: rows 2i / 2i+1 of B are the gate / up
    // projection of output channel i and C[m,i] = act(v_gate) * v_up, else C[m,n] = act(v); then + residual[m, channel]; one rounding
    const float* bias;
    const uint16_t* residual;
    uint32_t ld_res;
    uint32_t fused;        // 0: off; bit 0: on; bit 1: gated
    uint32_t act;          // AFB_ACT_*
    uint32_t push_rows, push_rank;
    // optional (pipelined reduce-scatter): the tiles are taken in units of (owner's row tiles) x (n_tiles / push_sub channel tiles);
    // unit u covers column chunk u / world of the rows of owner (rank + u % world) % world, so that after every `world` units one
    // more column chunk is complete on EVERY owner.  Each finished tile is counted in push_cnt[owner][chunk] (system-scope release).
    uint32_t push_sub, push_world;
    uint32_t* push_cnt[AFB_MAX_RANKS];
    uint32_t xchg_on;      // pipelined reduce-scatter finished in this kernel: two extra warps per CTA sum and broadcast the chunks
    PushExchange x;
    uint32_t push_on;      // 0: off; 1: the epilogue stores to the owner directly; 2: the epilogue stores to p.c (local) and the
                           // forwarder warps copy each finished tile to its owner while the next tile is being computed
    int32_t* status;
    unsigned long long* ts;   // optional phase timestamps: [0] start of CTA 0, [1] latest end of any CTA (nullptr = off)
};

template <int BITS, int BMA>
struct TsLayout {
    static constexpr int kStages = BMA == 256 ? 5 : 8;
    static constexpr int kRawRowBytes = BK * BITS / 8;
    static constexpr int kActBytes = BMA * BK * 2;              // 32 KiB at BMA = 256
    static constexpr int kRawBytes = BNW * kRawRowBytes;         // 8 KiB (int8) / 4 KiB (int4)
    static constexpr int kOffAct = 0;
    static constexpr int kOffRaw = kStages * kActBytes;
    static constexpr int kOffBars = kOffRaw + kStages * kRawBytes;
    static constexpr int kNumBars = 3 * kStages + 2 * kSlotsA + 6;
    static constexpr int kOffMisc = kOffBars + kNumBars * 8;
    // epilogue staging: one [32 activation rows][32 channels] bf16 block (2 KiB) per converter warp, the source of a tile store
    static constexpr int kStageOutBytes = 32 * 32 * 2;
    static constexpr int kOffOut = (kOffMisc + 32 + 127) / 128 * 128;   // 8 words of flags and counters before it
    static constexpr int kDynamic = kOffOut + kWorkerWarps * kStageOutBytes + 1024;
    static constexpr uint32_t kTmemCols = 512;                   // accumulator [0, BMA) + weight slots [256, 256 + kSlotsA * 32)
    static constexpr uint32_t kColA = 256;
};

// Tile t -> (row tile, channel tile).  Consecutive tiles (= the CTAs of one wave) share group_m activation row tiles and
// walk the channel tiles, so the activations of a group stay in L2 while the weights stream past once per group.
__device__ __forceinline__ void tile_coords(const TsParams& p, uint32_t t, uint32_t& m_tile, uint32_t& n_tile) {
    if (p.push_sub) {
        const uint32_t rt = p.m_tiles / p.push_world, cn = p.n_tiles / p.push_sub, per_unit = rt * cn;
        const uint32_t u = t / per_unit, i = t - u * per_unit;
        const uint32_t chunk = u / p.push_world, owner = (p.push_rank + (u - chunk * p.push_world)) % p.push_world;
        n_tile = chunk * cn + i / rt;
        m_tile = owner * rt + (i - (i / rt) * rt);
        return;
    }
    const uint32_t per_group = p.group_m * p.n_tiles;
    const uint32_t g = t / per_group, r = t - g * per_group;
    const uint32_t gsz = min(p.group_m, p.m_tiles - g * p.group_m);
    n_tile = r / gsz;
    m_tile = g * p.group_m + (r - n_tile * gsz) + p.m_rot;
    if (m_tile >= p.m_tiles) m_tile -= p.m_tiles;
}

__device__ __forceinline__ void report_timeout(int32_t* status, int where, int a, int b) {
    if (atomicCAS(status, 0, AFB_ERR_TIMEOUT) == 0) { status[1] = where; status[2] = a; status[3] = b; }
}
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

template <int BITS, bool GROUPED, int BMA>
__global__ void __launch_bounds__(kThreadsFwd, 1)
prefill_ts_kernel(const __grid_constant__ CUtensorMap tmap_act, const __grid_constant__ CUtensorMap tmap_w,
                  const __grid_constant__ CUtensorMap tmap_c, const TsParams p) {
    using L = TsLayout<BITS, BMA>;
    constexpr int S = L::kStages;
    extern __shared__ uint8_t smem_raw_base[];
    const uint32_t smem_base = (ptx::smem_u32(smem_raw_base) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw_base + (smem_base - ptx::smem_u32(smem_raw_base));

    const uint32_t bar_base = smem_base + L::kOffBars;
    auto bar_full      = [&](int s) { return bar_base + 8u * s; };                       // TMA landed (act + raw)
    auto bar_empty_act = [&](int s) { return bar_base + 8u * (S + s); };                 // MMA done with the activation tile
    auto bar_empty_raw = [&](int s) { return bar_base + 8u * (2 * S + s); };             // converters done with the raw tile
    auto bar_full_a    = [&](int s) { return bar_base + 8u * (3 * S + s); };             // converted weights are in TMEM slot s
    auto bar_empty_a   = [&](int s) { return bar_base + 8u * (3 * S + kSlotsA + s); };   // MMA done with TMEM slot s
    const uint32_t bar_acc_full = bar_base + 8u * (3 * S + 2 * kSlotsA);
    const uint32_t bar_acc_empty = bar_acc_full + 8u;
    const uint32_t bar_tile_stored = bar_acc_full + 16u;   // forward mode: the epilogue has stored a tile to local memory
    const uint32_t bar_tile_fwd = bar_acc_full + 24u;      // forward mode: the forwarder warps have copied it out
    const uint32_t bar_tail_stored = bar_acc_full + 32u;   // tail stretch: every converter warp has published its part of the tile
    const uint32_t bar_tail_verdict = bar_acc_full + 40u;  // tail stretch: the arrival count has been taken
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem_gen + L::kOffMisc);
    volatile uint32_t* abort_flag = tmem_slot + 1;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t num_kb = p.k / BK;
    const uint32_t num_tiles = p.m_tiles * p.n_tiles;
    // Work items of this CTA: its full tiles (t = blockIdx.x, + gridDim.x, ... below tail_first), then at most one stretch of K of
    // a tail tile.  Every role walks the same list.
    struct Item { uint32_t t, kb0, kb1, tail_r, part; bool tail; };
    auto get_item = [&](uint32_t it, Item& w) -> bool {
        const uint32_t t_full = blockIdx.x + it * gridDim.x;
        if (t_full < p.tail_first) { w.t = t_full; w.kb0 = 0; w.kb1 = num_kb; w.tail = false; w.tail_r = 0; w.part = 0; return true; }
        if (p.tail_parts && it == p.tail_first / gridDim.x && blockIdx.x < p.tail_tiles * p.tail_parts) {
            w.tail_r = blockIdx.x / p.tail_parts; w.part = blockIdx.x - w.tail_r * p.tail_parts;
            w.t = p.tail_first + w.tail_r;
            w.kb0 = w.part * num_kb / p.tail_parts; w.kb1 = (w.part + 1) * num_kb / p.tail_parts;
            w.tail = true;
            return true;
        }
        return false;
    };

    if (threadIdx.x == 0) {
        if (p.ts && blockIdx.x == 0) p.ts[0] = ptx::globaltimer();
        for (int s = 0; s < S; ++s) { ptx::mbar_init(bar_full(s), 1); ptx::mbar_init(bar_empty_act(s), 1); ptx::mbar_init(bar_empty_raw(s), kWorkerWarps); }
        for (int s = 0; s < kSlotsA; ++s) { ptx::mbar_init(bar_full_a(s), kWorkerWarps); ptx::mbar_init(bar_empty_a(s), 1); }
        ptx::mbar_init(bar_acc_full, 1);
        ptx::mbar_init(bar_acc_empty, kWorkerWarps);
        ptx::mbar_init(bar_tile_stored, kWorkerWarps);
        ptx::mbar_init(bar_tile_fwd, kFwdWarps);
        ptx::mbar_init(bar_tail_stored, kWorkerWarps);
        ptx::mbar_init(bar_tail_verdict, 1);
        *abort_flag = 0;
        tmem_slot[4] = 0; tmem_slot[5] = 0;   // converter warps that have reported the tile being counted (pipelined reduce-scatter), by tile parity
        ptx::fence_mbar_init();
        ptx::prefetch_tmap(&tmap_act);
        ptx::prefetch_tmap(&tmap_w);
        if (p.c_tma) ptx::prefetch_tmap(&tmap_c);
    }
    if (warp == 1) {
        ptx::tmem_alloc(ptx::smem_u32(const_cast<uint32_t*>(tmem_slot)), L::kTmemCols);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ======================= TMA producer =======================
        if (lane == 0) {
            uint32_t stage = 0, phase = 0, issued = 0, issued_parity = 0;
            bool ok = true;
            Item w;
            for (uint32_t it = 0; ok && get_item(it, w); ++it) {
                const uint32_t t = w.t;
                uint32_t mt_, nt_;
                tile_coords(p, t, mt_, nt_);
                const int m0 = (int)mt_ * BMA, n0 = (int)nt_ * BNW;
                for (uint32_t kb = w.kb0; kb < w.kb1; ++kb) {
                    if (!wait_or_abort(bar_empty_act(stage), phase ^ 1u, abort_flag) ||
                        !wait_or_abort(bar_empty_raw(stage), phase ^ 1u, abort_flag)) {
                        if (!*abort_flag) { report_timeout(p.status, 21, (int)t, (int)kb); *abort_flag = 1; }
                        ok = false; break;
                    }
                    ptx::mbar_arrive_expect_tx(bar_full(stage), L::kActBytes + L::kRawBytes);
                    ptx::tma_load_2d(smem_base + L::kOffAct + stage * L::kActBytes, &tmap_act, (int)(kb * BK), m0, bar_full(stage));
                    ptx::tma_load_2d(smem_base + L::kOffRaw + stage * L::kRawBytes, &tmap_w, (int)(kb * L::kRawRowBytes), n0, bar_full(stage));
                    issued |= 1u << stage;
                    issued_parity = (issued_parity & ~(1u << stage)) | (phase << stage);
                    if (++stage == S) { stage = 0; phase ^= 1u; }
                }
            }
            for (int s = 0; s < S; ++s)   // never leave with a bulk copy still writing this CTA's shared memory
                if (issued & (1u << s)) ptx::mbar_wait(bar_full(s), (issued_parity >> s) & 1u);
        }
    } else if (warp == 1) {
        // ======================= MMA issuer =======================
        if (lane == 0) {
            constexpr uint32_t idesc = ptx::umma_idesc_bf16_f32(BNW, BMA);
            uint32_t st = 0, ph = 0, sa = 0, pa = 0, it = 0;
            bool ok = true;
            Item w;
            for (; ok && get_item(it, w); ++it) {
                const uint32_t t = w.t;
                if (!wait_or_abort(bar_acc_empty, (it & 1u) ^ 1u, abort_flag)) {   // the epilogue of the previous tile has drained the accumulator
                    if (!*abort_flag) { report_timeout(p.status, 22, (int)t, -1); *abort_flag = 1; }
                    break;
                }
                ptx::tc_fence_after_sync();
                for (uint32_t kb = w.kb0; kb < w.kb1; ++kb) {
                    const bool two_terms = GROUPED && p.exact;   // slots sa (hi) and sa + 1 (lo) move in lockstep
                    if (!wait_or_abort(bar_full(st), ph, abort_flag) || !wait_or_abort(bar_full_a(sa), pa, abort_flag) ||
                        (two_terms && !wait_or_abort(bar_full_a(sa + 1), pa, abort_flag))) {
                        if (!*abort_flag) { report_timeout(p.status, 23, (int)t, (int)kb); *abort_flag = 1; }
                        ok = false; break;
                    }
                    ptx::tc_fence_after_sync();
                    const uint64_t db = ptx::umma_desc_kmajor_sw128(smem_base + L::kOffAct + st * L::kActBytes);
                    const uint32_t ta = tmem_base + L::kColA + sa * 32;
#pragma unroll
                    for (int j = 0; j < BK / 16; ++j)   // 16 k per instruction: 8 TMEM columns of weights, 32 bytes of each activation row
                        ptx::umma_bf16_ts(tmem_base, ta + 8 * j, db + 2u * j, idesc, ((kb - w.kb0) | (uint32_t)j) ? 1u : 0u);
                    if (two_terms) {
#pragma unroll
                        for (int j = 0; j < BK / 16; ++j) ptx::umma_bf16_ts(tmem_base, ta + 32 + 8 * j, db + 2u * j, idesc, 1u);
                    }
                    ptx::umma_commit(bar_empty_act(st));
                    ptx::umma_commit(bar_empty_a(sa));
                    if (two_terms) ptx::umma_commit(bar_empty_a(sa + 1));
                    if (++st == S) { st = 0; ph ^= 1u; }
                    sa += two_terms ? 2 : 1;
                    if (sa == kSlotsA) { sa = 0; pa ^= 1u; }
                }
                if (ok) ptx::umma_commit(bar_acc_full);
            }
        }
    } else if (warp < 2 + kWorkerWarps) {
        // ======================= converters + epilogue =======================
        const uint32_t q = (uint32_t)(warp & 3);             // TMEM lane quarter this warp may touch
        const uint32_t kq = (uint32_t)(warp - 2) >> 2;        // which part of the 64-wide K step / which part of the columns
        const uint32_t ch = q * 32 + lane;                    // channel (TMEM lane) of this thread inside the tile
        const uint32_t xormask = (BITS == 8 && p.enc == AFB_ENC_OFFSET_BINARY) ? 0x80808080u : 0u;
        const uint32_t magic4 = p.enc == AFB_ENC_OFFSET_BINARY ? 0x43004300u : 0x43084308u;
        const bool packed = p.packed != 0;
        const uint32_t groups_per_row = GROUPED ? p.k / p.group : 0;
        const bool has_zero = p.zero != nullptr;
        // raw tile in shared memory: rows of 64 (int8) / 32 (int4) bytes, stored by TMA with the 64- / 32-byte swizzle
        // (16-byte piece index XOR row bits); this thread converts kKPer consecutive k of its row
        constexpr int kRawPer = kKPer * BITS / 8;                 // bytes per thread and stage: 32/16 (int8), 16/8 (int4)
        constexpr int kPieces = kRawPer >= 16 ? kRawPer / 16 : 1;  // 16-byte pieces (an 8-byte read stays inside one piece)
        uint32_t raw_off[kPieces];
#pragma unroll
        for (int i = 0; i < kPieces; ++i) {
            const uint32_t byte = kq * kRawPer + i * 16;           // offset inside the row before the swizzle
            const uint32_t piece = byte >> 4;
            raw_off[i] = BITS == 8 ? ch * 64 + ((piece ^ ((ch >> 1) & 3)) << 4) + (byte & 15)
                                   : ch * 32 + ((piece ^ ((ch >> 2) & 1)) << 4) + (byte & 15);
        }
        uint32_t st = 0, ph = 0, sa = 0, pa = 0, it = 0;
        bool ok = true;
        Item w;
        // Pipelined reduce-scatter: a finished tile is counted at its owner only after this warp's peer stores of the tile are
        // visible system-wide, and a fence right after the stores would wait for them to drain over NVLink (tens of microseconds
        // at a CTA's share of the link) with the accumulator and the converters held up.  The count of a tile is therefore taken
        // one tile later, at the start of the next epilogue, when those stores have long drained and the fence is cheap; the last
        // tile of the CTA is counted after the loop.
        // The eight converter warps of the CTA meet at a word in shared memory and the last one reports the whole tile with ONE
        // remote addition of 8: the counters are few (one per owner and column chunk), and an addition per warp means thousands of
        // system-scope atomics from every GPU on the same few words.
        // (two words, used in turn: a warp can be at most one tile ahead of another, so the arrivals of consecutive tiles never mix)
        uint32_t* pending_cnt = nullptr;
        uint32_t pending_parity = 0;
        // Ordering: a warp's lanes meet (__syncwarp), its lane 0 fences at CTA scope and arrives at the word; the last arrival fences
        // at CTA scope again and performs the ONE system-scope release of the tile (cumulative over everything synchronised into
        // it).  A system-scope fence per thread instead cost the GEMM 30 % on 4 GPUs (0.50 against 0.385 ms, whatever the chunk count).
        auto count_pending = [&]() {
            if (!pending_cnt) return;
            __syncwarp();
            if (lane == 0) {
                uint32_t* arrivals = const_cast<uint32_t*>(tmem_slot) + 4 + pending_parity;
                __threadfence_block();
                if (atomicAdd(arrivals, 1u) == (uint32_t)kWorkerWarps - 1) {   // every warp of the CTA has stored its part of the tile
                    atomicExch(arrivals, 0u);   // this word is used again two tiles from now
                    __threadfence_block();
                    asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(pending_cnt), "r"((uint32_t)kWorkerWarps) : "memory");
                }
            }
            pending_cnt = nullptr;
        };
        for (; ok && get_item(it, w); ++it) {
            const uint32_t t = w.t;
            uint32_t mt_, nt_;
            tile_coords(p, t, mt_, nt_);
            const uint32_t m0 = mt_ * BMA, n0 = nt_ * BNW;
            const uint32_t nn = n0 + ch;
            // Scale (and zero-point) of the group this thread's kKPer consecutive k of the step lie in (groups are multiples of kKPer,
            // so a thread never straddles one).  The next group's values are fetched one group ahead.
            uint32_t sc_cur = 0, sc_nxt = 0, zb_cur = 0, zb_nxt = 0;
            auto load_group = [&](uint32_t gidx, uint32_t& sc, uint32_t& zb) {
                sc = 0; zb = 0;
                if (nn >= p.n || gidx >= groups_per_row) return;
                sc = bf16_dup(reinterpret_cast<const uint16_t*>(p.scale)[(size_t)nn * groups_per_row + gidx]);
                if (has_zero) zb = p.zero[(size_t)nn * groups_per_row + gidx];
            };
            uint32_t kpos = w.kb0 * BK + kq * kKPer;            // first k this thread converts in the coming step
            const uint32_t gstep = (GROUPED && p.group < (uint32_t)BK) ? BK / p.group : 1u;   // groups a 64-wide step advances by (2 for groups of 32)
            uint32_t gcur = GROUPED ? kpos / p.group : 0, gend = GROUPED ? (gcur + 1) * p.group : 0xffffffffu;
            uint32_t z8 = 0u, sub4 = 0x43084308u;               // zero-point constants of the unpack (dequant.cuh)
            if (GROUPED) {
                load_group(gcur, sc_cur, zb_cur);
                load_group(gcur + gstep, sc_nxt, zb_nxt);
            } else if (has_zero && nn < p.n) {
                zb_cur = p.zero[nn];
            }
            if (has_zero) { if (BITS == 8) z8 = zero8_const(zb_cur, p.enc); else sub4 = zero4_const(zb_cur, p.enc); }
            for (uint32_t kb = w.kb0; kb < w.kb1; ++kb, kpos += BK) {
                if (GROUPED && kpos >= gend) {
                    gcur += gstep; gend += gstep * p.group;
                    sc_cur = sc_nxt; zb_cur = zb_nxt;
                    load_group(gcur + gstep, sc_nxt, zb_nxt);
                    if (has_zero) { if (BITS == 8) z8 = zero8_const(zb_cur, p.enc); else sub4 = zero4_const(zb_cur, p.enc); }
                }
                const bool two_terms = GROUPED && p.exact;
                if (!wait_or_abort(bar_full(st), ph, abort_flag) || !wait_or_abort(bar_empty_a(sa), pa ^ 1u, abort_flag) ||
                    (two_terms && !wait_or_abort(bar_empty_a(sa + 1), pa ^ 1u, abort_flag))) {
                    if (!*abort_flag) { report_timeout(p.status, 24, (int)t, (int)kb); *abort_flag = 1; }
                    ok = false; break;
                }
                ptx::tc_fence_after_sync();
                const uint8_t* raw = smem_gen + L::kOffRaw + st * L::kRawBytes;
                constexpr int kWords = kRawPer / 4;     // 32-bit words of raw weights per thread
                constexpr int kOut = kKPer / 2;         // packed bf16 pairs = TMEM columns per thread
                uint32_t w[kWords], o[kOut];
                if (kRawPer >= 16) {
#pragma unroll
                    for (int i = 0; i < kPieces; ++i) {
                        const uint4 v = *reinterpret_cast<const uint4*>(raw + raw_off[i]);
                        w[4 * i] = v.x; w[4 * i + 1] = v.y; w[4 * i + 2] = v.z; w[4 * i + 3] = v.w;
                    }
                } else {
                    const uint2 v = *reinterpret_cast<const uint2*>(raw + raw_off[0]);
                    w[0] = v.x; w[1] = v.y;
                }
#pragma unroll
                for (int j = 0; j < kWords; ++j) {
                    if (BITS == 8) {
                        s8x4_to_bf16_pairs(w[j] ^ xormask, packed, o[2 * j], o[2 * j + 1]);
                        if (has_zero) { o[2 * j] = bf16x2_sub(o[2 * j], z8); o[2 * j + 1] = bf16x2_sub(o[2 * j + 1], z8); }
                    } else {
                        uint32_t qv[4];
                        s4x8_to_bf16_pairs(w[j], magic4, packed, qv, sub4);
                        o[4 * j] = qv[0]; o[4 * j + 1] = qv[1]; o[4 * j + 2] = qv[2]; o[4 * j + 3] = qv[3];
                    }
                }
                const uint32_t taddr = tmem_base + ((q * 32u) << 16) + L::kColA + sa * 32 + kq * kOut;
                if (two_terms) {
                    uint32_t lo[kOut];
#pragma unroll
                    for (int j = 0; j < kOut; ++j) {
                        const uint32_t hi = bf16x2_mul(o[j], sc_cur);
                        lo[j] = bf16x2_fma(o[j], sc_cur, hi ^ 0x80008000u);   // q * s - hi: the fused product is exact, the difference fits bf16
                        o[j] = hi;
                    }
                    ptx::tmem_st_cols(taddr + 32, lo);
                } else if (GROUPED) {
#pragma unroll
                    for (int j = 0; j < kOut; ++j) o[j] = bf16x2_mul(o[j], sc_cur);
                }
                ptx::tmem_st_cols(taddr, o);
                ptx::tmem_st_wait();
                ptx::tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) {
                    ptx::mbar_arrive(bar_full_a(sa));
                    if (two_terms) ptx::mbar_arrive(bar_full_a(sa + 1));
                    ptx::mbar_arrive(bar_empty_raw(st));
                }
                if (++st == S) { st = 0; ph ^= 1u; }
                sa += two_terms ? 2 : 1;
                if (sa == kSlotsA) { sa = 0; pa ^= 1u; }
            }
            if (!ok) break;
            // ---- epilogue of this tile: the accumulator is complete once the last MMA has been committed ----
            if (!wait_or_abort(bar_acc_full, it & 1u, abort_flag)) {
                if (!*abort_flag) { report_timeout(p.status, 25, (int)t, -1); *abort_flag = 1; }
                break;
            }
            ptx::tc_fence_after_sync();
            count_pending();   // the previous tile of this CTA (pipelined reduce-scatter only)
            float scale = 1.f;
            if (!GROUPED && nn < p.n)
                scale = p.scale_dtype == AFB_SCALE_BF16 ? __uint_as_float((uint32_t)reinterpret_cast<const uint16_t*>(p.scale)[nn] << 16)
                                                       : reinterpret_cast<const float*>(p.scale)[nn];
            if (p.push_on == 2 && !wait_or_abort(bar_tile_fwd, (it & 1u) ^ 1u, abort_flag)) {   // the previous tile has left
                if (!*abort_flag) { report_timeout(p.status, 26, (int)t, -1); *abort_flag = 1; }
                break;
            }
            constexpr int kColsPerWarp = BMA / kKParts;   // the warps of a lane quarter split the activation rows
#pragma unroll 1
            for (int c0 = 0; c0 < kColsPerWarp; c0 += 32) {
                uint32_t r[32];
                const uint32_t col = kq * kColsPerWarp + c0;
                ptx::tmem_ld_32x32(tmem_base + ((q * 32u) << 16) + col, r);
                ptx::tmem_ld_wait();
                if (w.tail) {   // a stretch of K of a tail tile: the raw fp32 sums go to the workspace, [part][row][channel]
                    float* wsp = p.tail_ws + ((size_t)(w.tail_r * p.tail_parts + w.part) * BMA + col) * BNW + ch;
#pragma unroll
                    for (int j = 0; j < 32; ++j) __stcg(wsp + (size_t)j * BNW, __uint_as_float(r[j]));
                } else if (p.fused) {
                    // every lane takes part (the gated form exchanges values between the two lanes of a pair): range checks only guard the accesses
                    const uint32_t mrow = m0 + col;
                    const bool gated = (p.fused & 2u) != 0;
                    const float bias = (p.bias && nn < p.n) ? p.bias[nn] : 0.f;
                    const uint32_t nout = gated ? (nn >> 1) : nn;
                    const bool writer = nn < p.n && (!gated || (lane & 1) == 0);
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        float v = fmaf(__uint_as_float(r[j]), scale, bias);
                        if (gated) {   // even lane: gate, odd lane: up
                            const float other = __shfl_xor_sync(0xffffffffu, v, 1);
                            if (p.act == AFB_ACT_SILU) v = v / (1.f + __expf(-v));
                            v *= other;
                        } else if (p.act == AFB_ACT_SILU) {
                            v = v / (1.f + __expf(-v));
                        }
                        if (writer && mrow + j < p.m) {
                            if (p.residual) v += __uint_as_float((uint32_t)p.residual[(size_t)(mrow + j) * p.ld_res + nout] << 16);
                            p.c[(size_t)(mrow + j) * p.ldc + nout] = __bfloat16_as_ushort(__float2bfloat16_rn(v));
                        }
                    }
                } else if (p.c_tma) {
                    // bf16 result through shared memory: lane = channel writes its 32 rows into a [row][channel] block (64 contiguous
                    // bytes per warp instruction, no bank conflicts), one lane hands the block to the copy engine as a 32 x 32 tile
                    // store (clipped at the edges of C), and the warp goes on with the next 32 columns while that store drains.
                    const uint32_t out = smem_base + L::kOffOut + (uint32_t)(warp - 2) * L::kStageOutBytes;
                    if (lane == 0) ptx::bulk_wait_group_read0();   // the previous block of this warp has been read out
                    __syncwarp();
#pragma unroll
                    for (int j = 0; j < 32; ++j)
                        asm volatile("st.shared.u16 [%0], %1;" ::"r"(out + (uint32_t)j * 64u + (uint32_t)lane * 2u),
                                     "h"(__bfloat16_as_ushort(__float2bfloat16_rn(__uint_as_float(r[j]) * scale))) : "memory");
                    ptx::fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) {
                        ptx::tma_store_2d(&tmap_c, out, (int)(n0 + q * 32u), (int)(m0 + col));
                        ptx::bulk_commit_group();
                    }
                } else if (nn < p.n) {
                    const uint32_t mrow = m0 + col;
                    if (p.c_f32) {
                        float* dst = reinterpret_cast<float*>(p.c) + (size_t)mrow * p.ldc + nn;
                        if (p.push_on == 1) {   // a tile never straddles two owners (push_rows is a multiple of the tile height)
                            const uint32_t owner = mrow / p.push_rows;
                            dst = p.push[owner] + ((size_t)p.push_rank * p.push_rows + (mrow - owner * p.push_rows)) * p.ldc + nn;
                        }
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            if (mrow + j < p.m) dst[(size_t)j * p.ldc] = __uint_as_float(r[j]) * scale;
                    } else {
                        uint16_t* dst = p.c + (size_t)mrow * p.ldc + nn;
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            if (mrow + j < p.m) dst[(size_t)j * p.ldc] = __bfloat16_as_ushort(__float2bfloat16_rn(__uint_as_float(r[j]) * scale));
                    }
                }
            }
            ptx::tc_fence_before_sync();
            if (p.tile_done) __threadfence_system();   // this lane's stores of the tile are visible to every GPU before the count below
            if (p.push_on == 2) __threadfence();       // ... and to the forwarder warps, which read them back through L2
            __syncwarp();
            if (w.tail) {
                // All stretches of the tile meet here.  The CTA that arrives last adds them in part order (so the bits do not
                // depend on who that is), applies the channel scales, rounds and stores the tile.
                // (a CTA has at most one such stretch per launch, so both barriers are used once: parity 0; every wait is bounded)
                __threadfence();
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(bar_tail_stored);
                if (warp == 2 && lane == 0) {
                    if (wait_or_abort(bar_tail_stored, 0u, abort_flag)) {
                        const uint32_t old = atomicAdd(p.tail_counters + w.tail_r, 1u);
                        tmem_slot[2] = (old == p.tail_parts - 1) ? 1u : 0u;
                    } else {
                        tmem_slot[2] = 0u;
                        if (!*abort_flag) { report_timeout(p.status, 28, (int)t, -1); *abort_flag = 1; }
                    }
                    ptx::mbar_arrive(bar_tail_verdict);
                }
                if (!wait_or_abort(bar_tail_verdict, 0u, abort_flag)) {
                    if (!*abort_flag) { report_timeout(p.status, 29, (int)t, -1); *abort_flag = 1; }
                    break;
                }
                if (tmem_slot[2]) {
                    __threadfence();
                    const uint32_t tid = threadIdx.x - 64;                  // 0 .. 255 over the converter warps
                    const uint32_t c4 = tid & 31u, nv = n0 + c4 * 4;        // this thread's four channels (the same in every row)
                    float sc4[4] = {1.f, 1.f, 1.f, 1.f};
                    if (!GROUPED) {
#pragma unroll
                        for (int e = 0; e < 4; ++e)
                            if (nv + e < p.n)
                                sc4[e] = p.scale_dtype == AFB_SCALE_BF16 ? __uint_as_float((uint32_t)reinterpret_cast<const uint16_t*>(p.scale)[nv + e] << 16)
                                                                         : reinterpret_cast<const float*>(p.scale)[nv + e];
                    }
                    const float* wst = p.tail_ws + (size_t)w.tail_r * p.tail_parts * BMA * BNW;
                    constexpr uint32_t kVecs = BMA * (BNW / 4), kMaxParts = 4, kU = 4;
                    for (uint32_t base = tid; base < kVecs; base += 256 * kU) {
                        float4 v[kMaxParts][kU];
#pragma unroll
                        for (uint32_t j = 0; j < kMaxParts; ++j)
#pragma unroll
                            for (uint32_t u2 = 0; u2 < kU; ++u2)
                                v[j][u2] = j < p.tail_parts ? __ldcg(reinterpret_cast<const float4*>(wst + (size_t)j * BMA * BNW) + base + u2 * 256)
                                                            : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                        for (uint32_t u2 = 0; u2 < kU; ++u2) {
                            float4 a4 = v[0][u2];
#pragma unroll
                            for (uint32_t j = 1; j < kMaxParts; ++j)
                                if (j < p.tail_parts) { a4.x += v[j][u2].x; a4.y += v[j][u2].y; a4.z += v[j][u2].z; a4.w += v[j][u2].w; }
                            const uint32_t row = (base + u2 * 256) >> 5, mrow = m0 + row;
                            if (mrow < p.m && nv < p.n) {
                                a4.x *= sc4[0]; a4.y *= sc4[1]; a4.z *= sc4[2]; a4.w *= sc4[3];
                                if (p.c_f32) {
                                    *reinterpret_cast<float4*>(reinterpret_cast<float*>(p.c) + (size_t)mrow * p.ldc + nv) = a4;
                                } else {
                                    const __nv_bfloat162 lo = __floats2bfloat162_rn(a4.x, a4.y), hi = __floats2bfloat162_rn(a4.z, a4.w);
                                    uint2 o2;
                                    o2.x = *reinterpret_cast<const uint32_t*>(&lo); o2.y = *reinterpret_cast<const uint32_t*>(&hi);
                                    *reinterpret_cast<uint2*>(p.c + (size_t)mrow * p.ldc + nv) = o2;
                                }
                            }
                        }
                    }
                    if (tid == 0) p.tail_counters[w.tail_r] = 0u;   // ready for the next launch
                }
            }
            if (lane == 0) {
                ptx::mbar_arrive(bar_acc_empty);
                if (p.push_on == 2) ptx::mbar_arrive(bar_tile_stored);
                if (p.tile_done) asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p.tile_done + t), "r"(1u) : "memory");
            }
            if (p.push_sub) {   // one count per converter warp and tile, at the owner of the tile's rows, for the tile's column chunk
                const uint32_t owner = m0 / p.push_rows, chunk = nt_ / (p.n_tiles / p.push_sub);
                pending_cnt = p.push_cnt[owner] + chunk;
                pending_parity = it & 1u;
            }
        }
        count_pending();   // the last tile of this CTA: here the fence does wait for the tile's stores to drain
    }

    else if (p.xchg_on) {
        // ======================= exchange warps (only launched with the in-kernel exchange) =======================
        // The other half of the pipelined reduce-scatter, done here instead of by a second kernel (which would have to share SMs
        // with this one): when a column chunk of THIS rank's rows is complete in its local slots (every rank's tiles of the chunk
        // counted), all the exchange warps of the grid add the slots in rank order, round once and broadcast the chunk, while the
        // rest of their CTAs compute the next chunks.  Reads are local; the result leaves as one multicast store (or one store per
        // rank).  The last warp of the grid to finish tells every rank that this rank's rows are in place and waits for theirs.
        const uint32_t fw = (uint32_t)(warp - (2 + kWorkerWarps));
        const uint32_t gw = blockIdx.x * kFwdWarps + fw, nw = gridDim.x * kFwdWarps;
        const uint32_t chunk_cols = p.n / p.push_sub, vec_per_row = chunk_cols / 8;
        const uint32_t total = p.push_rows * vec_per_row;
        const uint32_t row0 = p.push_rank * p.push_rows;
        const float* slots = p.push[p.push_rank];
        bool failed = false;
        for (uint32_t c = 0; c < p.push_sub && !failed; ++c) {
            uint32_t ok = 1u;
            if (lane == 0) {
                const unsigned long long t0 = ptx::globaltimer();
                uint32_t spins = 0;
                while ((int32_t)(xchg::ld_relaxed_sys(p.x.counters + c) - p.x.want) < 0) {
                    __nanosleep(500);
                    if ((++spins & 0xfu) == 0 && (*abort_flag || ptx::globaltimer() - t0 > p.x.wait_ns)) { ok = 0u; break; }
                }
                if (ok) (void)xchg::ld_acquire_sys(p.x.counters + c);   // the counted tiles are visible from here on
                else if (atomicCAS(p.status, 0, AFB_ERR_TIMEOUT) == 0) { p.status[1] = 16; p.status[2] = (int)c; p.status[3] = (int)p.x.epoch; }
            }
            ok = __shfl_sync(0xffffffffu, ok, 0);
            __syncwarp();   // the other lanes' loads below are ordered after lane 0's acquire
            if (!ok) { failed = true; break; }
            for (uint32_t i = gw * 32u + (uint32_t)lane; i < total; i += nw * 32u) {
                const uint32_t lr = i / vec_per_row, col = c * chunk_cols + (i - lr * vec_per_row) * 8u;
                float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int q0 = 0; q0 < AFB_MAX_RANKS; q0 += 4) {
                    uint4 lo[4], hi[4];
#pragma unroll
                    for (int q = 0; q < 4; ++q)
                        if (q0 + q < (int)p.push_world) {
                            const float* src = slots + ((size_t)(q0 + q) * p.push_rows + lr) * p.ldc + col;
                            lo[q] = __ldcg(reinterpret_cast<const uint4*>(src)); hi[q] = __ldcg(reinterpret_cast<const uint4*>(src + 4));
                        }
#pragma unroll
                    for (int q = 0; q < 4; ++q)   // fixed rank order: identical bits wherever it is computed
                        if (q0 + q < (int)p.push_world) {
                            acc[0] += __uint_as_float(lo[q].x); acc[1] += __uint_as_float(lo[q].y); acc[2] += __uint_as_float(lo[q].z); acc[3] += __uint_as_float(lo[q].w);
                            acc[4] += __uint_as_float(hi[q].x); acc[5] += __uint_as_float(hi[q].y); acc[6] += __uint_as_float(hi[q].z); acc[7] += __uint_as_float(hi[q].w);
                        }
                }
                const uint4 out = make_uint4(xchg::pack_bf16(acc[0], acc[1]), xchg::pack_bf16(acc[2], acc[3]), xchg::pack_bf16(acc[4], acc[5]), xchg::pack_bf16(acc[6], acc[7]));
                const size_t at = (size_t)(row0 + lr) * p.x.ldc + col;
                if (p.x.c_multicast) {
                    xchg::st16_multicast(p.x.c_multicast + at, out);
                } else {
#pragma unroll
                    for (int q = 0; q < AFB_MAX_RANKS; ++q)
                        if (q < (int)p.push_world) *reinterpret_cast<uint4*>(p.x.c[q] + at) = out;
                }
            }
        }
        __threadfence_system();
        __syncwarp();
        if (lane == 0) {
            if (failed) atomicExch(p.x.cta_done + 1, 1u);
            if (atomicAdd(p.x.cta_done, 1u) == nw - 1) {   // the last exchange warp of the grid
                const bool any_failed = atomicExch(p.x.cta_done + 1, 0u) != 0;
                *p.x.cta_done = 0u;
                __threadfence_system();
                if (!any_failed) {
                    for (uint32_t q = 0; q < p.push_world; ++q) xchg::st_release_sys(p.x.signals[q] + 1 * AFB_MAX_RANKS + p.push_rank, p.x.epoch);
                    const bool done = xchg::wait_all(p.x.signals[p.push_rank], 1, p.push_world, p.x.epoch, p.x.wait_ns);
                    if (!done && atomicCAS(p.status, 0, AFB_ERR_TIMEOUT) == 0) { p.status[1] = 17; p.status[2] = (int)p.push_rank; p.status[3] = (int)p.x.epoch; }
                }
            }
        }
    }

    else if (p.push_on == 2) {
        // ======================= forwarders (only launched in forward mode) =======================
        // Copy each finished 256 x 128 fp32 tile from local memory to the staging buffer of the rank owning its rows: 512
        // contiguous bytes per warp instruction, issued while the rest of the CTA computes the next tile.
        const uint32_t fw = (uint32_t)(warp - (2 + kWorkerWarps));
        uint32_t it = 0;
        for (uint32_t t = blockIdx.x; t < num_tiles; t += gridDim.x, ++it) {
            if (!wait_or_abort(bar_tile_stored, it & 1u, abort_flag)) {
                if (!*abort_flag) { report_timeout(p.status, 27, (int)t, -1); *abort_flag = 1; }
                break;
            }
            uint32_t mt_, nt_;
            tile_coords(p, t, mt_, nt_);
            const uint32_t m0 = mt_ * BMA, n0 = nt_ * BNW;
            const uint32_t owner = m0 / p.push_rows;
            const float* src = reinterpret_cast<const float*>(p.c) + (size_t)m0 * p.ldc + n0 + lane * 4;
            float* dst = p.push[owner] + ((size_t)p.push_rank * p.push_rows + (m0 - owner * p.push_rows)) * p.ldc + n0 + lane * 4;
            const bool col_ok = n0 + lane * 4 < p.n;
            constexpr int kBatch = 8;
            for (uint32_t r0 = fw * kBatch; r0 < (uint32_t)BMA; r0 += kFwdWarps * kBatch) {
                float4 v[kBatch];
#pragma unroll
                for (int j = 0; j < kBatch; ++j)
                    if (col_ok && m0 + r0 + j < p.m) v[j] = __ldcg(reinterpret_cast<const float4*>(src + (size_t)(r0 + j) * p.ldc));
#pragma unroll
                for (int j = 0; j < kBatch; ++j)
                    if (col_ok && m0 + r0 + j < p.m) *reinterpret_cast<float4*>(dst + (size_t)(r0 + j) * p.ldc) = v[j];
            }
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(bar_tile_fwd);
        }
    }

    // ---- teardown: every thread gets here, also after an abort ----
    if (p.c_tma && warp >= 2 && warp < 2 + kWorkerWarps && lane == 0) ptx::bulk_wait_group0();   // this warp's tile stores are complete
    ptx::tc_fence_before_sync();
    __syncthreads();
    if (p.ts && threadIdx.x == 0) atomicMax(p.ts + 1, ptx::globaltimer());
    if (warp == 1) {
        ptx::tc_fence_after_sync();
        ptx::tmem_dealloc(tmem_base, L::kTmemCols);
    }
}

int ts_tmap_2d(CUtensorMap* map, CUtensorMapDataType dt, const void* base, uint64_t inner, uint64_t outer, uint64_t row_stride_bytes,
               uint32_t box_inner, uint32_t box_outer, CUtensorMapSwizzle swz) {
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

// Row tiles per group of the tile order, from a simple model of the HBM traffic.  One wave of CTAs covers g row tiles and
// about sms / g channel tiles and re-reads both from HBM, unless the activations of the group (g * BMA * K * 2 bytes) are
// small enough to stay in L2 over the whole group, in which case they are read once per group.
uint32_t pick_group_m(const afb_gemm_args& a, uint32_t m_tiles, uint32_t n_tiles, uint32_t bma, int sms) {
    const double k = a.k, wbytes = a.b_bits / 8.0;
    const double tiles = (double)m_tiles * n_tiles;
    const double w_total = (double)a.n * k * wbytes, a_total = (double)a.m * k * 2.0;
    const double l2_keep = 36e6;   // what survives in L2 next to the streams (measured: 33.5 MB does, 67 MB does not)
    double best = 1e30;
    uint32_t best_g = m_tiles;
    for (uint32_t g = 1; g <= m_tiles; ++g) {
        if (g != m_tiles && g != 1 && (m_tiles % g) != 0) continue;
        const double a_slice = (double)g * bma * k * 2.0;
        const double groups = (double)((m_tiles + g - 1) / g);
        double bytes;
        if (a_slice <= l2_keep) {
            bytes = a_total + groups * w_total;                       // activations once, weights once per group
        } else {
            const double ng = (double)sms / g < 1.0 ? 1.0 : ((double)sms / g > n_tiles ? (double)n_tiles : (double)sms / g);
            const double per_wave = a_slice + ng * BNW * k * wbytes;
            bytes = tiles / ((double)g * ng) * per_wave;
        }
        if (bytes < best) { best = bytes; best_g = g; }
    }
    if (const char* e = getenv("AFB_PREFILL_GROUP_M")) { const uint32_t v = (uint32_t)atoi(e); if (v >= 1 && v <= m_tiles) best_g = v; }
    return best_g;
}

template <int BITS, bool GROUPED, int BMA>
int launch_ts_cfg(const afb_gemm_args& a, DeviceCtx* ctx, cudaStream_t s, uint32_t* tile_done = nullptr, void* const* push = nullptr,
                  uint32_t push_world = 0, uint32_t push_rank = 0, bool push_via_local = false, const afb_fused_args* fused = nullptr,
                  uint32_t* const* push_cnt = nullptr, uint32_t push_sub = 0, const PushExchange* xchg_desc = nullptr) {
    using L = TsLayout<BITS, BMA>;
    static_assert(L::kDynamic <= 232448, "shared memory budget");
    CUtensorMap ta, tw;
    int rc = ts_tmap_2d(&ta, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, a.ptr_a, a.k, a.m, (uint64_t)a.lda * 2, BK, BMA, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
    const uint64_t row_bytes = (uint64_t)a.k * BITS / 8, ld_bytes = (uint64_t)a.ldb * BITS / 8;
    rc = ts_tmap_2d(&tw, CU_TENSOR_MAP_DATA_TYPE_UINT8, a.ptr_b, row_bytes, a.n, ld_bytes, L::kRawRowBytes, BNW,
                    BITS == 8 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B);
    if (rc) return rc;
    TsParams p;
    // bf16 C of a plain GEMM leaves through tile stores (32 channels x 32 rows per store); every other form stores from registers
    CUtensorMap tc = ta;
    p.c_tma = 0;
    {
        const char* e = getenv("AFB_PREFILL_TILE_STORE");   // tuning aid: 0 switches it off
        const bool wanted = !(e && atoi(e) == 0);
        if (wanted && !(a.flags & AFB_FLAG_C_F32) && !tile_done && !push && !fused && a.ldc % 8 == 0 && (uintptr_t)a.ptr_c % 16 == 0 &&
            ts_tmap_2d(&tc, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, a.ptr_c, a.n, a.m, (uint64_t)a.ldc * 2, 32, 32, CU_TENSOR_MAP_SWIZZLE_NONE) == AFB_OK)
            p.c_tma = 1;
    }
    p.c = reinterpret_cast<uint16_t*>(a.ptr_c);
    p.scale = a.ptr_scale;
    p.zero = reinterpret_cast<const uint8_t*>(a.ptr_zero);
    p.m = a.m; p.n = a.n; p.k = a.k; p.ldc = a.ldc;
    p.enc = a.b_encoding; p.scale_dtype = a.scale_dtype; p.group = a.group_size;
    p.m_tiles = (a.m + BMA - 1) / BMA;
    p.n_tiles = (a.n + BNW - 1) / BNW;
    p.c_f32 = (a.flags & AFB_FLAG_C_F32) ? 1u : 0u;
    p.exact = (GROUPED && (a.flags & AFB_FLAG_GROUP_EXACT)) ? 1u : 0u;
    p.packed = a.b_layout == AFB_LAYOUT_COL_PACKED ? 1u : 0u;
    p.group_m = tile_done ? p.m_tiles : pick_group_m(a, p.m_tiles, p.n_tiles, BMA, ctx->sm_count);   // the exchange kernel assumes row-tile-fastest order
    p.tile_done = tile_done;
    // The tiles beyond the last full wave would keep a few SMs busy for a whole tile while the rest idle: cut each of them into
    // up to 4 stretches of K, one per CTA (up-projection shard on 8 GPUs: 448 tiles on 148 SMs = 3 waves + 4 tiles).  The same
    // when ALL the tiles are at most half a wave (8192 channels at M <= 128: 64 tiles, two stretches each on 128 SMs).
    p.tail_first = p.m_tiles * p.n_tiles; p.tail_tiles = 0; p.tail_parts = 0;
    p.tail_ws = nullptr; p.tail_counters = nullptr;
    {
        const uint32_t tiles_all = p.m_tiles * p.n_tiles, sms = (uint32_t)ctx->sm_count, nkb = a.k / BK;
        // (less than a wave: only for bf16 results -- fp32 results are the partial sums of a row-parallel GEMM, which the exchange forms
        // sum to identical bits only while every form adds along K in the same order)
        const uint32_t rest = tiles_all > sms ? tiles_all % sms : ((tiles_all < sms && !(a.flags & AFB_FLAG_C_F32)) ? tiles_all : 0);
        const char* e = getenv("AFB_PREFILL_SPLIT_TAIL");   // tuning aid: 0 switches it off
        const bool allowed = !(e && atoi(e) == 0) && !tile_done && !push && !fused && a.n % 4 == 0;
        if (allowed && rest > 0 && rest <= sms / 2) {
            uint32_t parts = sms / rest;
            if (parts > 4) parts = 4;
            const uint32_t kb_group = (GROUPED && a.group_size > (uint32_t)BK) ? a.group_size / BK : 1;
            while (parts >= 2 && (nkb % parts != 0 || (nkb / parts) % kb_group != 0 || nkb / parts < 8)) --parts;
            if (parts >= 2 && (size_t)rest * parts * BMA * BNW * sizeof(float) <= ctx->splitk_ws_bytes && rest <= ctx->splitk_counter_count) {
                int wrc = AFB_OK;
                const DeviceCtx::Workspace* wsp = workspace_for(ctx, s, &wrc);   // this stream's own workspace
                if (!wsp) return wrc;
                p.tail_ws = wsp->ws; p.tail_counters = wsp->counters;
                p.tail_first = tiles_all - rest; p.tail_tiles = rest; p.tail_parts = parts;
            }
        }
    }
    p.bias = fused ? reinterpret_cast<const float*>(fused->ptr_bias) : nullptr;
    p.residual = fused ? reinterpret_cast<const uint16_t*>(fused->ptr_residual) : nullptr;
    p.ld_res = fused ? fused->ld_residual : 0;
    p.fused = fused ? (1u | (fused->gated ? 2u : 0u)) : 0u;
    p.act = fused ? fused->activation : AFB_ACT_NONE;
    p.push_on = push ? (push_via_local ? 2u : 1u) : 0u;
    // every rank walks the row tiles from a different start, so that at any moment the ranks push to different owners
    // instead of all loading the same peer's NVLink ingress
    p.m_rot = 0;
    if (push) {
        const char* e = getenv("AFB_PUSH_ROTATE");   // tuning aid: 0 switches the rotation off
        if (!(e && atoi(e) == 0)) p.m_rot = (uint32_t)(((uint64_t)push_rank * p.m_tiles) / push_world) % p.m_tiles;
    }
    p.push_rank = push_rank;
    p.push_world = push_world;
    p.push_sub = (push && push_cnt) ? push_sub : 0;
    for (uint32_t q = 0; q < AFB_MAX_RANKS; ++q) p.push_cnt[q] = (p.push_sub && q < push_world) ? push_cnt[q] : nullptr;
    if (p.push_sub) p.m_rot = 0;   // the unit order already spreads the owners
    p.xchg_on = (p.push_sub && xchg_desc) ? 1u : 0u;
    p.x = xchg_desc ? *xchg_desc : PushExchange{};
    p.push_rows = push ? a.m / push_world : 0;
    for (uint32_t q = 0; q < AFB_MAX_RANKS; ++q) p.push[q] = (push && q < push_world) ? reinterpret_cast<float*>(push[q]) : nullptr;
    p.status = ctx->status;
    p.ts = push ? phase_ts_if_enabled(ctx) : nullptr;
    auto kern = prefill_ts_kernel<BITS, GROUPED, BMA>;
    static DeviceOnce attr_set;  // per template instance
    if (!attr_set.done(ctx->device)) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDynamic);
        if (e != cudaSuccess) return cuda_fail(e);
        attr_set.mark(ctx->device);
    }
    const uint32_t tiles = p.m_tiles * p.n_tiles;
    uint32_t grid = tiles < (uint32_t)ctx->sm_count ? tiles : (uint32_t)ctx->sm_count;
    // pipelined reduce-scatter: a few SMs are left to the kernel that sums and broadcasts the finished column chunks (ksplit.cu)
    // (always that many, also when there are fewer tiles than SMs: a CTA of that kernel on an SM this GEMM still needs would
    // wait for tiles that cannot be computed)
    if (p.push_sub && !p.xchg_on && (uint32_t)ctx->sm_count > 2 * sub_allreduce_sms() && grid > (uint32_t)ctx->sm_count - sub_allreduce_sms())
        grid = (uint32_t)ctx->sm_count - sub_allreduce_sms();
    if (grid < p.tail_tiles * p.tail_parts) grid = p.tail_tiles * p.tail_parts;   // less than a wave of tiles, all of them cut along K
    kern<<<grid, (p.push_on == 2 || p.xchg_on) ? kThreadsFwd : kThreads, L::kDynamic, s>>>(ta, tw, tc, p);
    count_launch();
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? AFB_OK : cuda_fail(e);
}

}  // namespace

// Tiles of the 256-row form, as the tile-granular exchange sees them: tile t covers rows (t % m_tiles) * 256 .. and
// channels (t / m_tiles) * 128 ..; every tile is counted kTileArrivals times in tile_done[t] per launch.
void prefill_ts_tile_info(uint32_t m, uint32_t n, uint32_t* tile_m, uint32_t* tile_n, uint32_t* m_tiles, uint32_t* n_tiles, uint32_t* arrivals) {
    *tile_m = 256; *tile_n = BNW; *m_tiles = (m + 255) / 256; *n_tiles = (n + BNW - 1) / BNW; *arrivals = kWorkerWarps;
}

int launch_prefill_ts_tiles(const afb_gemm_args& a, DeviceCtx* ctx, uint32_t* tile_done, cudaStream_t s) {
    if (!prefill_supports(a) || a.group_size != 0 || a.b_bits != 8 || a.m <= 128) return AFB_ERR_UNSUPPORTED;   // the row-parallel path: int8, per-channel
    return launch_ts_cfg<8, false, 256>(a, ctx, s, tile_done);
}

// Row-parallel GEMM whose epilogue is the reduce-scatter: every tile of fp32 partial sums is stored straight into the staging
// buffer of the rank that owns those rows (peer stores over NVLink), slot = this rank.
int launch_prefill_ts_push(const afb_gemm_args& a, DeviceCtx* ctx, void* const* stage, uint32_t world, uint32_t rank, cudaStream_t s,
                           uint32_t* const* counters, uint32_t sub_blocks, const PushExchange* x) {
    if (!prefill_supports(a) || a.group_size != 0 || a.b_bits != 8 || a.m <= 128) return AFB_ERR_UNSUPPORTED;
    if (world == 0 || world > AFB_MAX_RANKS || rank >= world || a.m % (world * 256) != 0 || a.ldc != a.n) return AFB_ERR_UNSUPPORTED;
    if (counters) {   // pipelined form: whole column chunks of channel tiles, epilogue stores straight to the owner
        const uint32_t n_tiles = (a.n + BNW - 1) / BNW;
        if (sub_blocks == 0 || n_tiles % sub_blocks != 0 || a.n % BNW != 0 || (a.flags & AFB_FLAG_PUSH_VIA_LOCAL)) return AFB_ERR_UNSUPPORTED;
    }
    if (x && !counters) return AFB_ERR_BAD_ARG;
    return launch_ts_cfg<8, false, 256>(a, ctx, s, nullptr, stage, world, rank, (a.flags & AFB_FLAG_PUSH_VIA_LOCAL) != 0, nullptr, counters, sub_blocks, x);
}

// `fused`: optional epilogue description (bias, activation, gate * up, residual); a.ptr_c / a.ldc describe the [M, N_out] result.
int launch_prefill_ts(const afb_gemm_args& a, DeviceCtx* ctx, cudaStream_t s, const afb_fused_args* fused) {
    if (!fused && !prefill_supports(a)) return AFB_ERR_UNSUPPORTED;   // the fused entry point has checked its own argument block
    const bool grouped = a.group_size != 0;
    const bool wide = a.m > 128;   // activation rows per tile: 256, or 128 when M is small
    uint32_t* const no_tiles = nullptr;
    void* const* const no_push = nullptr;
#define AFB_TS_LAUNCH(B, G, W) launch_ts_cfg<B, G, W>(a, ctx, s, no_tiles, no_push, 0, 0, false, fused)
    if (a.b_bits == 8) {
        if (wide) return grouped ? AFB_TS_LAUNCH(8, true, 256) : AFB_TS_LAUNCH(8, false, 256);
        return grouped ? AFB_TS_LAUNCH(8, true, 128) : AFB_TS_LAUNCH(8, false, 128);
    }
    if (wide) return grouped ? AFB_TS_LAUNCH(4, true, 256) : AFB_TS_LAUNCH(4, false, 256);
    return grouped ? AFB_TS_LAUNCH(4, true, 128) : AFB_TS_LAUNCH(4, false, 128);
#undef AFB_TS_LAUNCH
}

}  // namespace afb
