// Row-parallel (K-split) exchange: the all-reduce of per-GPU partial sums as one kernel per GPU over
// NVLink peer memory (reduce-scatter by peer loads, all-gather by peer stores), plus the fp32 -> bf16
// cast that finishes the NCCL comparison path.  The reference is single-GPU (bfAintBGemm.cc:63) and has
// no counterpart.  Only plain ld/st reach peer memory (no TMA); the broadcast of the result rows may instead be ONE
// multimem.st per 16 bytes to an NVSwitch multicast address, when the caller has one.
//
// Signals: every rank owns uint32 signals[2][AFB_MAX_RANKS]; rank q writes `epoch` into
// signals[phase][q] of every rank.  Phase 0: "my partial of this epoch is complete" (the GEMM that
// produced it precedes this kernel in stream order).  Phase 1: "I have stored my row block into your C".
// Epochs only grow, so nothing is ever reset and a late reader cannot mistake an old signal.
#include <cstdlib>
#include <cuda_bf16.h>
#include "afb_internal.h"
#include "sys_sync.cuh"

namespace afb {
namespace {

constexpr int kThreads = 512;
constexpr uint32_t BNW_TILE = 128;   // channels per GEMM tile (prefill_ts.cu)

struct ARParams {
    const void* partial[AFB_MAX_RANKS];
    uint16_t* c[AFB_MAX_RANKS];
    uint16_t* c_multicast;   // optional: one address that the NVSwitch replicates into every rank's C
    uint32_t* signals[AFB_MAX_RANKS];
    uint32_t rank, world, m, n, ld_partial, ldc, partial_f32, epoch;
    unsigned long long wait_ns;
    uint32_t* cta_done;   // local counter, zero between launches
    int32_t* status;
    unsigned long long* ts;   // optional phase timestamps (nullptr = off)
};

using namespace xchg;

template <bool F32>
__global__ void __launch_bounds__(kThreads) ksplit_allreduce_kernel(const ARParams p) {
    __shared__ uint32_t s_ok;
    __shared__ uint32_t s_last;
    const uint32_t* my_sig = p.signals[p.rank];
    if (threadIdx.x == 0) {
        if (blockIdx.x == 0) {
            if (p.ts) p.ts[2] = now_ns();
            __threadfence_system();
            for (uint32_t q = 0; q < p.world; ++q) st_release_sys(p.signals[q] + 0 * AFB_MAX_RANKS + p.rank, p.epoch);
        }
        const bool ok = wait_all(my_sig, 0, p.world, p.epoch, p.wait_ns);
        if (p.ts && blockIdx.x == 0) p.ts[3] = now_ns();
        if (!ok && atomicCAS(p.status, 0, AFB_ERR_TIMEOUT) == 0) { p.status[1] = 10; p.status[2] = (int)p.rank; p.status[3] = (int)p.epoch; }
        if (!ok) atomicExch(p.cta_done + 1, 1u);   // every CTA runs its own clock: one that gave up vetoes the completion signal
        s_ok = ok ? 1u : 0u;
    }
    __syncthreads();
    if (s_ok) {
        // rows [r0, r1) belong to this rank; 8 output columns (16 bytes of bf16) per thread per step
        const uint32_t r0 = (uint32_t)((uint64_t)p.m * p.rank / p.world), r1 = (uint32_t)((uint64_t)p.m * (p.rank + 1) / p.world);
        const uint32_t vec_per_row = p.n / 8;
        const uint64_t total = (uint64_t)(r1 - r0) * vec_per_row;
        for (uint64_t i = (uint64_t)blockIdx.x * kThreads + threadIdx.x; i < total; i += (uint64_t)gridDim.x * kThreads) {
            const uint32_t row = r0 + (uint32_t)(i / vec_per_row), col = (uint32_t)(i % vec_per_row) * 8;
            float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            if (F32) {
                uint4 lo[AFB_MAX_RANKS], hi[AFB_MAX_RANKS];
#pragma unroll
                for (int q = 0; q < AFB_MAX_RANKS; ++q)
                    if (q < (int)p.world) {
                        const float* src = reinterpret_cast<const float*>(p.partial[q]) + (size_t)row * p.ld_partial + col;
                        lo[q] = ld16(src); hi[q] = ld16(src + 4);
                    }
#pragma unroll
                for (int q = 0; q < AFB_MAX_RANKS; ++q)   // fixed rank order: identical bits wherever it is computed
                    if (q < (int)p.world) {
                        acc[0] += __uint_as_float(lo[q].x); acc[1] += __uint_as_float(lo[q].y); acc[2] += __uint_as_float(lo[q].z); acc[3] += __uint_as_float(lo[q].w);
                        acc[4] += __uint_as_float(hi[q].x); acc[5] += __uint_as_float(hi[q].y); acc[6] += __uint_as_float(hi[q].z); acc[7] += __uint_as_float(hi[q].w);
                    }
            } else {
                uint4 v[AFB_MAX_RANKS];
#pragma unroll
                for (int q = 0; q < AFB_MAX_RANKS; ++q)
                    if (q < (int)p.world) v[q] = ld16(reinterpret_cast<const uint16_t*>(p.partial[q]) + (size_t)row * p.ld_partial + col);
#pragma unroll
                for (int q = 0; q < AFB_MAX_RANKS; ++q)
                    if (q < (int)p.world) {
                        acc[0] += bf_lo(v[q].x); acc[1] += bf_hi(v[q].x); acc[2] += bf_lo(v[q].y); acc[3] += bf_hi(v[q].y);
                        acc[4] += bf_lo(v[q].z); acc[5] += bf_hi(v[q].z); acc[6] += bf_lo(v[q].w); acc[7] += bf_hi(v[q].w);
                    }
            }
            const uint4 out = make_uint4(pack_bf16(acc[0], acc[1]), pack_bf16(acc[2], acc[3]), pack_bf16(acc[4], acc[5]), pack_bf16(acc[6], acc[7]));
            if (p.c_multicast) {
                st16_multicast(p.c_multicast + (size_t)row * p.ldc + col, out);   // leaves this GPU once, lands in all C
            } else {
#pragma unroll
                for (int q = 0; q < AFB_MAX_RANKS; ++q)
                    if (q < (int)p.world) *reinterpret_cast<uint4*>(p.c[q] + (size_t)row * p.ldc + col) = out;
            }
        }
    }
    // the last CTA to finish tells every rank that this rank's block is in place, then waits for theirs
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        const uint32_t old = atomicAdd(p.cta_done, 1u);
        s_last = old == gridDim.x - 1 ? 1u : 0u;
    }
    __syncthreads();
    if (s_last && threadIdx.x == 0) {
        const bool any_failed = atomicExch(p.cta_done + 1, 0u) != 0;
        *p.cta_done = 0u;
        if (p.ts) p.ts[4] = now_ns();
        __threadfence_system();
        if (!any_failed) {   // after a timeout in ANY CTA part of the block was not stored: do not claim completion
            for (uint32_t q = 0; q < p.world; ++q) st_release_sys(p.signals[q] + 1 * AFB_MAX_RANKS + p.rank, p.epoch);
            const bool ok = wait_all(my_sig, 1, p.world, p.epoch, p.wait_ns);
            if (p.ts) p.ts[5] = now_ns();
            if (!ok && atomicCAS(p.status, 0, AFB_ERR_TIMEOUT) == 0) { p.status[1] = 11; p.status[2] = (int)p.rank; p.status[3] = (int)p.epoch; }
        }
    }
}

// ---------------------------------------------------------------------------------------------------------
// Pipelined form: runs NEXT TO the pushing GEMM (launched on another stream).  The GEMM delivers the partial sums column
// chunk by column chunk: after every `world` units of its tile order one more chunk of THIS rank's rows is complete in the
// local staging slots, and the GEMM has counted every tile of it in counters[chunk].  This kernel waits for a chunk's count,
// adds the `world` LOCAL slots in rank order, rounds once and broadcasts the bf16 rows (multimem.st or peer stores), while the
// GEMM computes the next chunk: only the last chunk's sum and broadcast remain after the GEMM.  It reads no peer memory.
// ---------------------------------------------------------------------------------------------------------
struct SubARParams {
    ARParams ar;
    const uint32_t* counters;   // local, one per column chunk, only grow
    uint32_t sub_blocks, want;  // want = counts per chunk and launch x launches so far
};

__global__ void __launch_bounds__(768, 1) ksplit_sub_allreduce_kernel(const SubARParams sp) {
    const ARParams& p = sp.ar;
    __shared__ uint32_t s_ok;
    __shared__ uint32_t s_last;
    const uint32_t r0 = (uint32_t)((uint64_t)p.m * p.rank / p.world), r1 = (uint32_t)((uint64_t)p.m * (p.rank + 1) / p.world);
    const uint32_t chunk_cols = p.n / sp.sub_blocks, vec_per_row = chunk_cols / 8;
    const uint64_t total = (uint64_t)(r1 - r0) * vec_per_row;
    bool failed = false;
    if (p.ts && blockIdx.x == 0 && threadIdx.x == 0) p.ts[2] = now_ns();
    for (uint32_t c = 0; c < sp.sub_blocks && !failed; ++c) {
        if (threadIdx.x == 0) {
            const unsigned long long t0 = now_ns();
            bool ok = true;
            uint32_t spins = 0;
            while ((int32_t)(ld_relaxed_sys(sp.counters + c) - sp.want) < 0) {
                __nanosleep(500);
                if ((++spins & 0xfu) == 0 && now_ns() - t0 > p.wait_ns) { ok = false; break; }
            }
            if (ok) (void)ld_acquire_sys(sp.counters + c);   // the one ordered load: the counted tiles are visible from here on
            if (!ok && atomicCAS(p.status, 0, AFB_ERR_TIMEOUT) == 0) { p.status[1] = 14; p.status[2] = (int)c; p.status[3] = (int)p.epoch; }
            s_ok = ok ? 1u : 0u;
            if (p.ts && blockIdx.x == 0 && c + 1 == sp.sub_blocks) p.ts[3] = now_ns();
        }
        __syncthreads();
        if (!s_ok) { failed = true; break; }
        for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (uint64_t)gridDim.x * blockDim.x) {
            const uint32_t row = r0 + (uint32_t)(i / vec_per_row), col = c * chunk_cols + (uint32_t)(i % vec_per_row) * 8;
            float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            // four slots at a time: few registers, so that a CTA of this kernel fits next to the GEMM's CTA on an SM
#pragma unroll
            for (int q0 = 0; q0 < AFB_MAX_RANKS; q0 += 4) {
                uint4 lo[4], hi[4];
#pragma unroll
                for (int q = 0; q < 4; ++q)
                    if (q0 + q < (int)p.world) {
                        const float* src = reinterpret_cast<const float*>(p.partial[q0 + q]) + (size_t)row * p.ld_partial + col;
                        lo[q] = __ldcg(reinterpret_cast<const uint4*>(src)); hi[q] = __ldcg(reinterpret_cast<const uint4*>(src + 4));
                    }
#pragma unroll
                for (int q = 0; q < 4; ++q)   // fixed rank order: identical bits wherever it is computed
                    if (q0 + q < (int)p.world) {
                        acc[0] += __uint_as_float(lo[q].x); acc[1] += __uint_as_float(lo[q].y); acc[2] += __uint_as_float(lo[q].z); acc[3] += __uint_as_float(lo[q].w);
                        acc[4] += __uint_as_float(hi[q].x); acc[5] += __uint_as_float(hi[q].y); acc[6] += __uint_as_float(hi[q].z); acc[7] += __uint_as_float(hi[q].w);
                    }
            }
            const uint4 out = make_uint4(pack_bf16(acc[0], acc[1]), pack_bf16(acc[2], acc[3]), pack_bf16(acc[4], acc[5]), pack_bf16(acc[6], acc[7]));
            if (p.c_multicast) {
                st16_multicast(p.c_multicast + (size_t)row * p.ldc + col, out);
            } else {
#pragma unroll
                for (int q = 0; q < AFB_MAX_RANKS; ++q)
                    if (q < (int)p.world) *reinterpret_cast<uint4*>(p.c[q] + (size_t)row * p.ldc + col) = out;
            }
        }
        __syncthreads();   // s_ok is rewritten for the next chunk
    }
    // the last CTA to finish tells every rank that this rank's rows are in place, then waits for theirs
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        if (failed) atomicExch(p.cta_done + 1, 1u);
        const uint32_t old = atomicAdd(p.cta_done, 1u);
        s_last = old == gridDim.x - 1 ? 1u : 0u;
    }
    __syncthreads();
    if (s_last && threadIdx.x == 0) {
        const bool any_failed = atomicExch(p.cta_done + 1, 0u) != 0;
        *p.cta_done = 0u;
        if (p.ts) p.ts[4] = now_ns();
        __threadfence_system();
        if (!any_failed) {
            for (uint32_t q = 0; q < p.world; ++q) st_release_sys(p.signals[q] + 1 * AFB_MAX_RANKS + p.rank, p.epoch);
            const bool ok = wait_all(p.signals[p.rank], 1, p.world, p.epoch, p.wait_ns);
            if (!ok && atomicCAS(p.status, 0, AFB_ERR_TIMEOUT) == 0) { p.status[1] = 15; p.status[2] = (int)p.rank; p.status[3] = (int)p.epoch; }
            if (p.ts) p.ts[5] = now_ns();
        }
    }
}

// ---------------------------------------------------------------------------------------------------------
// Tile-granular form: runs NEXT TO the K-split GEMM (launched after it, on another stream).  The GEMM counts every
// finished tile of its partial sum in tile_done[t]; this kernel takes the tiles this rank owns (t % world == rank) in
// the order the GEMM produces them, waits until all ranks have counted the tile, then pulls, adds, rounds and pushes it.
// The exchange of a tile thus overlaps the GEMM main loop of the following tiles.  The GEMM never waits for this kernel.
// ---------------------------------------------------------------------------------------------------------
struct TileARParams {
    ARParams ar;
    const uint32_t* tile_done[AFB_MAX_RANKS];
    uint32_t tile_m, tile_n, m_tiles, n_tiles, arrivals, tile_epoch;
};
constexpr int kTileThreads = 256;         // upper bound (launch bounds)
constexpr int kTileThreadsDefault = 128;
constexpr int kSubRows = 64;   // rows of a tile handled as one unit of work

__global__ void __launch_bounds__(kTileThreads, 2) ksplit_tile_allreduce_kernel(const TileARParams tp) {
    const ARParams& p = tp.ar;
    __shared__ uint32_t s_ok;
    __shared__ uint32_t s_last;
    const uint32_t tiles = tp.m_tiles * tp.n_tiles;
    const uint32_t owned = tiles > p.rank ? (tiles - p.rank + p.world - 1) / p.world : 0;
    const uint32_t subs = tp.tile_m / kSubRows;
    const uint32_t units = owned * subs;
    const uint32_t want = tp.arrivals * tp.tile_epoch;
    const uint32_t vec_per_row = tp.tile_n / 8;                    // 8 channels (32 bytes of fp32) per thread
    const uint32_t rows_per_pass = blockDim.x / vec_per_row;
    bool failed = false;
    for (uint32_t u = blockIdx.x; u < units && !failed; u += gridDim.x) {
        const uint32_t t = p.rank + (u / subs) * p.world, sub = u % subs;
        if (threadIdx.x < 32) {   // lane q watches rank q's counter: one NVLink round trip per poll, not one per rank
            const unsigned long long t0 = now_ns();
            const uint32_t* f = threadIdx.x < p.world ? tp.tile_done[threadIdx.x] + t : nullptr;
            bool ok = true;
            uint32_t spins = 0;
            while (true) {
                const bool ready = f == nullptr || (int32_t)(ld_acquire_sys(f) - want) >= 0;
                if (__all_sync(0xffffffffu, ready)) break;
                if ((++spins & 0x7u) == 0) {
                    const bool late = now_ns() - t0 > p.wait_ns;
                    if (__any_sync(0xffffffffu, late)) { ok = false; break; }
                    __nanosleep(100);
                }
            }
            if (threadIdx.x == 0) {
                if (!ok && atomicCAS(p.status, 0, AFB_ERR_TIMEOUT) == 0) { p.status[1] = 12; p.status[2] = (int)t; p.status[3] = (int)p.epoch; }
                s_ok = ok ? 1u : 0u;
            }
        }
        __syncthreads();
        if (!s_ok) { failed = true; break; }
        const uint32_t m0 = (t % tp.m_tiles) * tp.tile_m + sub * kSubRows, n0 = (t / tp.m_tiles) * tp.tile_n;
        const uint32_t col = n0 + (threadIdx.x % vec_per_row) * 8;
        for (uint32_t r = threadIdx.x / vec_per_row; r < (uint32_t)kSubRows; r += rows_per_pass) {
            const uint32_t row = m0 + r;
            if (row >= p.m || col >= p.n) continue;
            float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            uint4 lo[AFB_MAX_RANKS], hi[AFB_MAX_RANKS];
#pragma unroll
            for (int q = 0; q < AFB_MAX_RANKS; ++q)
                if (q < (int)p.world) {
                    const float* src = reinterpret_cast<const float*>(p.partial[q]) + (size_t)row * p.ld_partial + col;
                    lo[q] = ld16(src); hi[q] = ld16(src + 4);
                }
#pragma unroll
            for (int q = 0; q < AFB_MAX_RANKS; ++q)   // fixed rank order: identical bits wherever it is computed
                if (q < (int)p.world) {
                    acc[0] += __uint_as_float(lo[q].x); acc[1] += __uint_as_float(lo[q].y); acc[2] += __uint_as_float(lo[q].z); acc[3] += __uint_as_float(lo[q].w);
                    acc[4] += __uint_as_float(hi[q].x); acc[5] += __uint_as_float(hi[q].y); acc[6] += __uint_as_float(hi[q].z); acc[7] += __uint_as_float(hi[q].w);
                }
            const uint4 out = make_uint4(pack_bf16(acc[0], acc[1]), pack_bf16(acc[2], acc[3]), pack_bf16(acc[4], acc[5]), pack_bf16(acc[6], acc[7]));
#pragma unroll
            for (int q = 0; q < AFB_MAX_RANKS; ++q)
                if (q < (int)p.world) *reinterpret_cast<uint4*>(p.c[q] + (size_t)row * p.ldc + col) = out;
        }
        __syncthreads();   // s_ok is rewritten by the next unit
    }
    // the last CTA to finish tells every rank that this rank's tiles are in place, then waits for theirs
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        if (failed) atomicExch(p.cta_done + 1, 1u);
        const uint32_t old = atomicAdd(p.cta_done, 1u);
        s_last = old == gridDim.x - 1 ? 1u : 0u;
    }
    __syncthreads();
    if (s_last && threadIdx.x == 0) {
        const bool any_failed = atomicExch(p.cta_done + 1, 0u) != 0;
        *p.cta_done = 0u;
        __threadfence_system();
        if (!any_failed) {   // after a timeout some tiles were not stored: do not claim completion
            for (uint32_t q = 0; q < p.world; ++q) st_release_sys(p.signals[q] + 1 * AFB_MAX_RANKS + p.rank, p.epoch);
            const bool ok = wait_all(p.signals[p.rank], 1, p.world, p.epoch, p.wait_ns);
            if (!ok && atomicCAS(p.status, 0, AFB_ERR_TIMEOUT) == 0) { p.status[1] = 13; p.status[2] = (int)p.rank; p.status[3] = (int)p.epoch; }
        }
    }
}

__global__ void __launch_bounds__(256) cast_f32_bf16_kernel(uint16_t* __restrict__ dst, const float* __restrict__ src, uint32_t rows,
                                                            uint32_t cols, uint32_t ld_dst, uint32_t ld_src) {
    const uint32_t vec_per_row = cols / 8;
    const uint64_t total = (uint64_t)rows * vec_per_row;
    for (uint64_t i = (uint64_t)blockIdx.x * 256 + threadIdx.x; i < total; i += (uint64_t)gridDim.x * 256) {
        const uint32_t r = (uint32_t)(i / vec_per_row), c = (uint32_t)(i % vec_per_row) * 8;
        const float4 a = *reinterpret_cast<const float4*>(src + (size_t)r * ld_src + c);
        const float4 b = *reinterpret_cast<const float4*>(src + (size_t)r * ld_src + c + 4);
        *reinterpret_cast<uint4*>(dst + (size_t)r * ld_dst + c) =
            make_uint4(pack_bf16(a.x, a.y), pack_bf16(a.z, a.w), pack_bf16(b.x, b.y), pack_bf16(b.z, b.w));
    }
}

}  // namespace

}  // namespace afb

using namespace afb;

extern "C" int afb_ksplit_allreduce_launch(const afb_allreduce_args* a, void* stream) {
    if (!a) return AFB_ERR_BAD_ARG;
    if (a->world == 0 || a->world > AFB_MAX_RANKS || a->rank >= a->world) return AFB_ERR_BAD_ARG;
    if (a->m == 0 || a->n == 0 || a->n % 8 || a->ldc % 8 || a->ld_partial % 8 || a->ld_partial < a->n || a->ldc < a->n) return AFB_ERR_BAD_ARG;
    if (a->epoch == 0 || a->reserved != 0) return AFB_ERR_BAD_ARG;
    for (uint32_t q = 0; q < a->world; ++q) {
        if (!a->partial[q] || !a->c[q] || !a->signals[q]) return AFB_ERR_BAD_ARG;
        if ((uintptr_t)a->partial[q] % 16 || (uintptr_t)a->c[q] % 16) return AFB_ERR_BAD_ARG;
    }
    if ((uintptr_t)a->c_multicast % 16) return AFB_ERR_BAD_ARG;
    DeviceCtx* ctx = current_ctx();
    if (!ctx) return AFB_ERR_NOT_INIT;
    ARParams p;
    for (int q = 0; q < AFB_MAX_RANKS; ++q) {
        p.partial[q] = q < (int)a->world ? a->partial[q] : nullptr;
        p.c[q] = q < (int)a->world ? reinterpret_cast<uint16_t*>(a->c[q]) : nullptr;
        p.signals[q] = q < (int)a->world ? a->signals[q] : nullptr;
    }
    p.rank = a->rank; p.world = a->world; p.m = a->m; p.n = a->n; p.ld_partial = a->ld_partial; p.ldc = a->ldc;
    p.partial_f32 = a->partial_f32; p.epoch = a->epoch;
    p.c_multicast = reinterpret_cast<uint16_t*>(a->c_multicast);
    p.wait_ns = (unsigned long long)(a->wait_ms ? a->wait_ms : 2000u) * 1000000ull;
    p.cta_done = ctx->ar_words;          // words 0-1: this kernel
    p.status = ctx->status;
    p.ts = phase_ts_if_enabled(ctx);
    const int grid = ctx->sm_count;   // one CTA per SM: all CTAs are co-resident, so the last-CTA hand-off cannot starve
    if (a->partial_f32) ksplit_allreduce_kernel<true><<<grid, kThreads, 0, (cudaStream_t)stream>>>(p);
    else                ksplit_allreduce_kernel<false><<<grid, kThreads, 0, (cudaStream_t)stream>>>(p);
    count_launch();
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? AFB_OK : cuda_fail(e);
}

extern "C" int afb_cast_f32_to_bf16(void* dst, const void* src, uint32_t rows, uint32_t cols, uint32_t ld_dst, uint32_t ld_src, void* stream) {
    if (!dst || !src || rows == 0 || cols == 0 || cols % 8 || ld_dst % 8 || ld_src % 4) return AFB_ERR_BAD_ARG;
    if ((uintptr_t)dst % 16 || (uintptr_t)src % 16) return AFB_ERR_BAD_ARG;
    if (!current_ctx()) return AFB_ERR_NOT_INIT;
    cast_f32_bf16_kernel<<<592, 256, 0, (cudaStream_t)stream>>>(reinterpret_cast<uint16_t*>(dst), reinterpret_cast<const float*>(src), rows, cols, ld_dst, ld_src);
    count_launch();
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? AFB_OK : cuda_fail(e);
}

// ---- tile-granular exchange -----------------------------------------------------------------------------
extern "C" int afb_ksplit_tile_info(uint32_t m, uint32_t n, uint32_t* tile_m, uint32_t* tile_n, uint32_t* num_tiles, uint32_t* arrivals) {
    if (!tile_m || !tile_n || !num_tiles || !arrivals || m == 0 || n == 0) return AFB_ERR_BAD_ARG;
    uint32_t mt, nt;
    prefill_ts_tile_info(m, n, tile_m, tile_n, &mt, &nt, arrivals);
    *num_tiles = mt * nt;
    return AFB_OK;
}

extern "C" int afb_gemm_launch_tiles(const afb_gemm_args* args, uint32_t* tile_done, void* stream) {
    if (!args || !tile_done || !args->ptr_a || !args->ptr_b || !args->ptr_c || !args->ptr_scale) return AFB_ERR_BAD_ARG;
    if (args->m == 0 || args->n == 0 || args->k == 0 || args->reserved != 0) return AFB_ERR_BAD_ARG;
    if (args->lda < args->k || args->ldc < args->n || args->ldb < args->k || args->b_layout == AFB_LAYOUT_ROW || args->b_layout > 2) return AFB_ERR_BAD_ARG;
    if (!(args->flags & AFB_FLAG_C_F32)) return AFB_ERR_UNSUPPORTED;   // the partial sums travel as fp32
    DeviceCtx* ctx = current_ctx();
    if (!ctx) return AFB_ERR_NOT_INIT;
    return launch_prefill_ts_tiles(*args, ctx, tile_done, (cudaStream_t)stream);
}

extern "C" int afb_abi_sizes(uint32_t sizes[4]) {
    if (!sizes) return AFB_ERR_BAD_ARG;
    sizes[0] = (uint32_t)sizeof(afb_gemm_args);
    sizes[1] = (uint32_t)sizeof(afb_allreduce_args);
    sizes[2] = (uint32_t)sizeof(afb_tile_allreduce_args);
    sizes[3] = (uint32_t)sizeof(afb_fused_args);
    return AFB_OK;
}

extern "C" int afb_gemm_launch_push(const afb_gemm_args* args, void* const stage[AFB_MAX_RANKS], uint32_t world, uint32_t rank, void* stream) {
    if (!args || !stage || !args->ptr_a || !args->ptr_b || !args->ptr_scale) return AFB_ERR_BAD_ARG;
    if (args->m == 0 || args->n == 0 || args->k == 0 || args->reserved != 0) return AFB_ERR_BAD_ARG;
    if (args->lda < args->k || args->ldb < args->k || args->b_layout == AFB_LAYOUT_ROW || args->b_layout > 2) return AFB_ERR_BAD_ARG;
    if (!(args->flags & AFB_FLAG_C_F32)) return AFB_ERR_UNSUPPORTED;   // the partial sums travel as fp32
    if (world == 0 || world > AFB_MAX_RANKS || rank >= world) return AFB_ERR_BAD_ARG;
    for (uint32_t q = 0; q < world; ++q) if (!stage[q] || (uintptr_t)stage[q] % 16) return AFB_ERR_BAD_ARG;
    DeviceCtx* ctx = current_ctx();
    if (!ctx) return AFB_ERR_NOT_INIT;
    afb_gemm_args a = *args;
    if (a.flags & AFB_FLAG_PUSH_VIA_LOCAL) {
        if (!a.ptr_c || (uintptr_t)a.ptr_c % 16 || a.ldc != a.n || a.n % 4) return AFB_ERR_BAD_ARG;   // local fp32 [M,N] scratch
    } else {
        a.ptr_c = stage[rank];   // never written in this mode; keeps the common validation happy
        a.ldc = a.n;
    }
    return launch_prefill_ts_push(a, ctx, stage, world, rank, (cudaStream_t)stream);
}

extern "C" int afb_gemm_launch_push_pipelined(const afb_gemm_args* args, void* const stage[AFB_MAX_RANKS], uint32_t* const counters[AFB_MAX_RANKS],
                                              uint32_t world, uint32_t rank, uint32_t sub_blocks, void* stream) {
    if (!args || !stage || !counters || !args->ptr_a || !args->ptr_b || !args->ptr_scale) return AFB_ERR_BAD_ARG;
    if (args->m == 0 || args->n == 0 || args->k == 0 || args->reserved != 0) return AFB_ERR_BAD_ARG;
    if (args->lda < args->k || args->ldb < args->k || args->b_layout == AFB_LAYOUT_ROW || args->b_layout > 2) return AFB_ERR_BAD_ARG;
    if (!(args->flags & AFB_FLAG_C_F32)) return AFB_ERR_UNSUPPORTED;   // the partial sums travel as fp32
    if (world == 0 || world > AFB_MAX_RANKS || rank >= world || sub_blocks == 0) return AFB_ERR_BAD_ARG;
    for (uint32_t q = 0; q < world; ++q) if (!stage[q] || (uintptr_t)stage[q] % 16 || !counters[q]) return AFB_ERR_BAD_ARG;
    DeviceCtx* ctx = current_ctx();
    if (!ctx) return AFB_ERR_NOT_INIT;
    afb_gemm_args a = *args;
    a.ptr_c = stage[rank];   // never written in this mode; keeps the common validation happy
    a.ldc = a.n;
    return launch_prefill_ts_push(a, ctx, stage, world, rank, (cudaStream_t)stream, counters, sub_blocks);
}

// The pipelined reduce-scatter in ONE launch: the pushing GEMM of afb_gemm_launch_push_pipelined plus two extra warps per CTA that
// do what afb_ksplit_sub_allreduce_launch does (x describes it exactly as for that entry point).
extern "C" int afb_gemm_launch_push_exchange(const afb_gemm_args* args, void* const stage[AFB_MAX_RANKS], uint32_t* const counters[AFB_MAX_RANKS],
                                             uint32_t world, uint32_t rank, uint32_t sub_blocks, const afb_sub_allreduce_args* sa, void* stream) {
    if (!args || !stage || !counters || !sa || !args->ptr_a || !args->ptr_b || !args->ptr_scale) return AFB_ERR_BAD_ARG;
    if (args->m == 0 || args->n == 0 || args->k == 0 || args->reserved != 0) return AFB_ERR_BAD_ARG;
    if (args->lda < args->k || args->ldb < args->k || args->b_layout == AFB_LAYOUT_ROW || args->b_layout > 2) return AFB_ERR_BAD_ARG;
    if (!(args->flags & AFB_FLAG_C_F32)) return AFB_ERR_UNSUPPORTED;   // the partial sums travel as fp32
    if (world == 0 || world > AFB_MAX_RANKS || rank >= world || sub_blocks == 0) return AFB_ERR_BAD_ARG;
    for (uint32_t q = 0; q < world; ++q) if (!stage[q] || (uintptr_t)stage[q] % 16 || !counters[q]) return AFB_ERR_BAD_ARG;
    const afb_allreduce_args* x = &sa->base;
    if (x->world != world || x->rank != rank || x->m != args->m || x->n != args->n || x->ldc % 8 || x->ldc < x->n) return AFB_ERR_BAD_ARG;
    if (x->epoch == 0 || x->reserved != 0 || !x->partial_f32 || sa->counters != counters[rank] || sa->sub_blocks != sub_blocks || sa->launches == 0 || sa->reserved != 0)
        return AFB_ERR_BAD_ARG;
    uint32_t per_chunk = 0;
    if (afb_ksplit_sub_info(x->m, x->n, world, sub_blocks, &per_chunk) != AFB_OK) return AFB_ERR_UNSUPPORTED;
    for (uint32_t q = 0; q < world; ++q) if (!x->c[q] || (uintptr_t)x->c[q] % 16 || !x->signals[q]) return AFB_ERR_BAD_ARG;
    if ((uintptr_t)x->c_multicast % 16) return AFB_ERR_BAD_ARG;
    DeviceCtx* ctx = current_ctx();
    if (!ctx) return AFB_ERR_NOT_INIT;
    PushExchange px = {};
    for (uint32_t q = 0; q < world; ++q) { px.c[q] = reinterpret_cast<uint16_t*>(x->c[q]); px.signals[q] = x->signals[q]; }
    px.c_multicast = reinterpret_cast<uint16_t*>(x->c_multicast);
    px.counters = sa->counters;
    px.ldc = x->ldc; px.epoch = x->epoch; px.want = per_chunk * sa->launches;
    px.wait_ns = (unsigned long long)(x->wait_ms ? x->wait_ms : 2000u) * 1000000ull;
    px.cta_done = ctx->ar_words + 2;   // the pair of the exchange kernels that run next to a GEMM: one form at a time
    afb_gemm_args a = *args;
    a.ptr_c = stage[rank];   // never written in this mode; keeps the common validation happy
    a.ldc = a.n;
    return launch_prefill_ts_push(a, ctx, stage, world, rank, (cudaStream_t)stream, counters, sub_blocks, &px);
}

extern "C" int afb_ksplit_sub_info(uint32_t m, uint32_t n, uint32_t world, uint32_t sub_blocks, uint32_t* counts_per_chunk) {
    if (!counts_per_chunk || world == 0 || sub_blocks == 0 || m % (256 * world) || n % (BNW_TILE * sub_blocks)) return AFB_ERR_BAD_ARG;
    uint32_t tm, tn, mt, nt, arr;
    prefill_ts_tile_info(m, n, &tm, &tn, &mt, &nt, &arr);
    *counts_per_chunk = (mt / world) * (nt / sub_blocks) * world * arr;   // tiles of a chunk of one owner's rows x ranks x counts per tile
    return AFB_OK;
}

extern "C" int afb_ksplit_sub_allreduce_launch(const afb_sub_allreduce_args* sa, void* stream) {
    if (!sa) return AFB_ERR_BAD_ARG;
    const afb_allreduce_args* a = &sa->base;
    if (a->world == 0 || a->world > AFB_MAX_RANKS || a->rank >= a->world) return AFB_ERR_BAD_ARG;
    if (a->m == 0 || a->n == 0 || a->ldc % 8 || a->ld_partial % 8 || a->ld_partial < a->n || a->ldc < a->n) return AFB_ERR_BAD_ARG;
    if (a->epoch == 0 || a->reserved != 0 || !a->partial_f32 || !sa->counters || sa->sub_blocks == 0 || sa->launches == 0 || sa->reserved != 0) return AFB_ERR_BAD_ARG;
    uint32_t per_chunk = 0;
    if (afb_ksplit_sub_info(a->m, a->n, a->world, sa->sub_blocks, &per_chunk) != AFB_OK) return AFB_ERR_UNSUPPORTED;
    for (uint32_t q = 0; q < a->world; ++q) {
        if (!a->partial[q] || !a->c[q] || !a->signals[q]) return AFB_ERR_BAD_ARG;
        if ((uintptr_t)a->partial[q] % 16 || (uintptr_t)a->c[q] % 16) return AFB_ERR_BAD_ARG;
    }
    if ((uintptr_t)a->c_multicast % 16) return AFB_ERR_BAD_ARG;
    DeviceCtx* ctx = current_ctx();
    if (!ctx) return AFB_ERR_NOT_INIT;
    SubARParams sp;
    ARParams& p = sp.ar;
    for (int q = 0; q < AFB_MAX_RANKS; ++q) {
        const bool on = q < (int)a->world;
        p.partial[q] = on ? a->partial[q] : nullptr;
        p.c[q] = on ? reinterpret_cast<uint16_t*>(a->c[q]) : nullptr;
        p.signals[q] = on ? a->signals[q] : nullptr;
    }
    p.rank = a->rank; p.world = a->world; p.m = a->m; p.n = a->n; p.ld_partial = a->ld_partial; p.ldc = a->ldc;
    p.partial_f32 = 1; p.epoch = a->epoch;
    p.c_multicast = reinterpret_cast<uint16_t*>(a->c_multicast);
    p.wait_ns = (unsigned long long)(a->wait_ms ? a->wait_ms : 2000u) * 1000000ull;
    p.cta_done = ctx->ar_words + 2;      // shares the pair of the tile-granular kernel: the two forms are never used together
    p.status = ctx->status;
    p.ts = phase_ts_if_enabled(ctx);
    sp.counters = sa->counters; sp.sub_blocks = sa->sub_blocks; sp.want = per_chunk * sa->launches;
    // This kernel runs on SMs of its own: the pushing GEMM leaves sub_allreduce_sms() SMs free, and this kernel is as many CTAs
    // of 768 threads, each asking for most of an SM's shared memory (which it does not use): one CTA per SM, none fits next to a
    // CTA of the GEMM, and whichever kernel reaches the GPU first, the other still finds the SMs it needs (a CTA of this kernel
    // that sat on an SM the GEMM needs would wait for tiles that cannot be computed).  Next to one it cost the GEMM a factor 1.7 (measured on 2 GPUs, whatever it did there: polling, sleeping or
    // summing), and with the GEMM's static tile assignment one slowed CTA is the whole GEMM.
    constexpr int kThreads = 768, kSmemPerCta = 200 * 1024;
    static DeviceOnce carveout_set;
    if (!carveout_set.done(ctx->device)) {
        cudaError_t e = cudaFuncSetAttribute(ksplit_sub_allreduce_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(ksplit_sub_allreduce_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemPerCta);
        if (e != cudaSuccess) return cuda_fail(e);
        carveout_set.mark(ctx->device);
    }
    ksplit_sub_allreduce_kernel<<<sub_allreduce_sms(), kThreads, kSmemPerCta, (cudaStream_t)stream>>>(sp);
    count_launch();
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? AFB_OK : cuda_fail(e);
}

namespace afb {
uint32_t sub_allreduce_sms() {
    static const uint32_t n = [] { const char* e = getenv("AFB_SUB_AR_SMS"); const int v = e ? atoi(e) : 0; return (v >= 1 && v <= 64) ? (uint32_t)v : 16u; }();
    return n;
}
}  // namespace afb

extern "C" int afb_ksplit_tile_allreduce_launch(const afb_tile_allreduce_args* ta, void* stream) {
    if (!ta) return AFB_ERR_BAD_ARG;
    const afb_allreduce_args* a = &ta->base;
    if (a->world == 0 || a->world > AFB_MAX_RANKS || a->rank >= a->world) return AFB_ERR_BAD_ARG;
    if (a->m == 0 || a->n == 0 || a->n % 8 || a->ldc % 8 || a->ld_partial % 8 || a->ld_partial < a->n || a->ldc < a->n) return AFB_ERR_BAD_ARG;
    if (a->epoch == 0 || a->reserved != 0 || !a->partial_f32 || ta->tile_epoch == 0 || ta->reserved != 0) return AFB_ERR_BAD_ARG;
    uint32_t tm, tn, mt, nt, arr;
    prefill_ts_tile_info(a->m, a->n, &tm, &tn, &mt, &nt, &arr);
    for (uint32_t q = 0; q < a->world; ++q) {
        if (!a->partial[q] || !a->c[q] || !a->signals[q] || !ta->tile_done[q]) return AFB_ERR_BAD_ARG;
        if ((uintptr_t)a->partial[q] % 16 || (uintptr_t)a->c[q] % 16) return AFB_ERR_BAD_ARG;
    }
    DeviceCtx* ctx = current_ctx();
    if (!ctx) return AFB_ERR_NOT_INIT;
    TileARParams tp;
    ARParams& p = tp.ar;
    for (int q = 0; q < AFB_MAX_RANKS; ++q) {
        const bool on = q < (int)a->world;
        p.partial[q] = on ? a->partial[q] : nullptr;
        p.c[q] = on ? reinterpret_cast<uint16_t*>(a->c[q]) : nullptr;
        p.signals[q] = on ? a->signals[q] : nullptr;
        tp.tile_done[q] = on ? ta->tile_done[q] : nullptr;
    }
    p.rank = a->rank; p.world = a->world; p.m = a->m; p.n = a->n; p.ld_partial = a->ld_partial; p.ldc = a->ldc;
    p.partial_f32 = 1; p.epoch = a->epoch;
    p.c_multicast = nullptr;   // the tile-granular form stores to each peer
    p.wait_ns = (unsigned long long)(a->wait_ms ? a->wait_ms : 2000u) * 1000000ull;
    p.cta_done = ctx->ar_words + 2;      // words 2-3: the tile-granular kernel may overlap the plain one
    p.status = ctx->status;
    p.ts = nullptr;
    tp.tile_m = tm; tp.tile_n = tn; tp.m_tiles = mt; tp.n_tiles = nt; tp.arrivals = arr; tp.tile_epoch = ta->tile_epoch;
    // One CTA per SM next to the GEMM's CTA (256 threads, no dynamic shared memory, <= 128 registers per thread).
    // The GEMM needs the SM's largest shared-memory carve-out; an SM cannot change its carve-out while a CTA is resident,
    // so this kernel asks for the same carve-out: whichever of the two reaches an SM first, the other can join it.
    static DeviceOnce carveout_set;
    if (!carveout_set.done(ctx->device)) {
        cudaError_t e = cudaFuncSetAttribute(ksplit_tile_allreduce_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        if (e != cudaSuccess) return cuda_fail(e);
        carveout_set.mark(ctx->device);
    }
    // Few threads on purpose: the pulls are long-latency NVLink loads; a full-size CTA keeps so many of them in flight that the
    // SM's load/store path backs up and the GEMM's own shared-memory reads queue behind them (measured: the GEMM ran 2.3x slower).
    static const int threads = [] { const char* e = getenv("AFB_TILE_AR_THREADS"); const int v = e ? atoi(e) : 0; return (v == 32 || v == 64 || v == 128 || v == 256) ? v : kTileThreadsDefault; }();
    ksplit_tile_allreduce_kernel<<<ctx->sm_count, threads, 0, (cudaStream_t)stream>>>(tp);
    count_launch();
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? AFB_OK : cuda_fail(e);
}
