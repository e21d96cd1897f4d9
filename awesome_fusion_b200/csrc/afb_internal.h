// Internal declarations shared by the translation units of libafb.so.
#pragma once
#include <cuda_runtime.h>
#include <cuda.h>
#include <stdint.h>
#include <atomic>
#include "afb_capi.h"

namespace afb {

// Per-device state created by afb_init.
struct DeviceCtx {
    bool     ready = false;
    int      device = -1;
    int      sm_count = 0;
    int32_t* status = nullptr;        // device int32[4]: {code, where, a, b}
    // Split-K workspaces (fp32 partial sums + arrival counters, used by decode K-slices, the balanced decode form and the
    // prefill tail split): one per stream that has launched such a GEMM, so that launches on different streams never share
    // one.  Slot 0 is allocated by afb_init, the others on a stream's first launch (outside any stream capture).
    static constexpr int kMaxWorkspaces = 16;
    struct Workspace {
        bool          assigned = false;
        cudaStream_t  stream = nullptr;
        float*        ws = nullptr;
        uint32_t*     counters = nullptr;
    };
    Workspace workspaces[kMaxWorkspaces];
    size_t    splitk_ws_bytes = 0;        // size of every workspace
    size_t    splitk_counter_count = 0;   // counters of every workspace
    // optional phase timestamps (globaltimer ns of THIS GPU) written by the row-parallel GEMM and the exchange kernel when the
    // environment variable AFB_PHASE_TIMESTAMPS is set: [0] GEMM start, [1] GEMM end (latest CTA), [2] exchange start,
    // [3] all ranks' GEMMs seen complete, [4] sum + broadcast done (latest CTA), [5] all ranks' blocks seen in place
    unsigned long long* phase_ts = nullptr;
    uint32_t* ar_words = nullptr;         // device uint32[4]: hand-off words of the two exchange kernels (CTAs finished, any failed)
    // staging for afb_gemm_host (grow-only): two sets used in turn, so that the copies of one call overlap the other call's
    void*  stage[2][4] = {};
    size_t stage_bytes[2][4] = {};
    cudaEvent_t stage_free[2] = {};      // recorded when a call is done with its set
    unsigned host_calls = 0;
    // copy-in / copy-out streams and per-chunk events of the pipelined afb_gemm_host
    cudaStream_t host_in = nullptr, host_out = nullptr;
    cudaEvent_t host_ev[2 * 16 + 2] = {};
};

// "Done once per device" for function-local statics (kernel attributes, occupancy queries).  One bit per device; what it
// guards is idempotent, so two host threads that both find the bit clear simply both do the work.
struct DeviceOnce {
    std::atomic<uint32_t> mask{0};
    bool done(int dev) const { return (mask.load(std::memory_order_acquire) >> (dev & 31)) & 1u; }
    void mark(int dev) { mask.fetch_or(1u << (dev & 31), std::memory_order_release); }
};

unsigned long long* phase_ts_if_enabled(DeviceCtx* ctx);   // ctx->phase_ts when AFB_PHASE_TIMESTAMPS is set, else nullptr

DeviceCtx* current_ctx();           // nullptr when afb_init was not called on the current device
// The split-K workspace of `s` on this device (allocates it on the stream's first use); nullptr + *rc on failure.
const DeviceCtx::Workspace* workspace_for(DeviceCtx* ctx, cudaStream_t s, int* rc);
int  cuda_fail(cudaError_t e);      // records e, returns AFB_ERR_CUDA
void count_launch(unsigned n = 1);

// Driver entry point for tensor-map encoding, fetched once through the runtime.
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_tiled_fn();

// Launchers (each validates what only it can know and returns an AFB status).
int launch_naive(const afb_gemm_args& a, DeviceCtx* ctx, cudaStream_t s);
int launch_decode(const afb_gemm_args& a, DeviceCtx* ctx, cudaStream_t s);
int launch_decode_ws(const afb_gemm_args& a, DeviceCtx* ctx, float* ws, size_t ws_bytes, uint32_t* counters,
                     size_t counter_count, cudaStream_t s);
int launch_prefill(const afb_gemm_args& a, DeviceCtx* ctx, cudaStream_t s);      // converted weights through shared memory
// SMs the pushing GEMM of the pipelined reduce-scatter leaves free for the kernel that sums and broadcasts next to it
// (environment variable AFB_SUB_AR_SMS, default 16: on 2 GPUs 1.03 ms for the down-projection with 16, 1.13 with 8)
uint32_t sub_allreduce_sms();
int launch_prefill_ts(const afb_gemm_args& a, DeviceCtx* ctx, cudaStream_t s, const afb_fused_args* fused = nullptr);   // converted weights in tensor memory
int launch_prefill_ts_tiles(const afb_gemm_args& a, DeviceCtx* ctx, uint32_t* tile_done, cudaStream_t s);
// The sum and broadcast of the pipelined reduce-scatter done inside the pushing GEMM, by two extra warps of every CTA (so that no
// second kernel has to share SMs with the GEMM): where the finished rows go, the words of the closing signal round, the count
// every chunk counter of this rank has to reach.
struct PushExchange {
    uint16_t* c[AFB_MAX_RANKS];
    uint16_t* c_multicast;
    uint32_t* signals[AFB_MAX_RANKS];
    const uint32_t* counters;     // this rank's per-chunk counters
    uint32_t ldc, epoch, want;
    unsigned long long wait_ns;
    uint32_t* cta_done;           // device uint32[2]: warps finished, any failed (zero between launches)
};
int launch_prefill_ts_push(const afb_gemm_args& a, DeviceCtx* ctx, void* const* stage, uint32_t world, uint32_t rank, cudaStream_t s,
                           uint32_t* const* counters = nullptr, uint32_t sub_blocks = 0, const PushExchange* x = nullptr);
void prefill_ts_tile_info(uint32_t m, uint32_t n, uint32_t* tile_m, uint32_t* tile_n, uint32_t* m_tiles, uint32_t* n_tiles, uint32_t* arrivals);
int launch_probe(uint32_t kind, const void* src, size_t bytes, uint32_t ctas, uint32_t smem_bytes, bool pdl, uint32_t* sink, cudaStream_t s);
int launch_dequant_dump(const afb_gemm_args& a, void* out, cudaStream_t s);

bool decode_supports(const afb_gemm_args& a);
bool prefill_supports(const afb_gemm_args& a);
bool prefill_needs_ts(const afb_gemm_args& a);   // groups of 32 or zero-points: only the tensor-memory form

}  // namespace afb
