// Internal declarations shared by the translation units of libafb.so.
#pragma once
#include <cuda_runtime.h>
#include <cuda.h>
#include <stdint.h>
#include "afb_capi.h"

namespace afb {

// Per-device state created by afb_init.
struct DeviceCtx {
    bool     ready = false;
    int      device = -1;
    int      sm_count = 0;
    int32_t* status = nullptr;        // device int32[4]: {code, where, a, b}
    // split-K workspace of the decode kernel: fp32 partial sums + per-row-block arrival counters
    float*    splitk_ws = nullptr;
    size_t    splitk_ws_bytes = 0;
    uint32_t* splitk_counters = nullptr;
    size_t    splitk_counter_count = 0;
    // staging for afb_gemm_host (grow-only)
    void*  stage[4] = {nullptr, nullptr, nullptr, nullptr};
    size_t stage_bytes[4] = {0, 0, 0, 0};
    // copy-in / copy-out streams and per-chunk events of the pipelined afb_gemm_host
    cudaStream_t host_in = nullptr, host_out = nullptr;
    cudaEvent_t host_ev[2 * 16 + 2] = {};
};

DeviceCtx* current_ctx();           // nullptr when afb_init was not called on the current device
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
int launch_prefill_ts(const afb_gemm_args& a, DeviceCtx* ctx, cudaStream_t s);   // converted weights in tensor memory
int launch_prefill_ts_tiles(const afb_gemm_args& a, DeviceCtx* ctx, uint32_t* tile_done, cudaStream_t s);
int launch_prefill_ts_push(const afb_gemm_args& a, DeviceCtx* ctx, void* const* stage, uint32_t world, uint32_t rank, cudaStream_t s);
void prefill_ts_tile_info(uint32_t m, uint32_t n, uint32_t* tile_m, uint32_t* tile_n, uint32_t* m_tiles, uint32_t* n_tiles, uint32_t* arrivals);
int launch_dequant_dump(const afb_gemm_args& a, void* out, cudaStream_t s);

bool decode_supports(const afb_gemm_args& a);
bool prefill_supports(const afb_gemm_args& a);

}  // namespace afb
