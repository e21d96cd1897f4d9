// extern "C" layer of libafb.so: argument validation, variant selection, device context,
// and the memory / event / stream helpers that mirror the HIP calls of the reference
// driver (bfAintBGemm.cc:60-66,99-101,148-186; simple_device_mem.hpp:20,25).
#include <atomic>
#include <mutex>
#include <cstring>
#include <cstdlib>
#include "afb_internal.h"

namespace afb {

namespace {
constexpr int kMaxDevices = 32;
DeviceCtx g_ctx[kMaxDevices];
std::mutex g_mutex;
std::atomic<int> g_last_cuda_error{0};
std::atomic<unsigned long long> g_launches{0};
constexpr size_t kSplitKWorkspaceBytes = 32u << 20;
constexpr size_t kSplitKCounters = 4096;
constexpr int kPreallocatedWorkspaces = 4;
constexpr uint32_t kPrefillTsMinM = 128;   // measured: above 128 activation rows the tensor-memory form is 1.3x faster, at 128 it is slower
}  // namespace

int cuda_fail(cudaError_t e) {
    g_last_cuda_error.store((int)e);
    (void)cudaGetLastError();  // clear the sticky-free error state
    return AFB_ERR_CUDA;
}
void count_launch(unsigned n) { g_launches.fetch_add(n); }

DeviceCtx* current_ctx() {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
    return g_ctx[dev].ready ? &g_ctx[dev] : nullptr;
}

unsigned long long* phase_ts_if_enabled(DeviceCtx* ctx) {
    static const bool on = getenv("AFB_PHASE_TIMESTAMPS") != nullptr;
    return on ? ctx->phase_ts : nullptr;
}

const DeviceCtx::Workspace* workspace_for(DeviceCtx* ctx, cudaStream_t s, int* rc) {
    std::lock_guard<std::mutex> lock(g_mutex);
    DeviceCtx::Workspace* free_slot = nullptr;
    for (auto& w : ctx->workspaces) {
        if (w.assigned && w.stream == s) return &w;
        if (!w.assigned && (!free_slot || (w.ws && !free_slot->ws))) free_slot = &w;   // an unassigned slot that already has memory first
    }
    if (!free_slot) { *rc = AFB_ERR_TOO_LARGE; return nullptr; }   // more streams than workspaces
    if (!free_slot->ws) {
        cudaError_t e = cudaMalloc(&free_slot->ws, ctx->splitk_ws_bytes);
        if (e == cudaSuccess) e = cudaMalloc(&free_slot->counters, ctx->splitk_counter_count * sizeof(uint32_t));
        if (e == cudaSuccess) e = cudaMemset(free_slot->counters, 0, ctx->splitk_counter_count * sizeof(uint32_t));
        if (e != cudaSuccess) {
            if (free_slot->ws) cudaFree(free_slot->ws);
            if (free_slot->counters) cudaFree(free_slot->counters);
            free_slot->ws = nullptr; free_slot->counters = nullptr;
            *rc = cuda_fail(e);
            return nullptr;
        }
    }
    free_slot->assigned = true;
    free_slot->stream = s;
    return free_slot;
}

EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    });
    return fn;
}

// n_out: columns of C (differs from a->n, the rows of B, only for the gated fused launch)
static int validate(const afb_gemm_args* a, uint32_t n_out = 0) {
    if (!a) return AFB_ERR_BAD_ARG;
    if (n_out == 0) n_out = a->n;
    if (!a->ptr_a || !a->ptr_b || !a->ptr_c || !a->ptr_scale) return AFB_ERR_BAD_ARG;
    if (a->m == 0 || a->n == 0 || a->k == 0) return AFB_ERR_BAD_ARG;
    if (a->reserved != 0 || a->reserved2 != 0) return AFB_ERR_BAD_ARG;
    if (a->b_bits != 8 && a->b_bits != 4) return AFB_ERR_BAD_ARG;
    if (a->b_encoding > 1 || a->b_layout > 2 || a->scale_dtype > 1 || a->variant > 3) return AFB_ERR_BAD_ARG;
    if (a->flags & ~(AFB_FLAG_C_F32 | AFB_FLAG_PREFILL_SMEM_B | AFB_FLAG_PREFILL_TMEM_A | AFB_FLAG_GROUP_EXACT | AFB_FLAG_PDL)) return AFB_ERR_BAD_ARG;
    if ((a->flags & AFB_FLAG_GROUP_EXACT) && (a->flags & AFB_FLAG_PREFILL_SMEM_B) && a->group_size) return AFB_ERR_UNSUPPORTED;   // only the tensor-memory form has it
    if (a->lda < a->k || a->ldc < n_out) return AFB_ERR_BAD_ARG;
    if (a->b_layout != AFB_LAYOUT_ROW ? a->ldb < a->k : a->ldb < a->n) return AFB_ERR_BAD_ARG;
    if (a->b_bits == 4 && (a->b_layout == AFB_LAYOUT_ROW || (a->k & 1) || (a->ldb & 1))) return AFB_ERR_UNSUPPORTED;
    if (a->b_layout == AFB_LAYOUT_COL_PACKED && a->k % (a->b_bits == 8 ? 4u : 8u)) return AFB_ERR_BAD_ARG;   // whole words
    if (a->group_size && (a->k % a->group_size)) return AFB_ERR_BAD_ARG;
    // element alignment of what the kernels load and store as 2- or 4-byte words (a misaligned pointer would fault on the GPU)
    if ((uintptr_t)a->ptr_scale % (a->scale_dtype == AFB_SCALE_BF16 ? 2 : 4)) return AFB_ERR_BAD_ARG;
    if ((uintptr_t)a->ptr_c % ((a->flags & AFB_FLAG_C_F32) ? 4 : 2) || (uintptr_t)a->ptr_a % 2) return AFB_ERR_BAD_ARG;
    return AFB_OK;
}

static int resolve(const afb_gemm_args& a, uint32_t* out) {
    uint32_t v = a.variant;
    if (a.flags & AFB_FLAG_C_F32) {  // fp32 output: the prefill variant (K-split partial sums) or the naive variant
        if (v == AFB_VARIANT_DECODE) return AFB_ERR_UNSUPPORTED;
        if (v == AFB_VARIANT_AUTO) v = (a.m > 16 && prefill_supports(a)) ? AFB_VARIANT_PREFILL : AFB_VARIANT_NAIVE;
    }
    if (v == AFB_VARIANT_AUTO) {
        if (a.m <= 16 && decode_supports(a)) v = AFB_VARIANT_DECODE;
        else if (prefill_supports(a)) v = AFB_VARIANT_PREFILL;
        else v = AFB_VARIANT_NAIVE;
    } else if (v == AFB_VARIANT_DECODE) {
        if (!decode_supports(a)) return AFB_ERR_UNSUPPORTED;
    } else if (v == AFB_VARIANT_PREFILL) {
        if (!prefill_supports(a)) return AFB_ERR_UNSUPPORTED;
    }
    *out = v;
    return AFB_OK;
}

}  // namespace afb

using namespace afb;

#define AFB_CUDA(call)                                  \
    do {                                                \
        cudaError_t e__ = (call);                       \
        if (e__ != cudaSuccess) return cuda_fail(e__);  \
    } while (0)

extern "C" {

int afb_init(int device) {
    if (device < 0 || device >= kMaxDevices) return AFB_ERR_BAD_ARG;
    AFB_CUDA(cudaSetDevice(device));
    std::lock_guard<std::mutex> lock(g_mutex);
    DeviceCtx& c = g_ctx[device];
    if (c.ready) return AFB_OK;
    cudaDeviceProp prop;
    AFB_CUDA(cudaGetDeviceProperties(&prop, device));
    if (prop.major != 10) return AFB_ERR_UNSUPPORTED;  // the kernels are sm_100a only; no fallback
    c.device = device;
    c.sm_count = prop.multiProcessorCount;
    AFB_CUDA(cudaMalloc(&c.status, 4 * sizeof(int32_t)));
    AFB_CUDA(cudaMemset(c.status, 0, 4 * sizeof(int32_t)));
    c.splitk_ws_bytes = kSplitKWorkspaceBytes;
    c.splitk_counter_count = kSplitKCounters;
    // the first few workspaces exist from the start, so that a stream's first launch may also happen inside a stream capture
    // (frameworks capture on a fresh stream); further streams allocate theirs on first use, outside capture
    for (int i = 0; i < kPreallocatedWorkspaces; ++i) {
        AFB_CUDA(cudaMalloc(&c.workspaces[i].ws, kSplitKWorkspaceBytes));
        AFB_CUDA(cudaMalloc(&c.workspaces[i].counters, kSplitKCounters * sizeof(uint32_t)));
        AFB_CUDA(cudaMemset(c.workspaces[i].counters, 0, kSplitKCounters * sizeof(uint32_t)));
    }
    AFB_CUDA(cudaMalloc(&c.phase_ts, 8 * sizeof(unsigned long long)));
    AFB_CUDA(cudaMemset(c.phase_ts, 0, 8 * sizeof(unsigned long long)));
    AFB_CUDA(cudaMalloc(&c.ar_words, 4 * sizeof(uint32_t)));
    AFB_CUDA(cudaMemset(c.ar_words, 0, 4 * sizeof(uint32_t)));
    AFB_CUDA(cudaDeviceSynchronize());
    c.ready = true;
    return AFB_OK;
}

int afb_finalize(void) {
    int dev = -1;
    AFB_CUDA(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> lock(g_mutex);
    DeviceCtx& c = g_ctx[dev];
    if (!c.ready) return AFB_OK;
    cudaDeviceSynchronize();
    cudaFree(c.status); cudaFree(c.ar_words); cudaFree(c.phase_ts);
    for (auto& w : c.workspaces) { if (w.ws) cudaFree(w.ws); if (w.counters) cudaFree(w.counters); }
    for (int j = 0; j < 2; ++j) {
        for (int i = 0; i < 4; ++i) if (c.stage[j][i]) cudaFree(c.stage[j][i]);
        if (c.stage_free[j]) cudaEventDestroy(c.stage_free[j]);
    }
    if (c.host_in) {
        cudaStreamDestroy(c.host_in); cudaStreamDestroy(c.host_out);
        for (auto& e : c.host_ev) if (e) cudaEventDestroy(e);
    }
    c = DeviceCtx();
    return AFB_OK;
}

int afb_device_count(int* count) {
    if (!count) return AFB_ERR_BAD_ARG;
    AFB_CUDA(cudaGetDeviceCount(count));
    return AFB_OK;
}
int afb_sm_count(int* count) {
    DeviceCtx* c = current_ctx();
    if (!c) return AFB_ERR_NOT_INIT;
    if (!count) return AFB_ERR_BAD_ARG;
    *count = c->sm_count;
    return AFB_OK;
}

int afb_malloc(void** ptr, size_t bytes) {
    if (!ptr) return AFB_ERR_BAD_ARG;
    AFB_CUDA(cudaMalloc(ptr, bytes ? bytes : 1));
    return AFB_OK;
}
int afb_free(void* ptr) { AFB_CUDA(cudaFree(ptr)); return AFB_OK; }
int afb_malloc_host(void** ptr, size_t bytes) {
    if (!ptr) return AFB_ERR_BAD_ARG;
    AFB_CUDA(cudaMallocHost(ptr, bytes ? bytes : 1));
    return AFB_OK;
}
int afb_free_host(void* ptr) { AFB_CUDA(cudaFreeHost(ptr)); return AFB_OK; }
int afb_memcpy_h2d(void* dst, const void* src, size_t bytes) { AFB_CUDA(cudaMemcpy(dst, src, bytes, cudaMemcpyHostToDevice)); return AFB_OK; }
int afb_memcpy_d2h(void* dst, const void* src, size_t bytes) { AFB_CUDA(cudaMemcpy(dst, src, bytes, cudaMemcpyDeviceToHost)); return AFB_OK; }
int afb_memcpy_d2d(void* dst, const void* src, size_t bytes) { AFB_CUDA(cudaMemcpy(dst, src, bytes, cudaMemcpyDeviceToDevice)); return AFB_OK; }
int afb_memset(void* dst, int value, size_t bytes) { AFB_CUDA(cudaMemset(dst, value, bytes)); return AFB_OK; }

int afb_event_create(void** event) {
    if (!event) return AFB_ERR_BAD_ARG;
    cudaEvent_t e;
    AFB_CUDA(cudaEventCreate(&e));
    *event = e;
    return AFB_OK;
}
int afb_event_record(void* event, void* stream) { AFB_CUDA(cudaEventRecord((cudaEvent_t)event, (cudaStream_t)stream)); return AFB_OK; }
int afb_event_sync(void* event) { AFB_CUDA(cudaEventSynchronize((cudaEvent_t)event)); return AFB_OK; }
int afb_event_elapsed_ms(float* ms, void* start, void* stop) {
    if (!ms) return AFB_ERR_BAD_ARG;
    AFB_CUDA(cudaEventElapsedTime(ms, (cudaEvent_t)start, (cudaEvent_t)stop));
    return AFB_OK;
}
int afb_event_destroy(void* event) { AFB_CUDA(cudaEventDestroy((cudaEvent_t)event)); return AFB_OK; }
int afb_stream_create(void** stream) {
    if (!stream) return AFB_ERR_BAD_ARG;
    cudaStream_t s;
    AFB_CUDA(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
    *stream = s;
    return AFB_OK;
}
int afb_stream_sync(void* stream) { AFB_CUDA(cudaStreamSynchronize((cudaStream_t)stream)); return AFB_OK; }
int afb_stream_destroy(void* stream) { AFB_CUDA(cudaStreamDestroy((cudaStream_t)stream)); return AFB_OK; }
int afb_device_sync(void) { AFB_CUDA(cudaDeviceSynchronize()); return AFB_OK; }

int afb_gemm_resolve_variant(const afb_gemm_args* args, uint32_t* variant) {
    if (!variant) return AFB_ERR_BAD_ARG;
    int rc = validate(args);
    if (rc) return rc;
    return resolve(*args, variant);
}

int afb_gemm_launch(const afb_gemm_args* args, void* stream) {
    int rc = validate(args);
    if (rc) return rc;
    DeviceCtx* ctx = current_ctx();
    if (!ctx) return AFB_ERR_NOT_INIT;
    uint32_t v;
    rc = resolve(*args, &v);
    if (rc) return rc;
    cudaStream_t s = (cudaStream_t)stream;
    switch (v) {
        case AFB_VARIANT_DECODE:  return launch_decode(*args, ctx, s);
        case AFB_VARIANT_PREFILL: {
            // two implementations of the prefill variant; a flag or AFB_PREFILL_IMPL=ss|ts overrides the default
            static const int env_ts = [] { const char* e = getenv("AFB_PREFILL_IMPL"); return e ? (e[0] == 't' ? 1 : 0) : -1; }();
            bool ts = env_ts == 1;
            if (env_ts < 0) {
                ts = args->m > kPrefillTsMinM;
                if (!ts) {
                    // up to 128 rows both forms are bound by the weight conversion: the shared-memory form converts 256 channels
                    // per tile, the tensor-memory form 128 (about 0.7 of the time, measured); what decides is how many waves of
                    // tiles each needs (28672 channels: 112 vs 224 tiles on 148 SMs -> shared-memory form; 8192: 32 vs 64 -> the other)
                    const uint64_t sms = (uint64_t)ctx->sm_count, mt = (args->m + 127) / 128;
                    const uint64_t waves_ss = (mt * ((args->n + 255) / 256) + sms - 1) / sms;
                    const uint64_t tiles_ts = mt * ((args->n + 127) / 128), waves_ts = (tiles_ts + sms - 1) / sms;
                    // at most half a wave of tiles: the tensor-memory form cuts every tile into up to 4 stretches of K
                    const uint64_t parts_ts = tiles_ts * 2 <= sms ? (sms / tiles_ts < 4 ? sms / tiles_ts : 4) : 1;
                    ts = waves_ts * 7 < waves_ss * 10 * parts_ts;
                }
            }
            if (args->flags & AFB_FLAG_PREFILL_SMEM_B) ts = false;
            if (args->flags & AFB_FLAG_PREFILL_TMEM_A) ts = true;
            if ((args->flags & AFB_FLAG_GROUP_EXACT) && args->group_size) ts = true;
            if (prefill_needs_ts(*args)) {
                if (args->flags & AFB_FLAG_PREFILL_SMEM_B) return AFB_ERR_UNSUPPORTED;
                ts = true;
            }
            return ts ? launch_prefill_ts(*args, ctx, s) : launch_prefill(*args, ctx, s);
        }
        default:                  return launch_naive(*args, ctx, s);
    }
}

int afb_gemm_fused_launch(const afb_fused_args* f, void* stream) {
    if (!f || f->reserved != 0 || f->gated > 1 || f->activation > AFB_ACT_SILU) return AFB_ERR_BAD_ARG;
    const afb_gemm_args& a = f->gemm;
    if (f->gated && (a.n & 1u)) return AFB_ERR_BAD_ARG;
    const uint32_t n_out = f->gated ? a.n / 2 : a.n;
    int rc = validate(&a, n_out);
    if (rc) return rc;
    if (a.flags & ~(AFB_FLAG_GROUP_EXACT | AFB_FLAG_PREFILL_TMEM_A)) return AFB_ERR_UNSUPPORTED;   // bf16 output, tensor-memory form
    if (a.variant != AFB_VARIANT_AUTO && a.variant != AFB_VARIANT_PREFILL) return AFB_ERR_UNSUPPORTED;
    if ((uintptr_t)f->ptr_bias % 4 || (uintptr_t)f->ptr_residual % 2) return AFB_ERR_BAD_ARG;
    if (f->ptr_residual && f->ld_residual < n_out) return AFB_ERR_BAD_ARG;
    if (!prefill_supports(a)) return AFB_ERR_UNSUPPORTED;   // [N,K] layout (plain or pre-packed), K % 64 == 0, aligned pointers and pitches
    DeviceCtx* ctx = current_ctx();
    if (!ctx) return AFB_ERR_NOT_INIT;
    return launch_prefill_ts(a, ctx, (cudaStream_t)stream, f);
}

static size_t b_bytes(const afb_gemm_args& a) {
    const size_t ld_bytes = (size_t)a.ldb * a.b_bits / 8;
    const size_t rows = a.b_layout != AFB_LAYOUT_ROW ? a.n : a.k;
    const size_t cols_bytes = (size_t)(a.b_layout != AFB_LAYOUT_ROW ? a.k : a.n) * a.b_bits / 8;
    return (rows - 1) * ld_bytes + cols_bytes;  // the size rule of bfAintBGemm.cc:68-76
}

// wait = true: returns when C is in host memory; false: returns when everything is queued (afb_stream_sync(stream) completes it).
static int gemm_host_impl(const afb_gemm_args* h, void* stream, bool wait) {
    int rc = validate(h);
    if (rc) return rc;
    DeviceCtx* ctx = current_ctx();
    if (!ctx) return AFB_ERR_NOT_INIT;
    const size_t c_elt = (h->flags & AFB_FLAG_C_F32) ? 4 : 2;
    const size_t scale_elt = h->scale_dtype == AFB_SCALE_BF16 ? 2 : 4;
    const size_t scale_cnt = h->group_size ? (size_t)h->n * (h->k / h->group_size) : h->n;
    const size_t need[4] = {((size_t)(h->m - 1) * h->ldc + h->n) * c_elt, ((size_t)(h->m - 1) * h->lda + h->k) * 2,
                            b_bytes(*h), scale_cnt * scale_elt};
    if (h->ptr_zero) return AFB_ERR_UNSUPPORTED;   // zero-points: copy them yourself and use afb_gemm_launch
    cudaStream_t s = (cudaStream_t)stream;
    if (!ctx->host_in) {
        AFB_CUDA(cudaStreamCreateWithFlags(&ctx->host_in, cudaStreamNonBlocking));
        AFB_CUDA(cudaStreamCreateWithFlags(&ctx->host_out, cudaStreamNonBlocking));
        for (auto& e : ctx->host_ev) AFB_CUDA(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
        for (auto& e : ctx->stage_free) AFB_CUDA(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
    }
    // two staging sets used in turn: this call's copies may run while the previous call (on the other set) still computes
    // or copies out; the set's previous user, two calls back, must be done with it
    const unsigned set = ctx->host_calls++ & 1u;
    void** stage = ctx->stage[set];
    for (int i = 0; i < 4; ++i) {
        if (ctx->stage_bytes[set][i] < need[i]) {
            if (stage[i]) AFB_CUDA(cudaFree(stage[i]));   // waits for everything in flight
            stage[i] = nullptr; ctx->stage_bytes[set][i] = 0;
            AFB_CUDA(cudaMalloc(&stage[i], need[i]));
            ctx->stage_bytes[set][i] = need[i];
        }
    }
    AFB_CUDA(cudaStreamWaitEvent(s, ctx->stage_free[set], 0));
    afb_gemm_args d = *h;
    d.ptr_c = stage[0]; d.ptr_a = stage[1]; d.ptr_b = stage[2]; d.ptr_scale = stage[3];

    // Pipelined form for B in [N,K] layout with per-channel scales: the channels are cut into chunks; while chunk i is
    // multiplied, chunk i+1 of the weights travels host -> device and chunk i-1 of C travels device -> host (PCIe is full duplex).
    constexpr uint32_t kChunks = 8;
    const bool pipelined = h->b_layout != AFB_LAYOUT_ROW && h->group_size == 0 && h->m > 16 && h->n >= kChunks * 512 && h->n % (kChunks * 128) == 0;
    if (!pipelined) {
        AFB_CUDA(cudaMemcpyAsync(stage[1], h->ptr_a, need[1], cudaMemcpyHostToDevice, s));
        AFB_CUDA(cudaMemcpyAsync(stage[2], h->ptr_b, need[2], cudaMemcpyHostToDevice, s));
        AFB_CUDA(cudaMemcpyAsync(stage[3], h->ptr_scale, need[3], cudaMemcpyHostToDevice, s));
        rc = afb_gemm_launch(&d, stream);
        if (rc) return rc;
        AFB_CUDA(cudaMemcpyAsync(h->ptr_c, stage[0], need[0], cudaMemcpyDeviceToHost, s));
        AFB_CUDA(cudaEventRecord(ctx->stage_free[set], s));
        if (wait) AFB_CUDA(cudaStreamSynchronize(s));
        return AFB_OK;
    }
    cudaEvent_t* ev_in = ctx->host_ev;                 // [kChunks]: chunk i of B and scale is on the device
    cudaEvent_t* ev_mm = ctx->host_ev + 16;            // [kChunks]: chunk i of C is computed
    cudaEvent_t ev_start = ctx->host_ev[32], ev_end = ctx->host_ev[33];
    AFB_CUDA(cudaEventRecord(ev_start, s));            // everything below happens after what the caller queued on `stream`
    AFB_CUDA(cudaStreamWaitEvent(ctx->host_in, ev_start, 0));
    AFB_CUDA(cudaStreamWaitEvent(ctx->host_out, ev_start, 0));
    AFB_CUDA(cudaMemcpyAsync(stage[1], h->ptr_a, need[1], cudaMemcpyHostToDevice, ctx->host_in));
    const uint32_t nc = h->n / kChunks;
    const size_t ldb_bytes = (size_t)h->ldb * h->b_bits / 8, b_chunk = (size_t)nc * ldb_bytes;
    for (uint32_t i = 0; i < kChunks; ++i) {
        const size_t b_off = (size_t)i * b_chunk;
        const size_t b_len = i + 1 < kChunks ? b_chunk : need[2] - b_off;
        AFB_CUDA(cudaMemcpyAsync((char*)stage[2] + b_off, (const char*)h->ptr_b + b_off, b_len, cudaMemcpyHostToDevice, ctx->host_in));
        AFB_CUDA(cudaMemcpyAsync((char*)stage[3] + (size_t)i * nc * scale_elt, (const char*)h->ptr_scale + (size_t)i * nc * scale_elt,
                                 (size_t)nc * scale_elt, cudaMemcpyHostToDevice, ctx->host_in));
        AFB_CUDA(cudaEventRecord(ev_in[i], ctx->host_in));
        AFB_CUDA(cudaStreamWaitEvent(s, ev_in[i], 0));
        afb_gemm_args c = d;
        c.n = nc;
        c.ptr_b = (char*)stage[2] + b_off;
        c.ptr_scale = (char*)stage[3] + (size_t)i * nc * scale_elt;
        c.ptr_c = (char*)stage[0] + (size_t)i * nc * c_elt;
        rc = afb_gemm_launch(&c, stream);
        if (rc) return rc;
        AFB_CUDA(cudaEventRecord(ev_mm[i], s));
        AFB_CUDA(cudaStreamWaitEvent(ctx->host_out, ev_mm[i], 0));
        AFB_CUDA(cudaMemcpy2DAsync((char*)h->ptr_c + (size_t)i * nc * c_elt, (size_t)h->ldc * c_elt, (char*)stage[0] + (size_t)i * nc * c_elt,
                                   (size_t)h->ldc * c_elt, (size_t)nc * c_elt, h->m, cudaMemcpyDeviceToHost, ctx->host_out));
    }
    AFB_CUDA(cudaEventRecord(ev_end, ctx->host_out));
    if (wait) {
        AFB_CUDA(cudaStreamWaitEvent(s, ev_end, 0));
        AFB_CUDA(cudaEventRecord(ctx->stage_free[set], s));
        AFB_CUDA(cudaStreamSynchronize(s));
    } else {
        // `stream` must not wait for the copy-out here, or the next call's GEMMs would queue behind it: the set is released,
        // and completion is reported, on the copy-out stream; afb_gemm_host_wait joins it
        AFB_CUDA(cudaEventRecord(ctx->stage_free[set], ctx->host_out));
    }
    return AFB_OK;
}

int afb_gemm_host(const afb_gemm_args* h, void* stream) { return gemm_host_impl(h, stream, true); }
int afb_gemm_host_async(const afb_gemm_args* h, void* stream) { return gemm_host_impl(h, stream, false); }
int afb_gemm_host_wait(void* stream) {
    DeviceCtx* ctx = current_ctx();
    if (!ctx) return AFB_ERR_NOT_INIT;
    AFB_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
    if (ctx->host_out) AFB_CUDA(cudaStreamSynchronize(ctx->host_out));
    return AFB_OK;
}

int afb_dequant_dump(const afb_gemm_args* args, void* out_bf16, void* stream) {
    if (!args || !args->ptr_b || !out_bf16 || args->n == 0 || args->k == 0) return AFB_ERR_BAD_ARG;
    if (args->b_bits != 8 && args->b_bits != 4) return AFB_ERR_BAD_ARG;
    if (args->group_size && !args->ptr_scale) return AFB_ERR_BAD_ARG;
    if (args->b_bits == 4 && args->b_layout == AFB_LAYOUT_ROW) return AFB_ERR_UNSUPPORTED;
    if (args->b_layout > 2) return AFB_ERR_BAD_ARG;
    if (!current_ctx()) return AFB_ERR_NOT_INIT;
    return launch_dequant_dump(*args, out_bf16, (cudaStream_t)stream);
}

int afb_read_status(int32_t out[4]) {
    DeviceCtx* ctx = current_ctx();
    if (!ctx) return AFB_ERR_NOT_INIT;
    if (!out) return AFB_ERR_BAD_ARG;
    AFB_CUDA(cudaDeviceSynchronize());
    AFB_CUDA(cudaMemcpy(out, ctx->status, 4 * sizeof(int32_t), cudaMemcpyDeviceToHost));
    AFB_CUDA(cudaMemset(ctx->status, 0, 4 * sizeof(int32_t)));
    if (out[0] != 0) {
        // A wait that gave up may have left arrival counters half way (a CTA that aborted never counted itself): launches that
        // were in flight with it are void, and the counters go back to zero so that the next launch starts clean.
        std::lock_guard<std::mutex> lock(g_mutex);
        for (auto& w : ctx->workspaces)
            if (w.counters) AFB_CUDA(cudaMemset(w.counters, 0, ctx->splitk_counter_count * sizeof(uint32_t)));
        AFB_CUDA(cudaMemset(ctx->ar_words, 0, 4 * sizeof(uint32_t)));
    }
    return AFB_OK;
}

int afb_probe_launch(uint32_t kind, const void* src, size_t bytes, uint32_t ctas, uint32_t smem_bytes, uint32_t flags, void* stream) {
    if (kind > 1 || ctas == 0 || ctas > 65535 || smem_bytes > 200 * 1024 || (kind == 1 && (!src || (uintptr_t)src % 16 || bytes % 16))) return AFB_ERR_BAD_ARG;
    if (flags & ~AFB_FLAG_PDL) return AFB_ERR_BAD_ARG;
    DeviceCtx* ctx = current_ctx();
    if (!ctx) return AFB_ERR_NOT_INIT;
    return launch_probe(kind, src, bytes, ctas, smem_bytes, (flags & AFB_FLAG_PDL) != 0, ctx->ar_words + 0 /* never written in practice */, (cudaStream_t)stream);
}

int afb_phase_timestamps(unsigned long long out[8]) {
    DeviceCtx* ctx = current_ctx();
    if (!ctx) return AFB_ERR_NOT_INIT;
    if (!out) return AFB_ERR_BAD_ARG;
    AFB_CUDA(cudaDeviceSynchronize());
    AFB_CUDA(cudaMemcpy(out, ctx->phase_ts, 8 * sizeof(unsigned long long), cudaMemcpyDeviceToHost));
    AFB_CUDA(cudaMemset(ctx->phase_ts, 0, 8 * sizeof(unsigned long long)));
    return AFB_OK;
}

int afb_ipc_export(void* dev_ptr, unsigned char handle[AFB_IPC_HANDLE_BYTES]) {
    static_assert(sizeof(cudaIpcMemHandle_t) == AFB_IPC_HANDLE_BYTES, "handle size");
    if (!dev_ptr || !handle) return AFB_ERR_BAD_ARG;
    cudaIpcMemHandle_t h;
    AFB_CUDA(cudaIpcGetMemHandle(&h, dev_ptr));
    memcpy(handle, &h, sizeof(h));
    return AFB_OK;
}
int afb_ipc_import(const unsigned char handle[AFB_IPC_HANDLE_BYTES], void** dev_ptr) {
    if (!dev_ptr || !handle) return AFB_ERR_BAD_ARG;
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, sizeof(h));
    AFB_CUDA(cudaIpcOpenMemHandle(dev_ptr, h, cudaIpcMemLazyEnablePeerAccess));
    return AFB_OK;
}
int afb_ipc_release(void* dev_ptr) { AFB_CUDA(cudaIpcCloseMemHandle(dev_ptr)); return AFB_OK; }

const char* afb_status_string(int status) {
    switch (status) {
        case AFB_OK: return "ok";
        case AFB_ERR_BAD_ARG: return "bad argument";
        case AFB_ERR_UNSUPPORTED: return "unsupported shape, layout or mode for the requested variant";
        case AFB_ERR_CUDA: return "CUDA call failed";
        case AFB_ERR_TIMEOUT: return "a bounded device-side wait gave up";
        case AFB_ERR_NOT_INIT: return "afb_init was not called on the current device";
        case AFB_ERR_TOO_LARGE: return "request exceeds a fixed capacity";
        default: return "unknown status";
    }
}
int afb_last_cuda_error(void) { return g_last_cuda_error.load(); }
const char* afb_last_cuda_error_string(void) { return cudaGetErrorString((cudaError_t)g_last_cuda_error.load()); }
unsigned long long afb_launch_count(void) { return g_launches.load(); }
const char* afb_version(void) { return "afb 0.1 (sm_100a)"; }

}  // extern "C"
