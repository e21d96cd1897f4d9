// afb_gemm_launch_static: the decode GEMM for callers that must not allocate.
//
// Who that is: a host program whose framework has already claimed the whole device for its own
// memory pool (a late cudaMalloc from a library then fails, or forces the pool to give memory back),
// and a latency-critical serving loop, where cudaMalloc / cudaFree synchronise the device and stall
// every stream that is running.  Such callers cannot use afb_init + afb_gemm_launch, because afb_init
// allocates the split-K workspace.  This entry point needs no afb_init and never calls cudaMalloc,
// cudaFree or any allocating routine: the split-K scratch (fp32 partial sums and the per-row-block
// arrival counters) lives in a fixed array inside the library image.  Every GPU on which the image
// has been placed holds that array (kScratchBytes + kCounters * 4 bytes) until the process exits.
// With CUDA's default lazy module loading the driver places the image -- this array and the decode
// kernels -- when they are first touched, i.e. inside the FIRST call of this entry point on a device
// (cudaGetSymbolAddress, then the first launch).  That one call can therefore still fail for lack of
// memory on a device whose pool has taken everything, and it is not free of driver-side
// synchronisation: it belongs at start-up.  Every later call allocates nothing.
//
// Rules that follow from the array being shared:
//   * capacity: M * N <= kMaxOutputs (two K-slices of fp32 partial sums always fit) and
//     ceil(N / 128) <= kCounters; anything larger is refused with AFB_ERR_TOO_LARGE;
//   * every call on a device uses the same array, so two calls that overlap on the GPU (different
//     streams, or different host threads) race: issue them on one stream, or serialise them;
//   * the array keeps what the last call left in it.  Partial sums are fully overwritten before
//     they are read; the counters must be zero when a kernel starts: they are zero when the library
//     is loaded, each kernel puts them back to zero, and the first call on a device clears them again;
//   * that first call on each device also looks up the array's device address
//     (cudaGetSymbolAddress, with that device current) and enqueues the clearing memset: make it
//     before the framework claims the remaining device memory and before any stream capture begins.
#include <mutex>
#include "afb_internal.h"

namespace afb {
namespace {

constexpr size_t kMaxOutputs = 512u * 1024u;               // M * N
constexpr size_t kScratchBytes = 2 * kMaxOutputs * 4;      // 4 MiB of fp32 partial sums
constexpr size_t kCounters = 4096;

// In host code this name is only a handle for the runtime; the device address comes from cudaGetSymbolAddress.
static __device__ __align__(256) unsigned char g_static_scratch[kScratchBytes + kCounters * sizeof(uint32_t)];

struct StaticSlot {
    bool ready = false;
    unsigned char* base = nullptr;   // device address of g_static_scratch on this device
    int sm_count = 0;
};
StaticSlot g_slots[32];
std::mutex g_slot_mutex;

}  // namespace
}  // namespace afb

using namespace afb;

extern "C" int afb_gemm_launch_static(const afb_gemm_args* args, void* stream) {
    if (!args || !args->ptr_a || !args->ptr_b || !args->ptr_c || !args->ptr_scale) return AFB_ERR_BAD_ARG;
    if (args->m == 0 || args->n == 0 || args->k == 0 || args->reserved != 0 || args->flags != 0) return AFB_ERR_BAD_ARG;
    if (args->lda < args->k || args->ldc < args->n || args->ldb < args->k) return AFB_ERR_BAD_ARG;
    if (args->variant != AFB_VARIANT_AUTO && args->variant != AFB_VARIANT_DECODE) return AFB_ERR_UNSUPPORTED;
    if (args->b_bits != 8 && args->b_bits != 4) return AFB_ERR_BAD_ARG;
    if (args->b_encoding > 1 || args->b_layout > 2 || args->scale_dtype > 1) return AFB_ERR_BAD_ARG;
    if ((uintptr_t)args->ptr_scale % (args->scale_dtype == AFB_SCALE_BF16 ? 2 : 4) || (uintptr_t)args->ptr_c % 2) return AFB_ERR_BAD_ARG;
    if (!decode_supports(*args)) return AFB_ERR_UNSUPPORTED;           // M <= 16, [N,K] layout, see afb_capi.h
    if ((size_t)args->m * args->n > kMaxOutputs) return AFB_ERR_TOO_LARGE;
    if (((size_t)args->n + 127) / 128 > kCounters) return AFB_ERR_TOO_LARGE;

    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return cuda_fail(e);
    if (dev < 0 || dev >= 32) return AFB_ERR_BAD_ARG;
    StaticSlot& slot = g_slots[dev];
    {
        std::lock_guard<std::mutex> lock(g_slot_mutex);
        if (!slot.ready) {   // once per device, with that device current
            void* p = nullptr;
            e = cudaGetSymbolAddress(&p, g_static_scratch);
            if (e != cudaSuccess) return cuda_fail(e);
            int sms = 0;
            e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
            if (e != cudaSuccess) return cuda_fail(e);
            e = cudaMemsetAsync(static_cast<unsigned char*>(p) + kScratchBytes, 0, kCounters * sizeof(uint32_t), (cudaStream_t)stream);
            if (e != cudaSuccess) return cuda_fail(e);
            slot.base = static_cast<unsigned char*>(p);
            slot.sm_count = sms;
            slot.ready = true;
        }
    }
    DeviceCtx local;              // only the SM count is read by the decode launcher
    local.device = dev;
    local.sm_count = slot.sm_count;
    return launch_decode_ws(*args, &local, reinterpret_cast<float*>(slot.base), kScratchBytes,
                            reinterpret_cast<uint32_t*>(slot.base + kScratchBytes), kCounters, (cudaStream_t)stream);
}
