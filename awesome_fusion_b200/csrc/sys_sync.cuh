// System-scope synchronisation and store helpers shared by the exchange kernels (ksplit.cu) and by the exchange warps inside the
// pushing GEMM (prefill_ts.cu): flag loads and stores that other GPUs observe, the bounded wait on a row of epoch words, the
// NVSwitch multicast store, bf16 packing.
#pragma once
#include <cuda_bf16.h>
#include <stdint.h>
#include "afb_capi.h"

namespace afb {
namespace xchg {

// Polling load without ordering: a kernel that polls NEXT TO a GEMM on the same SM must not issue an acquire per probe (every
// system-scope acquire disturbs the caches the GEMM's CTA lives on: measured 1.85 x on the co-resident CTA, and with a static
// tile assignment on the whole GEMM); it probes with this, sleeps between probes, and orders once after the value has shown.
__device__ __forceinline__ uint32_t ld_relaxed_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned long long now_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// Waits until signals[phase][q] >= epoch for every rank q.  One thread calls it.  false = gave up.
__device__ __forceinline__ bool wait_all(const uint32_t* my_signals, int phase, uint32_t world, uint32_t epoch, unsigned long long limit_ns) {
    const unsigned long long t0 = now_ns();
    for (uint32_t q = 0; q < world; ++q) {
        const uint32_t* f = my_signals + phase * AFB_MAX_RANKS + q;
        uint32_t spins = 0;
        while ((int32_t)(ld_acquire_sys(f) - epoch) < 0) {
            if ((++spins & 0x3fu) == 0 && now_ns() - t0 > limit_ns) return false;
        }
    }
    return true;
}

// One 16-byte store to a multicast address: the switch writes it into every rank's copy of the buffer.
__device__ __forceinline__ void st16_multicast(void* p, const uint4& v) {
    asm volatile("multimem.st.weak.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(__uint_as_float(v.x)), "f"(__uint_as_float(v.y)),
                 "f"(__uint_as_float(v.z)), "f"(__uint_as_float(v.w)) : "memory");
}
__device__ __forceinline__ uint4 ld16(const void* p) { return *reinterpret_cast<const uint4*>(p); }
__device__ __forceinline__ float bf_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf_hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }
__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&h);
}

}  // namespace xchg
}  // namespace afb
