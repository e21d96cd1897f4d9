// Sharded GEMM across the GPUs of one box from a SINGLE process: the multi-GPU extension of the reference driver's
// one-device set-up (bfAintBGemm.cc:63 selects device 0 and never leaves it).  One host thread drives every GPU through
// its own stream; the GPUs reach each other's memory directly (peer access), so no handle exchange is needed.
//   * AFB_SPLIT_N (column-parallel): GPU r computes its own channels C[:, n_r] = A x B[n_r, :]^T.  Independent launches.
//   * AFB_SPLIT_K (row-parallel): GPU r multiplies A[:, K_r] by B[:, K_r]; the fp32 partial sums are combined by the
//     peer-memory exchange of ksplit.cu (reduce-scatter in the GEMM epilogue when M allows it, else an exchange kernel
//     that pulls), and every GPU ends up with the complete bf16 C.
// The kernels of different GPUs wait for one another through flags in peer memory (bounded waits); they are launched
// back to back without any host synchronisation in between, one kernel of each kind per GPU.
#include <mutex>
#include "afb_internal.h"

namespace afb {

struct DistCtx {
    uint32_t world = 0;
    cudaStream_t stream[AFB_MAX_RANKS] = {};
    float* stage[AFB_MAX_RANKS] = {};       // per GPU: float[world][M / world][N] (push form) or float[M][N] (pull form)
    size_t stage_bytes = 0;
    uint32_t* signals[AFB_MAX_RANKS] = {};  // per GPU: uint32[2 * AFB_MAX_RANKS]
    uint32_t epoch = 0;
};

}  // namespace afb

using namespace afb;

#define AFB_CUDA(call)                                  \
    do {                                                \
        cudaError_t e__ = (call);                       \
        if (e__ != cudaSuccess) return cuda_fail(e__);  \
    } while (0)

extern "C" {

int afb_dist_init(uint32_t ngpus, afb_dist** out) {
    if (!out || ngpus == 0 || ngpus > AFB_MAX_RANKS) return AFB_ERR_BAD_ARG;
    int count = 0;
    AFB_CUDA(cudaGetDeviceCount(&count));
    if ((int)ngpus > count) return AFB_ERR_UNSUPPORTED;
    DistCtx* d = new DistCtx();
    d->world = ngpus;
    for (uint32_t r = 0; r < ngpus; ++r) {
        int rc = afb_init((int)r);   // makes device r current
        if (rc) { delete d; return rc; }
        for (uint32_t q = 0; q < ngpus; ++q) {
            if (q == r) continue;
            int can = 0;
            cudaError_t e = cudaDeviceCanAccessPeer(&can, (int)r, (int)q);
            if (e != cudaSuccess || !can) { delete d; return e != cudaSuccess ? cuda_fail(e) : AFB_ERR_UNSUPPORTED; }
            e = cudaDeviceEnablePeerAccess((int)q, 0);
            if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled) { delete d; return cuda_fail(e); }
            (void)cudaGetLastError();
        }
        cudaError_t e = cudaStreamCreateWithFlags(&d->stream[r], cudaStreamNonBlocking);
        if (e == cudaSuccess) e = cudaMalloc(&d->signals[r], 2 * AFB_MAX_RANKS * sizeof(uint32_t));
        if (e == cudaSuccess) e = cudaMemset(d->signals[r], 0, 2 * AFB_MAX_RANKS * sizeof(uint32_t));
        if (e == cudaSuccess) e = cudaDeviceSynchronize();
        if (e != cudaSuccess) { delete d; return cuda_fail(e); }
    }
    AFB_CUDA(cudaSetDevice(0));
    *out = reinterpret_cast<afb_dist*>(d);
    return AFB_OK;
}

int afb_dist_world(const afb_dist* dist, uint32_t* world) {
    if (!dist || !world) return AFB_ERR_BAD_ARG;
    *world = reinterpret_cast<const DistCtx*>(dist)->world;
    return AFB_OK;
}

int afb_dist_sync(afb_dist* dist) {
    if (!dist) return AFB_ERR_BAD_ARG;
    DistCtx* d = reinterpret_cast<DistCtx*>(dist);
    for (uint32_t r = 0; r < d->world; ++r) {
        AFB_CUDA(cudaSetDevice((int)r));
        AFB_CUDA(cudaStreamSynchronize(d->stream[r]));
    }
    AFB_CUDA(cudaSetDevice(0));
    return AFB_OK;
}

int afb_dist_finalize(afb_dist* dist) {
    if (!dist) return AFB_OK;
    DistCtx* d = reinterpret_cast<DistCtx*>(dist);
    for (uint32_t r = 0; r < d->world; ++r) {
        if (cudaSetDevice((int)r) != cudaSuccess) continue;
        cudaDeviceSynchronize();
        if (d->stream[r]) cudaStreamDestroy(d->stream[r]);
        if (d->stage[r]) cudaFree(d->stage[r]);
        if (d->signals[r]) cudaFree(d->signals[r]);
    }
    cudaSetDevice(0);
    delete d;
    return AFB_OK;
}

// The partition arithmetic of the shards: [lo, hi) of `total` owned by `rank`, in whole units of `multiple`, the remainder
// going to the first ranks (the same rule the multi-process launcher uses).
int afb_dist_split_range(uint32_t total, uint32_t world, uint32_t rank, uint32_t multiple, uint32_t* lo, uint32_t* hi) {
    if (!lo || !hi || world == 0 || rank >= world || multiple == 0 || total % multiple) return AFB_ERR_BAD_ARG;
    const uint32_t units = total / multiple, base = units / world, rem = units % world;
    const uint32_t first = rank * base + (rank < rem ? rank : rem);
    *lo = first * multiple;
    *hi = (first + base + (rank < rem ? 1u : 0u)) * multiple;
    return AFB_OK;
}

int afb_dist_gemm_launch(afb_dist* dist, const afb_dist_gemm_args* a) {
    if (!dist || !a) return AFB_ERR_BAD_ARG;
    DistCtx* d = reinterpret_cast<DistCtx*>(dist);
    const uint32_t world = d->world;
    if (a->split != AFB_SPLIT_N && a->split != AFB_SPLIT_K) return AFB_ERR_BAD_ARG;
    if (a->split == AFB_SPLIT_N || world == 1) {
        for (uint32_t r = 0; r < world; ++r) {
            AFB_CUDA(cudaSetDevice((int)r));
            const int rc = afb_gemm_launch(&a->shard[r], d->stream[r]);
            if (rc) { cudaSetDevice(0); return rc; }
        }
        AFB_CUDA(cudaSetDevice(0));
        return AFB_OK;
    }
    // ---- K-split: every shard has the same M, N; its own K range
    const uint32_t m = a->shard[0].m, n = a->shard[0].n;
    for (uint32_t r = 0; r < world; ++r) {
        if (a->shard[r].m != m || a->shard[r].n != n || !a->c[r] || (uintptr_t)a->c[r] % 16) return AFB_ERR_BAD_ARG;
        if (a->shard[r].group_size || a->shard[r].b_bits != 8 || a->shard[r].ptr_zero) return AFB_ERR_UNSUPPORTED;   // per-channel int8: the scale is applied per rank
    }
    if (n % 8) return AFB_ERR_UNSUPPORTED;
    const size_t need = (size_t)m * n * sizeof(float);
    if (d->stage_bytes < need) {
        for (uint32_t r = 0; r < world; ++r) {
            AFB_CUDA(cudaSetDevice((int)r));
            AFB_CUDA(cudaStreamSynchronize(d->stream[r]));
            if (d->stage[r]) { AFB_CUDA(cudaFree(d->stage[r])); d->stage[r] = nullptr; }
            AFB_CUDA(cudaMalloc(&d->stage[r], need));
        }
        d->stage_bytes = need;
    }
    const bool push = m > 128 && m % (256 * world) == 0;   // the reduce-scatter can live in the GEMM epilogue
    ++d->epoch;
    const uint32_t rows = m / world;
    for (uint32_t r = 0; r < world; ++r) {
        AFB_CUDA(cudaSetDevice((int)r));
        afb_gemm_args g = a->shard[r];
        g.flags |= AFB_FLAG_C_F32;
        int rc;
        if (push) {
            void* stage[AFB_MAX_RANKS] = {};
            for (uint32_t q = 0; q < world; ++q) stage[q] = d->stage[q];
            g.ptr_c = d->stage[r]; g.ldc = n;
            rc = afb_gemm_launch_push(&g, stage, world, r, d->stream[r]);
        } else {
            g.ptr_c = d->stage[r]; g.ldc = n;
            rc = afb_gemm_launch(&g, d->stream[r]);
        }
        if (rc) { cudaSetDevice(0); return rc; }
    }
    for (uint32_t r = 0; r < world; ++r) {
        AFB_CUDA(cudaSetDevice((int)r));
        afb_allreduce_args x = {};
        for (uint32_t q = 0; q < world; ++q) {
            // push form: rank r's own staging buffer holds slot q at row offset q * rows; the exchange kernel addresses rows
            // [r * rows, (r + 1) * rows) of an [M, N] matrix, so slot q is presented as if it began r * rows rows earlier
            x.partial[q] = push ? reinterpret_cast<void*>(reinterpret_cast<intptr_t>(d->stage[r]) + ((intptr_t)q * rows - (intptr_t)r * rows) * (intptr_t)n * (intptr_t)sizeof(float))
                                : (void*)d->stage[q];
            x.c[q] = a->c[q];
            x.signals[q] = d->signals[q];
        }
        x.rank = r; x.world = world; x.m = m; x.n = n; x.ld_partial = n; x.ldc = n;
        x.partial_f32 = 1; x.epoch = d->epoch; x.wait_ms = a->wait_ms; x.reserved = 0; x.c_multicast = nullptr;
        const int rc = afb_ksplit_allreduce_launch(&x, d->stream[r]);
        if (rc) { cudaSetDevice(0); return rc; }
    }
    AFB_CUDA(cudaSetDevice(0));
    return AFB_OK;
}

int afb_dist_stream(afb_dist* dist, uint32_t rank, void** stream) {
    if (!dist || !stream) return AFB_ERR_BAD_ARG;
    DistCtx* d = reinterpret_cast<DistCtx*>(dist);
    if (rank >= d->world) return AFB_ERR_BAD_ARG;
    *stream = d->stream[rank];
    return AFB_OK;
}

}  // extern "C"
