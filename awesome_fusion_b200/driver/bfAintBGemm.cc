// Host driver of the bf16 x int GEMM benchmark: the command line, buffer set-up, timing loop, metric line and
// optional validation of the reference's bfAintBGemm/bfAintBGemm.cc:36-217, re-targeted from HIP + a hand-loaded
// gfx90a code object to the C ABI of libafb.so (B200, sm_100a).
//
//   bfAintBGemm [validation [m n k [lda ldb ldc]]] [key=value ...]
//
// The positional arguments mean what they mean in the reference (:38-58; defaults 0, 32, 128, 512, k, n, n).
// Options the reference fixed at compile time are key=value pairs, so old invocations keep working:
//   b_layout=row|col   row: B is [K,N] as in the reference (default); col: B is [N,K], the layout of the fast kernels
//   enc=offset|twos    int8 stored as value+128 as in the reference (default) or two's complement
//   bits=8|4  group=G  4-bit weights (col layout), one bf16 scale per G weights along K (0 = one fp32 scale per channel)
//   data=int|real      int: every value an integer in {-2,-1,0,1} as the reference's generators (default);
//                      real: A ~ N(0,1), B uniform integers over the full range, scales uniform[0.001,0.01]
//   a_dist=normal|uniform   real data: A ~ N(0,1) (default) or uniform[-1,1]
//   scale_lo=X scale_hi=Y   real data: range of the scales (defaults 0.001..0.01 per channel, 0.005..0.05 per group)
//   exact=0|1          group scales, prefill variant: two bf16 terms per weight (AFB_FLAG_GROUP_EXACT) instead of one rounded term
//   prepack=0|1        run afb_prepack on B first (outside the timed loop) and multiply the pre-packed weights: this is how
//                      the reference's own [K,N] layout (b_layout=row) reaches the fast kernels
//   gpus=G split=n|k   shard the GEMM over G GPUs of the box from this one process (afb_dist_*): n = output channels
//                      (column-parallel, no collective), k = the K dimension (row-parallel, partial sums added over NVLink);
//                      needs b_layout=col, bits=8, group=0
//   seed=S  iters=I  warmup=W  variant=auto|decode|prefill|naive
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "afb_capi.h"
#include "bfAintBGemm/datatype.hpp"
#include "bfAintBGemm/gemm_tensor_layout.hpp"
#include "bfAintBGemm/gpu_utils.hpp"
#include "bfAintBGemm/host_ref.hpp"
#include "bfAintBGemm/mem_transfer.hpp"
#include "bfAintBGemm/random_gen.hpp"
#include "bfAintBGemm/simple_device_mem.hpp"
#include "bfAintBGemm/validation.hpp"

using Row = gemm_layout::gemm::RowMajor;
using Col = gemm_layout::gemm::ColumnMajor;

using ADataType = bfloat16;
using BDataType = std::int8_t;
using ScaleDataType = float;
using CDataType = bfloat16;

namespace {
constexpr float kGroupedOneTermBound = 0.25f;   // group-scaled prefill, one rounded term per weight, against the fp32 formula at the 0.05 x RMS floor
struct Options {
    int validation = 0, m = 32, n = 128, k = 512, lda = -1, ldb = -1, ldc = -1;
    bool b_col = false, offset_enc = true, real_data = false, a_uniform = false, exact = false, prepack = false, split_k = false;
    int gpus = 1;
    float scale_lo = -1.f, scale_hi = -1.f;
    int bits = 8, group = 0, iters = 10, warmup = 10;
    unsigned long long seed = 0;
    unsigned variant = AFB_VARIANT_AUTO;
};

bool parse(int argc, char** argv, Options& o) {
    std::vector<const char*> pos;
    for (int i = 1; i < argc; ++i) {
        const char* eq = std::strchr(argv[i], '=');
        if (!eq) { pos.push_back(argv[i]); continue; }
        const std::string key(argv[i], eq - argv[i]), val(eq + 1);
        if (key == "b_layout") o.b_col = val == "col";
        else if (key == "enc") o.offset_enc = val != "twos";
        else if (key == "bits") o.bits = std::atoi(val.c_str());
        else if (key == "group") o.group = std::atoi(val.c_str());
        else if (key == "data") o.real_data = val == "real";
        else if (key == "a_dist") o.a_uniform = val == "uniform";
        else if (key == "scale_lo") o.scale_lo = (float)std::atof(val.c_str());
        else if (key == "scale_hi") o.scale_hi = (float)std::atof(val.c_str());
        else if (key == "exact") o.exact = std::atoi(val.c_str()) != 0;
        else if (key == "prepack") o.prepack = std::atoi(val.c_str()) != 0;
        else if (key == "gpus") o.gpus = std::atoi(val.c_str());
        else if (key == "split") o.split_k = val == "k";
        else if (key == "seed") o.seed = std::strtoull(val.c_str(), nullptr, 10);
        else if (key == "iters") o.iters = std::atoi(val.c_str());
        else if (key == "warmup") o.warmup = std::atoi(val.c_str());
        else if (key == "variant") o.variant = val == "decode" ? AFB_VARIANT_DECODE : val == "prefill" ? AFB_VARIANT_PREFILL : val == "naive" ? AFB_VARIANT_NAIVE : AFB_VARIANT_AUTO;
        else { std::printf("unknown option %s\n", argv[i]); return false; }
    }
    if (pos.size() >= 1) o.validation = std::atoi(pos[0]);
    if (pos.size() >= 4) { o.m = std::atoi(pos[1]); o.n = std::atoi(pos[2]); o.k = std::atoi(pos[3]); }
    o.lda = o.k; o.ldb = o.b_col ? o.k : o.n; o.ldc = o.n;
    if (pos.size() >= 7) { o.lda = std::atoi(pos[4]); o.ldb = std::atoi(pos[5]); o.ldc = std::atoi(pos[6]); }
    if (o.bits == 4 && !o.b_col) { std::printf("bits=4 needs b_layout=col\n"); return false; }
    if (o.m <= 0 || o.n <= 0 || o.k <= 0 || o.iters <= 0) return false;
    if (o.gpus < 1 || o.gpus > AFB_MAX_RANKS) { std::printf("gpus must be 1..%d\n", AFB_MAX_RANKS); return false; }
    if (o.gpus > 1 && (!o.b_col || o.bits != 8 || o.group != 0 || o.lda != o.k || o.ldb != o.k || o.ldc != o.n)) {
        std::printf("gpus=G needs b_layout=col, bits=8, group=0 and default leading dimensions\n");
        return false;
    }
    return true;
}

// The sharded run: the same timing loop and metric line, with the GEMM cut over o.gpus GPUs by afb_dist_*.
// a_dev / b_dev / s_host are the device-format host copies (bf16 A [M,K], int8 B [N,K], fp32 scales [N]); ref_inputs are the
// fp32 masters the check multiplies.  Returns the process exit code.
int run_sharded(const Options& o, const void* a_dev, const void* b_dev, const float* s_host, const float* a_f32, const float* b_f32) {
    const int m = o.m, n = o.n, k = o.k, world = o.gpus;
    afb_dist* dist = nullptr;
    GPU_CHECK_ERROR(afb_dist_init((uint32_t)world, &dist));
    struct Rank { void *a = nullptr, *b = nullptr, *s = nullptr, *c = nullptr; uint32_t lo = 0, hi = 0; void *ev0 = nullptr, *ev1 = nullptr, *stream = nullptr; };
    std::vector<Rank> rk(world);
    afb_dist_gemm_args da = {};
    da.split = o.split_k ? AFB_SPLIT_K : AFB_SPLIT_N;
    for (int r = 0; r < world; ++r) {
        GPU_CHECK_ERROR(afb_init(r));   // also makes device r current for the allocations below
        GPU_CHECK_ERROR(afb_dist_split_range(o.split_k ? k : n, world, r, o.split_k ? 64 : 8, &rk[r].lo, &rk[r].hi));
        // every GPU gets the whole A; B and the scales are cut (N-split) or addressed with an offset and the full pitch (K-split)
        GPU_CHECK_ERROR(afb_malloc(&rk[r].a, (std::size_t)m * k * 2));
        GPU_CHECK_ERROR(afb_memcpy_h2d(rk[r].a, a_dev, (std::size_t)m * k * 2));
        const std::size_t b_rows = o.split_k ? n : rk[r].hi - rk[r].lo, b_row0 = o.split_k ? 0 : rk[r].lo;
        GPU_CHECK_ERROR(afb_malloc(&rk[r].b, b_rows * k));
        GPU_CHECK_ERROR(afb_memcpy_h2d(rk[r].b, static_cast<const char*>(b_dev) + b_row0 * k, b_rows * k));
        GPU_CHECK_ERROR(afb_malloc(&rk[r].s, b_rows * 4));
        GPU_CHECK_ERROR(afb_memcpy_h2d(rk[r].s, s_host + b_row0, b_rows * 4));
        const std::size_t c_cols = o.split_k ? n : rk[r].hi - rk[r].lo;
        GPU_CHECK_ERROR(afb_malloc(&rk[r].c, (std::size_t)m * c_cols * 2));
        GPU_CHECK_ERROR(afb_memset(rk[r].c, 0, (std::size_t)m * c_cols * 2));
        afb_gemm_args& g = da.shard[r];
        g.ptr_c = rk[r].c; g.ptr_scale = rk[r].s;
        g.m = m;
        g.b_bits = 8; g.b_encoding = o.offset_enc ? AFB_ENC_OFFSET_BINARY : AFB_ENC_TWOS_COMPLEMENT; g.b_layout = AFB_LAYOUT_COL;
        g.scale_dtype = AFB_SCALE_F32; g.variant = o.variant;
        if (o.split_k) {
            g.ptr_a = static_cast<char*>(rk[r].a) + (std::size_t)rk[r].lo * 2; g.ptr_b = static_cast<char*>(rk[r].b) + rk[r].lo;
            g.n = n; g.k = rk[r].hi - rk[r].lo; g.lda = k; g.ldb = k; g.ldc = n;
            da.c[r] = rk[r].c;
        } else {
            g.ptr_a = rk[r].a; g.ptr_b = rk[r].b;
            g.n = rk[r].hi - rk[r].lo; g.k = k; g.lda = k; g.ldb = k; g.ldc = g.n;
        }
        GPU_CHECK_ERROR(afb_dist_stream(dist, r, &rk[r].stream));
        GPU_CHECK_ERROR(afb_event_create(&rk[r].ev0));
        GPU_CHECK_ERROR(afb_event_create(&rk[r].ev1));
    }
    for (int i = 0; i < o.warmup; ++i) GPU_CHECK_ERROR(afb_dist_gemm_launch(dist, &da));
    GPU_CHECK_ERROR(afb_dist_sync(dist));
    for (int r = 0; r < world; ++r) { GPU_CHECK_ERROR(afb_init(r)); GPU_CHECK_ERROR(afb_event_record(rk[r].ev0, rk[r].stream)); }
    for (int i = 0; i < o.iters; ++i) GPU_CHECK_ERROR(afb_dist_gemm_launch(dist, &da));
    for (int r = 0; r < world; ++r) { GPU_CHECK_ERROR(afb_init(r)); GPU_CHECK_ERROR(afb_event_record(rk[r].ev1, rk[r].stream)); }
    GPU_CHECK_ERROR(afb_dist_sync(dist));
    float elapsed_ms = 0.f;   // the slowest GPU decides
    for (int r = 0; r < world; ++r) {
        float ms = 0.f;
        GPU_CHECK_ERROR(afb_init(r));
        GPU_CHECK_ERROR(afb_event_elapsed_ms(&ms, rk[r].ev0, rk[r].ev1));
        if (ms > elapsed_ms) elapsed_ms = ms;
        int32_t status[4] = {0, 0, 0, 0};
        GPU_CHECK_ERROR(afb_read_status(status));
        if (status[0] != 0) { std::printf("device %d status %d (%s) at %d/%d/%d\n", r, status[0], afb_status_string(status[0]), status[1], status[2], status[3]); return 1; }
    }
    const double time_per_loop = elapsed_ms / o.iters, flops = 2.0 * m * n * k;
    const double bytes = 2.0 * ((double)m * k + (double)m * n) + (double)n * k + 4.0 * n;
    std::printf("m: %d, n: %d, k: %d, time: %.3f ms, tflops: %.3f, bw: %.3f GB/s, variant: sharded over %d GPUs (%s-split)\n", m, n, k, time_per_loop,
                flops / time_per_loop / 1e9, bytes / time_per_loop / 1e6, world, o.split_k ? "k" : "n");
    std::printf("\n");
    int rc = 0;
    if (o.validation) {
        std::vector<float> ref((std::size_t)m * n);
        gemm_ref(ref.data(), a_f32, b_f32, s_host, m, n, k, k, k, n, true, 0);
        std::vector<CDataType> got((std::size_t)m * n), part;
        const float nrms = o.real_data ? 5e-3f : 2e-3f, rel = o.real_data ? 1e-2f : 4e-3f;
        bool res = true;
        if (o.split_k) {   // every GPU holds the complete result: check them all
            for (int r = 0; r < world && res; ++r) {
                GPU_CHECK_ERROR(afb_init(r));
                GPU_CHECK_ERROR(afb_memcpy_d2h(got.data(), rk[r].c, got.size() * 2));
                res = valid_vector<CDataType>(ref.data(), got.data(), m * n, nrms, rel, 0.05f);
            }
        } else {           // the channel shards side by side
            for (int r = 0; r < world; ++r) {
                const std::size_t cols = rk[r].hi - rk[r].lo;
                part.resize((std::size_t)m * cols);
                GPU_CHECK_ERROR(afb_init(r));
                GPU_CHECK_ERROR(afb_memcpy_d2h(part.data(), rk[r].c, part.size() * 2));
                for (int row = 0; row < m; ++row) std::memcpy(&got[(std::size_t)row * n + rk[r].lo], &part[(std::size_t)row * cols], cols * 2);
            }
            res = valid_vector<CDataType>(ref.data(), got.data(), m * n, nrms, rel, 0.05f);
        }
        std::printf(",%s \n", res ? "valid" : "fail");
        rc = res ? 0 : 1;
    }
    for (int r = 0; r < world; ++r) {
        (void)afb_event_destroy(rk[r].ev0); (void)afb_event_destroy(rk[r].ev1);
        (void)afb_free(rk[r].a); (void)afb_free(rk[r].b); (void)afb_free(rk[r].s); (void)afb_free(rk[r].c);
    }
    GPU_CHECK_ERROR(afb_dist_finalize(dist));
    return rc;
}
}  // namespace

int main(int argc, char** argv) {
    Options o;
    if (!parse(argc, argv, o)) return 2;
    const int m = o.m, n = o.n, k = o.k;
    rand_seed(o.seed);
    GPU_CHECK_ERROR(afb_init(0));

    // fp32 masters; B's master is kept in the layout the GEMM reads
    const std::size_t a_elems = gemm_layout::matrix_space_size(m, k, o.lda, Row{});
    const std::size_t b_elems = o.b_col ? gemm_layout::matrix_space_size(k, n, o.ldb, Col{}) : gemm_layout::matrix_space_size(k, n, o.ldb, Row{});
    const std::size_t c_elems = gemm_layout::matrix_space_size(m, n, o.ldc, Row{});
    const std::size_t groups = o.group ? (std::size_t)k / o.group : 1;
    const std::size_t s_elems = (std::size_t)n * groups;
    const bool scale_bf16 = o.group != 0;

    SimpleHostMem a_host_buf(sizeof(float) * a_elems), b_host_buf(sizeof(float) * b_elems), c_host_buf(sizeof(float) * c_elems),
        scale_host_buf(sizeof(float) * s_elems);
    float* a_f32 = static_cast<float*>(a_host_buf.GetBuffer());
    float* b_f32 = static_cast<float*>(b_host_buf.GetBuffer());
    float* s_f32 = static_cast<float*>(scale_host_buf.GetBuffer());
    const int b_rows = o.b_col ? n : k, b_cols = o.b_col ? k : n;
    if (!o.real_data) {
        rand_vector_2d_int_a(a_f32, m, k, o.lda);
        rand_vector_2d_int_b(b_f32, b_rows, b_cols, o.ldb);
        rand_vector_2d_int_scale(s_f32, n, (int)groups, (int)groups);
    } else {
        if (o.a_uniform) rand_vector_2d_uniform(a_f32, m, k, o.lda, -1.f, 1.f, 1);
        else rand_vector_2d_normal(a_f32, m, k, o.lda);
        if (o.bits == 8) rand_vector_2d_int_range(b_f32, b_rows, b_cols, o.ldb, -127, 127);
        else rand_vector_2d_int_range(b_f32, b_rows, b_cols, o.ldb, -8, 7);
        rand_vector_2d_uniform(s_f32, n, (int)groups, (int)groups, o.scale_lo >= 0.f ? o.scale_lo : (o.group ? 0.005f : 0.001f),
                               o.scale_hi >= 0.f ? o.scale_hi : (o.group ? 0.05f : 0.01f));
    }

    // device formats
    const std::size_t b_bytes = o.bits == 8 ? b_elems : (b_elems + 1) / 2;
    SimpleHostMem a_host_buf_to_device(sizeof(ADataType) * a_elems), b_host_buf_to_device(b_bytes),
        scale_host_buf_to_device((scale_bf16 ? 2 : 4) * s_elems), c_host_buf_from_device(sizeof(CDataType) * c_elems);
    if (o.real_data) mem_transfer_bf16_rne(a_host_buf_to_device, a_host_buf, a_elems);                    // rounds the master too
    else mem_transfer<ADataType, float, SimpleHostMem, SimpleHostMem>(a_host_buf_to_device, a_host_buf, a_elems);
    if (o.bits == 4) mem_transfer_int4(b_host_buf_to_device, b_host_buf, b_elems, o.offset_enc);
    else if (o.offset_enc) mem_transfer<BDataType, float, SimpleHostMem, SimpleHostMem>(b_host_buf_to_device, b_host_buf, b_elems);
    else mem_transfer_int8_twos(b_host_buf_to_device, b_host_buf, b_elems);
    if (scale_bf16) mem_transfer_bf16_rne(scale_host_buf_to_device, scale_host_buf, s_elems);
    else std::memcpy(scale_host_buf_to_device.GetBuffer(), s_f32, 4 * s_elems);

    if (o.gpus > 1) {
        if (scale_bf16) { std::printf("gpus=G needs per-channel fp32 scales\n"); return 2; }
        return run_sharded(o, a_host_buf_to_device.GetBuffer(), b_host_buf_to_device.GetBuffer(), s_f32, a_f32, b_f32);
    }

    SimpleDeviceMem a_device_buf(sizeof(ADataType) * a_elems), b_device_buf(b_bytes), c_device_buf(sizeof(CDataType) * c_elems),
        scale_device_buf((scale_bf16 ? 2 : 4) * s_elems);
    if (!a_device_buf.ok() || !b_device_buf.ok() || !c_device_buf.ok() || !scale_device_buf.ok()) { std::printf("device allocation failed\n"); return 1; }
    GPU_CHECK_ERROR(afb_memcpy_h2d(a_device_buf.GetBuffer(), a_host_buf_to_device.GetBuffer(), sizeof(ADataType) * a_elems));
    GPU_CHECK_ERROR(afb_memcpy_h2d(b_device_buf.GetBuffer(), b_host_buf_to_device.GetBuffer(), b_bytes));
    GPU_CHECK_ERROR(afb_memcpy_h2d(scale_device_buf.GetBuffer(), scale_host_buf_to_device.GetBuffer(), (scale_bf16 ? 2 : 4) * s_elems));
    GPU_CHECK_ERROR(afb_memset(c_device_buf.GetBuffer(), 0, sizeof(CDataType) * c_elems));

    afb_gemm_args args = {};
    args.ptr_c = c_device_buf.GetBuffer();
    args.ptr_a = a_device_buf.GetBuffer();
    args.ptr_b = b_device_buf.GetBuffer();
    args.ptr_scale = scale_device_buf.GetBuffer();
    args.m = m; args.n = n; args.k = k;
    args.lda = o.lda; args.ldb = o.ldb; args.ldc = o.ldc;
    args.b_bits = o.bits;
    args.b_encoding = o.offset_enc ? AFB_ENC_OFFSET_BINARY : AFB_ENC_TWOS_COMPLEMENT;
    args.b_layout = o.b_col ? AFB_LAYOUT_COL : AFB_LAYOUT_ROW;
    args.scale_dtype = scale_bf16 ? AFB_SCALE_BF16 : AFB_SCALE_F32;
    args.group_size = o.group;
    args.variant = o.variant;
    args.flags = o.exact ? AFB_FLAG_GROUP_EXACT : 0u;
    // optional offline step: the weights re-ordered (and, from the reference's [K,N] layout, transposed) for the fast kernels
    SimpleDeviceMem packed_device_buf(o.prepack ? (std::size_t)n * k * o.bits / 8 : 1);
    if (o.prepack) {
        if (!packed_device_buf.ok()) { std::printf("device allocation failed\n"); return 1; }
        GPU_CHECK_ERROR(afb_prepack(&args, packed_device_buf.GetBuffer(), (uint32_t)k, nullptr));
        args.ptr_b = packed_device_buf.GetBuffer();
        args.ldb = k;
        args.b_layout = AFB_LAYOUT_COL_PACKED;
    }
    unsigned chosen = 0;
    GPU_CHECK_ERROR(afb_gemm_resolve_variant(&args, &chosen));

    for (int i = 0; i < o.warmup; ++i) GPU_CHECK_ERROR(afb_gemm_launch(&args, nullptr));

    void *evt_00 = nullptr, *evt_11 = nullptr;
    GPU_CHECK_ERROR(afb_event_create(&evt_00));
    GPU_CHECK_ERROR(afb_event_create(&evt_11));
    GPU_CHECK_ERROR(afb_device_sync());
    GPU_CHECK_ERROR(afb_event_record(evt_00, nullptr));
    for (int i = 0; i < o.iters; ++i) GPU_CHECK_ERROR(afb_gemm_launch(&args, nullptr));
    GPU_CHECK_ERROR(afb_event_record(evt_11, nullptr));
    GPU_CHECK_ERROR(afb_event_sync(evt_11));
    GPU_CHECK_ERROR(afb_device_sync());
    float elapsed_ms = 0.f;
    GPU_CHECK_ERROR(afb_event_elapsed_ms(&elapsed_ms, evt_00, evt_11));
    GPU_CHECK_ERROR(afb_event_destroy(evt_00));
    GPU_CHECK_ERROR(afb_event_destroy(evt_11));
    int32_t status[4] = {0, 0, 0, 0};
    GPU_CHECK_ERROR(afb_read_status(status));
    if (status[0] != 0) { std::printf("device status %d (%s) at %d/%d/%d\n", status[0], afb_status_string(status[0]), status[1], status[2], status[3]); return 1; }

    // the metric line of the reference (bfAintBGemm.cc:186-195), in units of 1e12 flop/s and 1e9 byte/s, scale bytes included
    const double time_per_loop = elapsed_ms / o.iters;
    const double flops = 2.0 * m * n * k;
    const double bytes = 2.0 * ((double)m * k + (double)m * n) + (double)n * k * o.bits / 8.0 + (double)s_elems * (scale_bf16 ? 2 : 4);
    static const char* names[] = {"auto", "decode", "prefill", "naive"};
    std::printf("m: %d, n: %d, k: %d, time: %.3f ms, tflops: %.3f, bw: %.3f GB/s, variant: %s\n", m, n, k, time_per_loop,
                flops / time_per_loop / 1e9, bytes / time_per_loop / 1e6, names[chosen & 3]);
    std::printf("\n");

    if (o.validation) {
        gemm_ref(static_cast<float*>(c_host_buf.GetBuffer()), a_f32, b_f32, s_f32, m, n, k, o.lda, o.ldb, o.ldc, o.b_col, o.group);
        GPU_CHECK_ERROR(afb_memcpy_d2h(c_host_buf_from_device.GetBuffer(), c_device_buf.GetBuffer(), sizeof(CDataType) * c_elems));
        // Integer data: products and sums are exact, so the only error is the final rounding of C to bf16 (at most 2^-8
        // relative; the reference's own 1e-3 bound only holds while every |C| < 256 is an exact bf16).  Real data: the 1e-2 contract.
        // Group scales on the prefill variant without exact=1: each weight reaches the tensor cores as ONE rounded bf16 term
        // bf16_rn(q * s), which the fp32 formula does not round; that mode is held to its own stated bound, not to 1e-2.
        const bool one_term = o.group && chosen == AFB_VARIANT_PREFILL && !o.exact;
        const float nrms = o.real_data ? 5e-3f : 2e-3f, rel = o.real_data ? (one_term ? kGroupedOneTermBound : 1e-2f) : 4e-3f;
        const float floor_frac = 0.05f;
        if (one_term && o.real_data) std::printf("note: one rounded bf16 term per weight (exact=0): bound %.2g instead of 1e-2\n", kGroupedOneTermBound);
        bool res = true;
        const float* ref = static_cast<const float*>(c_host_buf.GetBuffer());
        const CDataType* got = static_cast<const CDataType*>(c_host_buf_from_device.GetBuffer());
        if (o.ldc == n) res = valid_vector<CDataType>(ref, got, m * n, nrms, rel, floor_frac);
        else for (int r = 0; r < m && res; ++r) res = valid_vector<CDataType>(ref + (std::size_t)r * o.ldc, got + (std::size_t)r * o.ldc, n, nrms, rel, floor_frac);
        std::printf(",%s \n", res ? "valid" : "fail");
        return res ? 0 : 1;
    }
    return 0;
}
