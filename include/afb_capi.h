/*
 * afb_capi.h — C ABI of the B200 (sm_100a) bfAintBGemm library (libafb.so).
 *
 * The reference host driver (bfAintBGemm/bfAintBGemm.cc) reaches its GPU through the
 * HIP runtime and a hand-loaded code object.  Every HIP entry point that driver uses
 * has exactly one counterpart here, so a host program written against the reference's
 * headers can be re-targeted by swapping the calls one for one.  All functions take
 * plain pointers and sizes, return an int status (0 = AFB_OK, negative = AFB_ERR_*)
 * and never abort or trap.  No CUDA or torch type appears in a signature: streams and
 * events are opaque void*.
 *
 * The computation:  C[M,N] (bf16) = A[M,K] (bf16) x dequant(B)^T, fp32 accumulation,
 * where B holds 8-bit or 4-bit integers and dequant multiplies by a per-output-channel
 * scale[N] or a per-group scale[N][K/group].
 */
#ifndef AFB_CAPI_H_
#define AFB_CAPI_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes ------------------------------------------------------------- */
#define AFB_OK               0
#define AFB_ERR_BAD_ARG     (-1)  /* null pointer, zero dimension, misaligned pointer/ld */
#define AFB_ERR_UNSUPPORTED (-2)  /* legal request that no kernel variant covers       */
#define AFB_ERR_CUDA        (-3)  /* a CUDA runtime/driver call failed; see afb_last_cuda_error */
#define AFB_ERR_TIMEOUT     (-4)  /* a bounded device-side wait gave up                 */
#define AFB_ERR_NOT_INIT    (-5)  /* afb_init was not called for the current device     */
#define AFB_ERR_TOO_LARGE   (-6)  /* request exceeds a fixed capacity (e.g. static scratch) */

/* ---- enumerations carried in afb_gemm_args ------------------------------------ */
#define AFB_ENC_TWOS_COMPLEMENT 0u /* int8 in [-128,127]; int4 in [-8,7]                */
#define AFB_ENC_OFFSET_BINARY   1u /* byte = value + 128 (reference: mem_transfer.hpp:30); nibble = value + 8 */

#define AFB_LAYOUT_ROW 0u /* B is [K,N], N contiguous — the reference's "rrr" (bfAintBGemm.cc:20-23,51) */
#define AFB_LAYOUT_COL 1u /* B is [N,K], K contiguous — ColumnMajor tag of gemm_tensor_layout.hpp:16-19 */
#define AFB_LAYOUT_COL_PACKED 2u /* [N,K] as written by afb_prepack: same rows and pitch, weights reordered inside every 32-bit word */

#define AFB_SCALE_F32  0u
#define AFB_SCALE_BF16 1u

#define AFB_VARIANT_AUTO    0u /* decode for M <= 16, prefill above, naive where neither applies */
#define AFB_VARIANT_DECODE  1u /* memory-bound small-M kernel                                   */
#define AFB_VARIANT_PREFILL 2u /* TMA + tcgen05/TMEM kernel                                    */
#define AFB_VARIANT_NAIVE   3u /* one thread per output element, fp32, order of host_ref.hpp:15-24 */

#define AFB_FLAG_C_F32 1u /* C is fp32 [M,N] instead of bf16: prefill variant (partial sums of a K-split) and naive variant */
#define AFB_FLAG_PREFILL_SMEM_B 2u /* prefill variant: force the form that stages the converted weights in shared memory */
#define AFB_FLAG_PREFILL_TMEM_A 4u /* prefill variant: force the form that keeps the converted weights in tensor memory  */
#define AFB_FLAG_PUSH_VIA_LOCAL 8u /* afb_gemm_launch_push only: ptr_c is a local fp32 [M,N] scratch (ldc = N); the epilogue stores there and two
                                      extra warps per CTA forward each finished tile to its owner while the next tile is computed */

#define AFB_FLAG_GROUP_EXACT 32u /* prefill variant with per-group scales: feed each weight q * s to the tensor cores as two bf16 terms
                                   (hi = bf16_rn(q * s), lo = q * s - hi, exact) instead of the one rounded term: twice the tensor-core
                                   work, and the result is that of the fp32 formula of host_ref.hpp:15-24 up to summation order.
                                   No effect where the scale never touches the weights (per-channel scales, decode variant). */
#define AFB_FLAG_PDL 64u /* decode variant: launch with programmatic stream serialisation.  The kernel starts streaming B while the preceding
                           kernel of the stream is still running and waits for it only before it touches A, C or the workspace; it
                           also lets its own successor start early.  The caller promises that B and the scales are NOT written by
                           the kernel that precedes this launch on the stream (weights are constants in a decode loop). */
#define AFB_FLAG_DUMP_DECODE_PAIRING 16u /* afb_dequant_dump only ([N,K] layout): unpack with the decode kernel's routines (strided pairing,
                                         integer values, no scale) instead of the prefill kernel's; the output is in natural k order either way */

/*
 * Kernel argument block.  The first ten fields are the reference's packed kernarg
 * block, same order and types (bfAintBGemm.cc:119-133; bf16gemm_kernel_gfx90a.s:97-108).
 * Leading dimensions are in ELEMENTS (for 4-bit B: in 4-bit elements, so bytes = ldb/2).
 * The appended fields select what the reference fixed at compile time.
 */
typedef struct afb_gemm_args {
    void*    ptr_c;      /* bf16 [M,N] row-major, ldc                                   */
    void*    ptr_a;      /* bf16 [M,K] row-major, lda                                   */
    void*    ptr_b;      /* packed integers, see b_layout / b_bits / b_encoding         */
    void*    ptr_scale;  /* group_size == 0: [N];  else [N][K/group_size] (n-major)      */
    uint32_t m, n, k;
    uint32_t lda, ldb, ldc;
    uint32_t b_bits;      /* 8 or 4 (4: two per byte along K, low nibble = even k; COL layout only) */
    uint32_t b_encoding;  /* AFB_ENC_*                                                   */
    uint32_t b_layout;    /* AFB_LAYOUT_*                                                */
    uint32_t scale_dtype; /* AFB_SCALE_*                                                 */
    uint32_t group_size;  /* 0 = one scale per output channel; else K-elements per scale */
    uint32_t variant;     /* AFB_VARIANT_*                                               */
    uint32_t flags;       /* AFB_FLAG_*                                                  */
    uint32_t reserved;    /* must be 0                                                   */
    void*    ptr_zero;    /* optional zero-points (NULL = symmetric quantisation): one BYTE per scale entry, same shape as the scales
                             ([N] or [N][K/group_size], n-major), in the weights' own encoding (int8: like a stored byte; int4: like a
                             stored nibble, in the low 4 bits).  The weight value is decode(stored) - decode(zero): the reference's fixed
                             "stored - 128" (bf16gemm_kernel_gfx90a.s:210, mem_transfer.hpp:30) made a per-channel / per-group quantity */
    uint64_t reserved2;   /* must be 0                                                   */
} afb_gemm_args;

/* ---- device / memory / events: one per HIP call of the reference driver --------- */
/* hipSetDevice (bfAintBGemm.cc:63) + module load (:65-66): selects the device, creates
 * the per-device context (status word, split-K workspace, tensor-map entry point).   */
int afb_init(int device);
int afb_finalize(void);
int afb_device_count(int* count);
int afb_sm_count(int* count);
/* hipMalloc / hipFree (simple_device_mem.hpp:20,25) */
int afb_malloc(void** ptr, size_t bytes);
int afb_free(void* ptr);
/* pinned host memory for the end-to-end path (no reference counterpart: the reference uses malloc) */
int afb_malloc_host(void** ptr, size_t bytes);
int afb_free_host(void* ptr);
/* hipMemcpy H2D / D2H (bfAintBGemm.cc:99-101,158,211) */
int afb_memcpy_h2d(void* dst, const void* src, size_t bytes);
int afb_memcpy_d2h(void* dst, const void* src, size_t bytes);
int afb_memcpy_d2d(void* dst, const void* src, size_t bytes);
int afb_memset(void* dst, int value, size_t bytes);
/* hipEventCreate / Record / Synchronize / ElapsedTime / Destroy (bfAintBGemm.cc:171-184) */
int afb_event_create(void** event);
int afb_event_record(void* event, void* stream);
int afb_event_sync(void* event);
int afb_event_elapsed_ms(float* ms, void* start, void* stop);
int afb_event_destroy(void* event);
int afb_stream_create(void** stream);
int afb_stream_sync(void* stream);
int afb_stream_destroy(void* stream);
/* hipDeviceSynchronize (bfAintBGemm.cc:173,181) */
int afb_device_sync(void);

/* ---- the hot path ------------------------------------------------------------- */
/* hipModuleLaunchKernel (bfAintBGemm.cc:152,176): validates args, picks the variant,
 * decides grid/block/shared memory/tensor maps itself and launches asynchronously on
 * `stream` (NULL = the default stream).  Pointers are DEVICE pointers.
 * GEMMs that split K between CTAs (decode K-slices, short last wave of prefill tiles) meet in an
 * fp32 workspace that belongs to the STREAM they are launched on: launches on one stream are
 * serialised by the stream, launches on different streams use different workspaces (32 MiB each).
 * afb_init allocates four of them; a fifth and later stream allocates its own on its first such
 * launch, which then must not happen inside a stream capture; at most 16 streams per device, after
 * that AFB_ERR_TOO_LARGE.  A captured graph keeps using the workspace of the stream it was captured on. */
int afb_gemm_launch(const afb_gemm_args* args, void* stream);
/* Which variant AFB_VARIANT_AUTO resolves to for these args (no launch). */
int afb_gemm_resolve_variant(const afb_gemm_args* args, uint32_t* variant);
/* The whole reference sequence "H2D x3, launch, D2H" (bfAintBGemm.cc:99-101,152,211)
 * as one call on HOST pointers: copies A, B, scale to library-owned device staging,
 * launches, copies C back, and returns when C is in host memory.                     */
int afb_gemm_host(const afb_gemm_args* host_args, void* stream);
/* The same without the final wait: returns when the copies and launches are queued, so that the next call's copy-in overlaps
 * this call's GEMM and copy-out (two staging sets are used in turn; at most two calls in flight make progress at once).
 * The host buffers must stay untouched until afb_gemm_host_wait(stream) has returned: it waits for every queued call. */
int afb_gemm_host_async(const afb_gemm_args* host_args, void* stream);
int afb_gemm_host_wait(void* stream);
/* No counterpart in the reference.  The decode GEMM (M <= 16, B in [N,K] layout) for callers that must not
 * allocate: programs whose framework already owns all device memory, and latency-critical loops that cannot
 * afford the device-wide synchronisation of cudaMalloc.  Needs no afb_init and calls no cudaMalloc / cudaFree or
 * other allocating routine: its split-K scratch is a fixed array inside the library image (about 4 MiB).
 * Limits: M * N <= 524288 and N <= 524288, else AFB_ERR_TOO_LARGE.  All calls on a device share the array:
 * calls that overlap on the GPU race, so keep them on one stream.
 * The first call on each device is the set-up call: it looks up the array's device address and enqueues a
 * clearing memset on `stream`.  With CUDA's default lazy module loading that first call is also the moment the
 * driver places this library's image -- the array and the kernel code -- in device memory, so it is not free of
 * driver-side allocation or synchronisation: make it once per device at start-up, before the host framework
 * takes the rest of the memory and before any stream capture (or run with CUDA_MODULE_LOADING=EAGER).  From
 * the second call on, nothing is allocated by anyone. */
int afb_gemm_launch_static(const afb_gemm_args* args, void* stream);
/* Weight pre-packing, the offline step before the GEMM (extends the reference's host-side format conversion,
 * mem_transfer.hpp:12-32 called at bfAintBGemm.cc:96-97).  Reads args->ptr_b / n / k / ldb / b_bits / b_layout
 * (AFB_LAYOUT_ROW [K,N] int8, or AFB_LAYOUT_COL [N,K] int8 / int4) and writes the same integers as
 * AFB_LAYOUT_COL_PACKED into out_b: [N,K], pitch out_ldb elements, inside every 32-bit word the order
 *   int8: bytes [k0,k2,k1,k3]      int4: nibbles [k0,k2,k4,k6,k1,k3,k5,k7]
 * which is the order the kernels' unpack reads as pairs, so they skip the re-pairing of the activations (decode)
 * or of the weights (prefill).  A GEMM on the result sets b_layout = AFB_LAYOUT_COL_PACKED, ptr_b = out_b,
 * ldb = out_ldb; its result is bit-identical to the GEMM on the plain [N,K] weights.  [N,K] input may be packed
 * in place (out_b == ptr_b, out_ldb == ldb).  Asynchronous on `stream`. */
int afb_prepack(const afb_gemm_args* args, void* out_b, uint32_t out_ldb, void* stream);
/* ---- fused neighbours of the GEMM ------------------------------------------------ */
/* The reference's stated purpose is "gemm fusion for llm" (README.md:2); its kernel fuses dequantisation into the GEMM
 * (bf16gemm_kernel_gfx90a.s:410-489).  These entry points fuse what stands on the other side of it in a gated MLP:
 *     v[m,r]  = (A x dequant(B)^T)[m,r] + bias[r]                        r = row of B, bias optional
 *     plain:    C[m,r] = act(v[m,r]) + residual[m,r]
 *     gated:    C[m,i] = act(v[m,2i]) * v[m,2i+1] + residual[m,i]          rows 2i / 2i+1 of B = gate / up projection of channel i
 * all in fp32 from the fp32 accumulator, rounded to bf16 once.  gemm.n counts the rows of B (twice the output channels when
 * gated), gemm.ptr_c / gemm.ldc describe the bf16 result [M, N_out].  B in [N,K] layout, plain or pre-packed.            */
#define AFB_ACT_NONE 0u
#define AFB_ACT_SILU 1u   /* x / (1 + exp(-x)) */
typedef struct afb_fused_args {
    afb_gemm_args gemm;
    uint32_t gated;          /* 0 / 1 */
    uint32_t activation;     /* AFB_ACT_* */
    void*    ptr_bias;       /* optional fp32 [gemm.n] */
    void*    ptr_residual;   /* optional bf16 [M, N_out] */
    uint32_t ld_residual;    /* elements */
    uint32_t reserved;       /* must be 0 */
} afb_fused_args;
int afb_gemm_fused_launch(const afb_fused_args* args, void* stream);
/* Builds the B of a gated launch from two separate projections of equal shape and format ([N,K] plain layout): row 2i of the
 * output is row i of the gate projection, row 2i+1 row i of the up projection, in the pre-packed word order (AFB_LAYOUT_COL_PACKED,
 * pitch out_ldb elements); scales (and zero-points, when gate->ptr_zero is set) are interleaved the same way into out_scale
 * (and out_zero).  gate->n is N, the output has 2N rows.  Asynchronous on `stream`. */
int afb_prepack_gated(const afb_gemm_args* gate, const void* b_up, const void* scale_up, const void* zero_up, void* out_b,
                      uint32_t out_ldb, void* out_scale, void* out_zero, void* stream);
/* Dequantised weights exactly as the kernels feed them to the tensor cores:
 * out is bf16 with B's logical shape and layout ([N,K] ld=K for COL, [K,N] ld=N for ROW).
 * group_size == 0: the exact integer value; else bf16_rn(float(q) * float(scale)).
 * This is the bit-exact unpack + dequant contract (reference: .dequant_int8_4x1,
 * bf16gemm_kernel_gfx90a.s:18-55, constants :204-210).                                */
int afb_dequant_dump(const afb_gemm_args* args, void* out_bf16, void* stream);
/* Reads (synchronously) the status words the last kernels on this device wrote:
 * out[0] = 0 or AFB_ERR_TIMEOUT, out[1..3] = where the wait gave up.  Clears them.   */
int afb_read_status(int32_t out[4]);

/* ---- row-parallel (K-split) exchange over peer memory --------------------------- */
/* No reference counterpart (the reference is single-GPU, bfAintBGemm.cc:63).  One process per GPU;
 * buffers allocated with afb_malloc are exported to the other processes of the box and mapped there. */
#define AFB_IPC_HANDLE_BYTES 64
#define AFB_MAX_RANKS 8
int afb_ipc_export(void* dev_ptr, unsigned char handle[AFB_IPC_HANDLE_BYTES]);
int afb_ipc_import(const unsigned char handle[AFB_IPC_HANDLE_BYTES], void** dev_ptr);
int afb_ipc_release(void* dev_ptr);

/* All-reduce of the K-split partial sums as ONE kernel per GPU over peer memory (plain peer
 * loads/stores through NVLink; the broadcast of the result may use an NVSwitch multicast store): rank r waits until every rank's partial is complete,
 * sums rows block r of all `world` partials in rank order (fp32), rounds to bf16 and stores the
 * result into every rank's C, then waits until every rank has stored its block here.  When the
 * kernel ends on a rank, that rank's C holds the complete sum and no peer reads its partial any more.
 * Pointer arrays are indexed by rank and hold addresses valid in THIS process (own buffers: the
 * local pointer; peers': afb_ipc_import).  `signals[r]` is rank r's uint32[2 * AFB_MAX_RANKS] array,
 * zero before first use.  `epoch` must increase by one per call, identically on all ranks, from 1.
 * Every wait is bounded; on expiry the kernel returns and afb_read_status reports AFB_ERR_TIMEOUT. */
typedef struct afb_allreduce_args {
    void*     partial[AFB_MAX_RANKS]; /* [M,N] ld = ld_partial; fp32 (partial_f32 = 1) or bf16 */
    void*     c[AFB_MAX_RANKS];       /* bf16 [M,N], ldc */
    uint32_t* signals[AFB_MAX_RANKS];
    uint32_t  rank, world;
    uint32_t  m, n, ld_partial, ldc;
    uint32_t  partial_f32;
    uint32_t  epoch;
    uint32_t  wait_ms;                /* bound of each wait in milliseconds (0 = 2000) */
    uint32_t  reserved;
    void*     c_multicast;            /* optional (NULL = unused): an NVLink multicast address bound to the same bytes as every
                                       * c[q] (same offset in all of them).  The result rows then leave this GPU once, as
                                       * multimem.st, and the switch writes them into every rank's C; c[] is not written. */
} afb_allreduce_args;
int afb_ksplit_allreduce_launch(const afb_allreduce_args* args, void* stream);
/* Tile-granular form of the same exchange, fused with the K-split GEMM: afb_gemm_launch_tiles is the prefill GEMM
 * (int8, per-channel scales, fp32 partial sums, M > 128) that also adds `arrivals` to tile_done[t] when tile t of its
 * output is stored (release at system scope; counters only grow, start them at zero).  afb_ksplit_tile_allreduce_launch,
 * launched AFTER it on another stream, handles the tiles this rank owns (t % world == rank) as soon as every rank has
 * counted them (tile_done[r][t] >= arrivals * tile_epoch), so the NVLink traffic overlaps the GEMM main loop.  The GEMM never
 * waits for the exchange kernel; if the two are serialised, launch order makes the GEMM run first.  Tile geometry and the
 * number of counters come from afb_ksplit_tile_info.  Same signals, epochs and bounded waits as above. */
typedef struct afb_tile_allreduce_args {
    afb_allreduce_args base;                 /* partial_f32 must be 1; base.epoch orders the "block in place" signals */
    uint32_t*          tile_done[AFB_MAX_RANKS];
    uint32_t           tile_epoch;           /* how many afb_gemm_launch_tiles have been issued on these counters (same on all ranks) */
    uint32_t           reserved;
} afb_tile_allreduce_args;
int afb_ksplit_tile_info(uint32_t m, uint32_t n, uint32_t* tile_m, uint32_t* tile_n, uint32_t* num_tiles, uint32_t* arrivals);
int afb_gemm_launch_tiles(const afb_gemm_args* args, uint32_t* tile_done, void* stream);
int afb_ksplit_tile_allreduce_launch(const afb_tile_allreduce_args* args, void* stream);
/* Reduce-scatter fused into the GEMM epilogue: the prefill GEMM (int8, per-channel scales, M a multiple of 256 * world) stores
 * every tile of its fp32 partial sums straight into the staging buffer of the rank that owns those rows, over NVLink:
 * stage[o] is rank o's float[world][M / world][N] buffer (mapped in this process), and this rank fills slot `rank` of each.
 * args->ptr_c is ignored unless AFB_FLAG_PUSH_VIA_LOCAL is set.  Follow it, on the same stream, with afb_ksplit_allreduce_launch whose partial[q] point at the
 * LOCAL slots (partial[q] = own_stage + (q * (M/world) - rank * (M/world)) * N floats, ld_partial = N): its first phase then
 * waits for every rank's GEMM, its sum reads local memory only, and its second phase broadcasts the bf16 rows. */
int afb_gemm_launch_push(const afb_gemm_args* args, void* const stage[AFB_MAX_RANKS], uint32_t world, uint32_t rank, void* stream);
/* ---- the sharded GEMM from ONE process (one host thread, one stream per GPU, peer access instead of IPC) ---------
 * The multi-GPU extension of the reference driver's single-device set-up (bfAintBGemm.cc:63).  afb_dist_init(ngpus)
 * initialises devices 0 .. ngpus-1 (afb_init on each), enables peer access between all pairs and creates one stream per
 * GPU; afb_dist_gemm_launch issues one sharded GEMM on those streams and returns without waiting; afb_dist_sync waits
 * for all of them.  shard[r] holds DEVICE-r pointers.
 *   AFB_SPLIT_N  column-parallel: shard[r] is an ordinary GEMM on GPU r's channels, written to its own ptr_c.  No collective.
 *   AFB_SPLIT_K  row-parallel (int8, per-channel scales): shard[r] multiplies A[:, K_r] by B[:, K_r] (same m and n on every
 *                rank; shard[r].ptr_c is ignored); the fp32 partial sums are added in rank order over NVLink peer memory and
 *                every c[r] (bf16 [M,N], ld = N, on GPU r) receives the complete result.  The reduce-scatter runs in the
 *                GEMM epilogue when M is a multiple of 256 * ngpus, else in the exchange kernel. */
#define AFB_SPLIT_N 0u
#define AFB_SPLIT_K 1u
typedef struct afb_dist afb_dist;
typedef struct afb_dist_gemm_args {
    afb_gemm_args shard[AFB_MAX_RANKS];
    void*    c[AFB_MAX_RANKS];   /* AFB_SPLIT_K only */
    uint32_t split;              /* AFB_SPLIT_* */
    uint32_t wait_ms;            /* bound of each cross-GPU wait (0 = 2000) */
} afb_dist_gemm_args;
int afb_dist_init(uint32_t ngpus, afb_dist** dist);
int afb_dist_world(const afb_dist* dist, uint32_t* world);
int afb_dist_stream(afb_dist* dist, uint32_t rank, void** stream);   /* GPU `rank`'s stream: for events and copies ordered with the GEMMs */
int afb_dist_gemm_launch(afb_dist* dist, const afb_dist_gemm_args* args);
int afb_dist_sync(afb_dist* dist);
int afb_dist_finalize(afb_dist* dist);
/* [lo, hi) of `total` owned by `rank`: whole units of `multiple`, the remainder to the first ranks.  Needs no GPU. */
int afb_dist_split_range(uint32_t total, uint32_t world, uint32_t rank, uint32_t multiple, uint32_t* lo, uint32_t* hi);
/* Pipelined form of the epilogue reduce-scatter: the pushing GEMM takes its tiles column chunk by column chunk (the N channels
 * cut into `sub_blocks` chunks) and, inside a chunk, owner by owner starting with its own rank, so that every `world` units one
 * more chunk of EVERY rank's rows is complete in that rank's staging slots; each finished tile is counted in
 * counters[owner][chunk] (uint32[sub_blocks] per rank, zero before first use, only grow).  afb_ksplit_sub_allreduce_launch,
 * launched on ANOTHER stream so that it runs next to the GEMM (on SMs of its own: the pipelined GEMM's grid leaves
 * AFB_SUB_AR_SMS of them free, default 16, and the two kernels never share an SM), waits for a chunk's count, sums the LOCAL
 * slots in rank order, rounds and broadcasts it while the GEMM works on the next chunk: only the last chunk is left after the GEMM.  base.partial[q]
 * are the local slots as for afb_gemm_launch_push; base.signals / epoch as for afb_ksplit_allreduce_launch; `launches` = how
 * many pipelined GEMMs have been issued on these counters (same on all ranks).  N must be a multiple of 128 * sub_blocks. */
typedef struct afb_sub_allreduce_args {
    afb_allreduce_args base;
    uint32_t* counters;      /* this rank's counters */
    uint32_t  sub_blocks;
    uint32_t  launches;
    uint32_t  reserved;
} afb_sub_allreduce_args;
int afb_ksplit_sub_info(uint32_t m, uint32_t n, uint32_t world, uint32_t sub_blocks, uint32_t* counts_per_chunk);
int afb_gemm_launch_push_pipelined(const afb_gemm_args* args, void* const stage[AFB_MAX_RANKS], uint32_t* const counters[AFB_MAX_RANKS],
                                   uint32_t world, uint32_t rank, uint32_t sub_blocks, void* stream);
int afb_ksplit_sub_allreduce_launch(const afb_sub_allreduce_args* args, void* stream);
/* Both halves in ONE launch: the pushing GEMM of afb_gemm_launch_push_pipelined with two extra warps per CTA that do what
 * afb_ksplit_sub_allreduce_launch does (x: exactly as for that entry point, with x->counters == counters[rank]), so that no second
 * kernel shares the SMs with the GEMM.  When the launch has completed, this rank's C holds the complete result.  No counterpart in
 * the reference (single GPU). */
int afb_gemm_launch_push_exchange(const afb_gemm_args* args, void* const stage[AFB_MAX_RANKS], uint32_t* const counters[AFB_MAX_RANKS],
                                  uint32_t world, uint32_t rank, uint32_t sub_blocks, const afb_sub_allreduce_args* x, void* stream);
/* sizeof(afb_gemm_args), sizeof(afb_allreduce_args), sizeof(afb_tile_allreduce_args), sizeof(afb_fused_args) as this library was
 * compiled: a binding in another language compares them with its own declarations before the first call.  Needs no GPU. */
int afb_abi_sizes(uint32_t sizes[4]);
/* fp32 [rows, cols] (ld_src) -> bf16 (ld_dst), round to nearest even: finishes a K-split whose partial
 * sums were combined by a library collective instead of afb_ksplit_allreduce_launch. */
int afb_cast_f32_to_bf16(void* dst_bf16, const void* src_f32, uint32_t rows, uint32_t cols, uint32_t ld_dst, uint32_t ld_src, void* stream);

/* ---- diagnostics ------------------------------------------------------------- */
const char* afb_status_string(int status);
int afb_last_cuda_error(void);             /* cudaError_t of the last failing CUDA call */
const char* afb_last_cuda_error_string(void);
/* Launch-floor probes (measurement aid): kind 0 launches a kernel with the given grid (256 threads per CTA) and dynamic shared
 * memory that does nothing; kind 1 one that only reads `bytes` at `src` with the decode kernel's access pattern.  flags:
 * AFB_FLAG_PDL or 0.  Timed like the decode kernels they show how much of a few-microsecond GEMM is launch and ramp. */
int afb_probe_launch(uint32_t kind, const void* src, size_t bytes, uint32_t ctas, uint32_t smem_bytes, uint32_t flags, void* stream);
/* Phase timestamps of the last row-parallel GEMM + exchange on the current device (measurement aid; written only while the
 * environment variable AFB_PHASE_TIMESTAMPS is set).  Nanoseconds of this GPU's own timer: out[0] GEMM start, [1] GEMM end,
 * [2] exchange kernel start, [3] every rank's GEMM seen complete, [4] sum and broadcast done, [5] every rank's block seen in
 * place.  Synchronises the device and clears the record. */
int afb_phase_timestamps(unsigned long long out[8]);
/* Number of kernels this library launched since afb_init (all variants). */
unsigned long long afb_launch_count(void);
const char* afb_version(void);

#ifdef __cplusplus
}
#endif
#endif /* AFB_CAPI_H_ */
