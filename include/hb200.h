/*
 * hb200 - C ABI of the B200 implementation of herbert-metal-bf16's bf16
 * matrix-multiply path (prefill GEMM, decode matvec, MoE grouped GEMM) and of
 * the load-time loop that chooses among kernel candidates.
 *
 * The reference engine has no FFI for this path: its seam is the internal
 * Rust API between the engine (src/metal/qwen.rs) and the kernel emitter plus
 * device layer (src/msl, src/metal/gpu.rs). Each entry point below names the
 * reference item it stands for (path:line inside the reference project).
 *
 * Conventions: every function returns an hb_status (0 = ok) and never aborts
 * or throws across the boundary (reference: Result<T, HerbertError>,
 * src/core/error.rs:9-27). hb_last_error() gives the message of the last
 * failure on a context. A context is not thread-safe: one context, one host
 * thread, one CUDA stream (reference: one engine, one queue,
 * src/metal/gpu.rs:59-74). A process may hold contexts on several devices:
 * every call that allocates, copies, builds or launches makes its context's
 * device the calling thread's current one. Buffers are device memory; the reference's
 * host-visible shared buffers become explicit hb_upload/hb_download copies.
 * All matrices are row-major; bf16 values are passed as uint16_t bits.
 */
#ifndef HB200_H
#define HB200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct hb_ctx hb_ctx;
typedef struct hb_kernel hb_kernel;

typedef enum {
    HB_OK = 0,
    HB_INVALID = 1,     /* bad argument, range too small, misaligned pointer */
    HB_UNSUPPORTED = 2, /* a kernel that cannot be built for this shape/tile: the caller skips the candidate
                           (reference: Gpu::pipeline -> Err, "not built", src/metal/qwen.rs:2266) */
    HB_BACKEND = 3,     /* CUDA failure (reference: HerbertError::Backend, src/core/error.rs:19) */
    HB_OOM = 4,
    HB_KERNEL = 5       /* a kernel reported a failed bounded wait through the status buffer */
} hb_status;

/* Epilogue of a projection (reference: enum Out, src/metal/kernels.rs:30-42). */
typedef enum {
    HB_OUT_BF16 = 0,     /* y = bf16(acc) */
    HB_OUT_F32 = 1,      /* y = acc */
    HB_OUT_RESIDUAL = 2, /* y = bf16(f32(y) + f32(bf16(acc))) */
    HB_OUT_SWIGLU = 3    /* W = [gate | up] rows; y[.., n/2] = bf16(g*sigmoid(g)*u), g and u rounded to bf16 first */
} hb_out;

/* Which rows a GEMM reads and writes (reference: enum MmaRows, src/metal/prefill.rs:317-328). */
typedef enum {
    HB_ROWS_DENSE = 0,
    HB_ROWS_GATHER = 1, /* expert tiles: sorted row p reads X[list[p] / top_k], writes Y[p] */
    HB_ROWS_SCATTER = 2, /* expert tiles: sorted row p reads X[p], writes Y[list[p]] */
    HB_ROWS_SORTED = 3   /* expert tiles over rows gathered beforehand (moe_gather): reads X[p], writes Y[p]
                            (reference: the expert branch of gemm_mm2d_rows, src/metal/prefill.rs:534-552) */
} hb_rows_mode;

/* A range of device memory (reference: Range{buf, offset, size}, src/metal/gpu.rs:32-47). */
typedef struct {
    void* ptr;
    size_t size;
} hb_range;

/* One recorded launch (reference: Op{pipe, ranges, groups}, src/metal/qwen.rs:650). The grid is derived
 * from `m`, the row count the reference keeps in state[STATE_ROWS] (src/metal/kernels.rs:10-15). */
typedef struct {
    const hb_kernel* kernel;
    const hb_range* args;
    int nargs;
    uint32_t m;
} hb_op;

/* ---- device and buffers ------------------------------------------------ */

/* Gpu::open, src/metal/gpu.rs:70. Fails with HB_BACKEND when no sm_100 device is present:
 * there is no CPU fallback. */
int hb_open(int device, hb_ctx** out);
/* Buffers and kernels of the context are freed here (the reference never frees, gpu.rs:62). */
int hb_close(hb_ctx* ctx);
/* Message of the last failure; ctx may be NULL for a failed hb_open. */
const char* hb_last_error(const hb_ctx* ctx);
/* Gpu::summary, src/metal/gpu.rs:81. */
int hb_describe(hb_ctx* ctx, char* buf, size_t len);
/* Use an existing CUDA stream (cudaStream_t) for every later launch and copy; NULL restores the
 * context's own stream. For callers that order these kernels with their own collectives. */
int hb_set_stream(hb_ctx* ctx, void* cuda_stream);
/* Gpu::alloc, src/metal/gpu.rs:92-123: zero-initialised, 256-byte aligned, owned by the context. */
int hb_alloc(hb_ctx* ctx, size_t bytes, void** dptr);
/* Test hook: hb_alloc fails with HB_OOM once the context holds more than `bytes` (0 = no limit). */
int hb_set_alloc_limit(hb_ctx* ctx, size_t bytes);
/* The reference writes and reads its shared buffers through raw pointers while the GPU is idle
 * (src/metal/qwen.rs:2764); here these are stream-ordered copies followed by a synchronisation. */
int hb_upload(hb_ctx* ctx, void* dst_device, const void* src_host, size_t bytes);
int hb_download(hb_ctx* ctx, void* dst_host, const void* src_device, size_t bytes);
int hb_memset(hb_ctx* ctx, void* dst_device, int value, size_t bytes);
/* Waits for the stream and checks the kernels' status words (command-buffer status, gpu.rs:215-218). */
int hb_sync(hb_ctx* ctx);
/* Number of kernels this context has enqueued so far. */
uint64_t hb_launch_count(const hb_ctx* ctx);

/* ---- peer memory ---------------------------------------------------------
 * One process per GPU: a buffer of hb_alloc is made visible to the other processes of the node by passing the
 * 64-byte handle of hb_ipc_export to them (any channel) and opening it there; the pointer hb_ipc_open returns is
 * valid in kernels of that process (loads and stores cross NVLink). Close before the owner frees. No reference
 * counterpart. */
#define HB_IPC_HANDLE_BYTES 64
int hb_ipc_export(hb_ctx* ctx, void* dptr, void* handle64);
int hb_ipc_open(hb_ctx* ctx, const void* handle64, void** dptr);
int hb_ipc_close(hb_ctx* ctx, void* dptr);

/* A barrier among the ranks of one node (one process and one GPU each) as a kernel on the stream, with an optional
 * all-gather of a small table riding on it. Every rank owns flags u32[64] (256 bytes, zeroed) in a buffer the others
 * have opened; `peers_flags` is a device array u64[world] of their addresses. The barrier numbers itself (word 32 of
 * a rank's own flags counts the barriers it has passed: 1, 2, 3, ... in the same sequence on every rank), so
 * hb_launch's m is ignored and a recorded launch can be replayed. With words > 0 the kernel first copies `payload` u32[words] into
 * slot `rank` of every rank's gather buffer u32[world][words] (`peers_gather`: their addresses); use two gather
 * buffers in turn, a rank may start the next gather while another still reads this one. What a rank wrote before
 * the barrier, to its own or a peer's memory, is visible to all after it. A rank that does not arrive within a few
 * seconds turns into HB_KERNEL on the others at their next hb_sync. Never launch it for two ranks on one GPU.
 * Bindings: peers_flags[, payload, peers_gather]. */
int hb_peer_sync_get(hb_ctx* ctx, uint32_t words, uint32_t world, uint32_t rank, hb_kernel** res);
/* How long a barrier waits for its peers before it gives up (default 5000 ms; 1..60000). */
int hb_set_peer_wait_ms(hb_ctx* ctx, uint32_t ms);

/* ---- copy lanes ---------------------------------------------------------
 * The reference's buffers are shared between CPU and GPU (src/metal/gpu.rs:92-110), so its engine
 * never copies activations. On a discrete GPU a prompt block crosses PCIe both ways; these calls let
 * the engine overlap the copies of one block with the kernels of another. A context has three lanes,
 * each an in-order queue: the kernels' lane (hb_launch, hb_run, hb_memset and the synchronous copies
 * above), an upload lane and a download lane. Nothing orders one lane against another except events:
 * hb_lane_record marks the work a lane holds so far, hb_lane_wait makes a lane's later work wait for
 * a mark on the device (the host does not block), hb_event_sync makes the host wait. Waiting for an
 * event that was never recorded returns at once. Host memory of the asynchronous copies must come
 * from hb_host_alloc (page-locked); with pageable memory the copies still happen but do not overlap. */
typedef struct hb_event hb_event;
enum { HB_LANE_KERNELS = 0, HB_LANE_UPLOAD = 1, HB_LANE_DOWNLOAD = 2 };
int hb_event_new(hb_ctx* ctx, hb_event** out);
int hb_event_free(hb_ctx* ctx, hb_event* ev);
int hb_lane_record(hb_ctx* ctx, int lane, hb_event* ev);
int hb_lane_wait(hb_ctx* ctx, int lane, const hb_event* ev);
int hb_event_sync(hb_ctx* ctx, const hb_event* ev);
int hb_upload_async(hb_ctx* ctx, void* dst_device, const void* src_host, size_t bytes);   /* upload lane */
int hb_download_async(hb_ctx* ctx, void* dst_host, const void* src_device, size_t bytes); /* download lane */
int hb_host_alloc(hb_ctx* ctx, size_t bytes, void** host_ptr);
int hb_host_free(hb_ctx* ctx, void* host_ptr);

/* ---- kernels ------------------------------------------------------------ */

/* Prefill GEMM Y[m][n] = out(X[m][k] . W[n][k]^T), bf16 inputs, f32 accumulation on the tensor cores.
 * Stands for the emitters gemm_mma_rows / gemm_mm2d / gemm_nax_swiglu and the expert-tile forms
 * (src/metal/prefill.rs:838,852-1301,442-567,755-822; rows modes :317-328,889-941,1206-1209).
 * Bindings: DENSE  W, X, Y             (reference order state, W, X, Y; prefill.rs:416-417)
 *           GATHER / SCATTER / SORTED  W, X, Y, list, tiles   (prefill.rs:836-837)
 * For GATHER/SCATTER `n` is the rows of ONE expert in W ([experts*n][k]) and `m` is the number of token rows
 * of the block; the tile table tells the kernel how many sorted rows there are. */
typedef struct {
    uint32_t k, n;
    uint32_t out;       /* hb_out */
    uint32_t rows_mode; /* hb_rows_mode */
    uint32_t top_k;     /* GATHER: slots per token row */
    uint32_t experts;   /* GATHER/SCATTER */
    uint32_t bm;        /* GATHER/SCATTER: rows of an expert tile, 16/32/64 (moe.tile) */
    uint32_t tile_n;    /* DENSE: accumulator columns per tile, 64/128/256 (0 = default 256); with cta_pair also 192
                           (256 x 192 tiles: for shapes whose 256 x 256 tiles leave the last wave of SM pairs nearly empty) */
    uint32_t stages;    /* shared-memory pipeline depth, 0 = as many as fit */
    uint32_t cta_pair;  /* DENSE: 1 = two CTAs share a 256-row tile (tcgen05 cta_group::2) */
    uint32_t m_first;   /* tile order: 1 = walk the row tiles of a column tile first (gemm.mfirst, prefill.rs:26-42) */
    uint32_t rows_max;  /* largest m this kernel will be launched with (sizes the tile table in expert modes) */
    uint32_t stream_k;  /* DENSE: 1 = the (tile, k-block) units are divided evenly among the CTAs of a persistent grid;
                           a tile cut by a boundary is completed through f32 partial tiles in scratch memory owned by
                           the context (allocated at the first such hb_gemm_get). Removes the idle tail when the tile
                           count is not a multiple of the SM count, and splits K for short row buckets. */
    uint32_t merge_runs; /* expert modes: 1 = the consecutive tiles of one expert are merged into work items of up to
                            128 rows, so that an expert's weights are read once whatever the tile size */
    uint32_t y_shards;   /* DENSE, cta_pair, Out::F32: P > 1 = Y is cut into P blocks of ceil(m / P) rows and the Y binding
                            is a device array u64[P] of the blocks' addresses (16-byte aligned, row stride n), which may be
                            other GPUs' memory opened with hb_ipc_open: the GEMM of a row-parallel projection stores every
                            block of its partial product straight into the buffer of the rank that sums it, tile by tile
                            while it computes; the CTA-pair form stores whole 128-byte row segments (the form to use when
                            the blocks are peers' memory). No reference counterpart */
    uint32_t y_group_rows; /* with y_shards = P: 0 = block b holds the contiguous rows [b * ceil(m / P), ...); G > 0 (a
                            multiple of 32 * P, at most 256) = the rows are dealt in groups of G: block b holds, for every
                            group g, the G / P rows [g * G + b * G / P, ...) at its rows [g * G / P, ...). Every rank then
                            sums a slice of every group, and the sum of a group can start while the GEMM works on the next */
    uint32_t y_signal;   /* with y_group_rows = 256: r + 1 = this GEMM runs on rank r of the y_shards ranks and tells the
                            summing ranks when a group of rows is complete (0 = it tells nobody). Two more bindings follow Y: flag_table, a device array u64[P] of the addresses of every rank's
                            flags u32[P][HB_TP_MAX_GROUPS], and ctl, this rank's own control words u32[HB_TP_CTL_WORDS]
                            (zeroed once). When the last tile of group g is stored, flag [rank][g] of every rank is set to
                            ctl[0] + 1, the step's number, which hb_tp_sum_stream_get's kernel waits for and then writes
                            to ctl[0]. The tiles are walked group by group (m_first is ignored). */
    uint32_t split_k;    /* DENSE, cta_pair: S = 2..64 = every 256 x 256 tile is computed as S work items, one per equal slice
                            of K, so that a short block (few tiles) still gives every SM work at the tile size that reads
                            the operands least often; the slices of a tile hand a running f32 sum from one to the next
                            through scratch memory of the context (slice order, so the same bits whoever runs when) and the
                            last one applies the output mode. For blocks of at most 1024 rows. */
} hb_gemm_desc;
int hb_gemm_get(hb_ctx* ctx, const hb_gemm_desc* desc, hb_kernel** out);

typedef enum { HB_X_PLAIN = 0, HB_X_NORM = 1, HB_X_SWIGLU = 2 } hb_x_src;

/* Decode matvec y[r][n] = out(W[n][k] . x[r][k]) for m = 1..8 activation rows, an HBM-streaming kernel on the
 * CUDA cores: 128-bit loads, f32 FMA chains, warp-shuffle sums. Stands for matvec / matvec_split
 * (src/metal/kernels.rs:146-214,502-981). Bindings: W, x, y (kernels.rs:145). The reference is m = 1 only;
 * rows 2..8 apply the same per-row contract. */
typedef struct {
    uint32_t k, n;
    uint32_t out;           /* BF16, F32, RESIDUAL, SWIGLU (y of n/2, kernels.rs:934-944) */
    uint32_t rows_max;      /* 1..8 activation rows (1..64 with tensor_core) */
    uint32_t rows_per_warp; /* W rows one warp reduces: 1, 2, 4 or 8 (the reference's `rows`) */
    uint32_t split;         /* K split across the warps of a block: 1, 2 or 4 (mv.split) */
    uint32_t persist;       /* 1 = a fixed grid that loops over the row groups (mv.persist) */
    uint32_t x_stationary;  /* 1 = for 2..8 activation rows: K is split across the threads of a persistent block and
                               each thread keeps its slice of the activations widened in registers; rows_per_warp
                               (2 or 4) is then the W rows reduced per step; needs K * rows <= 32768 */
    uint32_t tensor_core;   /* > 0 = the product runs on the tensor cores as a weight stream (W rows are the 128-row
                               operand of tcgen05.mma, the activation rows its narrow side): rows_max up to 64.
                               1 = a CTA takes blocks of 128 features over all of K; 2 = the (feature block, 64-element
                               K block) units are dealt evenly, one contiguous range per SM, and blocks shared by
                               several SMs are summed from f32 partials in K order; 3 = as 1 with blocks of fewer
                               features (n / (SMs x waves), at most 128), so that the blocks fill whole waves of
                               SMs (one SM takes in 60-76 GB/s: 96 blocks of 128 features cannot stream 12288
                               features at the HBM rate, 147 blocks of 84 can). Accumulation order inside a
                               range is the tensor core's, as in the prefill GEMM. `split` (1, 2 or 4) is then the
                               number of neighbouring K blocks one pipeline stage holds (longer runs per weight row
                               in DRAM) and `persist` >= 2 caps the number of stages (with half the shared memory
                               or less two consecutive kernels share an SM, see hb_set_launch_overlap); the other
                               form fields are ignored. */
    uint32_t argmax;        /* Out::Bf16 only: 1 = also the index of the largest output of every row, the first on a tie
                               (argmax_partial + argmax_final, src/metal/kernels.rs:1461-1565, folded into the
                               projection: no pass over the logits, no launch of its own); 2 = the index only, y is
                               not written. A fourth binding, index u32[m], follows y. */
    uint32_t x_src;         /* hb_x_src: what the x binding holds (enum XSrc, src/metal/kernels.rs:236-252). HB_X_NORM: x is
                               the residual stream and the input of the product is its RMSNorm, made by every block in
                               shared memory first with rmsnorm_rows' sums in their order (norm_into, kernels.rs:355-442;
                               the engine's dec.fnorm, src/metal/qwen.rs:224-228,1603): one launch less a norm, the same
                               bits; k a multiple of 256, at most 8192; a binding norm_w (bf16 [k]) follows y.
                               HB_X_SWIGLU: x rows are [gate (k) | up (k)] and the input is bf16(g * sigmoid(g) * u)
                               (dec.fswi). Built for the CUDA-core form with 2 or 4 weight rows per warp, and HB_X_NORM
                               also for the tensor-core stream with at most 16 activation rows. */
    uint32_t norm_eps_bits; /* HB_X_NORM: the f32 bits of eps (the reference passes them so, XSrc::Norm{eps}) */
    uint32_t norm_plus_one; /* HB_X_NORM: 1 = the weights are w + 1 */
} hb_matvec_desc;
int hb_matvec_get(hb_ctx* ctx, const hb_matvec_desc* desc, hb_kernel** out);

/* h = bf16(g*sigmoid(g)*u) over rows of [gate(n) | up(n)]: swiglu_rows, src/metal/prefill.rs:2790-2818 (and
 * swiglu_slots over sorted expert rows, src/metal/qwen_kernels.rs:2087). Bindings: gate_up, h. */
int hb_swiglu_get(hb_ctx* ctx, uint32_t n, hb_kernel** out);
/* route_qwen, src/metal/qwen_kernels.rs:1802-1878. Bindings: scores (bf16 [m][experts]),
 * route (u32 [m][2*top_k]: experts ascending, then the f32 bits of their bf16 weights). */
int hb_route_get(hb_ctx* ctx, uint32_t experts, uint32_t top_k, hb_kernel** out);
/* moe_sort, src/metal/prefill.rs:1315-1442: stable counting sort of the (row, slot) pairs by expert and the
 * expert-tile table. Bindings: route, list (u32 [m*top_k]), tiles (u32 [1 + 3*hb_moe_tiles()]). */
int hb_moe_sort_get(hb_ctx* ctx, uint32_t experts, uint32_t top_k, uint32_t rows_max, uint32_t bm, hb_kernel** out);
/* moe_tiles, src/metal/prefill.rs:832: upper bound of the number of expert tiles. */
uint32_t hb_moe_tiles(uint32_t rows_max, uint32_t top_k, uint32_t experts, uint32_t bm);
/* moe_gather, src/metal/prefill.rs:579: XS[p] = X[list[p] / top_k]. Bindings: X, list, XS. m = token rows. */
int hb_moe_gather_get(hb_ctx* ctx, uint32_t h, uint32_t top_k, hb_kernel** out);
/* experts_matvec, src/metal/qwen_kernels.rs:1880-1990 (the engine's moe.grouped = 0, src/metal/qwen.rs:2085-2088,
 * 2725-2729, and its decode step): one matvec per (row, slot) against the rows of the slot's expert in W
 * ([experts * n][k]); slot s of row r reads its input at r * x_row + s * x_stride elements of x (x_stride 0: every slot
 * the row's input) and writes y[(r * top_k + s) * n ..] in bf16, the matvec's arithmetic and bits.
 * Bindings W, x, y, route. rows_per_warp 1, 2, 4 or 8 (0 = 2). */
int hb_experts_matvec_get(hb_ctx* ctx, uint32_t k, uint32_t n, uint32_t top_k, uint32_t experts, uint32_t x_row, uint32_t x_stride, uint32_t rows_per_warp,
                          hb_kernel** out);
/* moe_combine, src/metal/qwen_kernels.rs:2119-2161: acc = bf16(acc + bf16(y*w)) over the slots in route order.
 * f32_sum = 1 is the variant that keeps the sum in f32 and rounds once. Bindings: y ([m][top_k][d]), route, out. */
int hb_moe_combine_get(hb_ctx* ctx, uint32_t d, uint32_t top_k, uint32_t f32_sum, hb_kernel** out);
/* ---- the rows around the products (the steps on either side of the GEMMs in the reference's op list) ----
 * rmsnorm_rows, src/metal/prefill.rs:70-117 (decode twin: norm_into, src/metal/kernels.rs:355-442):
 * y = bf16((x / sqrt(mean(x^2) + eps)) * (w + plus_one)), the sums in the reference's order. Bindings x, w, y
 * (y may be x). */
int hb_rmsnorm_get(hb_ctx* ctx, uint32_t d, float eps, uint32_t plus_one, hb_kernel** out);
/* argmax_partial + argmax_final, src/metal/kernels.rs:1461-1565, in one launch: index[r] = the first index of the
 * largest logit of row r (0xffffffff when no logit is greater than -inf). Bindings logits (bf16 [m][n]), index
 * (u32 [m]; the reference writes state[STATE_ARGMAX] for its single row). */
int hb_argmax_get(hb_ctx* ctx, uint32_t n, uint32_t rows_max, hb_kernel** out);
/* moe_out, src/metal/qwen_kernels.rs:2163-2214: g = bf16(sigmoid(bf16(xn . gate))),
 * x = bf16(x + bf16(experts + bf16(g * shared))), in place. Bindings xn, gate (bf16 [d]), experts, shared, x. */
int hb_moe_out_get(hb_ctx* ctx, uint32_t d, hb_kernel** out);

/* ---- Q4_0 weights (src/metal/q4.rs:7-24: per block of 32 weights 16 bytes of nibbles + an f16 scale) ----
 * dequant_q4, src/metal/kernels.rs:1074-1102: W as bf16 [n][k], every value bf16(d * q); what the reference's prefill
 * GEMM stages from Q4 weights (prefill.rs:1058-1076), so this kernel followed by hb_gemm_get gives its bits.
 * Bindings W (nibbles, n*k/2 bytes), scales (f16, n*k/32), out (bf16 [n][k]); m is ignored. */
int hb_dequant_q4_get(hb_ctx* ctx, uint32_t k, uint32_t n, hb_kernel** out);
/* matvec_q4 (masks = 0) and matvec_q4s (masks = 1: "llama.cpp's masks", the tune key mv.masks), src/metal/kernels.rs:
 * 444-632, 1387-1424: y = out(W . x) for one activation row, the sums in the order of the form named (bit-exact with
 * either). rows_per_warp 1, 2 or 4 (0 = 2); out BF16, F32 or RESIDUAL. Bindings W, x, y, scales as there. */
int hb_matvec_q4_get(hb_ctx* ctx, uint32_t k, uint32_t n, uint32_t out, uint32_t rows_per_warp, uint32_t masks, hb_kernel** res);
/* matvec_q4_split, src/metal/kernels.rs:472-500, 896-928: the same product with the blocks of each row shared by `split`
 * (1, 2, 4 or 8) warps of a block (block b to warp (b / 32) % split), their sums added in warp order: `split` times the
 * warps on a matrix of few rows, the sums in another order (bit-exact with that order). persist > 0: only that many
 * blocks, each taking one row group after another (mv.persist). Bindings as hb_matvec_q4_get. */
int hb_matvec_q4_split_get(hb_ctx* ctx, uint32_t k, uint32_t n, uint32_t out, uint32_t rows_per_warp, uint32_t masks, uint32_t split, uint32_t persist,
                           hb_kernel** res);
/* matmul_q4, src/metal/kernels.rs:983-1071: Y[r] = bf16(W . X[r]) for the m (1..8) rows of a short block, row r of X at
 * r * ldx and of Y at r * ldy (bf16 elements; ldx a multiple of 8); each block of weights is decoded once for all
 * rows and every row is summed in matvec_q4's order (the decode step's bits). The kernel is built for m: launch it
 * with that m. Bindings W, X, Y, scales. */
int hb_matmul_q4_get(hb_ctx* ctx, uint32_t k, uint32_t n, uint32_t m, uint32_t ldx, uint32_t ldy, hb_kernel** res);

/* gemm_mma_q4, src/metal/prefill.rs:427-434, 1058-1076 (the engine's q4.fuse = 1, src/metal/qwen.rs:169-173): the
 * prefill GEMM on Q4_0 weights, every staged cell of W decoded to bf16(d * q) as dequant_q4 decodes it while the tile
 * is staged, so that the sums are those of hb_dequant_q4_get followed by hb_gemm_get, bit for bit, without the bf16
 * copy of W ever being written or read. k a multiple of 32; tile_n 128 or 256 (0 = 256); any 1 <= m <= rows_max.
 * Bindings W (Q4 data), X, Y, scales (the reference's order: state, W, X, Y, scales). */
int hb_gemm_q4_get(hb_ctx* ctx, uint32_t k, uint32_t n, uint32_t out, uint32_t tile_n, uint32_t m_first, uint32_t rows_max, hb_kernel** res);

/* ---- expert-parallel exchange over peer memory (no reference counterpart: the reference runs on one GPU) ----
 * Experts are partitioned contiguously over `world` ranks, the token rows are each rank's own. A rank sorts its
 * (row, slot) pairs by global expert with hb_moe_sort_get, binding a fourth range `offsets` u32[experts + 1] (first
 * sorted position of every expert, then the pair count); the host all-gathers these into u32[world][experts + 1].
 * `peers` is a device array u64[world] of the base addresses of every rank's buffer ([cap][h] bf16), the rank's own
 * included, obtained through hb_ipc_export / hb_ipc_open.
 *   dispatch, bindings X, peers, list, offsets_all: writes row X[list[p] / top_k] of every sorted position p into
 *     the receive buffer of the rank that owns p's expert (sources in rank order, each source's rows in its order).
 *   plan, bindings offsets_all, list, tiles: the list (sorted row -> receive-buffer row) and the tile table for this
 *     rank's experts, for expert GEMMs built with top_k = 1, experts / world experts and rows_max = cap, which are
 *     then launched with m = cap (the table, not m, says how many rows there are).
 *   return, bindings peers, EY, list, offsets_all: EY[list[p]] = the row of p in its owner's output buffer.
 *   combine (hb_ep_combine_get), bindings peers_ey, where, route, out: the return and moe_combine in one kernel:
 *     out[row] = the bf16 chain acc = bf16(acc + bf16(y * w)) over the row's slots in route order
 *     (src/metal/qwen_kernels.rs:2119-2161), every y read straight from its owner's output buffer; EY is never made.
 *     `where` u32[m * top_k] is written by the dispatch when it is bound to three more ranges (below).
 * The host orders the steps on the stream: all-gather of the offsets, then dispatch, a barrier, plan and the expert
 * GEMMs, a barrier, return (or combine). The barrier between dispatch and plan may be carried by the two kernels
 * themselves: dispatch bound to X, peers, list, offsets_all, where, peers_landed, ctl (peers_landed: u64[world], the
 * addresses of every rank's u32[world] flags, zeroed once; ctl: this rank's u32[2], zeroed once) numbers the step in
 * ctl[0] and stores the number into flag `rank` of every rank when its last row is out; plan bound to offsets_all,
 * list, tiles, landed (this rank's flags), ctl waits (bounded, hb_set_peer_wait_ms) until every rank's number has
 * arrived. No other kernel of the exchange waits for another GPU. A count that exceeds `cap` rows is reported
 * through the status words (HB_KERNEL at the next hb_sync) and nothing is written past the buffers. */
int hb_ep_dispatch_get(hb_ctx* ctx, uint32_t h, uint32_t top_k, uint32_t experts, uint32_t world, uint32_t rank, uint32_t cap, hb_kernel** out);
int hb_ep_plan_get(hb_ctx* ctx, uint32_t experts, uint32_t world, uint32_t rank, uint32_t bm, uint32_t cap, hb_kernel** out);
int hb_ep_return_get(hb_ctx* ctx, uint32_t h, uint32_t top_k, uint32_t experts, uint32_t world, uint32_t rank, uint32_t cap, hb_kernel** out);
int hb_ep_combine_get(hb_ctx* ctx, uint32_t h, uint32_t top_k, uint32_t world, hb_kernel** out);
/* The combine with the barrier before it ("every rank's expert outputs are complete") inside: bindings peers_ey,
 * where, route, out, peers_done, done, ctl (peers_done: u64[world], the addresses of every rank's u32[world] flags,
 * zeroed once; done: this rank's flags; ctl: this rank's u32[2], zeroed once). Its first block stores the step's
 * number (kept in ctl[0] by the kernel) into flag `rank` of every rank, every block waits (bounded,
 * hb_set_peer_wait_ms) until all owners' numbers have arrived, then combines. One process per GPU: never launched for
 * several ranks on one GPU. No counterpart in the reference (one GPU). */
int hb_ep_combine_sync_get(hb_ctx* ctx, uint32_t h, uint32_t top_k, uint32_t world, uint32_t rank, hb_kernel** out);
/* The direct form of dispatch and plan: every source owns a fixed region of cap / world rows in every rank's receive
 * and output buffers (source s at row s * cap / world), so a source needs nobody else's counts to place its rows and
 * the all-gather of the offsets before the dispatch falls away. The dispatch delivers this rank's offsets itself, into
 * row `rank` of every rank's table, before it flags its landing; the plan waits for the flags and lays the expert tiles
 * over the regions. A step is then route, sort, dispatch, plan, the two expert GEMMs, one barrier, combine.
 * dispatch bindings: X, peers, list, offsets (this rank's u32[experts + 1], as the sort wrote them), where,
 *   peers_landed, ctl, peers_offsets (u64[world]: the addresses of every rank's table u32[world][experts + 1]).
 * plan bindings: offsets_all (this rank's table), list, tiles, landed, ctl. cap must divide by world; a source that has
 * more than cap / world rows for one rank is reported through the status words. */
int hb_ep_dispatch_direct_get(hb_ctx* ctx, uint32_t h, uint32_t top_k, uint32_t experts, uint32_t world, uint32_t rank, uint32_t cap, hb_kernel** out);
int hb_ep_plan_direct_get(hb_ctx* ctx, uint32_t experts, uint32_t world, uint32_t rank, uint32_t bm, uint32_t cap, hb_kernel** out);
/* The output mode (BF16 or RESIDUAL: store, src/metal/kernels.rs:217-234) applied to an f32 accumulator array
 * [m][n] that was completed outside a GEMM: a row-parallel projection sums f32 partial products across GPUs
 * (hb_gemm_get with HB_OUT_F32 on each, then an all-reduce) and rounds once afterwards. Bindings: acc, y. */
int hb_epilogue_get(hb_ctx* ctx, uint32_t n, uint32_t out, hb_kernel** res);
/* The same, with the sum across GPUs and the distribution of the result inside the kernel (no reference
 * counterpart): every rank holds an f32 partial [m][n] and a Y [m][n] in buffers the other ranks have opened
 * (hb_ipc_open); `peers_acc` and `peers_y` are device arrays u64[world] of their addresses, the rank's own included.
 * Rank r sums rows [r * ceil(m / world), ...) of all partials in rank order through NVLink loads, rounds once,
 * applies the output mode with its own old Y and stores the result into every rank's Y. The host puts a barrier
 * before (partials complete everywhere) and after (Y complete everywhere). Bindings: peers_acc, peers_y. */
int hb_tp_reduce_get(hb_ctx* ctx, uint32_t n, uint32_t out, uint32_t world, uint32_t rank, hb_kernel** res);
/* The second half of the same step when the partials were pushed by the GEMMs (hb_gemm_desc.y_shards): this rank's
 * staging buffer f32 [world][ceil(m / world)][n] holds, from every rank s in slot s, the partial rows this rank sums.
 * Sums the slots in rank order, rounds once, applies the output mode with its own old Y and stores the rows into
 * every rank's Y. Bindings: staging (local), peers_y. The host puts a barrier before and after. */
int hb_tp_sum_get(hb_ctx* ctx, uint32_t n, uint32_t out, uint32_t world, uint32_t rank, hb_kernel** res);
/* hb_tp_sum_get's kernel with the step's two barriers inside: bindings staging, peers_y, peers_flags (u64[world]: the
 * addresses of every rank's u32[32] flags, zeroed once), ctl (this rank's u32[2], zeroed once). Its first block tells
 * every rank that this rank's partial has been pushed (the GEMM precedes the kernel on the stream), every block waits
 * (bounded, hb_set_peer_wait_ms) until all ranks have said so; the block that finishes last tells every rank that this
 * rank's rows of Y are stored and waits until all ranks have said that: when the kernel ends Y is complete on every
 * rank and the staging may be overwritten. The step's number is kept in ctl[0]. One process per GPU: never launched
 * for several ranks on one GPU. No counterpart in the reference (one GPU). */
int hb_tp_sum_sync_get(hb_ctx* ctx, uint32_t n, uint32_t out, uint32_t world, uint32_t rank, hb_kernel** res);
/* The sum as a kernel that runs beside the GEMM whose partial it sums (hb_gemm_desc.y_group_rows = group_rows,
 * y_signal = 1 on every rank): for each group of rows in turn it waits until every rank's GEMM has flagged the group,
 * sums this rank's slice of it from the staging slots in rank order, rounds once, applies the output mode and stores
 * the bf16 rows into every rank's Y, while the GEMMs work on the later groups. It is launched right behind the GEMM
 * and may start while the GEMM runs (programmatic stream serialization; the GEMM lets it go at its start); its blocks
 * share the SMs with the GEMM's. When the last group is stored it tells every rank, waits until every rank has said
 * the same (so that Y is complete everywhere and the staging may be overwritten when it returns: no barrier kernel
 * before or after), and writes the step's number to ctl[0]. All waits are bounded (hb_set_peer_wait_ms).
 * staging: this rank's f32 [world][groups][group_rows / world][n], groups = ceil(m / group_rows).
 * sync = 0: no flag is waited for and none is sent (the host orders the kernels: one process that holds every rank on
 * one GPU, or ranks ordered by a collective of the caller's).
 * sync = 2: for a GEMM that deals its rows in groups but flags nothing (y_group_rows = 256, y_signal = 0): the kernel
 * starts after the GEMM, its first block tells every rank that this rank's partial is out, every block waits for all
 * ranks (words 16.. of the `done` arrays, which must hold 16 + world words), then all groups are summed at once and
 * the kernel closes as with sync = 1: both barriers of the step inside the summing kernel.
 * Bindings: staging, peers_y, flags (this rank's u32[world][HB_TP_MAX_GROUPS]), peers_done (u64[world]: every rank's
 * u32[world], zeroed once), ctl (this rank's, the array the GEMM is bound to). No reference counterpart. */
#define HB_TP_MAX_GROUPS 64u
#define HB_TP_CTL_WORDS 128u
int hb_tp_sum_stream_get(hb_ctx* ctx, uint32_t n, uint32_t out, uint32_t world, uint32_t rank, uint32_t group_rows, uint32_t sync, hb_kernel** res);

/* The GEMM for callers that must not allocate device memory. (No counterpart in the reference: its buffers all
 * come from Gpu::alloc at load.)
 *
 * Some hosts of this library cannot call cudaMalloc where they call the GEMM: code running inside a region where
 * the allocator is off limits (a latency-critical serving loop that forbids any call that may synchronise the
 * device or take the allocator's lock), a plugin handed a fixed memory budget by its host engine, or a process
 * whose device memory is fully claimed by another allocator. hb_gemm_get with stream_k = 1 allocates its
 * partial-tile scratch from the context on first use; this entry point runs the same stream-K kernel (128x64
 * tiles, output modes BF16 / F32 / RESIDUAL / SWIGLU) with the scratch in a fixed array inside the library
 * instead, and calls no cudaMalloc, cudaFree or other allocating routine. The caller passes W, X and Y as for
 * hb_launch (W [n][k], X [m][k], Y [m][n] or [m][n/2]); the launch goes on the context's stream.
 *
 * Limits: the array serves HB_STATIC_SCRATCH_SLOTS CTAs (a GPU with more SMs runs that many CTAs) and costs
 * 5.0 MiB of device memory on every GPU that loads the library, until the process exits. Products beyond
 * HB_STATIC_SCRATCH_MAX_ROWS rows, HB_STATIC_SCRATCH_MAX_K or HB_STATIC_SCRATCH_MAX_N are refused with
 * HB_UNSUPPORTED: use hb_gemm_get for those.
 * The first call on a device looks up the array's device address (cudaGetSymbolAddress) and raises the kernel's
 * shared-memory limit.
 * All calls on a device share the one array: two calls whose kernels overlap on the GPU (different streams or
 * contexts) race on it. Calls on one stream are ordered and safe; nothing needs clearing between them. */
#define HB_STATIC_SCRATCH_SLOTS 160u
#define HB_STATIC_SCRATCH_MAX_ROWS 2048u
#define HB_STATIC_SCRATCH_MAX_K 65536u
#define HB_STATIC_SCRATCH_MAX_N 262144u
int hb_gemm_static_scratch(hb_ctx* ctx, uint32_t k, uint32_t n, uint32_t out, uint32_t m, hb_range w, hb_range x, hb_range y);

/* Emitted.name, src/msl/mod.rs:1461: deterministic, encodes the description. */
const char* hb_kernel_name(const hb_kernel* k);
/* Gpu::dispatch, src/metal/gpu.rs:166: enqueue on the context's stream. Any 1 <= m <= rows_max. */
int hb_launch(hb_ctx* ctx, const hb_kernel* k, const hb_range* args, int nargs, uint32_t m);
/* Runs the sequence once (asynchronously). */
int hb_run(hb_ctx* ctx, const hb_op* ops, int nops);
/* time_ops, src/metal/qwen.rs:2593: `reps` runs of the sequence, GPU seconds measured with events on the
 * stream (reference: Done.gpu of the command buffer, src/metal/gpu.rs:209-221). Synchronises. */
int hb_time(hb_ctx* ctx, const hb_op* ops, int nops, int reps, double* gpu_seconds);
/* A sequence recorded once and replayed with one call (a CUDA graph): the decode step launches a dozen kernels of
 * 10-200 us each, and enqueueing them one by one costs the host about as long as the GPU takes to run them. The
 * reference encodes its ops into one command buffer per step (src/metal/gpu.rs:151-221) for the same reason. The
 * bound ranges and m are fixed at recording. Every kernel of this library can be recorded (none of them carries a
 * host-side counter: the stream-K GEMM's flags are cleared by their reader, the peer barrier counts itself);
 * hb_gemm_static_scratch is a direct call, not an hb_kernel: it is not an entry of an hb_op list. */
/* Overlapped launches (off by default): the decode kernels (hb_matvec_get in all its forms, hb_rmsnorm_get) are then
 * launched with programmatic stream serialization: a kernel may start while the one before it on the stream is
 * still finishing, sets up, prefetches weights, and waits inside for its predecessor's completion before it reads
 * an activation or writes an output. Results are unchanged; a chain of 15-20 us kernels loses its launch gaps.
 * Applies to plain launches and to sequences recorded afterwards. */
int hb_set_launch_overlap(hb_ctx* ctx, int on);
typedef struct hb_graph hb_graph;
int hb_graph_record(hb_ctx* ctx, const hb_op* ops, int nops, hb_graph** out);
int hb_graph_launch(hb_ctx* ctx, hb_graph* g);
int hb_graph_time(hb_ctx* ctx, hb_graph* g, int reps, double* gpu_seconds);
int hb_graph_free(hb_ctx* ctx, hb_graph* g);

/* ---- the load-time selection loop (host library) ------------------------- */

/* Tune, src/metal/qwen.rs:62-397. Acted on by the selection loop: gemm.auto gemm.mma gemm.tn gemm.mform gemm.mfirst
 * prefill.block moe.grouped moe.tile pf.fswi q4.fuse mv.auto mv.split mv.splitauto mv.persist mv.persists mv.cold auto.heat, and through
 * hb_select_axis dec.auto dec.fnorm dec.fswi. Every other key of the reference is parsed, range-checked where the
 * reference checks it, stored and ignored: among the keys of this path that is gemm.simt (the layouts of a CUDA-core
 * GEMM that does not exist here) and gemm.half (half-staged Q4 tiles: the tensor cores take bf16 here).
 * moe.grouped = 0 makes hb_select_experts return the per-slot form (experts_matvec). */
typedef struct hb_tune hb_tune;
int hb_tune_new(hb_tune** out);
void hb_tune_free(hb_tune* t);
/* Tune::apply, qwen.rs:296-389: "key=value[,key=value]"; unknown key, non-u32 value or a value out of range
 * returns HB_INVALID with the reference's message in err. */
int hb_tune_apply(hb_tune* t, const char* list, char* err, size_t errlen);
int hb_tune_get(const hb_tune* t, const char* key, uint32_t* value);
/* Tune::summary, qwen.rs:391-396 (the keys of this path, in the reference's order). */
int hb_tune_summary(const hb_tune* t, char* buf, size_t len);
/* 1 when GEMM candidates are timed at load: gemm.auto != 0 and none of gemm.mma/gemm.tn/gemm.mform given
 * (qwen.rs:902,2229). */
int hb_tune_gemm_timed(const hb_tune* t);

typedef struct hb_selector hb_selector;
int hb_selector_new(hb_ctx* ctx, const hb_tune* tune, hb_selector** out);
void hb_selector_free(hb_selector* s);
/* The "[autotune] ..." lines produced so far (also written to stderr), newline separated. */
const char* hb_selector_log(const hb_selector* s);
/* Row buckets of the prefill GEMMs: 64, 128, .. < block, then block (qwen.rs:1049-1052). Returns the count. */
int hb_selector_buckets(const hb_selector* s, uint32_t* buckets, int cap);
/* autotune_inputs / fill_random16, qwen.rs:2605-2626: fills a device range with xorshift32 bf16 in [-1, 1). */
int hb_fill_random16(hb_ctx* ctx, hb_range dst, uint32_t seed);
/* QwenEngine::gemm, qwen.rs:2200-2315: the kernel for (k, n, out) at m rows. With timing on, candidates are
 * built, checked against the first one (check_candidates, qwen.rs:2497-2543: full and partial block from a
 * zeroed output, rejected when max|diff| > max|ref|/64), timed (pick_flagged, qwen.rs:2547-2573: 5 interleaved
 * rounds, median) and the pick cached under "{k}x{n} {Out}, {m} rows". With timing off the tune keys name it. */
int hb_select_gemm(hb_selector* s, uint32_t k, uint32_t n, uint32_t out, hb_range w, hb_range x, hb_range y, uint32_t m,
                   const hb_kernel** picked);
/* gate_up_pipes, qwen.rs:2148-2191: [gate|up] GEMM + swiglu_rows ("apart") against the fused epilogue,
 * per pf.fswi (0 apart, 1 fused, 2 timed). ops_out receives 1 or 2 ops bound to the given ranges;
 * gu is the [m][2*inter] intermediate of the apart form. */
int hb_select_gate_up(hb_selector* s, uint32_t k, uint32_t inter, hb_range w, hb_range x, hb_range gu, hb_range h, uint32_t m,
                      const hb_kernel** kernels_out, int* nkernels);
/* mv_full, qwen.rs:1311-1505: the matvec form for (k, n, out) at `rows` activation rows. `w_copies` same-shaped
 * matrices are walked in turn so that weights come from memory, not cache (mv.cold, qwen.rs:248-251,1177). */
int hb_select_matvec(hb_selector* s, uint32_t k, uint32_t n, uint32_t out, uint32_t rows, const hb_range* w_copies, int ncopies,
                     hb_range x, hb_range y, const hb_kernel** picked);
/* QwenEngine::gemm for a Q4_0 matrix (qwen.rs:2200-2315 with q4; the key gets " q4", qwen.rs:2239): with q4.fuse given,
 * 0 = dequant_q4 into `w_bf16` and then the GEMM the keys name (2 kernels), 1 = the GEMM that decodes while it stages
 * (1 kernel); with timing on both are built ("dequant+" the picked bf16 form, and the fused tiles), checked against the
 * first (check_candidates) and timed. kernels_out receives 1 or 2 kernels: [fused] with bindings W (Q4 data), X, Y,
 * scales, or [dequant, gemm] with bindings W (Q4 data), scales, w_bf16 and w_bf16, X, Y. w_bf16 is the scratch for the
 * decoded matrix (bf16 [n][k]); it may be empty, and then only the fused form is built. */
int hb_select_gemm_q4(hb_selector* s, uint32_t k, uint32_t n, uint32_t out, hb_range wq, hb_range scales, hb_range w_bf16, hb_range x, hb_range y, uint32_t m,
                      const hb_kernel** kernels_out, int* nkernels);
/* The same for a projection whose input is made inside the kernel (mv_full with XSrc::Norm / XSrc::Swiglu,
 * qwen.rs:1308-1335; the pick is cached under the key with " norm" appended, qwen.rs:1410): x is the residual stream
 * and norm_w the norm's weights (HB_X_NORM), or x holds rows of [gate | up] (HB_X_SWIGLU, norm_w empty). */
int hb_select_matvec_x(hb_selector* s, uint32_t k, uint32_t n, uint32_t out, uint32_t rows, uint32_t x_src, uint32_t norm_eps_bits, uint32_t norm_plus_one,
                       const hb_range* w_copies, int ncopies, hb_range x, hb_range y, hb_range norm_w, const hb_kernel** picked);
/* One axis of tune_step, qwen.rs:3043-3170 (dec.auto): the decode step recorded once per value of a switch (axis
 * "fnorm" with key "dec.fnorm": the norms as kernels of their own, or made by the projections that follow them;
 * "fswi" with "dec.fswi": the SwiGLU as the gate/up projection's epilogue, or made by the down projection) is run
 * twice to warm and seven times for the median; the first strictly fastest value is returned and the line
 * "[autotune] decode step at position {p}, {axis}: {v} {ms} ms, ... -> {v}" logged. A key that --tune gives is
 * returned untimed, and so is the key's value when dec.auto = 0. variants[i] may be NULL (that form is unavailable). */
int hb_select_axis(hb_selector* s, const char* axis, const char* key, const hb_op* const* variants, const int* nops, const uint32_t* values, int nvariants,
                   uint32_t position, uint32_t* best_value);
/* expert_pipes, qwen.rs:2326-2386: for bm in {16, 32, 64} (moe.tile only, if given) the sort and the two expert
 * GEMMs are timed on a real route (the caller has run the router on its block); per tile size the fastest
 * checked gate/up form is kept, then the tile whose sort + gate/up + down time is least.
 * Gate/up forms: "fused" (GATHER GEMM with the SwiGLU epilogue, X -> EHB), "apart" (GATHER GEMM to EGU, then
 * swiglu over the sorted rows; needs egu), "gather+fused" (moe_gather to XS, then the SORTED GEMM with the
 * SwiGLU epilogue; needs xs). egu and xs may be empty ranges: their forms are then left out. */
typedef struct {
    uint32_t experts, top_k, h, mi, m;
    hb_range route, list, tiles, x, wgu, wdown, ehb, ey;
    hb_range egu; /* optional: bf16 [m*top_k][2*mi] */
    hb_range xs;  /* optional: bf16 [m*top_k][h] */
} hb_expert_io;
typedef struct {
    uint32_t bm;              /* 0: moe.grouped = 0, the per-slot form: sort and gather are NULL, gate_up is experts_matvec over X
                                 (bindings W, X, EGU, route; rows of [gate | up]), swiglu turns EGU into EHB, down is
                                 experts_matvec over EHB (bindings W, EHB, EY, route); io.egu is then required */
    const hb_kernel* sort;    /* bindings route, list, tiles */
    const hb_kernel* gather;  /* NULL, or moe_gather: X, list, XS */
    const hb_kernel* gate_up; /* W, X (or XS), EHB (or EGU), list, tiles */
    const hb_kernel* swiglu;  /* NULL, or swiglu over sorted rows: EGU, EHB; launched with m*top_k rows */
    const hb_kernel* down;    /* W, EHB, EY, list, tiles */
} hb_expert_pick;
int hb_select_experts(hb_selector* s, const hb_expert_io* io, hb_expert_pick* pick);
/* Test hook for the correctness gate: while enabled, hb_select_gemm adds a candidate named "wrong" that runs
 * the first candidate and then scales the output by 1.25 (builds, runs, plausible magnitudes, incorrect). The
 * 1/64 rule must reject it and log it (the reference's incident: README.md:65-73). */
int hb_selector_inject_wrong(hb_selector* s, int enable);
/* check_candidates' rule alone, on host arrays (bf16 bits or f32): returns HB_OK and sets *eligible. */
int hb_check_rule(const void* reference, const void* got, size_t count, int f32_out, int* eligible, float* err, float* scale);

#ifdef __cplusplus
}
#endif
#endif
