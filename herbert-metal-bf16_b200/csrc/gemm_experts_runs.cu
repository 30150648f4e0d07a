// Expert GEMM of the MoE layer, run-merging form (hb_gemm_desc.merge_runs = 1).
//
// Same contract and bindings as gemm_experts.cu (reference src/metal/prefill.rs:317-328, :889-941,
// :1206-1209, :534-552). An MoE block at 2048 tokens is weight-bandwidth bound (64 FLOP per weight
// byte), so this form is built around reading every expert's weights ONCE:
//   * the product is computed transposed: the expert's weight rows are the 128-row tcgen05 operand
//     (streamed by TMA), the token rows are the narrow N operand, the accumulator in tensor memory
//     is [128 features][tokens];
//   * the tiles of one expert are consecutive in the table and their sorted rows contiguous, so a CTA
//     merges them: a work item is (expert run of up to 128 rows, block of 128 features), N = the run's
//     rows rounded up to 16. The tile size of the table (16/32/64) then only sets the granularity of
//     the runs, not how often weights are re-read through L2.
// Warp roles (320 threads):
//   warp 0      TMA producer: weight slices, and the token slices when the sorted rows are contiguous
//               in memory (Scatter and Sorted modes)
//   warp 1      tcgen05.mma issuer, tensor-memory owner
//   warps 2-5   epilogue: tcgen05.ld, output mode, stores to row p or to row list[p]
//   warps 6-9   Gather mode: token rows X[list[p] / top_k] fetched with 16-byte cp.async straight into
//               the 128-byte-swizzled stage (the layout TMA would have produced); completion is
//               signalled on the stage's mbarrier by cp.async.mbarrier.arrive, so the gather runs as
//               many stages ahead as the ring allows
// With the fused SwiGLU form the gate rows and the matching up rows of the expert feed two
// accumulators, so one thread holds g and u of the same (feature, token). Every barrier wait is bounded.
#include <algorithm>

#include "hb_internal.hpp"
#include "tc05.cuh"

namespace hb {

struct RunParams {
    void* y;
    const uint16_t* x;  // Gather mode: token rows [m][k]
    const uint32_t* list;
    const uint32_t* tiles;
    uint32_t k_blocks;
    uint32_t n;         // W rows of one expert
    uint32_t n_feat;    // output features of one expert (n, or n/2 fused)
    uint32_t n_blocks;  // ceil(n_feat / 128)
    uint32_t k;         // row length of X
    uint32_t top_k;
    uint32_t stages;
    uint32_t max_tiles;
    uint32_t experts;
    uint32_t* status;
};

constexpr int RN_THREADS = 320;
constexpr int RN_MAX_STAGES = 8;
constexpr int RN_A_BYTES = 128 * 64 * 2;
constexpr int RN_NMAX = 128;               // token rows of a work item
constexpr int RN_B_BYTES = RN_NMAX * 128;  // 16 KiB
constexpr int RN_MAX_RUNS = 1024;          // runs a launch can hold in shared memory
constexpr int RN_MAX_EXPERTS = 1024;

struct __align__(8) RunBarriers {
    uint64_t full[RN_MAX_STAGES];
    uint64_t empty[RN_MAX_STAGES];
    uint64_t tmem_full[2];
    uint64_t tmem_empty[2];
    uint32_t tmem_base;
    uint32_t nruns;
};

enum { RSRC_GATHER = 0, RSRC_SORTED = 1 };   // where the token operand comes from
enum { RDST_SORTED = 0, RDST_SCATTER = 1 };  // where output row p goes

__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src, uint32_t src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
// One pending arrival of the mbarrier completes when all earlier cp.async of this thread have landed.
__device__ __forceinline__ void cp_async_mbar_arrive(uint32_t bar) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}

// Builds the run list in shared memory from the table's tiles: run = (expert, first sorted row, rows <= 128).
// A tile starts a run when it is the first of its expert or a multiple of 128 rows into the expert's rows.
// The table is copied to shared memory once (`tl`, room for 3 words per tile: the pipeline's stage buffers, not yet in
// use) and everything else works from there: one round trip to global memory, and the scan of the per-thread counts is
// a shuffle scan (a serial scan over 320 counts by one thread took longer than streaming an expert's weights).
__device__ __forceinline__ void build_runs(const RunParams& p, uint32_t ntiles, uint32_t* tl, uint32_t* run_first, uint32_t* run_end, uint32_t* runs, uint32_t* scratch,
                                           uint32_t* nruns_out) {
    const uint32_t tid = threadIdx.x, nthr = blockDim.x, lane = tid & 31u, warp = tid >> 5;
    for (uint32_t i = tid; i < 3 * ntiles; i += nthr) tl[i] = p.tiles[1 + i];
    __syncthreads();
    for (uint32_t t = tid; t < ntiles; t += nthr) {
        const uint32_t e = tl[3 * t], start = tl[3 * t + 1], rows = tl[3 * t + 2];
        if (e < RN_MAX_EXPERTS) {
            if (t == 0 || tl[3 * (t - 1)] != e) run_first[e] = start;
            if (t + 1 == ntiles || tl[3 * (t + 1)] != e) run_end[e] = start + rows;
        }
    }
    __syncthreads();
    // each thread owns a contiguous range of tiles: count the run starts in it, scan, then write them
    const uint32_t per = (ntiles + nthr - 1) / nthr;
    const uint32_t t0 = min(ntiles, tid * per), t1 = min(ntiles, t0 + per);
    uint32_t mine = 0;
    for (uint32_t t = t0; t < t1; ++t) {
        const uint32_t e = tl[3 * t], start = tl[3 * t + 1];
        if (e < RN_MAX_EXPERTS && (start - run_first[e]) % RN_NMAX == 0) mine++;
    }
    uint32_t incl = mine;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
        const uint32_t o = __shfl_up_sync(0xffffffffu, incl, off);
        if (lane >= (uint32_t)off) incl += o;
    }
    if (lane == 31) scratch[warp] = incl;
    __syncthreads();
    uint32_t before = 0, total = 0;
    for (uint32_t w = 0; w < nthr / 32; ++w) {
        const uint32_t c = scratch[w];
        if (w < warp) before += c;
        total += c;
    }
    if (tid == 0) *nruns_out = min(total, (uint32_t)RN_MAX_RUNS);
    uint32_t at = before + incl - mine;
    for (uint32_t t = t0; t < t1; ++t) {
        const uint32_t e = tl[3 * t], start = tl[3 * t + 1];
        if (e < RN_MAX_EXPERTS && (start - run_first[e]) % RN_NMAX == 0) {
            if (at < RN_MAX_RUNS) {
                runs[3 * at] = e;
                runs[3 * at + 1] = start;
                runs[3 * at + 2] = min((uint32_t)RN_NMAX, run_end[e] - start);
            }
            at++;
        }
    }
    // `tl` becomes a pipeline stage next: written by TMA (async proxy) after these reads
    fence_proxy_async();
    __syncthreads();
}

// ACCS: 1 = one block of 128 features per work item; 2 with FUSED = the gate block and its up block (SwiGLU);
// 2 without FUSED = two neighbouring feature blocks sharing the token operand (halves its traffic from L2).
template <int SRC, int DST, bool FUSED, int ACCS>
__global__ void __launch_bounds__(RN_THREADS, 1)
gemm_expert_runs_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x64, const __grid_constant__ CUtensorMap tm_x128, const RunParams p) {
    constexpr int NACC = ACCS;
    constexpr uint32_t FEAT_PER_ITEM = (ACCS == 2 && !FUSED) ? 256u : 128u;
    constexpr int A_STAGE = NACC * RN_A_BYTES;
    constexpr int STAGE_BYTES = A_STAGE + RN_B_BYTES;
    constexpr uint32_t ACC_COLS = NACC * RN_NMAX;  // 128 or 256 columns per accumulator set
    constexpr uint32_t TMEM_COLS = 2 * ACC_COLS;   // two sets: 256 or 512
    constexpr uint32_t FULL_ARRIVALS = SRC == RSRC_GATHER ? 1 + 128 : 1;

    extern __shared__ uint8_t smem_raw[];
    __shared__ RunBarriers bars;
    __shared__ uint32_t run_first[RN_MAX_EXPERTS];
    __shared__ uint32_t run_end[RN_MAX_EXPERTS];
    __shared__ uint32_t runs[3 * RN_MAX_RUNS];
    __shared__ uint32_t scratch[RN_THREADS];
    __shared__ uint32_t orow_s[4][RN_NMAX];  // per epilogue warp: the output row of each row of the run
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t S = p.stages;

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < S; ++s) {
            mbar_init(smem_u32(&bars.full[s]), FULL_ARRIVALS);
            mbar_init(smem_u32(&bars.empty[s]), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(smem_u32(&bars.tmem_full[a]), 1);
            mbar_init(smem_u32(&bars.tmem_empty[a]), 4);
        }
        fence_mbar_init();
        fence_proxy_async();
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(&bars.tmem_base), TMEM_COLS);
        tmem_relinquish();
    }
    // (an overlapped launch: barriers and tensor memory are set up under the tail of the kernel before this one; the
    // table, the list and the token rows are its outputs)
    griddep_wait();
    const uint32_t ntiles = min(p.tiles[0], p.max_tiles);
    build_runs(p, ntiles, reinterpret_cast<uint32_t*>(smem_raw), run_first, run_end, runs, scratch, &bars.nruns);  // ends with __syncthreads
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = bars.tmem_base;
    const uint32_t work_total = bars.nruns * p.n_blocks;

    if (warp == 0) {
        if (lane == 0) {
            tma_prefetch_desc(&tm_w);
            if (SRC == RSRC_SORTED) { tma_prefetch_desc(&tm_x64); tma_prefetch_desc(&tm_x128); }
            uint32_t s = 0, ph = 0;
            bool ok = true;
            for (uint32_t w = blockIdx.x; ok && w < work_total; w += gridDim.x) {
                const uint32_t r = w / p.n_blocks, nb = w % p.n_blocks;
                const uint32_t expert = runs[3 * r], start = runs[3 * r + 1], rows = runs[3 * r + 2];
                const int row_w0 = (int)(expert * p.n + nb * FEAT_PER_ITEM);
                const int row_w1 = FUSED ? (int)(expert * p.n + p.n_feat + nb * 128) : row_w0 + 128;
                const bool small = rows <= 64;
                const uint32_t b_bytes = small ? 64 * 128 : 128 * 128;
                for (uint32_t kb = 0; kb < p.k_blocks; ++kb) {
                    if (!mbar_wait(smem_u32(&bars.empty[s]), ph ^ 1u)) {
                        report(p.status, ST_WAIT_TIMEOUT, WHERE_EMPTY, s);
                        ok = false;
                        break;
                    }
                    const uint32_t full = smem_u32(&bars.full[s]);
                    const uint32_t dst = smem_base + s * STAGE_BYTES;
                    mbar_arrive_expect_tx(full, SRC == RSRC_SORTED ? A_STAGE + b_bytes : A_STAGE);
                    tma_load_2d(dst, &tm_w, full, (int)(kb * 64), row_w0);
                    if (NACC == 2) tma_load_2d(dst + RN_A_BYTES, &tm_w, full, (int)(kb * 64), row_w1);
                    if (SRC == RSRC_SORTED) tma_load_2d(dst + A_STAGE, small ? &tm_x64 : &tm_x128, full, (int)(kb * 64), (int)start);
                    if (++s == S) { s = 0; ph ^= 1u; }
                }
            }
            // every weight load of this CTA is requested: the kernel behind this one may take the SMs as they fall free
            // (let go at the kernel's start, its blocks sat on the SMs beside this kernel's for its whole length: slower)
            griddep_launch_dependents();
        }
    } else if (warp == 1) {
        if (lane == 0) {
            uint32_t s = 0, ph = 0, it = 0;
            bool ok = true;
            for (uint32_t w = blockIdx.x; ok && w < work_total; w += gridDim.x, ++it) {
                const uint32_t r = w / p.n_blocks;
                const uint32_t rows_pad = (runs[3 * r + 2] + 15u) & ~15u;
                const uint32_t idesc = umma_idesc_bf16(128, rows_pad);
                const uint32_t acc = it & 1u, acc_ph = (it >> 1) & 1u;
                if (!mbar_wait(smem_u32(&bars.tmem_empty[acc]), acc_ph ^ 1u)) {
                    report(p.status, ST_WAIT_TIMEOUT, WHERE_TMEM_EMPTY, acc);
                    break;
                }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * ACC_COLS;
                for (uint32_t kb = 0; kb < p.k_blocks; ++kb) {
                    if (!mbar_wait(smem_u32(&bars.full[s]), ph)) {
                        report(p.status, ST_WAIT_TIMEOUT, WHERE_FULL, s);
                        ok = false;
                        break;
                    }
                    if (SRC == RSRC_GATHER) fence_proxy_async();  // the token rows were written by cp.async (generic proxy)
                    tc_fence_after();
                    const uint32_t a_addr = smem_base + s * STAGE_BYTES;
                    const uint64_t a_desc = umma_desc_sw128(a_addr);
                    const uint64_t b_desc = umma_desc_sw128(a_addr + A_STAGE);
#pragma unroll
                    for (uint32_t k4 = 0; k4 < 4; ++k4) {
                        const uint32_t accumulate = (kb | k4) != 0 ? 1u : 0u;
                        umma_bf16(d_tmem, a_desc + 2 * k4, b_desc + 2 * k4, idesc, accumulate);
                        if (NACC == 2) umma_bf16(d_tmem + RN_NMAX, umma_desc_sw128(a_addr + RN_A_BYTES) + 2 * k4, b_desc + 2 * k4, idesc, accumulate);
                    }
                    umma_commit(smem_u32(&bars.empty[s]));
                    if (++s == S) { s = 0; ph ^= 1u; }
                }
                if (ok) umma_commit(smem_u32(&bars.tmem_full[acc]));
            }
        }
    } else if (warp < 6) {
        const uint32_t q = (uint32_t)warp & 3u;
        uint32_t it = 0;
        for (uint32_t w = blockIdx.x; w < work_total; w += gridDim.x, ++it) {
            const uint32_t r = w / p.n_blocks, nb = w % p.n_blocks;
            const uint32_t start = runs[3 * r + 1], rows = runs[3 * r + 2];
            // where each row of the run goes, fetched before the accumulator is waited for
            uint32_t* orow = orow_s[q];
            for (uint32_t i = lane; i < rows; i += 32) orow[i] = DST == RDST_SCATTER ? p.list[start + i] : start + i;
            __syncwarp();
            const uint32_t acc = it & 1u, acc_ph = (it >> 1) & 1u;
            const bool got = mbar_wait(smem_u32(&bars.tmem_full[acc]), acc_ph);
            if (!__all_sync(0xffffffffu, got)) {
                if (lane == 0) report(p.status, ST_WAIT_TIMEOUT, WHERE_TMEM_FULL, acc);
                break;
            }
            tc_fence_after();
            const uint32_t feat = nb * FEAT_PER_ITEM + q * 32 + lane;
            const uint32_t t_addr = tmem_base + ((q * 32u) << 16) + acc * ACC_COLS;
            uint16_t* y = reinterpret_cast<uint16_t*>(p.y) + feat;
            for (uint32_t c = 0; c * 32 < rows; ++c) {
                uint32_t g[32], u[32];
                tmem_ld_32x32(t_addr + c * 32, g);
                if (NACC == 2) tmem_ld_32x32(t_addr + RN_NMAX + c * 32, u);
                tmem_ld_wait();
                if (feat < p.n_feat) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        const uint32_t row = c * 32 + j;
                        if (row < rows) {
                            uint32_t o;
                            if (FUSED) o = swiglu_bf16(round_bf16(__uint_as_float(g[j])), round_bf16(__uint_as_float(u[j])));
                            else o = f32_to_bf16(__uint_as_float(g[j]));
                            y[(size_t)orow[row] * p.n_feat] = (uint16_t)o;
                        }
                    }
                }
                if (NACC == 2 && !FUSED && feat + 128 < p.n_feat) {  // the second feature block of the pair
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        const uint32_t row = c * 32 + j;
                        if (row < rows) y[(size_t)orow[row] * p.n_feat + 128] = (uint16_t)f32_to_bf16(__uint_as_float(u[j]));
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&bars.tmem_empty[acc]));
        }
    } else if (SRC == RSRC_GATHER) {
        // 128 threads: thread gt owns 16-byte chunk (gt & 7) of rows (gt >> 3) + 16 i. Chunk c of row r lands at
        // r*128 + ((c ^ (r & 7)) << 4): the 128-byte swizzle of the weight tiles. Rows past the run (padding to a
        // multiple of 16) are zero-filled (cp.async with a source size of 0).
        const uint32_t gt = threadIdx.x - 6 * 32;
        const uint32_t chunk = gt & 7u, row0 = gt >> 3;
        uint32_t s = 0, ph = 0;
        bool ok = true;
        for (uint32_t w = blockIdx.x; ok && w < work_total; w += gridDim.x) {
            const uint32_t r = w / p.n_blocks;
            const uint32_t start = runs[3 * r + 1], rows = runs[3 * r + 2];
            const uint32_t rows_pad = (rows + 15u) & ~15u;
            const uint16_t* src[RN_NMAX / 16];
#pragma unroll
            for (int i = 0; i < RN_NMAX / 16; ++i) {
                const uint32_t row = row0 + 16u * i;
                src[i] = row < rows ? p.x + (size_t)(p.list[start + row] / p.top_k) * p.k + chunk * 8 : nullptr;
            }
            for (uint32_t kb = 0; kb < p.k_blocks; ++kb) {
                const bool got = mbar_wait(smem_u32(&bars.empty[s]), ph ^ 1u);
                if (!__all_sync(0xffffffffu, got)) {
                    if (lane == 0) report(p.status, ST_WAIT_TIMEOUT, WHERE_EMPTY, 100 + s);
                    ok = false;
                    break;
                }
                const uint32_t b_dst = smem_base + s * STAGE_BYTES + A_STAGE;
                const bool k_in = kb * 64 + chunk * 8 < p.k;
#pragma unroll
                for (int i = 0; i < RN_NMAX / 16; ++i) {
                    const uint32_t row = row0 + 16u * i;
                    if (row < rows_pad) {
                        const uint32_t at = b_dst + row * 128u + ((chunk ^ (row & 7u)) << 4);
                        const bool real = src[i] != nullptr && k_in;
                        cp_async_16(at, real ? (const void*)(src[i] + (size_t)kb * 64) : (const void*)p.x, real ? 16u : 0u);
                    }
                }
                cp_async_mbar_arrive(smem_u32(&bars.full[s]));
                if (++s == S) { s = 0; ph ^= 1u; }
            }
        }
        asm volatile("cp.async.wait_all;" ::: "memory");
    }

    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
}

namespace {

typedef void (*run_fn)(const CUtensorMap, const CUtensorMap, const CUtensorMap, const RunParams);

// Unfused forms take two feature blocks per work item when the expert has at least 256 features.
run_fn run_pick(uint32_t rows_mode, bool fused, bool pair) {
    if (rows_mode == HB_ROWS_GATHER)
        return fused ? gemm_expert_runs_kernel<RSRC_GATHER, RDST_SORTED, true, 2>
                     : pair ? gemm_expert_runs_kernel<RSRC_GATHER, RDST_SORTED, false, 2> : gemm_expert_runs_kernel<RSRC_GATHER, RDST_SORTED, false, 1>;
    if (rows_mode == HB_ROWS_SORTED)
        return fused ? gemm_expert_runs_kernel<RSRC_SORTED, RDST_SORTED, true, 2>
                     : pair ? gemm_expert_runs_kernel<RSRC_SORTED, RDST_SORTED, false, 2> : gemm_expert_runs_kernel<RSRC_SORTED, RDST_SORTED, false, 1>;
    if (rows_mode == HB_ROWS_SCATTER)
        return fused ? nullptr : pair ? gemm_expert_runs_kernel<RSRC_SORTED, RDST_SCATTER, false, 2> : gemm_expert_runs_kernel<RSRC_SORTED, RDST_SCATTER, false, 1>;
    return nullptr;
}

struct ExpertRunsGemm : hb_kernel {
    hb_gemm_desc d{};
    run_fn fn = nullptr;
    bool fused = false, pair = false;
    uint32_t stages = 0;
    size_t smem = 0;
    const void* last_w = nullptr;
    const void* last_x = nullptr;
    uint32_t last_m = 0;
    CUtensorMap tm_w{}, tm_x64{}, tm_x128{};

    int launch(hb_ctx* ctx, const hb_range* a, int na, uint32_t m) override {
        if (na != 5) return fail(ctx, HB_INVALID, name + ": bindings are W, X, Y, list, tiles");
        if (m == 0 || m > d.rows_max) return fail(ctx, HB_INVALID, name + ": m outside 1.." + std::to_string(d.rows_max));
        const uint32_t pairs = m * d.top_k;
        const uint32_t n_feat = fused ? d.n / 2 : d.n;
        const uint32_t max_tiles = hb_moe_tiles(m, d.top_k, d.experts, d.bm);
        if ((size_t)d.experts + (pairs + RN_NMAX - 1) / RN_NMAX > RN_MAX_RUNS)
            return fail(ctx, HB_UNSUPPORTED, name + ": more expert runs than the kernel's table holds");
        if ((size_t)max_tiles * 12 + 1024 > smem) return fail(ctx, HB_UNSUPPORTED, name + ": the tile table does not fit in the shared memory the kernel stages it in");
        const size_t xrows = d.rows_mode == HB_ROWS_GATHER ? m : pairs;
        if (!range_ok(a[0], (size_t)d.experts * d.n * d.k * 2) || !range_ok(a[1], xrows * d.k * 2) || !range_ok(a[2], (size_t)pairs * n_feat * 2) ||
            !range_ok(a[3], (size_t)pairs * 4) || !range_ok(a[4], (1 + 3 * (size_t)max_tiles) * 4))
            return fail(ctx, HB_INVALID, name + ": a bound range is too small for " + std::to_string(m) + " rows");
        if (reinterpret_cast<uintptr_t>(a[1].ptr) & 15u) return fail(ctx, HB_INVALID, name + ": X must be 16-byte aligned");
        if (a[0].ptr != last_w || a[1].ptr != last_x || m != last_m) {
            int r = make_tmap_bf16(ctx, &tm_w, a[0].ptr, (uint64_t)d.experts * d.n, d.k, 128);
            if (r != HB_OK) return r;
            if ((r = make_tmap_bf16(ctx, &tm_x64, a[1].ptr, xrows, d.k, 64)) != HB_OK) return r;
            if ((r = make_tmap_bf16(ctx, &tm_x128, a[1].ptr, xrows, d.k, 128)) != HB_OK) return r;
            last_w = a[0].ptr;
            last_x = a[1].ptr;
            last_m = m;
        }
        RunParams p{};
        p.y = a[2].ptr;
        p.x = static_cast<const uint16_t*>(a[1].ptr);
        p.list = static_cast<const uint32_t*>(a[3].ptr);
        p.tiles = static_cast<const uint32_t*>(a[4].ptr);
        p.k_blocks = (d.k + 63) / 64;
        p.n = d.n;
        p.n_feat = n_feat;
        p.n_blocks = pair ? (n_feat + 255) / 256 : (n_feat + 127) / 128;
        p.k = d.k;
        p.top_k = d.top_k;
        p.stages = stages;
        p.max_tiles = max_tiles;
        p.experts = d.experts;
        p.status = ctx->status_dev;
        HB_CUDA(ctx, launch_kernel(ctx, true, fn, dim3(ctx->sm_count), dim3(RN_THREADS), smem, tm_w, tm_x64, tm_x128, p));
        ctx->launches++;
        return HB_OK;
    }
};

}  // namespace

int make_gemm_expert_runs(hb_ctx* ctx, const hb_gemm_desc* d, hb_kernel** out) {
    *out = nullptr;
    const bool fused = d->out == HB_OUT_SWIGLU;
    if (d->experts > RN_MAX_EXPERTS) return fail(ctx, HB_UNSUPPORTED, "expert gemm (merged runs): at most 1024 experts");
    const bool pair = !fused && d->n >= 256;
    run_fn fn = run_pick(d->rows_mode, fused, pair);
    if (!fn) return fail(ctx, HB_UNSUPPORTED, "expert gemm: this rows mode / output combination is not built");
    const size_t stage_bytes = (fused || pair ? 2 : 1) * (size_t)RN_A_BYTES + RN_B_BYTES;
    const size_t static_smem = sizeof(RunBarriers) + (2 * RN_MAX_EXPERTS + 3 * RN_MAX_RUNS + RN_THREADS + 4 * RN_NMAX) * 4;
    const size_t budget = std::min<size_t>(ctx->smem_optin, 227 * 1024) - 2048 - static_smem;
    const uint32_t max_stages = (uint32_t)std::min<size_t>(budget / stage_bytes, RN_MAX_STAGES);
    const uint32_t stages = d->stages ? d->stages : max_stages;
    if (stages < 2 || stages > max_stages) return fail(ctx, HB_UNSUPPORTED, "expert gemm (merged runs): stage count does not fit");
    auto k = std::make_unique<ExpertRunsGemm>();
    k->d = *d;
    k->fn = fn;
    k->fused = fused;
    k->pair = pair;
    k->stages = stages;
    k->smem = stages * stage_bytes + 1024;
    k->kind = 8;
    k->nargs = 5;
    const char* mode = d->rows_mode == HB_ROWS_GATHER ? "gather" : d->rows_mode == HB_ROWS_SCATTER ? "scatter" : "sorted";
    char nm[192];
    snprintf(nm, sizeof nm, "gemm_expert_runs_%ux%u_e%u_k%u_%s_%s_m%u_s%u", d->k, d->n, d->experts, d->top_k, out_tag(d->out), mode, d->bm, stages);
    k->name = nm;
    if (hb_kernel* have = find(ctx, k->name)) {
        auto* e = static_cast<ExpertRunsGemm*>(have);
        e->d.rows_max = std::max(e->d.rows_max, d->rows_max);
        *out = have;
        return HB_OK;
    }
    cudaError_t e = cudaFuncSetAttribute(reinterpret_cast<const void*>(fn), cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(ctx->smem_optin - static_smem - 256));
    if (e != cudaSuccess) return cuda_fail(ctx, e, "cudaFuncSetAttribute(max dynamic shared memory)");
    *out = intern(ctx, std::move(k));
    return HB_OK;
}

}  // namespace hb
