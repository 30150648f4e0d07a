// Expert-tile grouped GEMM of the MoE layer for sm_100a.
//
// Counterpart of the reference's gemm_mma_rows in its Gather / Scatter row modes and of the
// expert branch of gemm_mm2d_rows (src/metal/prefill.rs:317-328, :889-941, :1206-1209, :534-552).
// The sorted (row, slot) pairs arrive as `list` with a tile table (expert, first sorted row,
// rows <= bm) made by moe_sort. An MoE block at 2048 tokens is weight-bandwidth bound, and an
// expert tile has only 16/32/64 token rows, so the product is computed transposed: the expert's
// weight rows are the 128-row tcgen05 operand (streamed once by TMA) and the token tile is the
// narrow N = bm operand. The accumulator in tensor memory is [128 features][bm tokens].
//   warp 0      TMA producer: weight slices (and the token slices when the sorted rows are
//               contiguous in memory: Scatter and Sorted modes)
//   warp 1      tcgen05.mma issuer, tensor-memory owner
//   warps 2-5   epilogue: tcgen05.ld, output mode, stores to row p or to row list[p]
//   warps 6-7   Gather mode: fetch token rows X[list[p] / top_k] with 16-byte loads and write
//               them into the 128-byte-swizzled stage (the layout TMA would have produced)
// With the fused SwiGLU form the gate rows and the matching up rows of the expert feed two
// accumulators, so one thread holds g and u of the same (feature, token).
// Every barrier wait is bounded.
#include <algorithm>

#include "hb_internal.hpp"
#include "tc05.cuh"

namespace hb {

struct ExpertParams {
    void* y;
    const uint16_t* x;      // Gather mode: token rows [m][k]
    const uint32_t* list;
    const uint32_t* tiles;
    uint32_t k_blocks;
    uint32_t n;             // W rows of one expert
    uint32_t n_feat;        // output features of one expert (n, or n/2 fused)
    uint32_t n_blocks;      // ceil(n_feat / 128)
    uint32_t k;             // row length of X
    uint32_t top_k;
    uint32_t stages;
    uint32_t max_tiles;
    uint32_t* status;
};

constexpr int EX_THREADS = 256;
constexpr int EX_MAX_STAGES = 8;
constexpr int EX_A_BYTES = 128 * 64 * 2;

struct __align__(8) ExpertBarriers {
    uint64_t full[EX_MAX_STAGES];
    uint64_t empty[EX_MAX_STAGES];
    uint64_t tmem_full[2];
    uint64_t tmem_empty[2];
    uint32_t tmem_base;
};

enum { SRC_GATHER = 0, SRC_SORTED = 1 };   // where the token operand comes from
enum { DST_SORTED = 0, DST_SCATTER = 1 };  // where output row p goes

template <int BMT, int SRC, int DST, bool FUSED>
__global__ void __launch_bounds__(EX_THREADS, 1)
gemm_experts_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x, const ExpertParams p) {
    constexpr int NACC = FUSED ? 2 : 1;
    constexpr int A_STAGE = NACC * EX_A_BYTES;
    constexpr int B_STAGE = BMT * 128;  // bm rows of 64 bf16; at least 2 KiB, a multiple of 1 KiB
    constexpr int STAGE_BYTES = A_STAGE + B_STAGE;
    constexpr uint32_t ACC_COLS = NACC * BMT;
    constexpr uint32_t TMEM_COLS = (2 * ACC_COLS) < 32 ? 32 : 2 * ACC_COLS;  // 32, 64, 128 or 256: powers of two
    constexpr uint32_t IDESC = umma_idesc_bf16(128, BMT);
    constexpr uint32_t FULL_ARRIVALS = SRC == SRC_GATHER ? 3 : 1;

    extern __shared__ uint8_t smem_raw[];
    __shared__ ExpertBarriers bars;
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
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = bars.tmem_base;
    const uint32_t ntiles = min(p.tiles[0], p.max_tiles);
    const uint32_t work_total = ntiles * p.n_blocks;

    if (warp == 0) {
        if (lane == 0) {
            tma_prefetch_desc(&tm_w);
            if (SRC == SRC_SORTED) tma_prefetch_desc(&tm_x);
            uint32_t s = 0, ph = 0;
            bool ok = true;
            for (uint32_t w = blockIdx.x; ok && w < work_total; w += gridDim.x) {
                const uint32_t t = w / p.n_blocks, nb = w % p.n_blocks;
                const uint32_t expert = p.tiles[1 + 3 * t], start = p.tiles[2 + 3 * t];
                const int row_w0 = (int)(expert * p.n + nb * 128);
                const int row_w1 = (int)(expert * p.n + p.n_feat + nb * 128);
                for (uint32_t kb = 0; kb < p.k_blocks; ++kb) {
                    if (!mbar_wait(smem_u32(&bars.empty[s]), ph ^ 1u)) {
                        report(p.status, ST_WAIT_TIMEOUT, WHERE_EMPTY, s);
                        ok = false;
                        break;
                    }
                    const uint32_t full = smem_u32(&bars.full[s]);
                    const uint32_t dst = smem_base + s * STAGE_BYTES;
                    mbar_arrive_expect_tx(full, SRC == SRC_SORTED ? STAGE_BYTES : A_STAGE);
                    tma_load_2d(dst, &tm_w, full, (int)(kb * 64), row_w0);
                    if (FUSED) tma_load_2d(dst + EX_A_BYTES, &tm_w, full, (int)(kb * 64), row_w1);
                    if (SRC == SRC_SORTED) tma_load_2d(dst + A_STAGE, &tm_x, full, (int)(kb * 64), (int)start);
                    if (++s == S) { s = 0; ph ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            uint32_t s = 0, ph = 0, it = 0;
            bool ok = true;
            for (uint32_t w = blockIdx.x; ok && w < work_total; w += gridDim.x, ++it) {
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
                    tc_fence_after();
                    const uint32_t a_addr = smem_base + s * STAGE_BYTES;
                    const uint64_t a_desc = umma_desc_sw128(a_addr);
                    const uint64_t b_desc = umma_desc_sw128(a_addr + A_STAGE);
#pragma unroll
                    for (uint32_t k4 = 0; k4 < 4; ++k4) {
                        const uint32_t accumulate = (kb | k4) != 0 ? 1u : 0u;
                        umma_bf16(d_tmem, a_desc + 2 * k4, b_desc + 2 * k4, IDESC, accumulate);
                        if (FUSED) umma_bf16(d_tmem + BMT, umma_desc_sw128(a_addr + EX_A_BYTES) + 2 * k4, b_desc + 2 * k4, IDESC, accumulate);
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
            const uint32_t t = w / p.n_blocks, nb = w % p.n_blocks;
            const uint32_t start = p.tiles[2 + 3 * t], rows = min(p.tiles[3 + 3 * t], (uint32_t)BMT);
            const uint32_t acc = it & 1u, acc_ph = (it >> 1) & 1u;
            const bool got = mbar_wait(smem_u32(&bars.tmem_full[acc]), acc_ph);
            if (!__all_sync(0xffffffffu, got)) {
                if (lane == 0) report(p.status, ST_WAIT_TIMEOUT, WHERE_TMEM_FULL, acc);
                break;
            }
            tc_fence_after();
            const uint32_t feat = nb * 128 + q * 32 + lane;
            const uint32_t t_addr = tmem_base + ((q * 32u) << 16) + acc * ACC_COLS;
            uint16_t* y = reinterpret_cast<uint16_t*>(p.y);
#pragma unroll
            for (int c = 0; c < BMT / 16; ++c) {
                uint32_t g[16], u[16];
                tmem_ld_32x16(t_addr + c * 16, g);
                if (FUSED) tmem_ld_32x16(t_addr + BMT + c * 16, u);
                tmem_ld_wait();
                if (feat < p.n_feat) {
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const uint32_t r = c * 16 + j;
                        if (r < rows) {
                            const uint32_t prow = DST == DST_SCATTER ? p.list[start + r] : start + r;
                            uint32_t o;
                            if (FUSED) o = swiglu_bf16(round_bf16(__uint_as_float(g[j])), round_bf16(__uint_as_float(u[j])));
                            else o = f32_to_bf16(__uint_as_float(g[j]));
                            y[(size_t)prow * p.n_feat + feat] = (uint16_t)o;
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&bars.tmem_empty[acc]));
        }
    } else if (SRC == SRC_GATHER) {
        // Two warps fill the token operand: warp g takes rows g, g+2, .. of each group of 8; a lane
        // owns one 16-byte chunk of a row. Chunk c of row r lands at r*128 + ((c ^ (r & 7)) << 4),
        // the 128-byte swizzle of the weight tiles.
        const uint32_t gw = (uint32_t)warp - 6u;
        uint32_t s = 0, ph = 0;
        bool ok = true;
        for (uint32_t w = blockIdx.x; ok && w < work_total; w += gridDim.x) {
            const uint32_t t = w / p.n_blocks;
            const uint32_t start = p.tiles[2 + 3 * t], rows = min(p.tiles[3 + 3 * t], (uint32_t)BMT);
            constexpr int PASSES = BMT / 8;  // rows per warp pass: 4
            const uint32_t chunk = lane & 7u;
            const uint16_t* src[PASSES];
#pragma unroll
            for (int i = 0; i < PASSES; ++i) {
                const uint32_t r = (uint32_t)i * 8u + gw * 4u + (lane >> 3);
                src[i] = r < rows ? p.x + (size_t)(p.list[start + r] / p.top_k) * p.k + chunk * 8 : nullptr;
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
                for (int i = 0; i < PASSES; ++i) {
                    const uint32_t r = (uint32_t)i * 8u + gw * 4u + (lane >> 3);
                    uint4 v = make_uint4(0, 0, 0, 0);
                    if (src[i] != nullptr && k_in) v = __ldg(reinterpret_cast<const uint4*>(src[i] + (size_t)kb * 64));
                    const uint32_t at = b_dst + r * 128u + ((chunk ^ (r & 7u)) << 4);
                    asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(at), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
                }
                fence_proxy_async();
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&bars.full[s]));
                if (++s == S) { s = 0; ph ^= 1u; }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
}

namespace {

typedef void (*ex_fn)(const CUtensorMap, const CUtensorMap, const ExpertParams);

template <int BMT>
ex_fn ex_pick(uint32_t rows_mode, bool fused) {
    if (rows_mode == HB_ROWS_GATHER) return fused ? gemm_experts_kernel<BMT, SRC_GATHER, DST_SORTED, true> : gemm_experts_kernel<BMT, SRC_GATHER, DST_SORTED, false>;
    if (rows_mode == HB_ROWS_SORTED) return fused ? gemm_experts_kernel<BMT, SRC_SORTED, DST_SORTED, true> : gemm_experts_kernel<BMT, SRC_SORTED, DST_SORTED, false>;
    if (rows_mode == HB_ROWS_SCATTER) return fused ? nullptr : gemm_experts_kernel<BMT, SRC_SORTED, DST_SCATTER, false>;
    return nullptr;
}

struct ExpertGemm : hb_kernel {
    hb_gemm_desc d{};
    ex_fn fn = nullptr;
    bool fused = false;
    uint32_t stages = 0;
    size_t smem = 0;
    const void* last_w = nullptr;
    const void* last_x = nullptr;
    uint32_t last_m = 0;
    CUtensorMap tm_w{}, tm_x{};

    int launch(hb_ctx* ctx, const hb_range* a, int na, uint32_t m) override {
        if (na != 5) return fail(ctx, HB_INVALID, name + ": bindings are W, X, Y, list, tiles");
        if (m == 0 || m > d.rows_max) return fail(ctx, HB_INVALID, name + ": m outside 1.." + std::to_string(d.rows_max));
        const uint32_t pairs = m * d.top_k;
        const uint32_t n_feat = fused ? d.n / 2 : d.n;
        const uint32_t max_tiles = hb_moe_tiles(m, d.top_k, d.experts, d.bm);
        const size_t xrows = d.rows_mode == HB_ROWS_GATHER ? m : pairs;
        if (!range_ok(a[0], (size_t)d.experts * d.n * d.k * 2) || !range_ok(a[1], xrows * d.k * 2) || !range_ok(a[2], (size_t)pairs * n_feat * 2) ||
            !range_ok(a[3], (size_t)pairs * 4) || !range_ok(a[4], (1 + 3 * (size_t)max_tiles) * 4))
            return fail(ctx, HB_INVALID, name + ": a bound range is too small for " + std::to_string(m) + " rows");
        if (reinterpret_cast<uintptr_t>(a[1].ptr) & 15u) return fail(ctx, HB_INVALID, name + ": X must be 16-byte aligned");
        if (a[0].ptr != last_w || a[1].ptr != last_x || m != last_m) {
            int r = make_tmap_bf16(ctx, &tm_w, a[0].ptr, (uint64_t)d.experts * d.n, d.k, 128);
            if (r != HB_OK) return r;
            r = make_tmap_bf16(ctx, &tm_x, a[1].ptr, xrows, d.k, d.bm);
            if (r != HB_OK) return r;
            last_w = a[0].ptr;
            last_x = a[1].ptr;
            last_m = m;
        }
        ExpertParams p{};
        p.y = a[2].ptr;
        p.x = static_cast<const uint16_t*>(a[1].ptr);
        p.list = static_cast<const uint32_t*>(a[3].ptr);
        p.tiles = static_cast<const uint32_t*>(a[4].ptr);
        p.k_blocks = (d.k + 63) / 64;
        p.n = d.n;
        p.n_feat = n_feat;
        p.n_blocks = (n_feat + 127) / 128;
        p.k = d.k;
        p.top_k = d.top_k;
        p.stages = stages;
        p.max_tiles = max_tiles;
        p.status = ctx->status_dev;
        fn<<<ctx->sm_count, EX_THREADS, smem, ctx->stream>>>(tm_w, tm_x, p);
        HB_CUDA(ctx, cudaGetLastError());
        ctx->launches++;
        return HB_OK;
    }
};

}  // namespace

int make_gemm_expert_runs(hb_ctx* ctx, const hb_gemm_desc* d, hb_kernel** out);

int make_gemm_experts(hb_ctx* ctx, const hb_gemm_desc* d, hb_kernel** out) {
    *out = nullptr;
    if (d->k == 0 || d->n == 0 || d->rows_max == 0 || d->experts == 0 || d->top_k == 0)
        return fail(ctx, HB_INVALID, "expert gemm: k, n, rows_max, experts and top_k must be positive");
    if (d->k % 8 != 0) return fail(ctx, HB_UNSUPPORTED, "expert gemm: k must be a multiple of 8");
    if (d->bm != 16 && d->bm != 32 && d->bm != 64) return fail(ctx, HB_UNSUPPORTED, "expert gemm: tile rows 16, 32 or 64");
    const bool fused = d->out == HB_OUT_SWIGLU;
    if (d->out != HB_OUT_BF16 && !fused) return fail(ctx, HB_UNSUPPORTED, "expert gemm: output bf16, or the fused SwiGLU of the [gate | up] rows");
    if (fused && d->n % 2 != 0) return fail(ctx, HB_INVALID, "expert gemm: the SwiGLU form needs an even n");
    if (d->merge_runs) return make_gemm_expert_runs(ctx, d, out);
    ex_fn fn = nullptr;
    switch (d->bm) {
        case 16: fn = ex_pick<16>(d->rows_mode, fused); break;
        case 32: fn = ex_pick<32>(d->rows_mode, fused); break;
        case 64: fn = ex_pick<64>(d->rows_mode, fused); break;
    }
    if (!fn) return fail(ctx, HB_UNSUPPORTED, "expert gemm: this rows mode / output combination is not built");
    const size_t stage_bytes = (fused ? 2 : 1) * (size_t)EX_A_BYTES + (size_t)d->bm * 128;
    const size_t budget = std::min<size_t>(ctx->smem_optin, 227 * 1024) - 2048;
    const uint32_t max_stages = (uint32_t)std::min<size_t>(budget / stage_bytes, EX_MAX_STAGES);
    const uint32_t stages = d->stages ? d->stages : max_stages;
    if (stages < 2 || stages > max_stages) return fail(ctx, HB_UNSUPPORTED, "expert gemm: stage count does not fit");
    auto k = std::make_unique<ExpertGemm>();
    k->d = *d;
    k->fn = fn;
    k->fused = fused;
    k->stages = stages;
    k->smem = stages * stage_bytes + 1024;
    k->kind = 8;
    k->nargs = 5;
    const char* mode = d->rows_mode == HB_ROWS_GATHER ? "gather" : d->rows_mode == HB_ROWS_SCATTER ? "scatter" : "sorted";
    char nm[192];
    snprintf(nm, sizeof nm, "gemm_experts_%ux%u_e%u_k%u_%s_%s_m%u_s%u", d->k, d->n, d->experts, d->top_k, out_tag(d->out), mode, d->bm, stages);
    k->name = nm;
    if (hb_kernel* have = find(ctx, k->name)) {
        auto* e = static_cast<ExpertGemm*>(have);
        e->d.rows_max = std::max(e->d.rows_max, d->rows_max);
        *out = have;
        return HB_OK;
    }
    cudaError_t e = cudaFuncSetAttribute(reinterpret_cast<const void*>(fn), cudaFuncAttributeMaxDynamicSharedMemorySize, (int)ctx->smem_optin - 1024);  // (static shared memory counts too) the limit is per function, not per kernel object: always the most
    if (e != cudaSuccess) return cuda_fail(ctx, e, "cudaFuncSetAttribute(max dynamic shared memory)");
    *out = intern(ctx, std::move(k));
    return HB_OK;
}

}  // namespace hb
