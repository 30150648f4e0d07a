// Prefill GEMM Y[m][n] = out(X[m][k] . W[n][k]^T) for sm_100a.
//
// Counterpart of the reference's gemm_mma_rows / gemm_mm2d / gemm_nax_swiglu
// (src/metal/prefill.rs:838-1301, :442-567, :755-822), designed for Blackwell:
// both operands are K-major, which is what tcgen05.mma takes from shared memory
// without a transpose. One persistent CTA per SM walks output tiles of 128 x BN:
//   warp 0    TMA producer: 64-element K slices of X (128 rows) and W (BN rows)
//             into a ring of 128-byte-swizzled shared-memory stages;
//   warp 1    allocates tensor memory, one elected lane issues tcgen05.mma
//             (bf16 x bf16 -> f32 in TMEM) and commits stage-free / tile-done
//             barriers;
//   warps 2-5 epilogue: tcgen05.ld the accumulator (two TMEM buffers, so the
//             epilogue of tile i overlaps the main loop of tile i+1), apply the
//             output mode and store.
// Rows past m and columns past n are zero-filled by TMA and never stored (the
// reference clamps the loads instead, prefill.rs:927-941; the stored values are
// the same). Every barrier wait is bounded; on expiry the CTA reports through
// the status words and leaves.
#include <algorithm>
#include <cstring>

#include "gemm_common.cuh"

namespace hb {

template <int BN, int OUT>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_tn_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_w, const GemmParams p) {
    constexpr int B_BYTES = BN * BK * 2;
    constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    constexpr int HALF = BN / 2;           // W rows per TMA box; SWIGLU: gate columns per tile
    constexpr uint32_t TMEM_COLS = 2 * BN; // two accumulators
    constexpr uint32_t IDESC = umma_idesc_bf16(BM, BN);

    extern __shared__ uint8_t smem_raw[];
    __shared__ GemmBarriers bars;
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t S = p.stages;

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < S; ++s) {
            mbar_init(smem_u32(&bars.full[s]), 1);
            mbar_init(smem_u32(&bars.empty[s]), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(smem_u32(&bars.tmem_full[a]), 1);
            mbar_init(smem_u32(&bars.tmem_empty[a]), 4);
        }
        bars.abort = 0;
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

    if (warp == 0) {
        // ---------------------------------------------------------- producer
        // Overlapped launch (hb_set_launch_overlap): the kernel may have started while the kernel before it on the stream
        // still runs. W is not that kernel's output, so the W boxes of the first stages are requested at once; X may be,
        // so its boxes follow griddepcontrol.wait. In a plain launch the wait returns at once.
        if (lane == 0) {
            tma_prefetch_desc(&tm_x);
            tma_prefetch_desc(&tm_w);
            bool ok = true;
            for (int pass = 0; pass < 2 && ok; ++pass) {  // pass 0: the W boxes of the first S fills; pass 1: everything else
                uint32_t s = 0, ph = 0, fill = 0;
                for (uint32_t tile = blockIdx.x; ok && tile < p.num_tiles; tile += gridDim.x) {
                    const uint32_t tm = p.m_first ? tile % p.tiles_m : tile / p.tiles_n;
                    const uint32_t tn = p.m_first ? tile / p.tiles_m : tile % p.tiles_n;
                    const int row_x = (int)(tm * BM);
                    int row_w0, row_w1;
                    if constexpr (OUT == HB_OUT_SWIGLU) {
                        row_w0 = (int)(tn * HALF);
                        row_w1 = (int)(p.n_out + tn * HALF);
                    } else {
                        row_w0 = (int)(tn * BN);
                        row_w1 = row_w0 + HALF;
                    }
                    for (uint32_t kb = 0; kb < p.k_blocks; ++kb, ++fill) {
                        const bool early = fill < S;  // the stage is free: nothing to wait for
                        if (pass == 0 && !early) { ok = false; break; }  // (pass 0 ends here; ok is set again below)
                        if (pass == 1 && !early && !mbar_wait(smem_u32(&bars.empty[s]), ph ^ 1u)) {
                            report(p.status, ST_WAIT_TIMEOUT, WHERE_EMPTY, s);
                            ok = false;
                            break;
                        }
                        const uint32_t full = smem_u32(&bars.full[s]);
                        const uint32_t a_dst = smem_base + s * STAGE_BYTES;
                        const bool do_w = pass == 0 || !early, do_x = pass == 1;
                        if (do_w) mbar_arrive_expect_tx(full, STAGE_BYTES);
                        if (do_x) tma_load_2d(a_dst, &tm_x, full, (int)(kb * BK), row_x);
                        if (do_w) {
                            tma_load_2d(a_dst + A_BYTES, &tm_w, full, (int)(kb * BK), row_w0);
                            tma_load_2d(a_dst + A_BYTES + HALF * BK * 2, &tm_w, full, (int)(kb * BK), row_w1);
                        }
                        if (++s == S) { s = 0; ph ^= 1u; }
                    }
                }
                if (pass == 0) {
                    ok = true;
                    griddep_wait();
                }
            }
            // every load of this CTA is requested: the kernel behind this one may take the SMs as they fall free
            griddep_launch_dependents();
        }
    } else if (warp == 1) {
        // --------------------------------------------------------- MMA issuer
        if (lane == 0) {
            uint32_t s = 0, ph = 0, it = 0;
            bool ok = true;
            for (uint32_t tile = blockIdx.x; ok && tile < p.num_tiles; tile += gridDim.x, ++it) {
                const uint32_t acc = it & 1u, acc_ph = (it >> 1) & 1u;
                if (!mbar_wait(smem_u32(&bars.tmem_empty[acc]), acc_ph ^ 1u)) {
                    report(p.status, ST_WAIT_TIMEOUT, WHERE_TMEM_EMPTY, acc);
                    break;
                }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * BN;
                for (uint32_t kb = 0; kb < p.k_blocks; ++kb) {
                    if (!mbar_wait(smem_u32(&bars.full[s]), ph)) {
                        report(p.status, ST_WAIT_TIMEOUT, WHERE_FULL, s);
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t a_addr = smem_base + s * STAGE_BYTES;
                    const uint64_t a_desc = umma_desc_sw128(a_addr);
                    const uint64_t b_desc = umma_desc_sw128(a_addr + A_BYTES);
#pragma unroll
                    for (uint32_t k4 = 0; k4 < BK / 16; ++k4)
                        umma_bf16(d_tmem, a_desc + 2 * k4, b_desc + 2 * k4, IDESC, (kb | k4) != 0 ? 1u : 0u);
                    umma_commit(smem_u32(&bars.empty[s]));
                    if (++s == S) { s = 0; ph ^= 1u; }
                }
                if (ok) umma_commit(smem_u32(&bars.tmem_full[acc]));
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue
        const uint32_t q = (uint32_t)warp & 3u;  // the TMEM lane quarter this warp may read
        uint32_t it = 0;
        griddep_wait();  // Y may be read (residual) or still be in use by the kernel before this one
        for (uint32_t tile = blockIdx.x; tile < p.num_tiles; tile += gridDim.x, ++it) {
            const uint32_t tm = p.m_first ? tile % p.tiles_m : tile / p.tiles_n;
            const uint32_t tn = p.m_first ? tile / p.tiles_m : tile % p.tiles_n;
            const uint32_t acc = it & 1u, acc_ph = (it >> 1) & 1u;
            const bool got = mbar_wait(smem_u32(&bars.tmem_full[acc]), acc_ph);
            if (!__all_sync(0xffffffffu, got)) {
                if (lane == 0) report(p.status, ST_WAIT_TIMEOUT, WHERE_TMEM_FULL, acc);
                break;
            }
            tc_fence_after();
            const uint32_t row = tm * BM + q * 32 + lane;
            const uint32_t t_addr = tmem_base + ((q * 32u) << 16) + acc * BN;
            if constexpr (OUT == HB_OUT_SWIGLU) {
#pragma unroll 1
                for (int c = 0; c < HALF / 32; ++c) {
                    uint32_t g[32], u[32];
                    tmem_ld_32x32(t_addr + c * 32, g);
                    tmem_ld_32x32(t_addr + HALF + c * 32, u);
                    tmem_ld_wait();
                    store_chunk<OUT>(p, row, tn * HALF + c * 32, g, u);
                }
            } else {
#pragma unroll 1
                for (int c = 0; c < BN / 32; ++c) {
                    uint32_t v[32];
                    tmem_ld_32x32(t_addr + c * 32, v);
                    tmem_ld_wait();
                    store_chunk<OUT>(p, row, tn * BN + c * 32, v, v);
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&bars.tmem_empty[acc]));
        }
    }

    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
}

// ------------------------------------------------------------------ host side

namespace {

typedef void (*gemm_fn)(const CUtensorMap, const CUtensorMap, const GemmParams);

template <int BN>
gemm_fn pick_out(uint32_t out) {
    switch (out) {
        case HB_OUT_BF16: return gemm_bf16_tn_kernel<BN, HB_OUT_BF16>;
        case HB_OUT_F32: return gemm_bf16_tn_kernel<BN, HB_OUT_F32>;
        case HB_OUT_RESIDUAL: return gemm_bf16_tn_kernel<BN, HB_OUT_RESIDUAL>;
        case HB_OUT_SWIGLU: return gemm_bf16_tn_kernel<BN, HB_OUT_SWIGLU>;
    }
    return nullptr;
}

struct DenseGemm : hb_kernel {
    hb_gemm_desc d{};
    gemm_fn fn = nullptr;
    uint32_t bn = 0, stages = 0;
    size_t smem = 0;
    // Tensor maps depend on the bound pointers and on m; the last ones are kept.
    const void* last_w = nullptr;
    const void* last_x = nullptr;
    uint32_t last_m = 0;
    CUtensorMap tm_x{}, tm_w{};

    int launch(hb_ctx* ctx, const hb_range* a, int na, uint32_t m) override {
        if (na != 3) return fail(ctx, HB_INVALID, name + ": bindings are W, X, Y");
        if (m == 0 || m > d.rows_max) return fail(ctx, HB_INVALID, name + ": m = " + std::to_string(m) + " outside 1.." + std::to_string(d.rows_max));
        const uint32_t n_out = d.out == HB_OUT_SWIGLU ? d.n / 2 : d.n;
        const size_t ybytes = (size_t)m * n_out * (d.out == HB_OUT_F32 ? 4 : 2);
        if (!range_ok(a[0], (size_t)d.n * d.k * 2) || !range_ok(a[1], (size_t)m * d.k * 2) || !range_ok(a[2], ybytes))
            return fail(ctx, HB_INVALID, name + ": a bound range is too small for " + std::to_string(m) + " rows");
        if (a[0].ptr != last_w || a[1].ptr != last_x || m != last_m) {
            int r = make_tmap_bf16(ctx, &tm_w, a[0].ptr, d.n, d.k, bn / 2);
            if (r != HB_OK) return r;
            r = make_tmap_bf16(ctx, &tm_x, a[1].ptr, m, d.k, BM);
            if (r != HB_OK) return r;
            last_w = a[0].ptr;
            last_x = a[1].ptr;
            last_m = m;
        }
        GemmParams p{};
        p.y = a[2].ptr;
        p.m = m;
        p.n_w = d.n;
        p.n_out = n_out;
        p.k_blocks = (d.k + BK - 1) / BK;
        p.tiles_m = (m + BM - 1) / BM;
        const uint32_t cols_per_tile = d.out == HB_OUT_SWIGLU ? bn / 2 : bn;
        p.tiles_n = (n_out + cols_per_tile - 1) / cols_per_tile;
        p.num_tiles = p.tiles_m * p.tiles_n;
        p.stages = stages;
        p.m_first = d.m_first;
        const uint32_t elem = d.out == HB_OUT_F32 ? 4 : 2;
        p.vec_ok = ((reinterpret_cast<uintptr_t>(a[2].ptr) & 15u) == 0 && ((size_t)n_out * elem) % 16 == 0) ? 1u : 0u;
        p.status = ctx->status_dev;
        const uint32_t grid = std::min<uint32_t>(p.num_tiles, (uint32_t)ctx->sm_count);
        HB_CUDA(ctx, launch_kernel(ctx, true, fn, dim3(grid), dim3(GEMM_THREADS), smem, tm_x, tm_w, p));
        HB_CUDA(ctx, cudaGetLastError());
        ctx->launches++;
        return HB_OK;
    }
};

}  // namespace

int make_gemm_experts(hb_ctx* ctx, const hb_gemm_desc* d, hb_kernel** out);
int make_gemm_streamk(hb_ctx* ctx, const hb_gemm_desc* d, hb_kernel** out);
int make_gemm_pair(hb_ctx* ctx, const hb_gemm_desc* d, hb_kernel** out);

int make_gemm(hb_ctx* ctx, const hb_gemm_desc* d, hb_kernel** out) {
    *out = nullptr;
    if (d->rows_mode != HB_ROWS_DENSE) return make_gemm_experts(ctx, d, out);
    if (d->k == 0 || d->n == 0 || d->rows_max == 0) return fail(ctx, HB_INVALID, "gemm: k, n and rows_max must be positive");
    if (d->k % 8 != 0) return fail(ctx, HB_UNSUPPORTED, "gemm: k must be a multiple of 8 (16-byte rows for TMA)");
    if (d->out > HB_OUT_SWIGLU) return fail(ctx, HB_INVALID, "gemm: unknown output mode");
    if (d->out == HB_OUT_SWIGLU && d->n % 2 != 0) return fail(ctx, HB_INVALID, "gemm: the SwiGLU form needs an even n ([gate | up])");
    if (d->cta_pair) return make_gemm_pair(ctx, d, out);
    if (d->y_shards > 1) return fail(ctx, HB_UNSUPPORTED, "gemm: a Y in row blocks is built for the CTA-pair form only");
    if (d->stream_k) return make_gemm_streamk(ctx, d, out);
    const uint32_t bn = d->tile_n ? d->tile_n : 256;
    gemm_fn fn = nullptr;
    switch (bn) {
        case 64: fn = pick_out<64>(d->out); break;
        case 128: fn = pick_out<128>(d->out); break;
        case 256: fn = pick_out<256>(d->out); break;
        default: return fail(ctx, HB_UNSUPPORTED, "gemm: tile_n must be 64, 128 or 256");
    }
    const size_t stage_bytes = A_BYTES + (size_t)bn * BK * 2;
    const size_t budget = std::min<size_t>(ctx->smem_optin, 227 * 1024) - 2048;  // alignment slack + static barriers
    uint32_t max_stages = (uint32_t)std::min<size_t>(budget / stage_bytes, MAX_STAGES);
    uint32_t stages = d->stages ? d->stages : max_stages;
    if (stages < 2 || stages > max_stages)
        return fail(ctx, HB_UNSUPPORTED, "gemm: " + std::to_string(stages) + " stages of " + std::to_string(stage_bytes) + " bytes do not fit (2.." +
                                             std::to_string(max_stages) + ")");
    auto k = std::make_unique<DenseGemm>();
    k->d = *d;
    k->d.tile_n = bn;
    k->fn = fn;
    k->bn = bn;
    k->stages = stages;
    k->smem = stages * stage_bytes + 1024;
    k->kind = 1;
    k->nargs = 3;
    char nm[160];
    snprintf(nm, sizeof nm, "gemm_tc_%ux%u_%s%s_t128x%u_s%u", d->k, d->n, out_tag(d->out), d->m_first ? "_mf" : "", bn, stages);
    k->name = nm;
    if (hb_kernel* have = find(ctx, k->name)) {
        auto* g = static_cast<DenseGemm*>(have);
        g->d.rows_max = std::max(g->d.rows_max, d->rows_max);
        *out = have;
        return HB_OK;
    }
    cudaError_t e = cudaFuncSetAttribute(reinterpret_cast<const void*>(fn), cudaFuncAttributeMaxDynamicSharedMemorySize, (int)ctx->smem_optin - 1024);  // (static shared memory counts too) the limit is per function, not per kernel object: always the most
    if (e != cudaSuccess) return cuda_fail(ctx, e, "cudaFuncSetAttribute(max dynamic shared memory)");
    *out = intern(ctx, std::move(k));
    return HB_OK;
}

}  // namespace hb

