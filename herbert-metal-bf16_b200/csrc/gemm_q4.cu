// Prefill GEMM on Q4_0 weights, decoded while they are staged: Y[m][n] = out(X[m][k] . dq(W)[n][k]^T).
//
// Counterpart of the reference's gemm_mma_q4 (src/metal/prefill.rs:427-434, 1058-1076; engine switch q4.fuse,
// src/metal/qwen.rs:169-173): "each staged cell of W is one word of a block of 32, decoded there to bf16(d * q) as
// dequant_q4 decodes it, so the sums are those of dequant_q4 then the GEMM, bit for bit". The alternative, dequant_q4
// into a bf16 copy followed by the bf16 GEMM, writes and re-reads 2 bytes per weight; this form reads the 0.5625 bytes
// the weight occupies and nothing else. Both exist and the selection loop times them (hb_select_gemm_q4).
//
// Built on the one-CTA tcgen05 GEMM (gemm_dense.cu): 128 x BN output tiles, the same ring of 128-byte-swizzled
// stages, the same K order (so the same bits as that kernel on the decoded weights). The X slice of a stage comes by
// TMA; the W slice is written by eight decode warps: a thread fetches a block's 16 bytes of nibbles and its f16
// scale with ordinary loads one stage ahead, turns each word into eight bf16 (the nibble as the low byte of
// 0x4B000000 is the float 8388608 + nibble: no integer conversion; d * q in f32, one rounding) and stores the 16-byte
// chunk where TMA would have put it (chunk c of row r at r * 128 + ((c ^ (r & 7)) << 4)). Word i of block j of the
// stage's 64-element K slice is chunk 4 j + i of the row. The stage's barrier counts the TMA bytes and the eight warps.
//   warp 0      TMA producer (X)          warp 1      tcgen05.mma issuer, tensor-memory owner
//   warps 2-5   epilogue                  warps 6-13  W decode
// Every barrier wait is bounded; on expiry the CTA reports through the status words and leaves.
#include <algorithm>
#include <cstring>

#include <cuda_fp16.h>

#include "gemm_common.cuh"

namespace hb {

constexpr int Q4G_THREADS = 448;
constexpr int Q4G_DECODE_WARPS = 8;
constexpr int Q4G_DECODE_THREADS = Q4G_DECODE_WARPS * 32;

struct GemmQ4Params {
    GemmParams g;
    const uint4* wq;       // [n][k / 32] blocks of 16 bytes
    const uint16_t* sc;    // [n][k / 32] f16 scales
    uint32_t nblk;         // k / 32
};

// The eight weights of one word as four bf16 pairs, bf16(d * q) each: dequant_q4's arithmetic (src/metal/kernels.rs:
// 1074-1102, 1425-1450). Weights 8i + 0..3 are the low nibbles of bytes 0..3, weights 8i + 4..7 the high ones.
__device__ __forceinline__ uint4 q4_word_to_bf16(uint32_t ww, float d) {
    const uint32_t lo = (ww & 0x0F0F0F0Fu) ^ 0x08080808u, hi = ((ww >> 4) & 0x0F0F0F0Fu) ^ 0x08080808u;
    auto q = [](uint32_t bytes, uint32_t sel) { return __uint_as_float(__byte_perm(bytes, 0x4B000000u, 0x7650u + sel)) - 8388616.0f; };
    uint4 o;
    o.x = f32x2_to_bf16x2(__fmul_rn(d, q(lo, 0)), __fmul_rn(d, q(lo, 1)));
    o.y = f32x2_to_bf16x2(__fmul_rn(d, q(lo, 2)), __fmul_rn(d, q(lo, 3)));
    o.z = f32x2_to_bf16x2(__fmul_rn(d, q(hi, 0)), __fmul_rn(d, q(hi, 1)));
    o.w = f32x2_to_bf16x2(__fmul_rn(d, q(hi, 2)), __fmul_rn(d, q(hi, 3)));
    return o;
}

template <int BN, int OUT>
__global__ void __launch_bounds__(Q4G_THREADS, 1)
gemm_q4_tn_kernel(const __grid_constant__ CUtensorMap tm_x, const GemmQ4Params pp) {
    const GemmParams& p = pp.g;
    constexpr int B_BYTES = BN * BK * 2;
    constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    constexpr int HALF = BN / 2;
    constexpr uint32_t TMEM_COLS = 2 * BN;
    constexpr uint32_t IDESC = umma_idesc_bf16(BM, BN);
    constexpr int ITEMS = 2 * BN / Q4G_DECODE_THREADS;  // blocks a decode thread handles per stage (BN 128: 1, 256: 2)
    static_assert(ITEMS >= 1, "the decode warps are laid out for tiles of at least 128 columns");

    extern __shared__ uint8_t smem_raw[];
    __shared__ GemmBarriers bars;
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t S = p.stages;

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < S; ++s) {
            mbar_init(smem_u32(&bars.full[s]), 1 + Q4G_DECODE_WARPS);  // the producer's expect_tx arrival and the decode warps
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
        // ---------------------------------------------------------- producer: the X slice of every stage
        if (lane == 0) {
            tma_prefetch_desc(&tm_x);
            uint32_t s = 0, ph = 0;
            bool ok = true;
            for (uint32_t tile = blockIdx.x; ok && tile < p.num_tiles; tile += gridDim.x) {
                const uint32_t tm = p.m_first ? tile % p.tiles_m : tile / p.tiles_n;
                const int row_x = (int)(tm * BM);
                for (uint32_t kb = 0; kb < p.k_blocks; ++kb) {
                    if (!mbar_wait(smem_u32(&bars.empty[s]), ph ^ 1u)) {
                        report(p.status, ST_WAIT_TIMEOUT, WHERE_EMPTY, s);
                        ok = false;
                        break;
                    }
                    const uint32_t full = smem_u32(&bars.full[s]);
                    mbar_arrive_expect_tx(full, A_BYTES);
                    tma_load_2d(smem_base + s * STAGE_BYTES, &tm_x, full, (int)(kb * BK), row_x);
                    if (++s == S) { s = 0; ph ^= 1u; }
                }
            }
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
                    fence_proxy_async();  // the W slice was written with ordinary stores
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
    } else if (warp < 6) {
        // ------------------------------------------------------------ epilogue
        const uint32_t q = (uint32_t)warp & 3u;
        uint32_t it = 0;
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
    } else {
        // ------------------------------------------------------------ W decode
        const uint32_t t = threadIdx.x - 6 * 32;  // 0..255
        // this thread's blocks of a stage: item u covers tile row (t + 256 u) / 2, block (t + 256 u) % 2 of the K slice
        uint4 wv[ITEMS];
        uint32_t sv[ITEMS];
        auto fetch = [&](uint32_t tile, uint32_t kb) {
            const uint32_t tn = p.m_first ? tile / p.tiles_m : tile % p.tiles_n;
#pragma unroll
            for (int u = 0; u < ITEMS; ++u) {
                const uint32_t i = t + Q4G_DECODE_THREADS * u, r = i >> 1, j = i & 1u;
                uint32_t wrow;
                if constexpr (OUT == HB_OUT_SWIGLU) wrow = r < (uint32_t)HALF ? min(tn * HALF + r, p.n_out - 1) : min(p.n_out + tn * HALF + (r - HALF), p.n_w - 1);
                else wrow = min(tn * BN + r, p.n_w - 1);  // rows past the end read the last row and are not stored
                const uint32_t blk = kb * 2 + j;
                if (blk < pp.nblk) {
                    const size_t at = (size_t)wrow * pp.nblk + blk;
                    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(wv[u].x), "=r"(wv[u].y), "=r"(wv[u].z), "=r"(wv[u].w) : "l"(pp.wq + at));
                    sv[u] = __ldg(pp.sc + at);
                } else {  // K ends inside the slice: zeros, as TMA fills the X slice
                    wv[u] = make_uint4(0u, 0u, 0u, 0u);
                    sv[u] = 0u;
                }
            }
        };
        uint32_t s = 0, ph = 0;
        bool ok = true;
        uint32_t tile = blockIdx.x, kb = 0;
        if (tile < p.num_tiles) fetch(tile, 0);
        while (ok && tile < p.num_tiles) {
            // the blocks of this stage are in registers; ask for the next stage's before working on these
            uint4 cur_w[ITEMS];
            uint32_t cur_s[ITEMS];
#pragma unroll
            for (int u = 0; u < ITEMS; ++u) { cur_w[u] = wv[u]; cur_s[u] = sv[u]; }
            uint32_t ntile = tile, nkb = kb + 1;
            if (nkb == p.k_blocks) { nkb = 0; ntile = tile + gridDim.x; }
            if (ntile < p.num_tiles) fetch(ntile, nkb);
            const bool got = mbar_wait(smem_u32(&bars.empty[s]), ph ^ 1u);
            if (!__all_sync(0xffffffffu, got)) {
                if (lane == 0) report(p.status, ST_WAIT_TIMEOUT, WHERE_EMPTY, 16u + s);
                ok = false;
                break;
            }
            const uint32_t b_base = smem_base + s * STAGE_BYTES + A_BYTES;
#pragma unroll
            for (int u = 0; u < ITEMS; ++u) {
                const uint32_t i = t + Q4G_DECODE_THREADS * u, r = i >> 1, j = i & 1u;
                const float d = __half2float(__ushort_as_half((unsigned short)cur_s[u]));
                const uint32_t ww[4] = {cur_w[u].x, cur_w[u].y, cur_w[u].z, cur_w[u].w};
#pragma unroll
                for (uint32_t w4 = 0; w4 < 4; ++w4) {
                    const uint4 o = q4_word_to_bf16(ww[w4], d);
                    const uint32_t dst = b_base + r * 128u + (((4u * j + w4) ^ (r & 7u)) << 4);
                    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(o.x), "r"(o.y), "r"(o.z), "r"(o.w) : "memory");
                }
            }
            fence_proxy_async();  // ordinary stores, read by the tensor core through the async proxy
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&bars.full[s]));
            if (++s == S) { s = 0; ph ^= 1u; }
            tile = ntile;
            kb = nkb;
        }
    }

    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
}

// ------------------------------------------------------------------ host side

namespace {

typedef void (*q4g_fn)(const CUtensorMap, const GemmQ4Params);

template <int BN>
q4g_fn q4g_pick_out(uint32_t out) {
    switch (out) {
        case HB_OUT_BF16: return gemm_q4_tn_kernel<BN, HB_OUT_BF16>;
        case HB_OUT_F32: return gemm_q4_tn_kernel<BN, HB_OUT_F32>;
        case HB_OUT_RESIDUAL: return gemm_q4_tn_kernel<BN, HB_OUT_RESIDUAL>;
        case HB_OUT_SWIGLU: return gemm_q4_tn_kernel<BN, HB_OUT_SWIGLU>;
    }
    return nullptr;
}

struct GemmQ4 : hb_kernel {
    uint32_t k = 0, n = 0, out = 0, rows_max = 0, bn = 0, stages = 0, m_first = 1;
    q4g_fn fn = nullptr;
    size_t smem = 0;
    const void* last_x = nullptr;
    uint32_t last_m = 0;
    CUtensorMap tm_x{};

    int launch(hb_ctx* ctx, const hb_range* a, int na, uint32_t m) override {
        if (na != 4) return fail(ctx, HB_INVALID, name + ": bindings are W (Q4 data), X, Y, scales");
        if (m == 0 || m > rows_max) return fail(ctx, HB_INVALID, name + ": m = " + std::to_string(m) + " outside 1.." + std::to_string(rows_max));
        const uint32_t n_out = out == HB_OUT_SWIGLU ? n / 2 : n;
        const size_t blocks = (size_t)n * (k / 32);
        if (!range_ok(a[0], blocks * 16) || !range_ok(a[1], (size_t)m * k * 2) || !range_ok(a[2], (size_t)m * n_out * (out == HB_OUT_F32 ? 4 : 2)) || !range_ok(a[3], blocks * 2))
            return fail(ctx, HB_INVALID, name + ": a bound range is too small for " + std::to_string(m) + " rows");
        if (reinterpret_cast<uintptr_t>(a[0].ptr) & 15u) return fail(ctx, HB_INVALID, name + ": the Q4 data must be 16-byte aligned");
        if (a[1].ptr != last_x || m != last_m) {
            int r = make_tmap_bf16(ctx, &tm_x, a[1].ptr, m, k, BM);
            if (r != HB_OK) return r;
            last_x = a[1].ptr;
            last_m = m;
        }
        GemmQ4Params pp{};
        GemmParams& p = pp.g;
        p.y = a[2].ptr;
        p.m = m;
        p.n_w = n;
        p.n_out = n_out;
        p.k_blocks = (k + BK - 1) / BK;
        p.tiles_m = (m + BM - 1) / BM;
        const uint32_t cols_per_tile = out == HB_OUT_SWIGLU ? bn / 2 : bn;
        p.tiles_n = (n_out + cols_per_tile - 1) / cols_per_tile;
        p.num_tiles = p.tiles_m * p.tiles_n;
        p.stages = stages;
        p.m_first = m_first;
        const uint32_t elem = out == HB_OUT_F32 ? 4 : 2;
        p.vec_ok = ((reinterpret_cast<uintptr_t>(a[2].ptr) & 15u) == 0 && ((size_t)n_out * elem) % 16 == 0) ? 1u : 0u;
        p.status = ctx->status_dev;
        pp.wq = static_cast<const uint4*>(a[0].ptr);
        pp.sc = static_cast<const uint16_t*>(a[3].ptr);
        pp.nblk = k / 32;
        const uint32_t grid = std::min<uint32_t>(p.num_tiles, (uint32_t)ctx->sm_count);
        fn<<<grid, Q4G_THREADS, smem, ctx->stream>>>(tm_x, pp);
        HB_CUDA(ctx, cudaGetLastError());
        ctx->launches++;
        return HB_OK;
    }
};

}  // namespace

int make_gemm_q4(hb_ctx* ctx, uint32_t k, uint32_t n, uint32_t out, uint32_t tile_n, uint32_t m_first, uint32_t rows_max, hb_kernel** res) {
    *res = nullptr;
    if (k == 0 || n == 0 || rows_max == 0) return fail(ctx, HB_INVALID, "gemm_q4: k, n and rows_max must be positive");
    if (k % 32 != 0) return fail(ctx, HB_UNSUPPORTED, "gemm_q4: k must be a multiple of 32 (a Q4_0 block)");
    if (out > HB_OUT_SWIGLU) return fail(ctx, HB_INVALID, "gemm_q4: unknown output mode");
    if (out == HB_OUT_SWIGLU && n % 2 != 0) return fail(ctx, HB_INVALID, "gemm_q4: the SwiGLU form needs an even n ([gate | up])");
    const uint32_t bn = tile_n ? tile_n : 256;
    q4g_fn fn = bn == 256 ? q4g_pick_out<256>(out) : bn == 128 ? q4g_pick_out<128>(out) : nullptr;
    if (!fn) return fail(ctx, HB_UNSUPPORTED, "gemm_q4: tile_n must be 128 or 256");
    const size_t stage_bytes = A_BYTES + (size_t)bn * BK * 2;
    const size_t budget = std::min<size_t>(ctx->smem_optin, 227 * 1024) - 2048;
    const uint32_t stages = (uint32_t)std::min<size_t>(budget / stage_bytes, MAX_STAGES);
    if (stages < 2) return fail(ctx, HB_UNSUPPORTED, "gemm_q4: the pipeline does not fit in shared memory");
    auto kq = std::make_unique<GemmQ4>();
    kq->k = k;
    kq->n = n;
    kq->out = out;
    kq->rows_max = rows_max;
    kq->bn = bn;
    kq->stages = stages;
    kq->m_first = m_first ? 1u : 0u;
    kq->fn = fn;
    kq->smem = stages * stage_bytes + 1024;
    kq->kind = 1;
    kq->nargs = 4;
    char nm[160];
    // the reference's name for this emitter is gemm_mma_q4_{k}x{n}...: the tile and the stage count are ours
    snprintf(nm, sizeof nm, "gemm_q4_%ux%u_%s%s_t128x%u_s%u", k, n, out_tag(out), m_first ? "_mf" : "", bn, stages);
    kq->name = nm;
    if (hb_kernel* have = find(ctx, kq->name)) {
        auto* g = static_cast<GemmQ4*>(have);
        g->rows_max = std::max(g->rows_max, rows_max);
        *res = have;
        return HB_OK;
    }
    cudaError_t e = cudaFuncSetAttribute(reinterpret_cast<const void*>(fn), cudaFuncAttributeMaxDynamicSharedMemorySize, (int)ctx->smem_optin - 1024);
    if (e != cudaSuccess) return cuda_fail(ctx, e, "cudaFuncSetAttribute(max dynamic shared memory)");
    *res = intern(ctx, std::move(kq));
    return HB_OK;
}

}  // namespace hb

extern "C" int hb_gemm_q4_get(hb_ctx* ctx, uint32_t k, uint32_t n, uint32_t out, uint32_t tile_n, uint32_t m_first, uint32_t rows_max, hb_kernel** res) {
    if (!ctx || !res) return hb::fail(ctx, HB_INVALID, "hb_gemm_q4_get: bad argument");
    try {
        hb::bind(ctx);
        return hb::make_gemm_q4(ctx, k, n, out, tile_n, m_first, rows_max, res);
    } catch (const std::exception& e) {
        return hb::fail(ctx, HB_BACKEND, e.what());
    }
}
