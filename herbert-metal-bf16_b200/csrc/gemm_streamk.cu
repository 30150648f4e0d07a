// Prefill GEMM, stream-K form (hb_gemm_desc.stream_k = 1): same product, tiles, pipeline and epilogue as
// gemm_dense.cu, another division of the work.
//
// The tile-per-CTA form leaves SMs idle whenever the tile count is not a multiple of the SM count (256 tiles
// on 148 SMs is 1.73 waves: 14 % of the machine idle; a 64-row prefill bucket has 24 tiles). Here the
// whole waves of tiles are dealt tile-per-CTA as before (the CTAs of a wave share W and X tiles through L2);
// the tiles of the last, partial wave are cut into (tile, k-block) units, numbered tile-major and divided evenly
// among the CTAs, so every CTA streams the same number of k-blocks. A CTA's contiguous range of units is cut
// into pieces at tile boundaries; it runs its work in this order:
//   1. the piece at the END of its range when that tile continues in the next CTA (or the whole range when it
//      lies inside one tile): the f32 accumulator is written to this CTA's slot of a scratch buffer and a
//      flag is released - early, before anything else;
//   2. its tiles of the whole waves, then the whole tiles inside its range: as the tile-per-CTA kernel;
//   3. the piece at the START of its range that completes a tile begun by lower-numbered CTAs: computed last;
//      the epilogue waits (bounded) for those CTAs' flags, adds their partial tiles in CTA order and applies
//      the output mode.
// A CTA therefore only ever waits for lower-numbered CTAs, which published their partials as their first act:
// no cycle, whatever the order blocks are scheduled in. The sum of a split tile is (own k-range) + partials in a
// fixed order: deterministic, but a different association than the unsplit kernel's (within the contract).
// The scratch buffer and flags belong to the context (19.4 MB for 148 SMs and 128x256 tiles). A flag is set once
// per launch by the warp that publishes a partial and read by exactly one warp (the same-numbered warp of the tile's
// owner), which puts it back to 0: every launch finds the flags clear, nothing on the host counts launches, and a
// recorded launch can be replayed. (After a wait that ran out the host clears them: see check_status.)
#include <algorithm>
#include <mutex>
#include <cstring>

#include "gemm_common.cuh"

namespace hb {

struct StreamKParams {
    GemmParams g;
    float* scratch;    // [gridDim.x][4 quarters][BN/32 chunks][8][32 lanes] float4: partial tiles
    uint32_t* flags;   // [gridDim.x][4]: one per epilogue warp (lane quarter)
    uint32_t epoch;
    uint32_t total_units;  // num_tiles * k_blocks
};

enum : uint32_t { PIECE_FULL = 0, PIECE_PARTIAL = 1, PIECE_OWNED = 2 };

struct Piece {
    uint32_t tile, kb0, kb1, mode, first_contrib;
};

__device__ __forceinline__ uint32_t sk_bound(uint32_t j, uint32_t total, uint32_t grid) { return (uint32_t)(((uint64_t)j * total) / grid); }

// The number of pieces of CTA `cta`, and piece `idx` of them in processing order. Whole waves of tiles are dealt
// tile-per-CTA (tile = cta + wave * grid: the CTAs of a wave share W and X tiles through L2, as in the plain
// kernel); only the tiles of the last, partial wave are cut into (tile, k-block) units and divided evenly.
__device__ __forceinline__ uint32_t sk_pieces(const StreamKParams& p, uint32_t cta, uint32_t grid, uint32_t idx, Piece* out) {
    const uint32_t KB = p.g.k_blocks;
    const uint32_t waves = p.g.num_tiles / grid;       // whole waves
    const uint32_t dp_tiles = waves * grid;             // tiles dealt tile-per-CTA
    const uint32_t units = (p.g.num_tiles - dp_tiles) * KB;  // units of the partial wave
    const uint32_t s = sk_bound(cta, units, grid), e = sk_bound(cta + 1, units, grid);
    const bool any = e > s;
    const uint32_t tb = e / KB;  // the tile (of the partial wave) the range ends in
    const bool has_tail = any && e % KB != 0;
    const uint32_t tail_begin = max(s, tb * KB);
    const uint32_t ta = s / KB;
    const bool has_head = any && (s % KB != 0) && ((ta + 1) * KB <= e);
    const uint32_t first_full = (s + KB - 1) / KB, end_full = e / KB;
    const uint32_t n_full = any && end_full > first_full ? end_full - first_full : 0;
    const uint32_t n = (has_tail ? 1u : 0u) + waves + n_full + (has_head ? 1u : 0u);
    if (out == nullptr || idx >= n) return n;
    uint32_t i = idx;
    out->first_contrib = 0;
    if (has_tail) {  // first: the partial this CTA owes to a higher-numbered one
        if (i == 0) {
            out->tile = dp_tiles + tb;
            out->kb0 = tail_begin - tb * KB;
            out->kb1 = e - tb * KB;
            out->mode = PIECE_PARTIAL;
            return n;
        }
        --i;
    }
    if (i < waves) {
        out->tile = cta + i * grid;
        out->kb0 = 0;
        out->kb1 = KB;
        out->mode = PIECE_FULL;
        return n;
    }
    i -= waves;
    if (i < n_full) {
        out->tile = dp_tiles + first_full + i;
        out->kb0 = 0;
        out->kb1 = KB;
        out->mode = PIECE_FULL;
        return n;
    }
    out->tile = dp_tiles + ta;  // last: the piece that completes a tile begun by lower-numbered CTAs
    out->kb0 = s - ta * KB;
    out->kb1 = KB;
    out->mode = PIECE_OWNED;
    uint32_t j = (uint32_t)(((uint64_t)ta * KB * grid) / units);
    while (j > 0 && sk_bound(j, units, grid) > ta * KB) --j;
    while (sk_bound(j + 1, units, grid) <= ta * KB) ++j;
    out->first_contrib = j;
    return n;
}

template <int BN, int OUT>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_tn_streamk_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_w, const StreamKParams sp) {
    constexpr int B_BYTES = BN * BK * 2;
    constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    constexpr int HALF = BN / 2;
    constexpr uint32_t TMEM_COLS = 2 * BN;
    constexpr uint32_t IDESC = umma_idesc_bf16(BM, BN);
    const GemmParams& p = sp.g;

    extern __shared__ uint8_t smem_raw[];
    __shared__ GemmBarriers bars;
    __shared__ __align__(8) uint64_t fix_bar[4];  // one per epilogue warp: arrival of a partial-tile quarter
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t S = p.stages;
    const uint32_t cta = blockIdx.x, grid = gridDim.x;

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < S; ++s) {
            mbar_init(smem_u32(&bars.full[s]), 1);
            mbar_init(smem_u32(&bars.empty[s]), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(smem_u32(&bars.tmem_full[a]), 1);
            mbar_init(smem_u32(&bars.tmem_empty[a]), 4);
        }
        for (int a = 0; a < 4; ++a) mbar_init(smem_u32(&fix_bar[a]), 1);
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
    // Overlapped launch: barriers and tensor memory were set up under the tail of the kernel before this one. The
    // producer requests the W boxes of its first fills (weights are nobody's output) and then waits for that kernel;
    // the epilogue warps wait before they touch Y or the partial-tile scratch and flags, which all stream-K kernels of
    // the context share. A plain launch passes straight through the waits.
    const uint32_t tmem_base = bars.tmem_base;
    const uint32_t n_pieces = sk_pieces(sp, cta, grid, 0, nullptr);
    const uint32_t sk_units = (p.num_tiles - (p.num_tiles / grid) * grid) * p.k_blocks;  // units of the partial wave

    auto tile_mn = [&](uint32_t tile, uint32_t& tm, uint32_t& tn) {
        tm = p.m_first ? tile % p.tiles_m : tile / p.tiles_n;
        tn = p.m_first ? tile / p.tiles_m : tile % p.tiles_n;
    };

    if (warp == 0) {
        if (lane == 0) {
            tma_prefetch_desc(&tm_x);
            tma_prefetch_desc(&tm_w);
            bool ok = true;
            for (int pass = 0; pass < 2 && ok; ++pass) {  // pass 0: the W boxes of the first S fills; pass 1: everything else
                uint32_t s = 0, ph = 0, fill = 0;
                for (uint32_t i = 0; ok && i < n_pieces; ++i) {
                    Piece pc;
                    sk_pieces(sp, cta, grid, i, &pc);
                    uint32_t tm, tn;
                    tile_mn(pc.tile, tm, tn);
                    const int row_x = (int)(tm * BM);
                    int row_w0, row_w1;
                    if constexpr (OUT == HB_OUT_SWIGLU) {
                        row_w0 = (int)(tn * HALF);
                        row_w1 = (int)(p.n_out + tn * HALF);
                    } else {
                        row_w0 = (int)(tn * BN);
                        row_w1 = row_w0 + HALF;
                    }
                    for (uint32_t kb = pc.kb0; kb < pc.kb1; ++kb, ++fill) {
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
            griddep_launch_dependents();  // every load of this CTA is requested
        }
    } else if (warp == 1) {
        if (lane == 0) {
            uint32_t s = 0, ph = 0;
            bool ok = true;
            for (uint32_t i = 0; ok && i < n_pieces; ++i) {
                Piece pc;
                sk_pieces(sp, cta, grid, i, &pc);
                const uint32_t acc = i & 1u, acc_ph = (i >> 1) & 1u;
                if (!mbar_wait(smem_u32(&bars.tmem_empty[acc]), acc_ph ^ 1u)) {
                    report(p.status, ST_WAIT_TIMEOUT, WHERE_TMEM_EMPTY, acc);
                    break;
                }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * BN;
                for (uint32_t kb = pc.kb0; kb < pc.kb1; ++kb) {
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
                        umma_bf16(d_tmem, a_desc + 2 * k4, b_desc + 2 * k4, IDESC, (kb != pc.kb0 || k4 != 0) ? 1u : 0u);
                    umma_commit(smem_u32(&bars.empty[s]));
                    if (++s == S) { s = 0; ph ^= 1u; }
                }
                if (ok) umma_commit(smem_u32(&bars.tmem_full[acc]));
            }
        }
    } else {
        const uint32_t q = (uint32_t)warp & 3u;
        griddep_wait();  // Y, the scratch and the flags may still be in use by the kernel before this one
        for (uint32_t i = 0; i < n_pieces; ++i) {
            Piece pc;
            sk_pieces(sp, cta, grid, i, &pc);
            uint32_t tm, tn;
            tile_mn(pc.tile, tm, tn);
            const uint32_t acc = i & 1u, acc_ph = (i >> 1) & 1u;
            bool got = mbar_wait(smem_u32(&bars.tmem_full[acc]), acc_ph);
            if (pc.mode == PIECE_OWNED && got) {
                // the partial tiles of the lower CTAs that began this tile: published as their first act
                if (lane == 0) {
                    const long long t0 = clock64();
                    for (uint32_t j = pc.first_contrib; j < cta && got; ++j) {
                        if (sk_bound(j + 1, sk_units, grid) == sk_bound(j, sk_units, grid)) continue;  // a CTA without units
                        uint32_t v;
                        do {
                            asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(sp.flags + j * 4 + q) : "memory");
                            if (v != sp.epoch && clock64() - t0 > HB_WAIT_LIMIT_CYCLES) got = false;
                        } while (v != sp.epoch && got);
                        // this warp is the flag's only reader: taken, it goes back to 0 for the next launch
                        if (got) asm volatile("st.relaxed.gpu.global.u32 [%0], %1;" ::"l"(sp.flags + j * 4 + q), "r"(0u) : "memory");
                    }
                    asm volatile("fence.proxy.async;" ::: "memory");  // the bulk copies below read what those CTAs wrote
                }
                __syncwarp();
            }
            if (!__all_sync(0xffffffffu, got)) {
                if (lane == 0) report(p.status, ST_WAIT_TIMEOUT, WHERE_TMEM_FULL, 10 + pc.mode);
                break;
            }
            tc_fence_after();
            const uint32_t trow = q * 32 + lane;  // row inside the tile
            const uint32_t row = tm * BM + trow;
            const uint32_t t_addr = tmem_base + ((q * 32u) << 16) + acc * BN;
            // Partial tiles in scratch: [cta][lane quarter q][32-column chunk c][k: 0..7][lane] float4 - the four values
            // (columns 32c + 4k ..) of the 32 rows of a quarter lie together, so a warp's stores and loads are 512-byte
            // runs, and a quarter (32 rows x BN f32) is one contiguous block a bulk copy can fetch.
            constexpr uint32_t QFLOATS = 32u * BN;  // floats of a quarter
            if (pc.mode == PIECE_PARTIAL) {
                float4* dst = reinterpret_cast<float4*>(sp.scratch + ((size_t)cta * 4 + q) * QFLOATS);
#pragma unroll 1
                for (int c = 0; c < BN / 32; ++c) {
                    uint32_t v[32];
                    tmem_ld_32x32(t_addr + c * 32, v);
                    tmem_ld_wait();
#pragma unroll
                    for (int k = 0; k < 8; ++k)
                        dst[(c * 8 + k) * 32 + lane] = make_float4(__uint_as_float(v[4 * k]), __uint_as_float(v[4 * k + 1]), __uint_as_float(v[4 * k + 2]),
                                                                  __uint_as_float(v[4 * k + 3]));
                }
                // a flag per (CTA, lane quarter): the warp that completes this quarter of the tile reads only what the
                // same-numbered warp wrote, so no barrier across the epilogue warps is needed
                __threadfence();
                __syncwarp();
                if (lane == 0) asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(sp.flags + cta * 4 + q), "r"(sp.epoch) : "memory");
            } else if (pc.mode == PIECE_FULL) {
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
            } else {
                // The owned piece is this CTA's last: every MMA has read its stage and no load is in flight, so the
                // stage memory is free. Each epilogue warp bulk-copies its quarter of a contributor's partial tile
                // there, adds it to the accumulator in tensor memory, and with the last contributor applies the
                // output mode instead of writing back.
                const uint32_t buf = smem_base + q * (QFLOATS * 4u);
                const uint32_t fbar = smem_u32(&fix_bar[q]);
                const float4* land = reinterpret_cast<const float4*>(smem_raw + (buf - smem_u32(smem_raw)));
                uint32_t last = pc.first_contrib;
                for (uint32_t j = pc.first_contrib; j < cta; ++j)
                    if (sk_bound(j + 1, sk_units, grid) != sk_bound(j, sk_units, grid)) last = j;
                uint32_t fph = 0;
                bool fine = true;
                auto add_chunk = [&](uint32_t (&v)[32], int c) {
#pragma unroll
                    for (int k = 0; k < 8; ++k) {
                        const float4 f = land[(c * 8 + k) * 32 + lane];
                        v[4 * k] = __float_as_uint(__fadd_rn(__uint_as_float(v[4 * k]), f.x));
                        v[4 * k + 1] = __float_as_uint(__fadd_rn(__uint_as_float(v[4 * k + 1]), f.y));
                        v[4 * k + 2] = __float_as_uint(__fadd_rn(__uint_as_float(v[4 * k + 2]), f.z));
                        v[4 * k + 3] = __float_as_uint(__fadd_rn(__uint_as_float(v[4 * k + 3]), f.w));
                    }
                };
                for (uint32_t j = pc.first_contrib; j <= last && fine; ++j) {
                    if (sk_bound(j + 1, sk_units, grid) == sk_bound(j, sk_units, grid)) continue;  // a CTA without units
                    if (lane == 0) {
                        mbar_arrive_expect_tx(fbar, QFLOATS * 4u);
                        bulk_load(buf, sp.scratch + ((size_t)j * 4 + q) * QFLOATS, QFLOATS * 4u, fbar);
                    }
                    fine = __all_sync(0xffffffffu, mbar_wait(fbar, fph));
                    fph ^= 1u;
                    if (!fine) break;
                    if (j != last) {
#pragma unroll 1
                        for (int c = 0; c < BN / 32; ++c) {
                            uint32_t v[32];
                            tmem_ld_32x32(t_addr + c * 32, v);
                            tmem_ld_wait();
                            add_chunk(v, c);
                            tmem_st_32x32(t_addr + c * 32, v);
                        }
                        tmem_st_wait();
                    } else if constexpr (OUT == HB_OUT_SWIGLU) {
#pragma unroll 1
                        for (int c = 0; c < HALF / 32; ++c) {
                            uint32_t g[32], u[32];
                            tmem_ld_32x32(t_addr + c * 32, g);
                            tmem_ld_32x32(t_addr + HALF + c * 32, u);
                            tmem_ld_wait();
                            add_chunk(g, c);
                            add_chunk(u, HALF / 32 + c);
                            store_chunk<OUT>(p, row, tn * HALF + c * 32, g, u);
                        }
                    } else {
#pragma unroll 1
                        for (int c = 0; c < BN / 32; ++c) {
                            uint32_t v[32];
                            tmem_ld_32x32(t_addr + c * 32, v);
                            tmem_ld_wait();
                            add_chunk(v, c);
                            store_chunk<OUT>(p, row, tn * BN + c * 32, v, v);
                        }
                    }
                    __syncwarp();  // the landing buffer is read out before the next copy overwrites it
                }
                if (!fine) {
                    if (lane == 0) report(p.status, ST_WAIT_TIMEOUT, WHERE_TMEM_FULL, 20);
                    break;
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

typedef void (*sk_fn)(const CUtensorMap, const CUtensorMap, const StreamKParams);

template <int BN>
sk_fn sk_pick_out(uint32_t out) {
    switch (out) {
        case HB_OUT_BF16: return gemm_bf16_tn_streamk_kernel<BN, HB_OUT_BF16>;
        case HB_OUT_F32: return gemm_bf16_tn_streamk_kernel<BN, HB_OUT_F32>;
        case HB_OUT_RESIDUAL: return gemm_bf16_tn_streamk_kernel<BN, HB_OUT_RESIDUAL>;
        case HB_OUT_SWIGLU: return gemm_bf16_tn_streamk_kernel<BN, HB_OUT_SWIGLU>;
    }
    return nullptr;
}

struct StreamKGemm : hb_kernel {
    hb_gemm_desc d{};
    sk_fn fn = nullptr;
    uint32_t bn = 0, stages = 0;
    size_t smem = 0;
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
        StreamKParams sp{};
        GemmParams& p = sp.g;
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
        const uint64_t units = (uint64_t)p.num_tiles * p.k_blocks;
        if (units > 0xffffffffull) return fail(ctx, HB_UNSUPPORTED, name + ": too many (tile, k-block) units");
        sp.total_units = (uint32_t)units;
        sp.scratch = ctx->sk_scratch;
        sp.flags = ctx->sk_flags;
        sp.epoch = 1;
        const uint32_t grid = (uint32_t)std::min<uint64_t>(units, (uint64_t)ctx->sm_count);  // a whole wave or more: every SM
        HB_CUDA(ctx, launch_kernel(ctx, true, fn, dim3(grid), dim3(GEMM_THREADS), smem, tm_x, tm_w, sp));
        ctx->launches++;
        return HB_OK;
    }
};

}  // namespace

int make_gemm_streamk(hb_ctx* ctx, const hb_gemm_desc* d, hb_kernel** out) {
    *out = nullptr;
    const uint32_t bn = d->tile_n ? d->tile_n : 256;
    sk_fn fn = nullptr;
    switch (bn) {
        case 64: fn = sk_pick_out<64>(d->out); break;
        case 128: fn = sk_pick_out<128>(d->out); break;
        case 256: fn = sk_pick_out<256>(d->out); break;
        default: return fail(ctx, HB_UNSUPPORTED, "gemm: tile_n must be 64, 128 or 256");
    }
    const size_t stage_bytes = A_BYTES + (size_t)bn * BK * 2;
    const size_t budget = std::min<size_t>(ctx->smem_optin, 227 * 1024) - 2048;
    const uint32_t max_stages = (uint32_t)std::min<size_t>(budget / stage_bytes, MAX_STAGES);
    const uint32_t stages = d->stages ? d->stages : max_stages;
    if (stages < 2 || stages > max_stages) return fail(ctx, HB_UNSUPPORTED, "gemm: stage count does not fit");
    // the epilogue of an owned piece lands a contributor's whole f32 partial tile (BM x bn) in the pipeline's shared memory
    if ((size_t)stages * stage_bytes < (size_t)BM * bn * sizeof(float))
        return fail(ctx, HB_UNSUPPORTED, "gemm: the stream-K form needs a pipeline at least as large as one f32 partial tile (" + std::to_string(BM) + " x " +
                                             std::to_string(bn) + "): more stages or a narrower tile");
    auto k = std::make_unique<StreamKGemm>();
    k->d = *d;
    k->d.tile_n = bn;
    k->fn = fn;
    k->bn = bn;
    k->stages = stages;
    k->smem = stages * stage_bytes + 1024;
    k->kind = 1;
    k->nargs = 3;
    char nm[160];
    snprintf(nm, sizeof nm, "gemm_sk_%ux%u_%s%s_t128x%u_s%u", d->k, d->n, out_tag(d->out), d->m_first ? "_mf" : "", bn, stages);
    k->name = nm;
    if (hb_kernel* have = find(ctx, k->name)) {
        auto* g = static_cast<StreamKGemm*>(have);
        g->d.rows_max = std::max(g->d.rows_max, d->rows_max);
        *out = have;
        return HB_OK;
    }
    if (!ctx->sk_scratch) {
        // one slot per SM, sized for the widest tile; flags start at 0 and every launch leaves them at 0
        void* s = nullptr;
        void* f = nullptr;
        int r = hb_alloc(ctx, (size_t)ctx->sm_count * BM * 256 * sizeof(float), &s);
        if (r != HB_OK) return r;
        if ((r = hb_alloc(ctx, (size_t)ctx->sm_count * 4 * sizeof(uint32_t), &f)) != HB_OK) return r;
        zero_on_failure(ctx, f, (size_t)ctx->sm_count * 4 * sizeof(uint32_t));  // flags of partial tiles: their reader clears them
        ctx->sk_scratch = static_cast<float*>(s);
        ctx->sk_flags = static_cast<uint32_t*>(f);
    }
    cudaError_t e = cudaFuncSetAttribute(reinterpret_cast<const void*>(fn), cudaFuncAttributeMaxDynamicSharedMemorySize, (int)ctx->smem_optin - 1024);
    if (e != cudaSuccess) return cuda_fail(ctx, e, "cudaFuncSetAttribute(max dynamic shared memory)");
    *out = intern(ctx, std::move(k));
    return HB_OK;
}

}  // namespace hb

// ------------------------------------------------------------------ the entry point that allocates nothing
//
// hb_gemm_static_scratch runs the stream-K GEMM (128x64 tiles) with its partial-tile scratch in the two arrays
// below instead of memory obtained from the allocator. Every GPU that loads this library holds them (5.0 MiB)
// until the process exits.

namespace hb {
constexpr uint32_t STATIC_SLOTS = HB_STATIC_SCRATCH_SLOTS;  // CTAs the static scratch can serve
constexpr uint32_t STATIC_BN = 64;
}  // namespace hb

static __device__ __align__(256) float g_static_partials[hb::STATIC_SLOTS * hb::BM * hb::STATIC_BN];
static __device__ __align__(256) uint32_t g_static_flags[hb::STATIC_SLOTS * 4];

namespace {
static_assert((size_t)2 * (hb::A_BYTES + (size_t)hb::STATIC_BN * hb::BK * 2) >= (size_t)hb::BM * hb::STATIC_BN * sizeof(float),
              "the static form's pipeline holds one f32 partial tile at any stage count");
constexpr int MAX_DEVICES = 64;
// Per device: the device addresses of the arrays (their names are host-side stand-ins, not addresses a kernel
// could use) and the epoch that tells this device's launches apart.
float* s_partials[MAX_DEVICES];
uint32_t* s_flags[MAX_DEVICES];
uint32_t s_epoch[MAX_DEVICES];
bool s_ready[MAX_DEVICES];
// Host threads with contexts of their own may call the entry point at the same time: the set-up and the drawing of an
// epoch are serialised here. (The array itself stays shared: kernels that overlap on the GPU race, as the header says.)
std::mutex s_lock;
}  // namespace

extern "C" int hb_gemm_static_scratch(hb_ctx* ctx, uint32_t k, uint32_t n, uint32_t out, uint32_t m, hb_range w, hb_range x, hb_range y) {
    using namespace hb;
    if (!ctx) return HB_INVALID;
    bind(ctx);
    if (k == 0 || n == 0 || m == 0) return fail(ctx, HB_INVALID, "hb_gemm_static_scratch: k, n and m must be positive");
    if (k % 8 != 0) return fail(ctx, HB_UNSUPPORTED, "hb_gemm_static_scratch: k must be a multiple of 8");
    if (out > HB_OUT_SWIGLU || (out == HB_OUT_SWIGLU && n % 2 != 0)) return fail(ctx, HB_INVALID, "hb_gemm_static_scratch: bad output mode");
    if (m > HB_STATIC_SCRATCH_MAX_ROWS || k > HB_STATIC_SCRATCH_MAX_K || n > HB_STATIC_SCRATCH_MAX_N)
        return fail(ctx, HB_UNSUPPORTED, "hb_gemm_static_scratch: at most 2048 rows, k <= 65536 and n <= 262144 (larger products need hb_gemm_get, which allocates)");
    if (ctx->device < 0 || ctx->device >= MAX_DEVICES) return fail(ctx, HB_UNSUPPORTED, "hb_gemm_static_scratch: device index out of range");
    const uint32_t n_out = out == HB_OUT_SWIGLU ? n / 2 : n;
    if (!range_ok(w, (size_t)n * k * 2) || !range_ok(x, (size_t)m * k * 2) || !range_ok(y, (size_t)m * n_out * (out == HB_OUT_F32 ? 4 : 2)))
        return fail(ctx, HB_INVALID, "hb_gemm_static_scratch: a range is too small");
    sk_fn fn = sk_pick_out<STATIC_BN>(out);
    const int dev = ctx->device;
    HB_CUDA(ctx, cudaSetDevice(dev));
    std::lock_guard<std::mutex> guard(s_lock);
    if (!s_ready[dev]) {
        // Set-up, once per device, with that device current: ask the runtime where the arrays live on it.
        float* pp = nullptr;
        uint32_t* fp = nullptr;
        HB_CUDA(ctx, cudaGetSymbolAddress(reinterpret_cast<void**>(&pp), g_static_partials));
        HB_CUDA(ctx, cudaGetSymbolAddress(reinterpret_cast<void**>(&fp), g_static_flags));
        for (uint32_t o = HB_OUT_BF16; o <= HB_OUT_SWIGLU; ++o)
            HB_CUDA(ctx, cudaFuncSetAttribute(reinterpret_cast<const void*>(sk_pick_out<STATIC_BN>(o)), cudaFuncAttributeMaxDynamicSharedMemorySize,
                                              (int)ctx->smem_optin - 1024));
        // The flags keep whatever the last call left; launches are told apart by the epoch, and the arrays start
        // zeroed when the module loads, so epochs begin at 1 and nothing needs clearing. That also covers a launch
        // whose bounded wait ran out: the context's own stream-K flags are cleared when the failure is reported, these
        // are not, and need not be, because no later launch uses that launch's epoch again.
        s_partials[dev] = pp;
        s_flags[dev] = fp;
        s_epoch[dev] = 0;
        s_ready[dev] = true;
    }
    CUtensorMap tm_x, tm_w;
    int r = make_tmap_bf16(ctx, &tm_w, w.ptr, n, k, STATIC_BN / 2);
    if (r != HB_OK) return r;
    if ((r = make_tmap_bf16(ctx, &tm_x, x.ptr, m, k, BM)) != HB_OK) return r;
    const size_t stage_bytes = A_BYTES + (size_t)STATIC_BN * BK * 2;
    const size_t budget = std::min<size_t>(ctx->smem_optin, 227 * 1024) - 2048;
    const uint32_t stages = (uint32_t)std::min<size_t>(budget / stage_bytes, MAX_STAGES);
    StreamKParams sp{};
    GemmParams& p = sp.g;
    p.y = y.ptr;
    p.m = m;
    p.n_w = n;
    p.n_out = n_out;
    p.k_blocks = (k + BK - 1) / BK;
    p.tiles_m = (m + BM - 1) / BM;
    const uint32_t cols_per_tile = out == HB_OUT_SWIGLU ? STATIC_BN / 2 : STATIC_BN;
    p.tiles_n = (n_out + cols_per_tile - 1) / cols_per_tile;
    p.num_tiles = p.tiles_m * p.tiles_n;
    p.stages = stages;
    p.m_first = 1;
    const uint32_t elem = out == HB_OUT_F32 ? 4 : 2;
    p.vec_ok = ((reinterpret_cast<uintptr_t>(y.ptr) & 15u) == 0 && ((size_t)n_out * elem) % 16 == 0) ? 1u : 0u;
    p.status = ctx->status_dev;
    const uint64_t units = (uint64_t)p.num_tiles * p.k_blocks;
    if (units > 0xffffffffull) return fail(ctx, HB_UNSUPPORTED, "hb_gemm_static_scratch: too many (tile, k-block) units");
    sp.total_units = (uint32_t)units;
    sp.scratch = s_partials[dev];
    sp.flags = s_flags[dev];
    if (++s_epoch[dev] == 0) s_epoch[dev] = 1;  // after 2^32 calls: 0 is what a never-written flag holds
    sp.epoch = s_epoch[dev];
    const uint32_t grid = (uint32_t)std::min<uint64_t>(units, std::min<uint64_t>((uint64_t)ctx->sm_count, STATIC_SLOTS));
    fn<<<grid, GEMM_THREADS, stages * stage_bytes + 1024, ctx->stream>>>(tm_x, tm_w, sp);
    HB_CUDA(ctx, cudaGetLastError());
    ctx->launches++;
    return HB_OK;
}
