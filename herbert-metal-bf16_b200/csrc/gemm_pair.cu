// Prefill GEMM, CTA-pair form (hb_gemm_desc.cta_pair = 1): a cluster of two CTAs computes one 256 x 256 tile
// with tcgen05.mma.cta_group::2.
//
// Why: with one CTA per 128 x 256 tile a pipeline stage is 48 KB (128 rows of X + 256 rows of W) and only four
// fit in shared memory; the measured time still falls 6-10 % from three to four stages, i.e. the kernel is
// short of bytes in flight. In a pair each CTA stages 128 rows of X (its half of the tile's rows) and 128 rows
// of W (its half of the tile's columns): 32 KB per stage, seven stages, and every W row is read from shared
// memory by one CTA only. The MMA is issued by the leader CTA (cluster rank 0) and reads both CTAs' shared
// memory; each CTA's tensor memory receives its own 128 rows of the 256 x 256 accumulator and its own four
// epilogue warps write them out.
//
// No TMA multicast anywhere: each CTA loads its own halves with an ordinary tiled load whose completion is
// counted on the LEADER's stage barrier (cp.async.bulk.tensor with .cta_group::2 may signal the peer's
// mbarrier). The leader's tcgen05.commit arrives on both CTAs' barriers (commit with .multicast::cluster).
// SwiGLU: CTA 0 stages the gate rows, CTA 1 the matching up rows, so accumulator columns [0,128) are gate and
// [128,256) up, as in the single-CTA kernel.
// Every wait is bounded; both CTAs always reach the closing cluster barrier and free their tensor memory.
#include <algorithm>
#include <cstring>

#include "gemm_common.cuh"

namespace hb {

constexpr int PAIR_BN = 256;
constexpr int PAIR_B_BYTES = 128 * BK * 2;            // this CTA's half of the W tile
constexpr int PAIR_STAGE_BYTES = A_BYTES + PAIR_B_BYTES;  // 32 KiB

__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Arrival on a barrier that may live in the peer CTA (a shared::cluster address).
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// Tiled load into this CTA's shared memory, bytes counted on a barrier of either CTA of the pair. Not a multicast.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* d, uint32_t bar_cluster_addr, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"((uint64_t)d), "r"(bar_cluster_addr), "r"(x), "r"(y)
        : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t dst_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// One arrival on the barrier at this offset in BOTH CTAs once the MMAs issued so far are done.
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
    const uint16_t mask = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar), "h"(mask) : "memory");
}

template <int OUT, int BN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_tn_pair_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_w, const GemmParams p) {
    // BN: the tile's columns, 256 or 192 (a narrower tile where 256 columns leave the last wave of pairs nearly empty:
    // 2048 x 5120 is 160 tiles of 256 x 256 for 74 pairs, 2.2 waves run as 3, and 216 tiles of 256 x 192, 2.9 waves
    // of three quarters the length). A stage keeps its 32 KB slots; the W box is BN / 2 rows.
    static_assert(BN == 256 || BN == 192, "tile columns");
    constexpr uint32_t TMEM_COLS = 512;  // two accumulators of BN columns (this CTA's 128 rows of each), a power of two
    constexpr uint32_t IDESC = umma_idesc_bf16(256, BN);
    constexpr int HALF = BN / 2;
    constexpr uint32_t STAGE_TX = 2u * (A_BYTES + HALF * BK * 2);  // both CTAs' bytes of one stage

    extern __shared__ uint8_t smem_raw[];
    __shared__ GemmBarriers bars;
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t S = p.stages;
    const uint32_t rank = cluster_rank();
    const uint32_t pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;
    // y_signal: the kernel that sums the partials is next on the stream and may start now (it shares the SMs with
    // this one and waits for the flags sent below, not for this kernel's end)
    if (OUT == HB_OUT_F32 && p.flag_table) griddep_launch_dependents();

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < S; ++s) {
            mbar_init(smem_u32(&bars.full[s]), 1);   // used in the leader: its producer's expect_tx arrival
            mbar_init(smem_u32(&bars.empty[s]), 1);  // the leader's commit, in both CTAs
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(smem_u32(&bars.tmem_full[a]), 1);   // the leader's commit, in both CTAs
            mbar_init(smem_u32(&bars.tmem_empty[a]), 8);  // used in the leader: four epilogue warps of each CTA
        }
        fence_mbar_init();
        fence_proxy_async();
    }
    if (warp == 1) {
        tmem_alloc_pair(smem_u32(&bars.tmem_base), TMEM_COLS);
        tmem_relinquish_pair();
    }
    tc_fence_before();
    cluster_sync_all();  // both CTAs' barriers exist before anything signals them
    tc_fence_after();
    const uint32_t tmem_base = bars.tmem_base;
    // tiles: 256 rows x (256 columns, or 128 SwiGLU outputs)
    const uint32_t tiles_m = (p.m + 255u) / 256u;
    const uint32_t tiles_n = p.tiles_n;
    const uint32_t num_tiles = tiles_m * tiles_n;
    const uint32_t nsplit = p.split_k > 1 ? p.split_k : 1u;  // K slices per tile (hb_gemm_desc.split_k)
    const uint32_t num_items = num_tiles * nsplit;           // slice-major: the items that run together share a K slice

    if (warp == 0) {
        // ---------------------------------------------------------- producer (one per CTA)
        // Overlapped launch (hb_set_launch_overlap): this kernel may have started while the kernel before it on the
        // stream still runs. W is not that kernel's output, so the W halves of the first stages are requested at once;
        // X may be, so its halves follow griddepcontrol.wait. In a plain launch the wait returns at once.
        if (lane == 0) {
            tma_prefetch_desc(&tm_x);
            tma_prefetch_desc(&tm_w);
            uint32_t s = 0, ph = 0, fill = 0;
            bool ok = true, waited = false;
            for (int pass = 0; pass < 2 && ok; ++pass) {  // pass 0: the W halves of the first S fills; pass 1: everything else
                s = 0; ph = 0; fill = 0;
                for (uint32_t item = pair; ok && item < num_items; item += npairs) {
                    const uint32_t tile = item % num_tiles, slice = item / num_tiles;
                    const uint32_t tm = p.m_first ? tile % tiles_m : tile / tiles_n;
                    const uint32_t tn = p.m_first ? tile / tiles_m : tile % tiles_n;
                    const int row_x = (int)(tm * 256 + rank * 128);
                    int row_w;
                    if constexpr (OUT == HB_OUT_SWIGLU) row_w = (int)(rank * p.n_out + tn * HALF);  // rank 0: gate rows, rank 1: up rows
                    else row_w = (int)(tn * BN + rank * HALF);
                    const uint32_t kb0 = slice * p.k_blocks / nsplit, kb1 = (slice + 1) * p.k_blocks / nsplit;
                    for (uint32_t kb = kb0; kb < kb1; ++kb, ++fill) {
                        const bool early = fill < S;  // the stage is free: nothing to wait for
                        if (pass == 0 && !early) { ok = false; break; }  // (ok is set again below: pass 0 just ends here)
                        if (pass == 1 && !early && !mbar_wait(smem_u32(&bars.empty[s]), ph ^ 1u)) {
                            report(p.status, ST_WAIT_TIMEOUT, WHERE_EMPTY, s);
                            ok = false;
                            break;
                        }
                        const uint32_t full_leader = map_to_cta(smem_u32(&bars.full[s]), 0);
                        const uint32_t a_dst = smem_base + s * PAIR_STAGE_BYTES;
                        const bool do_w = pass == 0 || !early, do_x = pass == 1;
                        if (do_w && rank == 0) mbar_arrive_expect_tx(smem_u32(&bars.full[s]), STAGE_TX);
                        if (do_x) tma_load_2d_pair(a_dst, &tm_x, full_leader, (int)(kb * BK), row_x);
                        if (do_w) tma_load_2d_pair(a_dst + A_BYTES, &tm_w, full_leader, (int)(kb * BK), row_w);
                        if (++s == S) { s = 0; ph ^= 1u; }
                    }
                }
                if (pass == 0) {
                    ok = true;
                    griddep_wait();
                    waited = true;
                }
            }
            (void)waited;
            // every load of this CTA is requested: the kernel behind this one may take the SMs as they fall free
            griddep_launch_dependents();
        }
    } else if (warp == 1) {
        // --------------------------------------------------------- MMA issuer (leader CTA only)
        if (lane == 0 && rank == 0) {
            uint32_t s = 0, ph = 0, it = 0;
            bool ok = true;
            for (uint32_t item = pair; ok && item < num_items; item += npairs, ++it) {
                const uint32_t slice = item / num_tiles;
                const uint32_t kb0 = slice * p.k_blocks / nsplit, kb1 = (slice + 1) * p.k_blocks / nsplit;
                const uint32_t acc = it & 1u, acc_ph = (it >> 1) & 1u;
                if (!mbar_wait(smem_u32(&bars.tmem_empty[acc]), acc_ph ^ 1u)) {
                    report(p.status, ST_WAIT_TIMEOUT, WHERE_TMEM_EMPTY, acc);
                    break;
                }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * BN;
                for (uint32_t kb = kb0; kb < kb1; ++kb) {
                    if (!mbar_wait(smem_u32(&bars.full[s]), ph)) {
                        report(p.status, ST_WAIT_TIMEOUT, WHERE_FULL, s);
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t a_addr = smem_base + s * PAIR_STAGE_BYTES;
                    const uint64_t a_desc = umma_desc_sw128(a_addr);
                    const uint64_t b_desc = umma_desc_sw128(a_addr + A_BYTES);
#pragma unroll
                    for (uint32_t k4 = 0; k4 < BK / 16; ++k4)
                        umma_bf16_pair(d_tmem, a_desc + 2 * k4, b_desc + 2 * k4, IDESC, (kb != kb0 || k4 != 0) ? 1u : 0u);
                    umma_commit_pair(smem_u32(&bars.empty[s]));
                    if (++s == S) { s = 0; ph ^= 1u; }
                }
                if (ok) umma_commit_pair(smem_u32(&bars.tmem_full[acc]));
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue (both CTAs: their own 128 rows)
        const uint32_t q = (uint32_t)warp & 3u;
        uint32_t it = 0;
        griddep_wait();  // Y may be read (residual) or still be in use by the kernel before this one
        for (uint32_t item = pair; item < num_items; item += npairs, ++it) {
            const uint32_t tile = item % num_tiles, slice = item / num_tiles;
            const uint32_t tm = p.m_first ? tile % tiles_m : tile / tiles_n;
            const uint32_t tn = p.m_first ? tile / tiles_m : tile % tiles_n;
            const uint32_t acc = it & 1u, acc_ph = (it >> 1) & 1u;
            const bool got = mbar_wait(smem_u32(&bars.tmem_full[acc]), acc_ph);
            if (!__all_sync(0xffffffffu, got)) {
                if (lane == 0) report(p.status, ST_WAIT_TIMEOUT, WHERE_TMEM_FULL, acc);
                break;
            }
            tc_fence_after();
            const uint32_t row = tm * 256 + rank * 128 + q * 32 + lane;
            const uint32_t t_addr = tmem_base + ((q * 32u) << 16) + acc * BN;
            if (nsplit > 1) {
                // The slices of a tile hand a running f32 sum from one to the next through one block of scratch per
                // quarter of a CTA's half tile: slice 0 stores its accumulator, slice s adds its own to what the slices
                // before it left (waiting, bounded, until they are done: they come earlier in every pair's item order,
                // so they are running or finished), the last slice applies the output mode. The order of the sum is
                // the order of the slices, whoever runs when. 16-byte piece j of 32-column chunk c of the lane's row is
                // slot (c * 8 + j) * 32 + lane of the block: a warp's access is 512 contiguous bytes.
                constexpr uint32_t BLOCK16 = 32 * BN / 4;  // 16-byte slots of a 32 x 256 f32 block
                const uint32_t which = (tile * 2 + rank) * 4 + q;
                uint4* buf = reinterpret_cast<uint4*>(p.partial) + (size_t)which * BLOCK16 + lane;
                uint32_t* flag = p.split_counters + which;  // slices of this quarter done so far
                const bool first = slice == 0, last = slice + 1 == nsplit;
                bool ready = true;
                if (!first) {
                    if (lane == 0) {
                        const long long t0 = clock64();
                        uint32_t v;
                        do {
                            asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
                            if (v != slice && clock64() - t0 > HB_WAIT_LIMIT_CYCLES) ready = false;
                        } while (v != slice && ready);
                    }
                    ready = __shfl_sync(0xffffffffu, ready ? 1 : 0, 0) != 0;
                    if (!ready) {
                        if (lane == 0) report(p.status, ST_WAIT_TIMEOUT, WHERE_TMEM_FULL, 64u + slice);
                        break;
                    }
                }
                // own accumulator chunk c plus the running sum (if any): v[] as f32 bits. A chunk's loads of the running
                // sum take about a microsecond to come back, so AHEAD chunks are in flight at any time (the loops are
                // unrolled: the ring of registers is indexed at compile time).
                constexpr int NCHUNK = BN / 32;
                constexpr int AHEAD = OUT == HB_OUT_SWIGLU ? 3 : 4;
                uint4 ahead[AHEAD][8];
                auto ask = [&](int slot, int c) {
#pragma unroll
                    for (int j = 0; j < 8; ++j) ahead[slot][j] = __ldcg(buf + (c * 8 + j) * 32);
                };
                // the order the chunks are visited in: 0, 1, .. or, for the SwiGLU's last slice, gate and up chunks in turn
                auto nth = [&](int i) { return (last && OUT == HB_OUT_SWIGLU) ? ((i & 1) ? HALF / 32 + (i >> 1) : (i >> 1)) : i; };
                if (!first) {
#pragma unroll
                    for (int i = 0; i < AHEAD; ++i) ask(i, nth(i));
                }
                auto chunk = [&](int i, uint32_t (&v)[32]) {
                    tmem_ld_32x32(t_addr + nth(i) * 32, v);
                    tmem_ld_wait();
                    if (!first) {
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            const uint4 t = ahead[i % AHEAD][j];
                            const uint32_t w4[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
                            for (int e = 0; e < 4; ++e) v[4 * j + e] = __float_as_uint(__fadd_rn(__uint_as_float(w4[e]), __uint_as_float(v[4 * j + e])));
                        }
                        if (i + AHEAD < NCHUNK) ask(i % AHEAD, nth(i + AHEAD));
                    }
                };
                if (!last) {
#pragma unroll
                    for (int c = 0; c < NCHUNK; ++c) {
                        uint32_t v[32];
                        chunk(c, v);
#pragma unroll
                        for (int j = 0; j < 8; ++j) __stcg(buf + (c * 8 + j) * 32, make_uint4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]));
                    }
                } else if constexpr (OUT == HB_OUT_SWIGLU) {
#pragma unroll
                    for (int c = 0; c < HALF / 32; ++c) {
                        uint32_t g[32], u[32];
                        chunk(2 * c, g);
                        chunk(2 * c + 1, u);
                        store_chunk<OUT>(p, row, tn * HALF + c * 32, g, u);
                    }
                } else {
#pragma unroll
                    for (int c = 0; c < NCHUNK; ++c) {
                        uint32_t v[32];
                        chunk(c, v);
                        store_chunk<OUT>(p, row, tn * BN + c * 32, v, v);
                    }
                }
                tc_fence_before();
                if (!last) __threadfence();  // this lane's part of the running sum is out before the flag says so
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive_cluster(map_to_cta(smem_u32(&bars.tmem_empty[acc]), 0));
                    const uint32_t next = last ? 0u : slice + 1u;  // the last slice leaves the flag at zero for the next launch
                    asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(flag), "r"(next) : "memory");
                }
                continue;
            }
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
                    if (OUT == HB_OUT_F32 && p.y_shards)  // row blocks, possibly on other GPUs: whole row segments per store
                        store_chunk_f32_blocks(p, row - lane, tn * BN + c * 32, v, smem_base + S * PAIR_STAGE_BYTES + q * 4096u);
                    else
                        store_chunk<OUT>(p, row, tn * BN + c * 32, v, v);
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&bars.tmem_empty[acc]), 0));
            if (OUT == HB_OUT_F32 && p.flag_table && lane == 0) {
                // This warp's rows of the tile are stored (the __syncwarp above orders the other lanes' stores before
                // this fence). The tile's row group is complete when the eight epilogue warps of the pair have arrived
                // for each of its column tiles; whoever arrives last tells every summing rank, with the step's number.
                // (device scope here; the last arriver's system-scope fence is cumulative over the warps it has
                // synchronised with through the counter)
                __threadfence();
                uint32_t* cnt = p.ctl + TP_CTL_GROUP0 + tm;
                if (atomicAdd(cnt, 1u) == 8u * tiles_n - 1u) {
                    *cnt = 0u;  // for the next launch
                    __threadfence_system();
                    const uint32_t step = *reinterpret_cast<volatile uint32_t*>(p.ctl) + 1u;
                    for (uint32_t d = 0; d < p.world; ++d) {
                        uint32_t* flag = reinterpret_cast<uint32_t*>(p.flag_table[d]) + p.rank * TP_MAX_GROUPS + tm;
                        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(flag), "r"(step) : "memory");
                    }
                }
            }
        }
    }

    tc_fence_before();
    cluster_sync_all();  // nobody signals the peer's barriers or reads its shared memory after this
    tc_fence_after();
    if (warp == 1) tmem_dealloc_pair(tmem_base, TMEM_COLS);
}

// ------------------------------------------------------------------ host side

namespace {

typedef void (*pair_fn)(const CUtensorMap, const CUtensorMap, const GemmParams);

template <int BN>
pair_fn pair_pick_bn(uint32_t out) {
    switch (out) {
        case HB_OUT_BF16: return gemm_bf16_tn_pair_kernel<HB_OUT_BF16, BN>;
        case HB_OUT_F32: return gemm_bf16_tn_pair_kernel<HB_OUT_F32, BN>;
        case HB_OUT_RESIDUAL: return gemm_bf16_tn_pair_kernel<HB_OUT_RESIDUAL, BN>;
        case HB_OUT_SWIGLU: return gemm_bf16_tn_pair_kernel<HB_OUT_SWIGLU, BN>;
    }
    return nullptr;
}
pair_fn pair_pick(uint32_t out, uint32_t bn) { return bn == 192 ? pair_pick_bn<192>(out) : pair_pick_bn<256>(out); }

struct PairGemm : hb_kernel {
    hb_gemm_desc d{};
    pair_fn fn = nullptr;
    uint32_t stages = 0;
    size_t smem = 0;
    const void* last_w = nullptr;
    const void* last_x = nullptr;
    uint32_t last_m = 0;
    uint32_t rank_of_signal = 0;  // y_signal: which row of the flags this rank writes (hb_gemm_desc.y_signal - 1)
    uint32_t split_rows_cap = 0;  // split_k: the rows the context's partial-tile scratch was sized for
    CUtensorMap tm_x{}, tm_w{};

    int launch(hb_ctx* ctx, const hb_range* a, int na, uint32_t m) override {
        if (na != (d.y_signal ? 5 : 3)) return fail(ctx, HB_INVALID, name + (d.y_signal ? ": bindings are W, X, Y, flag_table, ctl" : ": bindings are W, X, Y"));
        if (m == 0 || m > d.rows_max) return fail(ctx, HB_INVALID, name + ": m = " + std::to_string(m) + " outside 1.." + std::to_string(d.rows_max));
        const uint32_t n_out = d.out == HB_OUT_SWIGLU ? d.n / 2 : d.n;
        const size_t ybytes = d.y_shards > 1 ? (size_t)d.y_shards * 8 : (size_t)m * n_out * (d.out == HB_OUT_F32 ? 4 : 2);
        if (!range_ok(a[0], (size_t)d.n * d.k * 2) || !range_ok(a[1], (size_t)m * d.k * 2) || !range_ok(a[2], ybytes))
            return fail(ctx, HB_INVALID, name + ": a bound range is too small for " + std::to_string(m) + " rows");
        if (a[0].ptr != last_w || a[1].ptr != last_x || m != last_m) {
            int r = make_tmap_bf16(ctx, &tm_w, a[0].ptr, d.n, d.k, d.tile_n / 2);  // a CTA's half of the tile's columns
            if (r != HB_OK) return r;
            r = make_tmap_bf16(ctx, &tm_x, a[1].ptr, m, d.k, 128);
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
        p.tiles_m = (m + 255) / 256;
        const uint32_t cols_per_tile = d.out == HB_OUT_SWIGLU ? d.tile_n / 2 : d.tile_n;
        p.tiles_n = (n_out + cols_per_tile - 1) / cols_per_tile;
        p.num_tiles = p.tiles_m * p.tiles_n;
        p.stages = stages;
        p.m_first = d.m_first;
        const uint32_t elem = d.out == HB_OUT_F32 ? 4 : 2;
        p.vec_ok = ((reinterpret_cast<uintptr_t>(a[2].ptr) & 15u) == 0 && ((size_t)n_out * elem) % 16 == 0) ? 1u : 0u;
        p.status = ctx->status_dev;
        if (d.y_shards > 1) {  // Y is a table of block addresses (every block 16-byte aligned by contract)
            p.y_shards = static_cast<const uint64_t*>(a[2].ptr);
            p.shard_rows = (m + d.y_shards - 1) / d.y_shards;
            p.y = nullptr;
            p.vec_ok = ((size_t)n_out * elem) % 16 == 0 ? 1u : 0u;
            p.group_rows = d.y_group_rows;
            p.group_part = d.y_group_rows / d.y_shards;
            p.world = d.y_shards;
            if (d.y_signal) {
                if (!range_ok(a[3], (size_t)d.y_shards * 8) || !range_ok(a[4], (size_t)HB_TP_CTL_WORDS * 4))
                    return fail(ctx, HB_INVALID, name + ": flag_table or ctl is too small");
                if (p.tiles_m > TP_MAX_GROUPS) return fail(ctx, HB_INVALID, name + ": more row groups than flags");
                p.flag_table = static_cast<const uint64_t*>(a[3].ptr);
                p.ctl = static_cast<uint32_t*>(a[4].ptr);
                p.rank = rank_of_signal;
                p.m_first = 0;  // group by group: all column tiles of a row tile before the next row tile
            }
        }
        if (d.split_k > 1) {
            if (m > split_rows_cap) return fail(ctx, HB_INVALID, name + ": the split-K form is built for blocks of at most " + std::to_string(split_rows_cap) + " rows");
            if (d.split_k > p.k_blocks) return fail(ctx, HB_INVALID, name + ": more K slices than 64-element K blocks");
            p.split_k = d.split_k;
            p.partial = ctx->splitk_partial;
            p.split_counters = ctx->splitk_counters;
        }
        const uint32_t pairs = std::min<uint32_t>(p.num_tiles * std::max(1u, d.split_k), (uint32_t)ctx->sm_count / 2);
        cudaLaunchConfig_t cfg{};
        cfg.gridDim = dim3(2 * pairs);
        cfg.blockDim = dim3(GEMM_THREADS);
        cfg.dynamicSmemBytes = smem;
        cfg.stream = ctx->stream;
        cudaLaunchAttribute attr[2];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        if (ctx->overlap_launches) {  // the kernel waits for its predecessor itself (griddepcontrol.wait before X and Y are touched)
            attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
            attr[1].val.programmaticStreamSerializationAllowed = 1;
            cfg.numAttrs = 2;
        }
        HB_CUDA(ctx, cudaLaunchKernelEx(&cfg, fn, tm_x, tm_w, p));
        ctx->launches++;
        return HB_OK;
    }
};

}  // namespace

// The running f32 sums of all split-K kernels of a context live in one scratch range (kernels on one stream run one
// after the other), grown when a shape needs more: one block of 256 x 256 f32 per tile, for blocks of at most 1024 rows
// (the form is for short blocks: few tiles for many SMs), and a flag per quarter of a CTA's half tile.
static int ensure_split_scratch(hb_ctx* ctx, const hb_gemm_desc* d, uint32_t* rows_cap_out) {
    const uint32_t rows_cap = std::min<uint32_t>(std::max<uint32_t>(d->rows_max, 256u), 1024u);
    const uint32_t n_out = d->out == HB_OUT_SWIGLU ? d->n / 2 : d->n;
    const uint32_t cols_per_tile = d->out == HB_OUT_SWIGLU ? PAIR_BN / 2 : PAIR_BN;
    const size_t tiles = (size_t)((rows_cap + 255) / 256) * ((n_out + cols_per_tile - 1) / cols_per_tile);
    const size_t need = tiles * 256 * 256 * sizeof(float), need_counters = tiles * 8 * sizeof(uint32_t);
    if (need > ctx->splitk_partial_bytes) {
        void* sc = nullptr;
        int r = hb_alloc(ctx, need, &sc);
        if (r != HB_OK) return r;
        ctx->splitk_partial = static_cast<float*>(sc);
        ctx->splitk_partial_bytes = need;
    }
    if (need_counters > ctx->splitk_counter_bytes) {
        void* cn = nullptr;
        int r = hb_alloc(ctx, need_counters, &cn);
        if (r != HB_OK) return r;
        zero_on_failure(ctx, cn, need_counters);
        ctx->splitk_counters = static_cast<uint32_t*>(cn);
        ctx->splitk_counter_bytes = need_counters;
    }
    *rows_cap_out = rows_cap;
    return HB_OK;
}

int make_gemm_pair(hb_ctx* ctx, const hb_gemm_desc* d, hb_kernel** out) {
    *out = nullptr;
    if (d->tile_n != 0 && d->tile_n != 256 && d->tile_n != 192) return fail(ctx, HB_UNSUPPORTED, "gemm: the CTA-pair form has tiles of 256 x 256 or 256 x 192");
    const uint32_t bn = d->tile_n == 192 ? 192u : 256u;
    if (bn != 256 && d->split_k > 1) return fail(ctx, HB_UNSUPPORTED, "gemm: split_k is built for the 256 x 256 tile");
    if (d->y_shards > 1 && d->out != HB_OUT_F32) return fail(ctx, HB_UNSUPPORTED, "gemm: a Y in row blocks is for f32 partial products (Out::F32)");
    if (d->y_shards > 16) return fail(ctx, HB_UNSUPPORTED, "gemm: at most 16 row blocks of Y");
    if (d->y_group_rows) {
        if (d->y_shards < 2 || d->y_group_rows > 256 || d->y_group_rows % (32 * d->y_shards) != 0)
            return fail(ctx, HB_UNSUPPORTED, "gemm: rows dealt in groups need y_shards >= 2 and a group of a multiple of 32 * y_shards rows, at most 256");
    }
    if (d->y_signal) {
        if (d->y_group_rows != 256) return fail(ctx, HB_UNSUPPORTED, "gemm: y_signal needs y_group_rows = 256 (a group is a row tile of the CTA pair)");
        if (d->y_signal > d->y_shards) return fail(ctx, HB_UNSUPPORTED, "gemm: y_signal is this rank's number + 1, at most y_shards");
    }
    if (d->split_k > 1 && (d->y_shards > 1 || d->split_k > 64)) return fail(ctx, HB_UNSUPPORTED, "gemm: split_k is 2..64 slices of K, not together with a Y in row blocks");
    pair_fn fn = pair_pick(d->out, bn);
    const size_t budget = std::min<size_t>(ctx->smem_optin, 227 * 1024) - 2048;
    // a Y in row blocks: 16 KB behind the ring (4 KB per epilogue warp) for the transposing store
    const size_t extra = d->y_shards > 1 ? 4 * 4096 : 0;
    const uint32_t max_stages = (uint32_t)std::min<size_t>((budget - extra) / PAIR_STAGE_BYTES, MAX_STAGES);
    const uint32_t stages = d->stages ? d->stages : max_stages;
    if (stages < 2 || stages > max_stages) return fail(ctx, HB_UNSUPPORTED, "gemm: stage count does not fit");
    auto k = std::make_unique<PairGemm>();
    k->d = *d;
    k->d.tile_n = bn;
    k->fn = fn;
    k->stages = stages;
    k->smem = (size_t)stages * PAIR_STAGE_BYTES + extra + 1024;
    k->kind = 1;
    k->nargs = d->y_signal ? 5 : 3;
    k->rank_of_signal = d->y_signal ? d->y_signal - 1 : 0;
    char nm[200];
    std::string ytag;
    if (d->y_shards > 1) ytag = "_y" + std::to_string(d->y_shards);
    if (d->y_group_rows) ytag += "g" + std::to_string(d->y_group_rows);
    if (d->y_signal) ytag += "_sig" + std::to_string(d->y_signal - 1);
    if (d->split_k > 1) ytag += "_k" + std::to_string(d->split_k);
    snprintf(nm, sizeof nm, "gemm_pair_%ux%u_%s%s_t256x%u_s%u%s", d->k, d->n, out_tag(d->out), d->m_first && !d->y_signal ? "_mf" : "", bn, stages, ytag.c_str());
    k->name = nm;
    if (hb_kernel* have = find(ctx, k->name)) {
        auto* g = static_cast<PairGemm*>(have);
        g->d.rows_max = std::max(g->d.rows_max, d->rows_max);
        if (d->split_k > 1) {
            int r = ensure_split_scratch(ctx, &g->d, &g->split_rows_cap);
            if (r != HB_OK) return r;
        }
        *out = have;
        return HB_OK;
    }
    if (d->split_k > 1) {
        int r = ensure_split_scratch(ctx, d, &k->split_rows_cap);
        if (r != HB_OK) return r;
    }
    cudaError_t e = cudaFuncSetAttribute(reinterpret_cast<const void*>(fn), cudaFuncAttributeMaxDynamicSharedMemorySize, (int)ctx->smem_optin - 1024);
    if (e != cudaSuccess) return cuda_fail(ctx, e, "cudaFuncSetAttribute(max dynamic shared memory)");
    *out = intern(ctx, std::move(k));
    return HB_OK;
}

}  // namespace hb
