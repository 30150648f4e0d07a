// moe_sort: stable counting sort of the routed (row, slot) pairs by expert, and the expert-tile table
// (reference src/metal/prefill.rs:1303-1442): list[p] = pair index (row*top_k + slot), experts ascending, pairs
// ascending inside an expert; tiles[0] = number of tiles, tile t = (expert, first sorted row, rows <= bm).
//
// One block of 1024 threads, no data-dependent ordering between threads, the same list on every run.
// Fast path (a route names an expert at most once per row, which a top-k route always does): one bitmask of
// rows per expert built with shared-memory atomicOr (the result does not depend on the order of the ORs), a
// prefix of popcounts per mask word, and every pair places itself at
//   first row of its expert + popcount of the expert's mask below its row.
// General path (an expert repeated inside a row, or masks too large for shared memory): every warp owns a
// contiguous segment of pairs and walks it 32 at a time in order; __match_any_sync ranks equal experts inside a
// step and per-warp per-expert counters carry the rank across steps and warps.
#include <algorithm>

#include "hb_internal.hpp"
#include "tc05.cuh"

namespace hb {

constexpr int SORT_THREADS = 1024;
constexpr int SORT_WARPS = SORT_THREADS / 32;

struct SortParams {
    const uint32_t* route;
    uint32_t* list;
    uint32_t* tiles;
    uint32_t* offsets;  // optional [experts + 1]: first sorted row of every expert, then the number of pairs
    uint32_t rows, rows_cap, experts, top_k, bm;
    uint32_t staged;    // the experts of all pairs fit in shared memory as 16-bit values
    uint32_t use_masks; // the per-expert row masks fit in shared memory
    uint32_t words;     // stride of an expert's mask in words: ceil(rows_max / 32) made odd
    uint32_t list_staged;  // the sorted list fits in shared memory as 16-bit pair numbers
};

__global__ void __launch_bounds__(SORT_THREADS) moe_sort_kernel(const SortParams p) {
    extern __shared__ uint32_t sm[];
    const uint32_t experts = p.experts, top_k = p.top_k, bm = p.bm;
    uint32_t* off = sm;                   // [experts] first sorted row of expert e
    uint32_t* tot = off + experts;        // [experts] pairs of expert e
    uint32_t* scan = tot + experts;       // [2][max(experts, 32)] scratch: the warps' totals of the two scans
    uint32_t* flag = scan + 2 * max(experts, 32u);  // [4]
    uint32_t* big = flag + 4;             // masks + prefixes, or the per-warp counters
    uint32_t* mask = big;                                     // [experts][words]
    uint32_t* pre = big + (p.use_masks ? experts * p.words : 0);  // [experts][words]
    uint32_t* cnt = big;                                      // [SORT_WARPS][experts] (general path)
    const size_t big_words = p.use_masks ? 2 * (size_t)experts * p.words : (size_t)SORT_WARPS * experts;
    const size_t counter_words = (size_t)SORT_WARPS * experts;
    uint16_t* ex16 = reinterpret_cast<uint16_t*>(big + (big_words > counter_words ? big_words : counter_words));
    uint16_t* list16 = ex16 + ((size_t)p.rows_cap * top_k + 7) / 8 * 8;  // after the staged experts
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t pairs = p.rows * top_k;
    const uint32_t words = (p.rows + 31) / 32;  // words in use this launch (<= p.words)

    auto expert_global = [&](uint32_t i) { return p.route[(size_t)(i / top_k) * 2 * top_k + (i % top_k)]; };
    if (tid == 0) flag[0] = 0;
    if (p.staged) {
        if (top_k % 4 == 0 && (reinterpret_cast<uintptr_t>(p.route) & 15u) == 0) {
            // a row's experts are top_k consecutive words: 16-byte loads, and all of a thread's loads issued before
            // the first is used (one memory round trip for the whole table instead of one per pair)
            const uint32_t q4 = top_k / 4, vecs = p.rows * q4;
            for (uint32_t v0 = tid; v0 < vecs; v0 += 4 * SORT_THREADS) {
                uint4 e[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const uint32_t v = v0 + u * SORT_THREADS;
                    if (v < vecs) e[u] = reinterpret_cast<const uint4*>(p.route + (size_t)(v / q4) * 2 * top_k)[v % q4];
                }
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const uint32_t v = v0 + u * SORT_THREADS;
                    if (v < vecs) {
                        const uint32_t at = (v / q4) * top_k + (v % q4) * 4;
                        ex16[at] = (uint16_t)e[u].x; ex16[at + 1] = (uint16_t)e[u].y; ex16[at + 2] = (uint16_t)e[u].z; ex16[at + 3] = (uint16_t)e[u].w;
                    }
                }
            }
        } else {
            for (uint32_t i = tid; i < pairs; i += SORT_THREADS) ex16[i] = (uint16_t)expert_global(i);
        }
    }
    auto expert_of = [&](uint32_t i) -> uint32_t { return p.staged ? (uint32_t)ex16[i] : expert_global(i); };

    bool fast = p.use_masks != 0;
    if (fast) {
        for (uint32_t i = tid; i < experts * p.words; i += SORT_THREADS) mask[i] = 0;
        __syncthreads();
        for (uint32_t i = tid; i < pairs; i += SORT_THREADS) {
            const uint32_t e = expert_of(i), r = i / top_k, bit = 1u << (r & 31);
            if (atomicOr(&mask[e * p.words + (r >> 5)], bit) & bit) flag[0] = 1;  // the expert twice in one row
        }
        __syncthreads();
        fast = flag[0] == 0;
    } else {
        __syncthreads();
    }

    uint32_t total_e = 0;
    if (fast) {
        // per expert: exclusive prefix of the popcounts of its mask words. `tpe` neighbouring threads share an expert,
        // each walks a contiguous run of the words, then the runs' totals are passed along the group by shuffles.
        const uint32_t tpe = experts <= 256 ? 4u : experts <= 512 ? 2u : 1u;
        const uint32_t seg = (words + tpe - 1) / tpe;
        {
            const uint32_t e = tid / tpe, part = tid % tpe;
            const uint32_t w0 = min(words, part * seg), w1 = min(words, w0 + seg);
            uint32_t run = 0;
            if (e < experts)
                for (uint32_t w = w0; w < w1; ++w) {
                    pre[e * p.words + w] = run;
                    run += __popc(mask[e * p.words + w]);
                }
            // exclusive scan of `run` over the tpe lanes of the group (groups are aligned inside a warp)
            uint32_t incl = run;
            for (uint32_t d = 1; d < tpe; d <<= 1) {
                const uint32_t v = __shfl_up_sync(0xffffffffu, incl, d);
                if (part >= d) incl += v;
            }
            const uint32_t base = incl - run;
            if (e < experts) {
                if (base)
                    for (uint32_t w = w0; w < w1; ++w) pre[e * p.words + w] += base;
                if (part == tpe - 1) tot[e] = incl;
            }
        }
        __syncthreads();
        if (tid < experts) total_e = tot[tid];
    } else {
        // general path, pass 1: per-warp histograms over contiguous segments
        for (uint32_t i = tid; i < SORT_WARPS * experts; i += SORT_THREADS) cnt[i] = 0;
        __syncthreads();
        const uint32_t seg = ((pairs + SORT_WARPS - 1) / SORT_WARPS + 31) / 32 * 32;
        const uint32_t s0 = min(pairs, warp * seg), s1 = min(pairs, s0 + seg);
        for (uint32_t b = s0; b < s1; b += 32) {
            const uint32_t i = b + lane;
            const bool in = i < s1;
            const uint32_t x = in ? expert_of(i) : 0xffffffffu;
            const uint32_t peers = __match_any_sync(0xffffffffu, x);
            if (in && (peers & ((1u << lane) - 1)) == 0) cnt[warp * experts + x] += __popc(peers);
            __syncwarp();
        }
        __syncthreads();
        if (tid < experts) {
            for (uint32_t w = 0; w < SORT_WARPS; ++w) {  // exclusive scan over the warps
                const uint32_t c = cnt[w * experts + tid];
                cnt[w * experts + tid] = total_e;
                total_e += c;
            }
        }
    }

    // exclusive scans over the experts of (pairs) and (tiles per expert); the tile table
    const uint32_t ntile_e = (total_e + bm - 1) / bm;
    // inclusive scans of both over the experts: inside each warp by shuffles, the warps' totals by warp 0
    uint32_t a = total_e, t = ntile_e;
    uint32_t* sa = scan;
    uint32_t* st = scan + max(experts, 32u);
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const uint32_t va = __shfl_up_sync(0xffffffffu, a, d), vt = __shfl_up_sync(0xffffffffu, t, d);
        if (lane >= (uint32_t)d) { a += va; t += vt; }
    }
    if (lane == 31) { sa[warp] = a; st[warp] = t; }
    __syncthreads();
    if (warp == 0) {
        uint32_t wa = sa[lane], wt = st[lane];
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const uint32_t va = __shfl_up_sync(0xffffffffu, wa, d), vt = __shfl_up_sync(0xffffffffu, wt, d);
            if (lane >= (uint32_t)d) { wa += va; wt += vt; }
        }
        sa[lane] = wa;
        st[lane] = wt;
    }
    __syncthreads();
    if (warp > 0) { a += sa[warp - 1]; t += st[warp - 1]; }
    if (tid < experts) {
        const uint32_t start = a - total_e, tfirst = t - ntile_e;
        off[tid] = start;
        if (p.offsets) {
            p.offsets[tid] = start;
            if (tid == experts - 1) p.offsets[experts] = a;
        }
        for (uint32_t j = 0, ti = tfirst; j < total_e; j += bm, ++ti) {
            p.tiles[1 + 3 * ti] = tid;
            p.tiles[2 + 3 * ti] = start + j;
            p.tiles[3 + 3 * ti] = min(bm, total_e - j);
        }
        if (tid == experts - 1) p.tiles[0] = t;
    }
    __syncthreads();

    if (fast && p.list_staged) {
        // the sorted list is put together in shared memory (16384 scattered 4-byte stores from one SM cost more
        // than everything else in this kernel) and written out in order
        for (uint32_t i = tid; i < pairs; i += SORT_THREADS) {
            const uint32_t e = expert_of(i), r = i / top_k;
            const uint32_t at = e * p.words + (r >> 5);
            list16[off[e] + pre[at] + __popc(mask[at] & ((1u << (r & 31)) - 1u))] = (uint16_t)i;
        }
        __syncthreads();
        if ((pairs & 1u) == 0 && (reinterpret_cast<uintptr_t>(p.list) & 7u) == 0) {
            for (uint32_t j = tid; j < pairs / 2; j += SORT_THREADS) {
                const uint32_t two = reinterpret_cast<const uint32_t*>(list16)[j];
                reinterpret_cast<uint2*>(p.list)[j] = make_uint2(two & 0xffffu, two >> 16);
            }
        } else {
            for (uint32_t j = tid; j < pairs; j += SORT_THREADS) p.list[j] = list16[j];
        }
    } else if (fast) {
        for (uint32_t i = tid; i < pairs; i += SORT_THREADS) {
            const uint32_t e = expert_of(i), r = i / top_k;
            const uint32_t at = e * p.words + (r >> 5);
            p.list[off[e] + pre[at] + __popc(mask[at] & ((1u << (r & 31)) - 1u))] = i;
        }
    } else {
        const uint32_t seg = ((pairs + SORT_WARPS - 1) / SORT_WARPS + 31) / 32 * 32;
        const uint32_t s0 = min(pairs, warp * seg), s1 = min(pairs, s0 + seg);
        for (uint32_t b = s0; b < s1; b += 32) {
            const uint32_t i = b + lane;
            const bool in = i < s1;
            const uint32_t x = in ? expert_of(i) : 0xffffffffu;
            const uint32_t peers = __match_any_sync(0xffffffffu, x);
            const uint32_t before = __popc(peers & ((1u << lane) - 1));
            uint32_t base = 0;
            if (in) base = off[x] + cnt[warp * experts + x];
            __syncwarp();
            if (in) {
                p.list[base + before] = i;
                if (before == 0) cnt[warp * experts + x] += __popc(peers);
            }
            __syncwarp();
        }
    }
}

// ---------------------------------------------------------------------------------------------------------------
// The same sort by a cluster of eight CTAs (distributed shared memory), for the case the fast path above covers: a
// route that names an expert at most once per row. The rows are dealt to the CTAs in contiguous blocks (a multiple of
// 32 rows each). Every CTA builds the masks of its own rows, counts its pairs per expert and stores the counts into
// the shared memory of all eight CTAs; after one cluster barrier each CTA knows, per expert, the total and how many
// pairs the CTAs before it hold, scans the totals itself and places its own pairs:
//   first row of the expert + pairs of that expert in the CTAs before + rank inside the CTA.
// The order is the single-CTA kernel's (and the reference's): experts ascending, pairs ascending inside an expert.
// One SM's shared-memory and store throughput bound the single-CTA form; eight SMs share the work here.
// A route with a repeated expert in a row is sorted by CTA 0 alone, serially (see below).
constexpr int CS_THREADS = 512;
constexpr int CS_CTAS = 8;

struct ClusterSortParams {
    const uint32_t* route;
    uint32_t* list;
    uint32_t* tiles;
    uint32_t* offsets;
    uint32_t rows, experts, top_k, bm;
    uint32_t rows_per_cta;  // a multiple of 32
    uint32_t words;         // stride of an expert's mask: rows_per_cta_max / 32, made odd
    uint32_t ex_cap;        // u16 slots of the staged experts
};

__device__ __forceinline__ uint32_t cs_map(uint32_t smem_addr, uint32_t cta) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(cta));
    return r;
}
__device__ __forceinline__ void cs_store(uint32_t cluster_addr, uint32_t v) {
    asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(cluster_addr), "r"(v) : "memory");
}

__global__ void __cluster_dims__(CS_CTAS, 1, 1) __launch_bounds__(CS_THREADS) moe_sort_cluster_kernel(const ClusterSortParams p) {
    extern __shared__ uint32_t sm[];
    const uint32_t experts = p.experts, top_k = p.top_k, bm = p.bm;
    uint32_t* cnt_all = sm;                          // [CS_CTAS][experts]: pairs of expert e in CTA c (written by CTA c)
    uint32_t* dup_all = cnt_all + CS_CTAS * experts; // [CS_CTAS]
    uint32_t* off = dup_all + CS_CTAS;               // [experts] first sorted row of e + pairs of e in the CTAs before
    uint32_t* sa = off + experts;                    // [32] warp totals of the scans
    uint32_t* st = sa + 32;                          // [32]
    uint32_t* mask = st + 32;                        // [experts][words]
    uint32_t* pre = mask + experts * p.words;        // [experts][words]
    uint16_t* ex16 = reinterpret_cast<uint16_t*>(pre + experts * p.words);
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    uint32_t cta;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(cta));
    const uint32_t r0 = min(p.rows, cta * p.rows_per_cta), r1 = min(p.rows, r0 + p.rows_per_cta);
    const uint32_t my_rows = r1 - r0, my_pairs = my_rows * top_k, words = p.rows_per_cta / 32;
    __shared__ uint32_t dup_s;

    for (uint32_t i = tid; i < experts * p.words; i += CS_THREADS) mask[i] = 0;
    if (tid == 0) dup_s = 0;
    griddep_wait();  // (an overlapped launch: the route is the output of the kernel before this one)
    griddep_launch_dependents();
    // the experts of this CTA's rows
    const uint32_t* rt = p.route + (size_t)r0 * 2 * top_k;
    if (top_k % 4 == 0 && (reinterpret_cast<uintptr_t>(p.route) & 15u) == 0) {
        const uint32_t q4 = top_k / 4, vecs = my_rows * q4;
        for (uint32_t v = tid; v < vecs; v += CS_THREADS) {
            const uint4 e = reinterpret_cast<const uint4*>(rt + (size_t)(v / q4) * 2 * top_k)[v % q4];
            const uint32_t at = (v / q4) * top_k + (v % q4) * 4;
            ex16[at] = (uint16_t)e.x; ex16[at + 1] = (uint16_t)e.y; ex16[at + 2] = (uint16_t)e.z; ex16[at + 3] = (uint16_t)e.w;
        }
    } else {
        for (uint32_t i = tid; i < my_pairs; i += CS_THREADS) ex16[i] = (uint16_t)rt[(size_t)(i / top_k) * 2 * top_k + (i % top_k)];
    }
    __syncthreads();
    for (uint32_t i = tid; i < my_pairs; i += CS_THREADS) {
        const uint32_t e = ex16[i], r = i / top_k, bit = 1u << (r & 31);
        if (e >= experts || (atomicOr(&mask[e * p.words + (r >> 5)], bit) & bit)) dup_s = 1;  // twice in a row (or not an expert)
    }
    __syncthreads();
    // per expert: prefix of the popcounts of its words; the count goes to every CTA of the cluster
    for (uint32_t e = tid; e < experts; e += CS_THREADS) {
        uint32_t run = 0;
        for (uint32_t w = 0; w < words; ++w) {
            pre[e * p.words + w] = run;
            run += __popc(mask[e * p.words + w]);
        }
        const uint32_t mine = smem_u32(&cnt_all[cta * experts + e]);
#pragma unroll
        for (uint32_t c = 0; c < CS_CTAS; ++c) cs_store(cs_map(mine, c), run);
    }
    if (tid < CS_CTAS) cs_store(cs_map(smem_u32(&dup_all[cta]), tid), dup_s);
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
    // (no CTA touches another's shared memory after this barrier, so none has to wait for the others to finish)
    uint32_t any_dup = 0;
#pragma unroll
    for (uint32_t c = 0; c < CS_CTAS; ++c) any_dup |= dup_all[c];
    // A route that repeats an expert inside a row (a top-k route never does) cannot use the masks: CTA 0 then sorts
    // alone, a thread per expert walking all pairs in order (every thread reads the same word: a broadcast) - slow
    // (two passes over the pairs) but exact, and taken by no route this library produces.
    const bool serial = any_dup != 0;
    if (serial && cta != 0) return;
    const uint32_t pairs_all = p.rows * top_k;
    // totals and the share of the CTAs before this one; scans of (pairs, tiles) over the experts
    // (thread e for e < CS_THREADS; the cluster form is built for at most CS_THREADS experts)
    uint32_t total_e = 0, before = 0;
    if (tid < experts) {
        if (serial) {
            for (uint32_t i = 0; i < pairs_all; ++i) total_e += p.route[(size_t)(i / top_k) * 2 * top_k + (i % top_k)] == tid ? 1u : 0u;
        } else {
#pragma unroll
            for (uint32_t c = 0; c < CS_CTAS; ++c) {
                const uint32_t v = cnt_all[c * experts + tid];
                total_e += v;
                if (c < cta) before += v;
            }
        }
    }
    const uint32_t ntile_e = (total_e + bm - 1) / bm;
    uint32_t a = total_e, t = ntile_e;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const uint32_t va = __shfl_up_sync(0xffffffffu, a, d), vt = __shfl_up_sync(0xffffffffu, t, d);
        if (lane >= (uint32_t)d) { a += va; t += vt; }
    }
    if (lane == 31) { sa[warp] = a; st[warp] = t; }
    __syncthreads();
    if (warp == 0) {
        uint32_t wa = lane < CS_THREADS / 32 ? sa[lane] : 0, wt = lane < CS_THREADS / 32 ? st[lane] : 0;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const uint32_t va = __shfl_up_sync(0xffffffffu, wa, d), vt = __shfl_up_sync(0xffffffffu, wt, d);
            if (lane >= (uint32_t)d) { wa += va; wt += vt; }
        }
        if (lane < CS_THREADS / 32) { sa[lane] = wa; st[lane] = wt; }
    }
    __syncthreads();
    if (warp > 0) { a += sa[warp - 1]; t += st[warp - 1]; }
    if (tid < experts) {
        const uint32_t start = a - total_e, tfirst = t - ntile_e;
        off[tid] = start + before;
        if (cta == 0) {  // the table and the offsets are the same in every CTA: one writes them
            if (p.offsets) {
                p.offsets[tid] = start;
                if (tid == experts - 1) p.offsets[experts] = a;
            }
            for (uint32_t j = 0, ti = tfirst; j < total_e; j += bm, ++ti) {
                p.tiles[1 + 3 * ti] = tid;
                p.tiles[2 + 3 * ti] = start + j;
                p.tiles[3 + 3 * ti] = min(bm, total_e - j);
            }
            if (tid == experts - 1) p.tiles[0] = t;
        }
    }
    __syncthreads();
    if (serial) {
        if (tid < experts) {
            uint32_t pos = off[tid];
            for (uint32_t i = 0; i < pairs_all; ++i)
                if (p.route[(size_t)(i / top_k) * 2 * top_k + (i % top_k)] == tid) p.list[pos++] = i;
        }
        return;
    }
    // placement: the pairs of one (expert, CTA) are neighbours in the list, so the stores fill whole sectors
    const uint32_t pair0 = r0 * top_k;
    for (uint32_t i = tid; i < my_pairs; i += CS_THREADS) {
        const uint32_t e = ex16[i], r = i / top_k;
        const uint32_t at = e * p.words + (r >> 5);
        p.list[off[e] + pre[at] + __popc(mask[at] & ((1u << (r & 31)) - 1u))] = pair0 + i;
    }
}

namespace {

struct MoeSort : hb_kernel {
    uint32_t experts = 0, top_k = 0, rows_max = 0, bm = 0, staged = 0, use_masks = 0, words = 0, list_staged = 0;
    size_t smem = 0;
    // the cluster form, when the shape allows it: its mask stride and shared memory
    uint32_t cl_words = 0, cl_ex_cap = 0;
    size_t cl_smem = 0;
    int launch(hb_ctx* ctx, const hb_range* a, int na, uint32_t m) override {
        if (na != 3 && na != 4) return fail(ctx, HB_INVALID, name + ": bindings are route, list, tiles[, offsets]");
        if (na == 4 && !range_ok(a[3], ((size_t)experts + 1) * 4)) return fail(ctx, HB_INVALID, name + ": the offsets range is too small");
        if (m == 0 || m > rows_max) return fail(ctx, HB_INVALID, name + ": m outside 1.." + std::to_string(rows_max));
        const size_t tiles_words = 1 + 3 * (size_t)hb_moe_tiles(m, top_k, experts, bm);
        if (!range_ok(a[0], (size_t)m * 2 * top_k * 4) || !range_ok(a[1], (size_t)m * top_k * 4) || !range_ok(a[2], tiles_words * 4))
            return fail(ctx, HB_INVALID, name + ": a bound range is too small");
        SortParams p{};
        p.route = static_cast<const uint32_t*>(a[0].ptr);
        p.list = static_cast<uint32_t*>(a[1].ptr);
        p.tiles = static_cast<uint32_t*>(a[2].ptr);
        p.offsets = na == 4 ? static_cast<uint32_t*>(a[3].ptr) : nullptr;
        p.rows = m;
        p.rows_cap = rows_max;
        p.list_staged = list_staged;
        p.experts = experts;
        p.top_k = top_k;
        p.bm = bm;
        p.staged = staged;
        p.use_masks = use_masks;
        p.words = words;
        if (cl_smem) {
            ClusterSortParams c{};
            c.route = p.route;
            c.list = p.list;
            c.tiles = p.tiles;
            c.offsets = p.offsets;
            c.rows = m;
            c.experts = experts;
            c.top_k = top_k;
            c.bm = bm;
            c.rows_per_cta = ((m + CS_CTAS - 1) / CS_CTAS + 31) / 32 * 32;
            c.words = cl_words;
            c.ex_cap = cl_ex_cap;
            HB_CUDA(ctx, launch_kernel(ctx, true, moe_sort_cluster_kernel, dim3(CS_CTAS), dim3(CS_THREADS), cl_smem, c));
            ctx->launches++;
            return HB_OK;
        }
        moe_sort_kernel<<<1, SORT_THREADS, smem, ctx->stream>>>(p);
        HB_CUDA(ctx, cudaGetLastError());
        ctx->launches++;
        return HB_OK;
    }
};

}  // namespace

int make_moe_sort(hb_ctx* ctx, uint32_t experts, uint32_t top_k, uint32_t rows_max, uint32_t bm, hb_kernel** out) {
    *out = nullptr;
    if (experts == 0 || experts > 1024 || top_k == 0 || rows_max == 0) return fail(ctx, HB_UNSUPPORTED, "moe_sort: 1..1024 experts, top_k and rows_max positive");
    if (bm != 16 && bm != 32 && bm != 64) return fail(ctx, HB_UNSUPPORTED, "moe_sort: tile rows 16, 32 or 64");
    auto k = std::make_unique<MoeSort>();
    k->experts = experts;
    k->top_k = top_k;
    k->rows_max = rows_max;
    k->bm = bm;
    k->kind = 5;
    k->nargs = 3;
    k->name = "moe_sort_" + std::to_string(experts) + "_k" + std::to_string(top_k) + "_r" + std::to_string(rows_max) + "_m" + std::to_string(bm);
    if (hb_kernel* have = find(ctx, k->name)) {
        *out = have;
        return HB_OK;
    }
    const size_t limit = 220 * 1024;
    const size_t fixed = (2 * (size_t)experts + 2 * std::max<size_t>(experts, 32) + 4) * 4;
    const size_t counters = (size_t)SORT_WARPS * experts * 4;
    k->words = ((rows_max + 31) / 32) | 1u;  // odd stride: the same word of different experts falls in different banks
    const size_t masks = 2 * (size_t)experts * k->words * 4;
    size_t big = counters;
    if (fixed + std::max(masks, counters) <= limit) {
        k->use_masks = 1;
        big = std::max(masks, counters);  // the general path stays available inside the same launch
    }
    const size_t stage = ((size_t)rows_max * top_k * 2 + 15) / 16 * 16;
    k->smem = fixed + big;
    if (k->smem + stage <= limit) {
        k->staged = 1;
        k->smem += stage;
        if (k->use_masks && (size_t)rows_max * top_k <= 65536 && k->smem + stage <= limit) {
            k->list_staged = 1;
            k->smem += stage;
        }
    }
    cudaError_t e = cudaFuncSetAttribute(reinterpret_cast<const void*>(moe_sort_kernel), cudaFuncAttributeMaxDynamicSharedMemorySize, (int)ctx->smem_optin - 1024);
    if (e != cudaSuccess) return cuda_fail(ctx, e, "cudaFuncSetAttribute(moe_sort)");
    // the cluster form: at most CS_THREADS experts (a thread per expert in the scans), at least a few rows per CTA,
    // and masks of one CTA's rows that fit its shared memory
    if (experts <= CS_THREADS && rows_max >= 256) {
        const uint32_t rpc = ((rows_max + CS_CTAS - 1) / CS_CTAS + 31) / 32 * 32;
        const uint32_t cw = (rpc / 32) | 1u;
        const size_t ex_cap = ((size_t)rpc * top_k + 7) / 8 * 8;
        const size_t need = ((size_t)CS_CTAS * experts + CS_CTAS + experts + 64 + 2 * (size_t)experts * cw) * 4 + ex_cap * 2 + 16;
        if (need <= limit) {
            k->cl_words = cw;
            k->cl_ex_cap = (uint32_t)ex_cap;
            k->cl_smem = need;
            e = cudaFuncSetAttribute(reinterpret_cast<const void*>(moe_sort_cluster_kernel), cudaFuncAttributeMaxDynamicSharedMemorySize, (int)ctx->smem_optin - 1024);
            if (e != cudaSuccess) return cuda_fail(ctx, e, "cudaFuncSetAttribute(moe_sort cluster)");
        }
    }
    *out = intern(ctx, std::move(k));
    return HB_OK;
}

}  // namespace hb
