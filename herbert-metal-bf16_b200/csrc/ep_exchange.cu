// Expert-parallel exchange over peer memory: the token rows of an MoE block travel to the GPUs that hold their
// experts, and the expert outputs travel back, as plain stores and loads through NVLink inside three small kernels -
// no host-side counts, no variable-size collective.
//
// Every rank sorts its (row, slot) pairs by GLOBAL expert (the sort kernel, which also writes the first sorted
// position of every expert: `offs[experts + 1]`). Experts are partitioned contiguously, `epr` per rank, so the sorted
// list is at the same time grouped by destination rank. After an all-gather of the offset vectors every rank knows,
// for every source s and expert e, how many rows s sends for e: cnt(s, e) = offs[s][e + 1] - offs[s][e].
//
//   receive buffer of rank d:  [rows of source 0 | rows of source 1 | ...], each source's rows in its sorted order
//                              (expert ascending, pair ascending within an expert)
//   ep_dispatch (source side): sorted position p -> d = rank of its expert, row base(d, s) + (p - first(s, d)) of d's
//                              receive buffer, where first(s, d) = offs[s][d * epr] and base(d, s) is the number of
//                              rows the sources below s send to d. The row X[list[p] / top_k] is written there.
//   ep_plan (owner side):      the list and the tile table the expert GEMMs need, built from the counts alone:
//                              local expert e owns, from source 0, 1, ..., a contiguous range of the receive buffer
//                              each. Expert-major, then source, then the source's pair order: the concatenation over
//                              the ranks is the order a single GPU's sort would give the same pairs.
//   ep_return (source side):   EY[list[p]] = row (base(d, s) + p - first(s, d)) of d's output buffer, read from d.
//
//   ep_combine (source side):  the return and moe_combine in one: out[row] = the bf16 chain over the row's slots in
//                              route order (src/metal/qwen_kernels.rs:2119-2161), every slot's expert output read
//                              straight from its owner's output buffer at the place the dispatch noted in `where`.
//                              EY is never written or re-read.
//
// Order between the ranks: the all-gather of the offsets before the dispatch, "every rank's rows have landed" before
// the expert GEMMs, "every rank's outputs are complete" before the return. The first and the last are barrier kernels
// on the stream. The middle one is either a barrier kernel too, or (dispatch and plan bound to their optional ranges)
// carried by the kernels themselves: the block of the dispatch that finishes last stores the step's number into a
// flag on every rank, and the plan, which runs before the expert GEMMs, waits (bounded) until every rank's number
// has arrived. No other kernel of this file waits for another GPU.
// No reference counterpart: the reference runs on one GPU.
#include <algorithm>

#include "hb_internal.hpp"
#include "tc05.cuh"

namespace hb {

constexpr int EP_MAX_WORLD = 16;

struct EpParams {
    const uint4* x;            // dispatch: X [rows][h]; return: unused
    uint4* ey;                 // return: EY [pairs][h]
    const uint32_t* list;      // this rank's sorted list
    const uint32_t* offs_all;  // [world][experts + 1]
    const uint64_t* peers;     // [world] base of every rank's receive (dispatch) or output (return) buffer
    uint32_t h8, top_k, experts, world, rank, epr, cap;
    uint32_t* status;
    // dispatch, optional: where[pair] = owner << 28 | row in the owner's buffers (0xffffffff: did not fit), and the
    // "my rows have landed" flag for every rank
    uint32_t* where;
    const uint64_t* peers_landed;  // [world] -> u32[world] on every rank
    uint32_t* ctl;                 // [0] dispatches completed (the step's number), [1] blocks finished
    // direct form: every source owns a fixed region of `region` rows in every receive buffer (source s at s * region),
    // so a source needs nobody else's counts to place its rows: no all-gather before the dispatch. The dispatch then
    // also delivers its own offsets (`offs_all` is this rank's u32[experts + 1]) into row `rank` of every rank's table.
    uint32_t region;
    const uint64_t* peers_offs;    // [world] -> u32[world][experts + 1] on every rank
};

constexpr uint32_t EP_WHERE_NONE = 0xffffffffu;

// first[d], base[d] for this rank as a source, in shared memory.
__device__ __forceinline__ void ep_source_tables(const EpParams& p, uint32_t* first, uint32_t* base) {
    const uint32_t stride = p.experts + 1;
    const uint32_t* mine = p.region ? p.offs_all : p.offs_all + p.rank * stride;  // direct form: the binding is this rank's own row
    if (threadIdx.x < p.world) {
        const uint32_t d = threadIdx.x;
        first[d] = mine[d * p.epr];
        uint32_t b = p.rank * p.region;
        if (!p.region)
            for (uint32_t s = 0; s < p.rank; ++s) b += p.offs_all[s * stride + (d + 1) * p.epr] - p.offs_all[s * stride + d * p.epr];
        base[d] = b;
    }
    if (threadIdx.x == 0) first[p.world] = mine[p.experts];
    __syncthreads();
}

template <bool RETURN>
__global__ void __launch_bounds__(256) ep_move_kernel(const EpParams p) {
    __shared__ uint32_t first[EP_MAX_WORLD + 1], base[EP_MAX_WORLD];
    griddep_wait();
    griddep_launch_dependents();
    ep_source_tables(p, first, base);
    const uint32_t pairs = first[p.world];
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    // a warp per sorted position: the destination is found once per row, the row moves as 16-byte pieces
    for (uint32_t pos = blockIdx.x * warps + warp; pos < pairs; pos += gridDim.x * warps) {
        uint32_t d = 0;
        while (d + 1 < p.world && pos >= first[d + 1]) ++d;
        const uint32_t r = base[d] + pos - first[d];
        if (r >= p.cap || (p.region && pos - first[d] >= p.region)) {  // the counts do not fit the buffers the host sized: report, move nothing
            if (lane == 0) {
                report(p.status, ST_BAD_TABLE, pos, r);
                if (!RETURN && p.where) p.where[p.list[pos]] = EP_WHERE_NONE;
            }
            continue;
        }
        const uint32_t pair = p.list[pos];
        if (!RETURN && p.where && lane == 0) p.where[pair] = (d << 28) | r;
        uint4* remote = reinterpret_cast<uint4*>(p.peers[d]) + (size_t)r * p.h8;
        if constexpr (RETURN) {
            uint4* dst = p.ey + (size_t)pair * p.h8;
            for (uint32_t c = lane; c < p.h8; c += 32) dst[c] = remote[c];
        } else {
            const uint4* src = p.x + (size_t)(pair / p.top_k) * p.h8;
            for (uint32_t c = lane; c < p.h8; c += 32) remote[c] = src[c];
        }
    }
    if (!RETURN && p.peers_landed) {
        // direct form: this rank's offsets into its row of every rank's table (the first blocks share the work)
        if (p.region) {
            const uint32_t words = p.experts + 1;
            for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < p.world * words; i += gridDim.x * blockDim.x) {
                const uint32_t d = i / words, e = i - d * words;
                reinterpret_cast<uint32_t*>(p.peers_offs[d])[(size_t)p.rank * words + e] = p.offs_all[e];
            }
        }
        // this block's rows are out; the block that gets here last numbers the step and tells every rank
        // A block's own fence is at device scope: it orders the block's stores before its count below. The block that
        // counts last has synchronised with all the others through that counter, and its system-scope fence before the
        // flags is cumulative: what the other blocks stored is visible to whoever acquires the flag. (A system-scope
        // fence in every block waits for that block's remote stores to be acknowledged: 8 us of a 26 us dispatch.)
        __shared__ uint32_t last_s;
        __threadfence();
        __syncthreads();
        if (threadIdx.x == 0) {
            last_s = atomicAdd(p.ctl + 1, 1u) == gridDim.x - 1u ? 1u : 0u;
            __threadfence();  // (the count is read before anything below)
        }
        __syncthreads();
        if (last_s && threadIdx.x < p.world) {
            __threadfence_system();
            const uint32_t step = *reinterpret_cast<volatile uint32_t*>(p.ctl) + 1u;
            uint32_t* flag = reinterpret_cast<uint32_t*>(p.peers_landed[threadIdx.x]) + p.rank;
            asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(flag), "r"(step) : "memory");
        }
        __syncthreads();
        if (last_s && threadIdx.x == 0) {
            p.ctl[1] = 0u;
            *reinterpret_cast<volatile uint32_t*>(p.ctl) += 1u;
        }
    }
}

// The return and the combine in one kernel: out[row][i] over the slots in route order, acc = bf16(acc + bf16(y * w))
// (reference src/metal/qwen_kernels.rs:2119-2161), y read from the output buffer of the rank that ran the slot's expert.
struct EpCombineParams {
    const uint64_t* peers_ey;  // [world] bf16 [cap][h] on every rank
    const uint32_t* where;     // [rows * top_k]
    const uint32_t* route;     // [rows][2 * top_k]
    uint16_t* out;             // [rows][h]
    uint32_t rows, h8, top_k, world;
    // optional (hb_ep_combine_sync_get): the barrier "every rank's expert outputs are complete" inside this kernel.
    // Block 0 tells every rank that this rank's expert GEMMs are done (they precede this kernel on the stream); every
    // block waits, bounded, until all owners have said so for this step. The step's number is kept in ctl[0] by the
    // kernel itself (the block that finishes last advances it), so a recorded launch replays.
    const uint64_t* peers_done;  // [world] -> u32[world] on every rank
    const uint32_t* done;        // this rank's u32[world]
    uint32_t* ctl;               // [0] combines completed, [1] blocks finished
    uint32_t rank;
    long long wait_cycles;
    uint32_t* status;
};

__global__ void __launch_bounds__(256) ep_combine_kernel(const EpCombineParams p) {
    __shared__ uint64_t ey_s[EP_MAX_WORLD];
    griddep_wait();  // (before the flag below says that this rank's expert outputs are complete)
    griddep_launch_dependents();
    if (threadIdx.x < p.world) ey_s[threadIdx.x] = p.peers_ey[threadIdx.x];
    uint32_t step = 0;
    if (p.peers_done) {
        step = *reinterpret_cast<volatile uint32_t*>(p.ctl) + 1u;
        if (threadIdx.x < p.world) {
            if (blockIdx.x == 0) {
                __threadfence_system();
                uint32_t* flag = reinterpret_cast<uint32_t*>(p.peers_done[threadIdx.x]) + p.rank;
                asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(flag), "r"(step) : "memory");
            }
            if (!wait_for_step(p.done + threadIdx.x, step, p.wait_cycles) && blockIdx.x == 0) report(p.status, ST_WAIT_TIMEOUT, WHERE_PEER, 64u + threadIdx.x);
        }
    }
    __syncthreads();
    const size_t total = (size_t)p.rows * p.h8;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const uint32_t row = (uint32_t)(i / p.h8), c = (uint32_t)(i % p.h8);
        uint32_t accp[4] = {0u, 0u, 0u, 0u};  // the running bf16 values, two per word
        for (uint32_t s0 = 0; s0 < p.top_k; s0 += 8) {
            uint4 v[8];
            float w[8];
            // all of a batch's loads (remote ones take a microsecond or two) before the first is used
#pragma unroll
            for (int b = 0; b < 8; ++b) {
                const uint32_t s = min(s0 + b, p.top_k - 1);
                const uint32_t loc = p.where[(size_t)row * p.top_k + s];
                v[b] = loc == EP_WHERE_NONE ? make_uint4(0u, 0u, 0u, 0u)
                                            : __ldcs(reinterpret_cast<const uint4*>(ey_s[loc >> 28]) + (size_t)(loc & 0x0fffffffu) * p.h8 + c);
                w[b] = __uint_as_float(p.route[(size_t)row * 2 * p.top_k + p.top_k + s]);
            }
#pragma unroll
            for (int b = 0; b < 8; ++b) {
                if (s0 + b < p.top_k) {
                    const uint32_t vw[4] = {v[b].x, v[b].y, v[b].z, v[b].w};
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const float lo = __uint_as_float(vw[j] << 16), hi = __uint_as_float(vw[j] & 0xffff0000u);
                        const uint32_t t = f32x2_to_bf16x2(__fmul_rn(lo, w[b]), __fmul_rn(hi, w[b]));
                        accp[j] = f32x2_to_bf16x2(__fadd_rn(__uint_as_float(accp[j] << 16), __uint_as_float(t << 16)),
                                                  __fadd_rn(__uint_as_float(accp[j] & 0xffff0000u), __uint_as_float(t & 0xffff0000u)));
                    }
                }
            }
        }
        *reinterpret_cast<uint4*>(p.out + ((size_t)row * p.h8 + c) * 8) = make_uint4(accp[0], accp[1], accp[2], accp[3]);
    }
    if (p.peers_done) {
        // every block has read ctl[0] before it gets here, so the last one may advance it
        __syncthreads();
        if (threadIdx.x == 0 && atomicAdd(p.ctl + 1, 1u) == gridDim.x - 1u) {
            p.ctl[1] = 0u;
            __threadfence();
            *reinterpret_cast<volatile uint32_t*>(p.ctl) = step;
        }
    }
}

struct PlanParams {
    const uint32_t* offs_all;
    uint32_t* list;
    uint32_t* tiles;
    uint32_t experts, world, rank, epr, bm, cap;
    uint32_t* status;
    // optional: wait until every rank's dispatch has flagged this step before the kernels behind the plan may run
    const uint32_t* landed;  // this rank's u32[world]
    const uint32_t* ctl;     // the dispatch's control words: [0] = the step's number
    long long wait_cycles;
    uint32_t region;         // direct form: source s's rows start at s * region of the receive buffer
};

constexpr int PLAN_THREADS = 1024;

__global__ void __launch_bounds__(PLAN_THREADS) ep_plan_kernel(const PlanParams p) {
    extern __shared__ uint32_t sm[];
    uint32_t* start = sm;                  // [epr] first sorted row of local expert e
    uint32_t* sa = start + p.epr;          // [epr] scan scratch (rows)
    uint32_t* st = sa + p.epr;             // [epr] scan scratch (tiles)
    uint32_t* recvbase = st + p.epr;       // [world] first receive row of source s
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t stride = p.experts + 1, e0 = p.rank * p.epr;
    griddep_wait();
    griddep_launch_dependents();
    // (in the direct form the table was written by the other GPUs' dispatch kernels: it is read from L2, not through a
    // read-only path)
    if (p.landed && tid < p.world) {
        const uint32_t step = *reinterpret_cast<const volatile uint32_t*>(p.ctl);  // this rank's dispatch has numbered the step
        if (!wait_for_step(p.landed + tid, step, p.wait_cycles)) report(p.status, ST_WAIT_TIMEOUT, WHERE_PEER, 32u + tid);
    }
    __syncthreads();  // (the waits above: the offsets the peers delivered are read below)
    // The part of the table this rank needs, every source's offsets of the local experts, goes to shared memory in one
    // round trip; everything below reads it there (read one by one from L2, a microsecond each, the serial loops over
    // the sources were most of this kernel's time).
    uint32_t* offs_s = recvbase + p.world;  // [world][epr + 1]
    for (uint32_t i = tid; i < p.world * (p.epr + 1); i += PLAN_THREADS) {
        const uint32_t s = i / (p.epr + 1), e = i - s * (p.epr + 1);
        offs_s[i] = __ldcg(p.offs_all + s * stride + e0 + e);
    }
    __syncthreads();
    auto offs = [&](uint32_t s, uint32_t e) { return offs_s[s * (p.epr + 1) + e]; };  // source s, local expert e (or epr: the end)
    if (tid == 0) {
        uint32_t b = 0;
        for (uint32_t s = 0; s < p.world; ++s) {
            recvbase[s] = p.region ? s * p.region : b;
            b += offs(s, p.epr) - offs(s, 0);
        }
    }
    uint32_t total_e = 0;
    if (tid < p.epr)
        for (uint32_t s = 0; s < p.world; ++s) total_e += offs(s, tid + 1) - offs(s, tid);
    const uint32_t ntile_e = (total_e + p.bm - 1) / p.bm;
    uint32_t a = total_e, t = ntile_e;
    if (tid < p.epr) { sa[tid] = a; st[tid] = t; }
    __syncthreads();
    for (uint32_t d = 1; d < p.epr; d <<= 1) {
        uint32_t va = 0, vt = 0;
        if (tid < p.epr && tid >= d) { va = sa[tid - d]; vt = st[tid - d]; }
        __syncthreads();
        if (tid < p.epr) { a += va; t += vt; sa[tid] = a; st[tid] = t; }
        __syncthreads();
    }
    if (tid < p.epr) {
        const uint32_t s0 = a - total_e, tfirst = t - ntile_e;
        start[tid] = s0;
        if (a <= p.cap) {
            for (uint32_t j = 0, ti = tfirst; j < total_e; j += p.bm, ++ti) {
                p.tiles[1 + 3 * ti] = tid;
                p.tiles[2 + 3 * ti] = s0 + j;
                p.tiles[3 + 3 * ti] = min(p.bm, total_e - j);
            }
        }
        if (tid == p.epr - 1) {
            if (a <= p.cap) {
                p.tiles[0] = t;
            } else {  // more rows than the buffers hold: an empty table, and the host learns why
                p.tiles[0] = 0;
                report(p.status, ST_BAD_TABLE, a, p.cap);
            }
        }
    }
    __syncthreads();
    if (sa[p.epr - 1] > p.cap) return;
    // the list: a warp per local expert, the sources in rank order, each a contiguous range of the receive buffer
    for (uint32_t e = warp; e < p.epr; e += PLAN_THREADS / 32) {
        uint32_t pos = start[e];
        for (uint32_t s = 0; s < p.world; ++s) {
            const uint32_t lo = offs(s, e), hi = offs(s, e + 1);
            const uint32_t src0 = recvbase[s] + lo - offs(s, 0);
            for (uint32_t j = lane; j < hi - lo; j += 32) p.list[pos + j] = src0 + j;
            pos += hi - lo;
        }
    }
}

namespace {

uint32_t ep_grid(hb_ctx* ctx, uint32_t rows) { return std::max(1u, std::min<uint32_t>((rows + 7) / 8, (uint32_t)ctx->sm_count * 8)); }

struct EpMove : hb_kernel {
    uint32_t h = 0, top_k = 0, experts = 0, world = 0, rank = 0, cap = 0;
    bool ret = false;
    bool direct = false;  // every source a fixed region of every receive buffer: no all-gather before the dispatch
    int launch(hb_ctx* ctx, const hb_range* a, int na, uint32_t m) override {
        if (direct ? na != 8 : (na != 4 && !(na == 7 && !ret)))
            return fail(ctx, HB_INVALID, name + (direct ? ": bindings are X, peers, list, offsets (this rank's), where, peers_landed, ctl, peers_offsets"
                                                    : ret ? ": bindings are peers, EY, list, offsets" : ": bindings are X, peers, list, offsets[, where, peers_landed, ctl]"));
        if (m == 0) return fail(ctx, HB_INVALID, name + ": m = 0");
        const uint32_t pairs = m * top_k;
        const hb_range& rows = ret ? a[1] : a[0];
        const hb_range& peers = ret ? a[0] : a[1];
        if (!range_ok(rows, (size_t)(ret ? pairs : m) * h * 2) || !range_ok(peers, (size_t)world * 8) || !range_ok(a[2], (size_t)pairs * 4) ||
            !range_ok(a[3], (size_t)(direct ? 1 : world) * (experts + 1) * 4))
            return fail(ctx, HB_INVALID, name + ": a bound range is too small");
        if (reinterpret_cast<uintptr_t>(rows.ptr) & 15u) return fail(ctx, HB_INVALID, name + ": rows must be 16-byte aligned");
        EpParams p{};
        p.x = ret ? nullptr : static_cast<const uint4*>(rows.ptr);
        p.ey = ret ? static_cast<uint4*>(rows.ptr) : nullptr;
        p.peers = static_cast<const uint64_t*>(peers.ptr);
        p.list = static_cast<const uint32_t*>(a[2].ptr);
        p.offs_all = static_cast<const uint32_t*>(a[3].ptr);
        p.h8 = h / 8;
        p.top_k = top_k;
        p.experts = experts;
        p.world = world;
        p.rank = rank;
        p.epr = experts / world;
        p.cap = cap;
        p.status = ctx->status_dev;
        if (na >= 7) {
            if (cap > 0x0fffffffu || world > 16) return fail(ctx, HB_UNSUPPORTED, name + ": `where` packs the owner in 4 bits and the row in 28");
            if (!range_ok(a[4], (size_t)pairs * 4) || !range_ok(a[5], (size_t)world * 8) || !range_ok(a[6], 8)) return fail(ctx, HB_INVALID, name + ": a bound range is too small");
            p.where = static_cast<uint32_t*>(a[4].ptr);
            p.peers_landed = static_cast<const uint64_t*>(a[5].ptr);
            p.ctl = static_cast<uint32_t*>(a[6].ptr);
        }
        if (direct) {
            if (!range_ok(a[7], (size_t)world * 8)) return fail(ctx, HB_INVALID, name + ": a bound range is too small");
            p.region = cap / world;
            p.peers_offs = static_cast<const uint64_t*>(a[7].ptr);
        }
        HB_CUDA(ctx, launch_kernel(ctx, true, ret ? ep_move_kernel<true> : ep_move_kernel<false>, dim3(ep_grid(ctx, pairs)), dim3(256), 0, p));
        ctx->launches++;
        return HB_OK;
    }
};

struct EpPlan : hb_kernel {
    uint32_t experts = 0, world = 0, rank = 0, bm = 0, cap = 0;
    bool direct = false;
    int launch(hb_ctx* ctx, const hb_range* a, int na, uint32_t m) override {
        if (direct ? na != 5 : (na != 3 && na != 5)) return fail(ctx, HB_INVALID, name + (direct ? ": bindings are offsets, list, tiles, landed, ctl" : ": bindings are offsets, list, tiles[, landed, ctl]"));
        (void)m;
        const uint32_t epr = experts / world;
        if (!range_ok(a[0], (size_t)world * (experts + 1) * 4) || !range_ok(a[1], (size_t)cap * 4) ||
            !range_ok(a[2], (1 + 3 * (size_t)hb_moe_tiles(cap, 1, epr, bm)) * 4))
            return fail(ctx, HB_INVALID, name + ": a bound range is too small");
        PlanParams p{};
        p.offs_all = static_cast<const uint32_t*>(a[0].ptr);
        p.list = static_cast<uint32_t*>(a[1].ptr);
        p.tiles = static_cast<uint32_t*>(a[2].ptr);
        p.experts = experts;
        p.world = world;
        p.rank = rank;
        p.epr = epr;
        p.bm = bm;
        p.cap = cap;
        p.status = ctx->status_dev;
        if (na == 5) {
            if (!range_ok(a[3], (size_t)world * 4) || !range_ok(a[4], 8)) return fail(ctx, HB_INVALID, name + ": a bound range is too small");
            p.landed = static_cast<const uint32_t*>(a[3].ptr);
            p.ctl = static_cast<const uint32_t*>(a[4].ptr);
            p.wait_cycles = (long long)ctx->peer_wait_ms * 2000000ll;
        }
        p.region = direct ? cap / world : 0;
        HB_CUDA(ctx, launch_kernel(ctx, true, ep_plan_kernel, dim3(1), dim3(PLAN_THREADS), (3 * epr + world + world * (epr + 1)) * 4, p));  // start, sa, st, recvbase, offs_s
        ctx->launches++;
        return HB_OK;
    }
};

struct EpCombine : hb_kernel {
    uint32_t h = 0, top_k = 0, world = 0, rank = 0;
    bool sync = false;
    int launch(hb_ctx* ctx, const hb_range* a, int na, uint32_t m) override {
        if (na != (sync ? 7 : 4)) return fail(ctx, HB_INVALID, name + (sync ? ": bindings are peers_ey, where, route, out, peers_done, done, ctl" : ": bindings are peers_ey, where, route, out"));
        if (m == 0) return fail(ctx, HB_INVALID, name + ": m = 0");
        if (!range_ok(a[0], (size_t)world * 8) || !range_ok(a[1], (size_t)m * top_k * 4) || !range_ok(a[2], (size_t)m * 2 * top_k * 4) || !range_ok(a[3], (size_t)m * h * 2))
            return fail(ctx, HB_INVALID, name + ": a bound range is too small");
        if (reinterpret_cast<uintptr_t>(a[3].ptr) & 15u) return fail(ctx, HB_INVALID, name + ": out must be 16-byte aligned");
        EpCombineParams p{};
        p.peers_ey = static_cast<const uint64_t*>(a[0].ptr);
        p.where = static_cast<const uint32_t*>(a[1].ptr);
        p.route = static_cast<const uint32_t*>(a[2].ptr);
        p.out = static_cast<uint16_t*>(a[3].ptr);
        p.rows = m;
        p.h8 = h / 8;
        p.top_k = top_k;
        p.world = world;
        if (sync) {
            if (!range_ok(a[4], (size_t)world * 8) || !range_ok(a[5], (size_t)world * 4) || !range_ok(a[6], 8)) return fail(ctx, HB_INVALID, name + ": a bound range is too small");
            p.peers_done = static_cast<const uint64_t*>(a[4].ptr);
            p.done = static_cast<const uint32_t*>(a[5].ptr);
            p.ctl = static_cast<uint32_t*>(a[6].ptr);
            p.rank = rank;
            p.wait_cycles = (long long)ctx->peer_wait_ms * 2000000ll;
            p.status = ctx->status_dev;
        }
        const size_t items = (size_t)m * p.h8;
        const uint32_t grid = (uint32_t)std::max<size_t>(1, std::min<size_t>((items + 255) / 256, (size_t)ctx->sm_count * 8));
        HB_CUDA(ctx, launch_kernel(ctx, true, ep_combine_kernel, dim3(grid), dim3(256), 0, p));
        ctx->launches++;
        return HB_OK;
    }
};

bool ep_shape_ok(uint32_t experts, uint32_t world, uint32_t rank) {
    return world >= 1 && world <= EP_MAX_WORLD && rank < world && experts >= world && experts % world == 0 && experts <= 1024;
}

}  // namespace

int make_ep_move(hb_ctx* ctx, bool ret, uint32_t h, uint32_t top_k, uint32_t experts, uint32_t world, uint32_t rank, uint32_t cap, hb_kernel** out, bool direct) {
    *out = nullptr;
    if (direct && (ret || cap % world != 0)) return fail(ctx, HB_UNSUPPORTED, "ep dispatch (direct): the buffers' rows must divide by the number of ranks");
    if (!ep_shape_ok(experts, world, rank) || h == 0 || h % 8 != 0 || top_k == 0 || cap == 0)
        return fail(ctx, HB_UNSUPPORTED, "ep exchange: 1..16 ranks dividing at most 1024 experts, h a positive multiple of 8");
    auto k = std::make_unique<EpMove>();
    k->h = h;
    k->top_k = top_k;
    k->experts = experts;
    k->world = world;
    k->rank = rank;
    k->cap = cap;
    k->ret = ret;
    k->direct = direct;
    k->kind = ret ? 12 : 11;
    k->nargs = direct ? 8 : 4;
    k->name = std::string(ret ? "ep_return_" : direct ? "ep_dispatch_direct_" : "ep_dispatch_") + std::to_string(h) + "_k" + std::to_string(top_k) + "_e" + std::to_string(experts) + "_r" +
              std::to_string(rank) + "of" + std::to_string(world) + "_c" + std::to_string(cap);
    *out = intern(ctx, std::move(k));
    return HB_OK;
}

int make_ep_combine(hb_ctx* ctx, uint32_t h, uint32_t top_k, uint32_t world, hb_kernel** out, bool sync, uint32_t rank) {
    *out = nullptr;
    if (world < 1 || world > EP_MAX_WORLD || h == 0 || h % 8 != 0 || top_k == 0) return fail(ctx, HB_UNSUPPORTED, "ep combine: 1..16 ranks, h a positive multiple of 8");
    if (sync && (world < 2 || rank >= world)) return fail(ctx, HB_UNSUPPORTED, "ep combine (with its barrier): 2..16 ranks, one GPU each");
    auto k = std::make_unique<EpCombine>();
    k->h = h;
    k->top_k = top_k;
    k->world = world;
    k->rank = rank;
    k->sync = sync;
    k->kind = 17;
    k->nargs = sync ? 7 : 4;
    k->name = "ep_combine_" + std::to_string(h) + "_k" + std::to_string(top_k) + "_w" + std::to_string(world) + (sync ? "_sync_r" + std::to_string(rank) : std::string());
    *out = intern(ctx, std::move(k));
    return HB_OK;
}

int make_ep_plan(hb_ctx* ctx, uint32_t experts, uint32_t world, uint32_t rank, uint32_t bm, uint32_t cap, hb_kernel** out, bool direct) {
    *out = nullptr;
    if (direct && cap % world != 0) return fail(ctx, HB_UNSUPPORTED, "ep plan (direct): the buffers' rows must divide by the number of ranks");
    if (!ep_shape_ok(experts, world, rank) || cap == 0) return fail(ctx, HB_UNSUPPORTED, "ep plan: 1..16 ranks dividing at most 1024 experts");
    if (bm != 16 && bm != 32 && bm != 64) return fail(ctx, HB_UNSUPPORTED, "ep plan: tile rows 16, 32 or 64");
    auto k = std::make_unique<EpPlan>();
    k->experts = experts;
    k->world = world;
    k->rank = rank;
    k->bm = bm;
    k->cap = cap;
    k->direct = direct;
    k->kind = 13;
    k->nargs = direct ? 5 : 3;
    k->name = std::string(direct ? "ep_plan_direct_e" : "ep_plan_e") + std::to_string(experts) + "_r" + std::to_string(rank) + "of" + std::to_string(world) + "_m" + std::to_string(bm) + "_c" + std::to_string(cap);
    *out = intern(ctx, std::move(k));
    return HB_OK;
}

}  // namespace hb
