// A barrier among the GPUs of one node, with an optional small all-gather riding on it, through peer memory.
//
// Every rank owns a flag array u32[64] (zeroed) in a buffer the other ranks have opened: words 0..world-1 are the
// ranks' arrivals, word 32 is the rank's own count of barriers passed, which only this kernel on this rank touches.
// The barrier's number `epoch` is that count plus one (so 1, 2, 3, ... in the same sequence on every rank, with
// nothing for the host to pass: a recorded launch can be replayed). A rank first copies its `words` payload words into slot `rank`
// of every rank's gather buffer (when there is a payload), then stores `epoch` into slot `rank` of every rank's
// flags with release semantics at system scope, then waits until all slots of its own flags have reached `epoch`
// (acquire, system scope). Writes a rank made before the barrier - by this kernel or by any kernel before it on the
// stream, to its own or to a peer's memory - are visible to every rank after it. Flags only grow, so a rank that
// runs ahead to the next barrier cannot confuse one that is still leaving this one; a payload buffer, however, may
// be overwritten by the next gather, so callers alternate between two of them.
//
// The wait is bounded (hb_set_peer_wait_ms, 5 s unless set): a rank that never arrives turns into a status word and
// HB_KERNEL on the waiting ranks, not a hang. Each rank is one process on its own GPU: this kernel must not be
// launched for several ranks on one GPU (the launches would wait for one another on one stream).
// No reference counterpart: the reference runs on one GPU.
#include "hb_internal.hpp"
#include "tc05.cuh"

namespace hb {

constexpr int SYNC_MAX_WORLD = 16;
constexpr long long SYNC_CYCLES_PER_MS = 2000000ll;  // clock64 counts SM cycles: at most 2 GHz
constexpr uint32_t SYNC_COUNT_WORD = 32;             // of a rank's own flag array: the barriers it has passed

struct SyncParams {
    const uint64_t* peers_flags;   // [world] -> u32[world]
    const uint64_t* peers_gather;  // [world] -> u32[world][words], or null
    const uint32_t* payload;       // [words]
    uint32_t words, world, rank;
    long long wait_cycles;
    uint32_t* status;
};

__global__ void __launch_bounds__(256) peer_sync_kernel(const SyncParams p) {
    const uint32_t t = threadIdx.x;
    __shared__ uint32_t epoch_s;
    if (t == 0) {
        uint32_t* own = reinterpret_cast<uint32_t*>(p.peers_flags[p.rank]) + SYNC_COUNT_WORD;
        epoch_s = *own + 1u;
        *own = epoch_s;
    }
    __syncthreads();
    const uint32_t epoch = epoch_s;
    if (p.words) {
        for (uint32_t d = 0; d < p.world; ++d) {
            uint32_t* dst = reinterpret_cast<uint32_t*>(p.peers_gather[d]) + (size_t)p.rank * p.words;
            for (uint32_t i = t; i < p.words; i += blockDim.x) dst[i] = p.payload[i];
        }
        __threadfence_system();
        __syncthreads();
    }
    if (t < p.world) {
        __threadfence_system();
        uint32_t* remote = reinterpret_cast<uint32_t*>(p.peers_flags[t]) + p.rank;
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(remote), "r"(epoch) : "memory");
        const uint32_t* mine = reinterpret_cast<const uint32_t*>(p.peers_flags[p.rank]) + t;
        const long long t0 = clock64();
        uint32_t v;
        bool ok = true;
        do {
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
            if ((int32_t)(v - epoch) < 0 && clock64() - t0 > p.wait_cycles) ok = false;
        } while ((int32_t)(v - epoch) < 0 && ok);
        if (!ok) report(p.status, ST_WAIT_TIMEOUT, WHERE_PEER, t);
    }
}

namespace {
struct PeerSync : hb_kernel {
    uint32_t words = 0, world = 0, rank = 0;
    int launch(hb_ctx* ctx, const hb_range* a, int na, uint32_t m) override {
        const int want = words ? 3 : 1;
        if (na != want) return fail(ctx, HB_INVALID, name + (words ? ": bindings are peers_flags, payload, peers_gather" : ": the binding is peers_flags"));
        (void)m;  // the barrier counts itself
        if (!range_ok(a[0], (size_t)world * 8)) return fail(ctx, HB_INVALID, name + ": a bound range is too small");
        SyncParams p{};
        p.peers_flags = static_cast<const uint64_t*>(a[0].ptr);
        if (words) {
            if (!range_ok(a[1], (size_t)words * 4) || !range_ok(a[2], (size_t)world * 8)) return fail(ctx, HB_INVALID, name + ": a bound range is too small");
            p.payload = static_cast<const uint32_t*>(a[1].ptr);
            p.peers_gather = static_cast<const uint64_t*>(a[2].ptr);
        }
        p.words = words;
        p.world = world;
        p.rank = rank;
        p.wait_cycles = (long long)ctx->peer_wait_ms * SYNC_CYCLES_PER_MS;
        p.status = ctx->status_dev;
        peer_sync_kernel<<<1, 256, 0, ctx->stream>>>(p);
        HB_CUDA(ctx, cudaGetLastError());
        ctx->launches++;
        return HB_OK;
    }
};
}  // namespace

int make_peer_sync(hb_ctx* ctx, uint32_t words, uint32_t world, uint32_t rank, hb_kernel** res) {
    *res = nullptr;
    if (world < 2 || world > SYNC_MAX_WORLD || rank >= world) return fail(ctx, HB_UNSUPPORTED, "peer_sync: 2..16 ranks, one GPU each");
    if (words > (1u << 20)) return fail(ctx, HB_UNSUPPORTED, "peer_sync: the payload is for small tables (at most 2^20 words)");
    auto k = std::make_unique<PeerSync>();
    k->words = words;
    k->world = world;
    k->rank = rank;
    k->kind = 15;
    k->nargs = words ? 3 : 1;
    k->name = std::string(words ? "peer_allgather_w" + std::to_string(words) : std::string("peer_barrier")) + "_r" + std::to_string(rank) + "of" + std::to_string(world);
    *res = intern(ctx, std::move(k));
    return HB_OK;
}

}  // namespace hb

extern "C" int hb_set_peer_wait_ms(hb_ctx* ctx, uint32_t ms) {
    if (!ctx || ms == 0 || ms > 60000) return hb::fail(ctx, HB_INVALID, "hb_set_peer_wait_ms: 1..60000 ms");
    ctx->peer_wait_ms = ms;
    return HB_OK;
}

extern "C" int hb_peer_sync_get(hb_ctx* ctx, uint32_t words, uint32_t world, uint32_t rank, hb_kernel** res) {
    if (!ctx || !res) return hb::fail(ctx, HB_INVALID, "hb_peer_sync_get: bad argument");
    try {
        hb::bind(ctx);
        return hb::make_peer_sync(ctx, words, world, rank, res);
    } catch (const std::exception& e) {
        return hb::fail(ctx, HB_BACKEND, e.what());
    }
}
