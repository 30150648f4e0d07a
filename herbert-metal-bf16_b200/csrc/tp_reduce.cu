// Reduce-scatter + output mode + all-gather of a row-parallel projection, in one kernel over peer memory.
//
// A tensor-parallel FFN leaves on every rank an f32 partial product [m][n] of its K slice (the down GEMM with
// Out::F32). The rows are dealt to the ranks in contiguous slices; a rank sums, for its slice only, the partials of
// all ranks in rank order (its own from local memory, the others through NVLink loads), rounds once, applies the
// output mode (src/metal/kernels.rs:217-234: Bf16, or Residual = a second rounding after adding the old Y), and
// stores the bf16 result into the Y of every rank (NVLink stores). Every element is computed by exactly one rank, so
// all copies of Y are bit-identical, and the sum order is fixed (rank 0 + rank 1 + ...) whatever the timing.
// The kernel never waits for another GPU: the host puts a barrier before it (all partials complete) and after it
// (all Y complete). No reference counterpart: the reference runs on one GPU.
#include <algorithm>

#include "gemm_common.cuh"

namespace hb {

constexpr int TP_MAX_WORLD = 8;
constexpr long long TP_CYCLES_PER_MS = 2000000ll;  // clock64 counts SM cycles: at most 2 GHz
constexpr uint32_t TP_START_WORD = 16;  // of a rank's `done` words: [0, world) the closing handshake, [16, 16 + world) the opening barrier

struct TpParams {
    const float* staging;       // STAGED: this rank's f32 [world][rows_per][n], slot s from rank s
    const uint64_t* peers_acc;  // [world] f32 [m][n] on every rank
    const uint64_t* peers_y;    // [world] bf16 [m][n] on every rank
    uint32_t m, n8, world, rank, rows_per;
    // optional (hb_tp_sum_sync_get): the two barriers of the step inside this kernel. Its first block tells every rank
    // that this rank's partial has been pushed (the GEMM precedes this kernel on the stream) and every block waits
    // until all ranks have said so; the block that finishes last tells every rank that this rank's rows of Y are out
    // and waits until all ranks have said that too. The step's number lives in ctl[0].
    const uint64_t* peers_flags;  // [world] -> u32[32] on every rank: [0, world) Y is out, [16, 16 + world) partial is out
    uint32_t* ctl;                // [0] steps completed, [1] blocks finished
    long long wait_cycles;
    uint32_t* status;
};

template <int OUT, bool STAGED>
__global__ void __launch_bounds__(256) tp_reduce_kernel(const TpParams p) {
    __shared__ uint64_t acc_s[TP_MAX_WORLD], y_s[TP_MAX_WORLD];
    uint32_t step = 0;
    if (p.peers_flags) {
        step = *reinterpret_cast<volatile uint32_t*>(p.ctl) + 1u;
        if (threadIdx.x < p.world) {
            if (blockIdx.x == 0) {
                __threadfence_system();
                uint32_t* remote = reinterpret_cast<uint32_t*>(p.peers_flags[threadIdx.x]) + TP_START_WORD + p.rank;
                asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(remote), "r"(step) : "memory");
            }
            if (!wait_for_step(reinterpret_cast<const uint32_t*>(p.peers_flags[p.rank]) + TP_START_WORD + threadIdx.x, step, p.wait_cycles) && blockIdx.x == 0)
                report(p.status, ST_WAIT_TIMEOUT, WHERE_PEER, 32u + threadIdx.x);
        }
    }
    if (threadIdx.x < p.world) {
        // STAGED: slot s of the local staging buffer, rebased so that the row index of the whole matrix applies
        acc_s[threadIdx.x] = STAGED ? reinterpret_cast<uint64_t>(p.staging + ((size_t)threadIdx.x * p.rows_per - (size_t)p.rank * p.rows_per) * p.n8 * 8)
                                    : p.peers_acc[threadIdx.x];
        y_s[threadIdx.x] = p.peers_y[threadIdx.x];
    }
    __syncthreads();
    const uint32_t r0 = min(p.m, p.rank * p.rows_per), r1 = min(p.m, r0 + p.rows_per);
    const size_t first = (size_t)r0 * p.n8, total = (size_t)(r1 - r0) * p.n8;  // units of 8 elements
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t at = first + i;
        float v[8];
        // all the loads first (the remote ones take a microsecond or two), the sums after, in rank order
        float4 part[TP_MAX_WORLD][2];
#pragma unroll
        for (uint32_t s = 0; s < TP_MAX_WORLD; ++s) {
            if (s < p.world) {
                const float4* src = reinterpret_cast<const float4*>(acc_s[s]) + at * 2;
                part[s][0] = __ldcs(src);
                part[s][1] = __ldcs(src + 1);
            }
        }
        v[0] = part[0][0].x; v[1] = part[0][0].y; v[2] = part[0][0].z; v[3] = part[0][0].w;
        v[4] = part[0][1].x; v[5] = part[0][1].y; v[6] = part[0][1].z; v[7] = part[0][1].w;
#pragma unroll
        for (uint32_t s = 1; s < TP_MAX_WORLD; ++s) {
            if (s < p.world) {
                v[0] = __fadd_rn(v[0], part[s][0].x); v[1] = __fadd_rn(v[1], part[s][0].y);
                v[2] = __fadd_rn(v[2], part[s][0].z); v[3] = __fadd_rn(v[3], part[s][0].w);
                v[4] = __fadd_rn(v[4], part[s][1].x); v[5] = __fadd_rn(v[5], part[s][1].y);
                v[6] = __fadd_rn(v[6], part[s][1].z); v[7] = __fadd_rn(v[7], part[s][1].w);
            }
        }
        uint32_t o[8];
        if (OUT == HB_OUT_RESIDUAL) {
            const uint4 old = reinterpret_cast<const uint4*>(y_s[p.rank])[at];
            const uint32_t ow[4] = {old.x, old.y, old.z, old.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                o[2 * j] = f32_to_bf16(__fadd_rn(bf16_to_f32(ow[j] & 0xffffu), round_bf16(v[2 * j])));
                o[2 * j + 1] = f32_to_bf16(__fadd_rn(bf16_to_f32(ow[j] >> 16), round_bf16(v[2 * j + 1])));
            }
        } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) o[j] = f32_to_bf16(v[j]);
        }
        const uint4 res = make_uint4(o[0] | (o[1] << 16), o[2] | (o[3] << 16), o[4] | (o[5] << 16), o[6] | (o[7] << 16));
        for (uint32_t d = 0; d < p.world; ++d) reinterpret_cast<uint4*>(y_s[d])[at] = res;
    }
    if (p.peers_flags) {
        // (a block's fence is at device scope; the last block's system-scope fence is cumulative over the blocks it has
        // synchronised with through the counter)
        __shared__ uint32_t last_s;
        __threadfence();
        __syncthreads();
        if (threadIdx.x == 0) {
            last_s = atomicAdd(p.ctl + 1, 1u) == gridDim.x - 1u ? 1u : 0u;
            __threadfence();
        }
        __syncthreads();
        if (!last_s) return;
        if (threadIdx.x == 0) p.ctl[1] = 0u;
        if (threadIdx.x < p.world) {
            __threadfence_system();
            uint32_t* remote = reinterpret_cast<uint32_t*>(p.peers_flags[threadIdx.x]) + p.rank;
            asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(remote), "r"(step) : "memory");
            if (!wait_for_step(reinterpret_cast<const uint32_t*>(p.peers_flags[p.rank]) + threadIdx.x, step, p.wait_cycles))
                report(p.status, ST_WAIT_TIMEOUT, WHERE_PEER, 16u + threadIdx.x);
        }
        __syncthreads();
        if (threadIdx.x == 0) *reinterpret_cast<volatile uint32_t*>(p.ctl) = step;
    }
}

// The sum that runs beside the GEMMs whose partials it sums (hb_tp_sum_stream_get). The rows are dealt in groups of
// group_rows (the GEMM's row tile); of every group this rank sums group_part = group_rows / world rows. For each
// group in turn: wait until every rank's GEMM has set this rank's flag [source][group] to the step's number (the
// stores of the group's partial rows into the staging slots precede the flag, release / acquire at system scope), then
// sum the slots in rank order, round once, apply the output mode and store the bf16 rows into every rank's Y. The block
// that finishes last tells every rank, waits until every rank has said the same, and writes the step's number to
// ctl[0]: when the kernel ends, Y is complete on every rank and every rank has read its staging, so the next step may
// overwrite both. Every wait is bounded; a wait that runs out is reported through the status words and the kernel
// carries on to its end.
struct TpStreamParams {
    const float* staging;        // f32 [world][groups][group_part][n]
    const uint64_t* peers_y;     // [world] bf16 [m][n] on every rank
    const uint32_t* flags;       // this rank's u32 [world][TP_MAX_GROUPS]
    const uint64_t* peers_done;  // [world] -> u32 [world] on every rank
    uint32_t* ctl;
    uint32_t m, n8, world, rank, group_rows, group_part, groups, sync;
    long long wait_cycles;
    uint32_t* status;
};

template <int OUT>
__global__ void __launch_bounds__(128) tp_sum_stream_kernel(const TpStreamParams p) {
    __shared__ uint64_t y_s[TP_MAX_WORLD];
    __shared__ uint32_t step_s, ok_s, last_s;
    if (threadIdx.x < p.world) y_s[threadIdx.x] = p.peers_y[threadIdx.x];
    if (threadIdx.x == 0) {
        step_s = *reinterpret_cast<volatile uint32_t*>(p.ctl) + 1u;
        ok_s = 1u;
    }
    __syncthreads();
    const uint32_t step = step_s;
    const size_t slot_units = (size_t)p.groups * p.group_part * p.n8;  // units of 8 elements in one source's slot
    // one unit: 8 elements of row j of this rank's part of group g
    auto unit = [&](uint32_t g, uint32_t row0, uint32_t i) {
        const uint32_t j = i / p.n8, c = i - j * p.n8;
        const size_t src = ((size_t)g * p.group_part + j) * p.n8 + c;
        const size_t at = (size_t)(row0 + j) * p.n8 + c;
        float4 part[TP_MAX_WORLD][2];
#pragma unroll
        for (uint32_t s = 0; s < TP_MAX_WORLD; ++s) {
            if (s < p.world) {
                const float4* q = reinterpret_cast<const float4*>(p.staging) + (s * slot_units + src) * 2;
                part[s][0] = __ldcs(q);
                part[s][1] = __ldcs(q + 1);
            }
        }
        float v[8] = {part[0][0].x, part[0][0].y, part[0][0].z, part[0][0].w, part[0][1].x, part[0][1].y, part[0][1].z, part[0][1].w};
#pragma unroll
        for (uint32_t s = 1; s < TP_MAX_WORLD; ++s) {
            if (s < p.world) {
                v[0] = __fadd_rn(v[0], part[s][0].x); v[1] = __fadd_rn(v[1], part[s][0].y);
                v[2] = __fadd_rn(v[2], part[s][0].z); v[3] = __fadd_rn(v[3], part[s][0].w);
                v[4] = __fadd_rn(v[4], part[s][1].x); v[5] = __fadd_rn(v[5], part[s][1].y);
                v[6] = __fadd_rn(v[6], part[s][1].z); v[7] = __fadd_rn(v[7], part[s][1].w);
            }
        }
        uint32_t o[8];
        if (OUT == HB_OUT_RESIDUAL) {
            const uint4 old = reinterpret_cast<const uint4*>(y_s[p.rank])[at];
            const uint32_t ow[4] = {old.x, old.y, old.z, old.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                o[2 * e] = f32_to_bf16(__fadd_rn(bf16_to_f32(ow[e] & 0xffffu), round_bf16(v[2 * e])));
                o[2 * e + 1] = f32_to_bf16(__fadd_rn(bf16_to_f32(ow[e] >> 16), round_bf16(v[2 * e + 1])));
            }
        } else {
#pragma unroll
            for (int e = 0; e < 8; ++e) o[e] = f32_to_bf16(v[e]);
        }
        const uint4 res = make_uint4(o[0] | (o[1] << 16), o[2] | (o[3] << 16), o[4] | (o[5] << 16), o[6] | (o[7] << 16));
        for (uint32_t d = 0; d < p.world; ++d) reinterpret_cast<uint4*>(y_s[d])[at] = res;
    };
    if (p.sync == 1) {
        // group by group, each as soon as every rank's GEMM has flagged it
        for (uint32_t g = 0; g < p.groups; ++g) {
            if (threadIdx.x < p.world && !wait_for_step(p.flags + threadIdx.x * TP_MAX_GROUPS + g, step, p.wait_cycles)) {
                report(p.status, ST_WAIT_TIMEOUT, WHERE_PEER, threadIdx.x);
                ok_s = 0u;
            }
            __syncthreads();
            if (!ok_s) break;
            const uint32_t row0 = g * p.group_rows + p.rank * p.group_part;
            if (row0 >= p.m) continue;
            const uint32_t units = min(p.group_part, p.m - row0) * p.n8;
            for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < units; i += gridDim.x * blockDim.x) unit(g, row0, i);
        }
    } else {
        if (p.sync == 2) {
            // the barrier "every rank's partial has been pushed" inside the kernel (the GEMMs precede it on every
            // rank's stream): block 0 says so for this rank, every block waits for all ranks
            if (threadIdx.x < p.world) {
                if (blockIdx.x == 0) {
                    __threadfence_system();
                    uint32_t* remote = reinterpret_cast<uint32_t*>(p.peers_done[threadIdx.x]) + TP_START_WORD + p.rank;
                    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(remote), "r"(step) : "memory");
                }
                if (!wait_for_step(reinterpret_cast<const uint32_t*>(p.peers_done[p.rank]) + TP_START_WORD + threadIdx.x, step, p.wait_cycles)) {
                    if (blockIdx.x == 0) report(p.status, ST_WAIT_TIMEOUT, WHERE_PEER, 32u + threadIdx.x);
                    ok_s = 0u;
                }
            }
            __syncthreads();
        }
        // all groups as one index space (every thread has work whatever the group's size)
        const uint32_t per_group = p.group_part * p.n8;
        const size_t total = ok_s ? (size_t)p.groups * per_group : 0;
        for (size_t t = (size_t)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (size_t)gridDim.x * blockDim.x) {
            const uint32_t g = (uint32_t)(t / per_group), i = (uint32_t)(t - (size_t)g * per_group);
            const uint32_t row0 = g * p.group_rows + p.rank * p.group_part;
            if (row0 < p.m && i < min(p.group_part, p.m - row0) * p.n8) unit(g, row0, i);
        }
    }
    // the closing handshake: this block's stores are ordered before its count (device scope), the last block to get
    // here speaks for the rank (its system-scope fence is cumulative over the blocks it has synchronised with)
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        last_s = atomicAdd(p.ctl + TP_CTL_DONE, 1u) == gridDim.x - 1u ? 1u : 0u;
        __threadfence();
    }
    __syncthreads();
    if (!last_s) return;
    if (threadIdx.x == 0) p.ctl[TP_CTL_DONE] = 0u;
    if (p.sync && threadIdx.x < p.world) {
        __threadfence_system();
        uint32_t* remote = reinterpret_cast<uint32_t*>(p.peers_done[threadIdx.x]) + p.rank;
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(remote), "r"(step) : "memory");
        if (!wait_for_step(reinterpret_cast<const uint32_t*>(p.peers_done[p.rank]) + threadIdx.x, step, p.wait_cycles))
            report(p.status, ST_WAIT_TIMEOUT, WHERE_PEER, 16u + threadIdx.x);
    }
    __syncthreads();
    if (threadIdx.x == 0) *reinterpret_cast<volatile uint32_t*>(p.ctl) = step;
}

namespace {
struct TpSumStream : hb_kernel {
    uint32_t n = 0, out = 0, world = 0, rank = 0, group_rows = 0, sync = 0;
    int launch(hb_ctx* ctx, const hb_range* a, int na, uint32_t m) override {
        if (na != 5) return fail(ctx, HB_INVALID, name + ": bindings are staging, peers_y, flags, peers_done, ctl");
        if (m == 0) return fail(ctx, HB_INVALID, name + ": m = 0");
        const uint32_t groups = (m + group_rows - 1) / group_rows, part = group_rows / world;
        if (groups > TP_MAX_GROUPS) return fail(ctx, HB_INVALID, name + ": more row groups than flags");
        if (!range_ok(a[0], (size_t)world * groups * part * n * 4) || !range_ok(a[1], (size_t)world * 8) || !range_ok(a[2], (size_t)world * TP_MAX_GROUPS * 4) ||
            !range_ok(a[3], (size_t)world * 8) || !range_ok(a[4], (size_t)HB_TP_CTL_WORDS * 4))
            return fail(ctx, HB_INVALID, name + ": a bound range is too small");
        TpStreamParams p{};
        p.staging = static_cast<const float*>(a[0].ptr);
        p.peers_y = static_cast<const uint64_t*>(a[1].ptr);
        p.flags = static_cast<const uint32_t*>(a[2].ptr);
        p.peers_done = static_cast<const uint64_t*>(a[3].ptr);
        p.ctl = static_cast<uint32_t*>(a[4].ptr);
        p.m = m;
        p.n8 = n / 8;
        p.world = world;
        p.rank = rank;
        p.group_rows = group_rows;
        p.group_part = part;
        p.groups = groups;
        p.sync = sync;
        p.wait_cycles = (long long)ctx->peer_wait_ms * TP_CYCLES_PER_MS;
        p.status = ctx->status_dev;
        // sync = 1: the kernel shares the SMs with the GEMM it follows, one block per SM, a group at a time; otherwise
        // all groups are one index space and four blocks per SM keep more loads in flight (all of them resident: they
        // may wait for the other ranks at their start)
        const size_t units = sync == 1 ? (size_t)part * p.n8 : (size_t)groups * part * p.n8;
        const uint32_t grid = (uint32_t)std::max<size_t>(1, std::min<size_t>((units + 127) / 128, (size_t)ctx->sm_count * (sync == 1 ? 1 : 4)));
        cudaLaunchConfig_t cfg{};
        cfg.gridDim = dim3(grid);
        cfg.blockDim = dim3(128);
        cfg.stream = ctx->stream;
        cudaLaunchAttribute attr[1];
        if (sync == 1) {  // may start while the GEMM before it on the stream runs: it waits for the GEMMs' flags, not for their end
            attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
            attr[0].val.programmaticStreamSerializationAllowed = 1;
            cfg.attrs = attr;
            cfg.numAttrs = 1;
        }
        if (out == HB_OUT_RESIDUAL) HB_CUDA(ctx, cudaLaunchKernelEx(&cfg, tp_sum_stream_kernel<HB_OUT_RESIDUAL>, p));
        else HB_CUDA(ctx, cudaLaunchKernelEx(&cfg, tp_sum_stream_kernel<HB_OUT_BF16>, p));
        ctx->launches++;
        return HB_OK;
    }
};

struct TpReduce : hb_kernel {
    uint32_t n = 0, out = 0, world = 0, rank = 0;
    bool staged = false, sync = false;
    int launch(hb_ctx* ctx, const hb_range* a, int na, uint32_t m) override {
        if (na != (sync ? 4 : 2))
            return fail(ctx, HB_INVALID, name + (sync ? ": bindings are staging, peers_y, peers_flags, ctl" : staged ? ": bindings are staging, peers_y" : ": bindings are peers_acc, peers_y (device arrays of one address per rank)"));
        if (m == 0) return fail(ctx, HB_INVALID, name + ": m = 0");
        const uint32_t rows_per = (m + world - 1) / world;
        if (!range_ok(a[0], staged ? (size_t)world * rows_per * n * 4 : (size_t)world * 8) || !range_ok(a[1], (size_t)world * 8))
            return fail(ctx, HB_INVALID, name + ": a bound range is too small");
        TpParams p{};
        if (staged) p.staging = static_cast<const float*>(a[0].ptr);
        else p.peers_acc = static_cast<const uint64_t*>(a[0].ptr);
        p.peers_y = static_cast<const uint64_t*>(a[1].ptr);
        p.m = m;
        p.n8 = n / 8;
        p.world = world;
        p.rank = rank;
        p.rows_per = rows_per;
        if (sync) {
            if (!range_ok(a[2], (size_t)world * 8) || !range_ok(a[3], 8)) return fail(ctx, HB_INVALID, name + ": a bound range is too small");
            p.peers_flags = static_cast<const uint64_t*>(a[2].ptr);
            p.ctl = static_cast<uint32_t*>(a[3].ptr);
            p.wait_cycles = (long long)ctx->peer_wait_ms * TP_CYCLES_PER_MS;
            p.status = ctx->status_dev;
        }
        const size_t units = (size_t)p.rows_per * p.n8;
        // (with the barriers inside, every block starts with a round trip to the flags: fewer, longer-lived blocks)
        const uint32_t grid = (uint32_t)std::max<size_t>(1, std::min<size_t>((units + 255) / 256, (size_t)ctx->sm_count * (sync ? 3 : 8)));
        if (staged) {
            if (out == HB_OUT_RESIDUAL) tp_reduce_kernel<HB_OUT_RESIDUAL, true><<<grid, 256, 0, ctx->stream>>>(p);
            else tp_reduce_kernel<HB_OUT_BF16, true><<<grid, 256, 0, ctx->stream>>>(p);
        } else {
            if (out == HB_OUT_RESIDUAL) tp_reduce_kernel<HB_OUT_RESIDUAL, false><<<grid, 256, 0, ctx->stream>>>(p);
            else tp_reduce_kernel<HB_OUT_BF16, false><<<grid, 256, 0, ctx->stream>>>(p);
        }
        HB_CUDA(ctx, cudaGetLastError());
        ctx->launches++;
        return HB_OK;
    }
};
}  // namespace

int make_tp_reduce(hb_ctx* ctx, uint32_t n, uint32_t out, uint32_t world, uint32_t rank, bool staged, hb_kernel** res, bool sync = false) {
    *res = nullptr;
    if (n == 0 || n % 8 != 0) return fail(ctx, HB_UNSUPPORTED, "tp_reduce: n a positive multiple of 8");
    if (out != HB_OUT_BF16 && out != HB_OUT_RESIDUAL) return fail(ctx, HB_UNSUPPORTED, "tp_reduce: output Bf16 or Residual");
    if (world < 1 || world > TP_MAX_WORLD || rank >= world) return fail(ctx, HB_UNSUPPORTED, "tp_reduce: 1..8 ranks");
    auto k = std::make_unique<TpReduce>();
    k->n = n;
    k->out = out;
    k->world = world;
    k->rank = rank;
    if (sync && (!staged || world < 2)) return fail(ctx, HB_UNSUPPORTED, "tp_sum (with its barriers): the staged form, 2..8 ranks, one GPU each");
    k->staged = staged;
    k->sync = sync;
    k->kind = 14;
    k->nargs = sync ? 4 : 2;
    k->name = std::string(staged ? "tp_sum_" : "tp_reduce_") + std::to_string(n) + "_" + out_tag(out) + "_r" + std::to_string(rank) + "of" + std::to_string(world) + (sync ? "_barriers" : "");
    *res = intern(ctx, std::move(k));
    return HB_OK;
}

}  // namespace hb

extern "C" int hb_tp_reduce_get(hb_ctx* ctx, uint32_t n, uint32_t out, uint32_t world, uint32_t rank, hb_kernel** res) {
    if (!ctx || !res) return hb::fail(ctx, HB_INVALID, "hb_tp_reduce_get: bad argument");
    try {
        hb::bind(ctx);
        return hb::make_tp_reduce(ctx, n, out, world, rank, false, res);
    } catch (const std::exception& e) {
        return hb::fail(ctx, HB_BACKEND, e.what());
    }
}

extern "C" int hb_tp_sum_stream_get(hb_ctx* ctx, uint32_t n, uint32_t out, uint32_t world, uint32_t rank, uint32_t group_rows, uint32_t sync, hb_kernel** res) {
    if (!ctx || !res) return hb::fail(ctx, HB_INVALID, "hb_tp_sum_stream_get: bad argument");
    try {
        hb::bind(ctx);
        *res = nullptr;
        if (n == 0 || n % 8 != 0) return hb::fail(ctx, HB_UNSUPPORTED, "tp_sum_stream: n a positive multiple of 8");
        if (out != HB_OUT_BF16 && out != HB_OUT_RESIDUAL) return hb::fail(ctx, HB_UNSUPPORTED, "tp_sum_stream: output Bf16 or Residual");
        if (world < 2 || world > (uint32_t)hb::TP_MAX_WORLD || rank >= world) return hb::fail(ctx, HB_UNSUPPORTED, "tp_sum_stream: 2..8 ranks");
        if (group_rows == 0 || group_rows > 256 || group_rows % (32 * world) != 0)
            return hb::fail(ctx, HB_UNSUPPORTED, "tp_sum_stream: a group of a multiple of 32 * world rows, at most 256");
        auto k = std::make_unique<hb::TpSumStream>();
        k->n = n;
        k->out = out;
        k->world = world;
        k->rank = rank;
        k->group_rows = group_rows;
        if (sync > 2) return hb::fail(ctx, HB_INVALID, "tp_sum_stream: sync is 0, 1 or 2");
        k->sync = sync;
        k->kind = 16;
        k->nargs = 5;
        k->name = "tp_sum_stream_" + std::to_string(n) + "_" + hb::out_tag(out) + "_g" + std::to_string(group_rows) + "_r" + std::to_string(rank) + "of" + std::to_string(world) +
                  (sync == 1 ? "" : sync == 2 ? "_barriers" : "_hostordered");
        *res = hb::intern(ctx, std::move(k));
        return HB_OK;
    } catch (const std::exception& e) {
        return hb::fail(ctx, HB_BACKEND, e.what());
    }
}

extern "C" int hb_tp_sum_sync_get(hb_ctx* ctx, uint32_t n, uint32_t out, uint32_t world, uint32_t rank, hb_kernel** res) {
    if (!ctx || !res) return hb::fail(ctx, HB_INVALID, "hb_tp_sum_sync_get: bad argument");
    try {
        hb::bind(ctx);
        return hb::make_tp_reduce(ctx, n, out, world, rank, true, res, true);
    } catch (const std::exception& e) {
        return hb::fail(ctx, HB_BACKEND, e.what());
    }
}

extern "C" int hb_tp_sum_get(hb_ctx* ctx, uint32_t n, uint32_t out, uint32_t world, uint32_t rank, hb_kernel** res) {
    if (!ctx || !res) return hb::fail(ctx, HB_INVALID, "hb_tp_sum_get: bad argument");
    try {
        hb::bind(ctx);
        return hb::make_tp_reduce(ctx, n, out, world, rank, true, res);
    } catch (const std::exception& e) {
        return hb::fail(ctx, HB_BACKEND, e.what());
    }
}
