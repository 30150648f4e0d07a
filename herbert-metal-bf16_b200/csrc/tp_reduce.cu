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

#include "hb_internal.hpp"
#include "tc05.cuh"

namespace hb {

constexpr int TP_MAX_WORLD = 8;

struct TpParams {
    const float* staging;       // STAGED: this rank's f32 [world][rows_per][n], slot s from rank s
    const uint64_t* peers_acc;  // [world] f32 [m][n] on every rank
    const uint64_t* peers_y;    // [world] bf16 [m][n] on every rank
    uint32_t m, n8, world, rank, rows_per;
};

template <int OUT, bool STAGED>
__global__ void __launch_bounds__(256) tp_reduce_kernel(const TpParams p) {
    __shared__ uint64_t acc_s[TP_MAX_WORLD], y_s[TP_MAX_WORLD];
    if (threadIdx.x < p.world) {
        // STAGED: slot s of the local staging buffer, rebased so that the row index of the whole matrix applies
        acc_s[threadIdx.x] = STAGED ? reinterpret_cast<uint64_t>(p.staging + ((size_t)threadIdx.x * p.rows_per - (size_t)p.rank * p.rows_per) * p.n8 * 8)
                                    : p.peers_acc[threadIdx.x];
        y_s[threadIdx.x] = p.peers_y[threadIdx.x];
    }
    __syncthreads();
    const uint32_t r0 = p.rank * p.rows_per, r1 = min(p.m, r0 + p.rows_per);
    if (r0 >= r1) return;
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
}

namespace {
struct TpReduce : hb_kernel {
    uint32_t n = 0, out = 0, world = 0, rank = 0;
    bool staged = false;
    int launch(hb_ctx* ctx, const hb_range* a, int na, uint32_t m) override {
        if (na != 2) return fail(ctx, HB_INVALID, name + (staged ? ": bindings are staging, peers_y" : ": bindings are peers_acc, peers_y (device arrays of one address per rank)"));
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
        const size_t units = (size_t)p.rows_per * p.n8;
        const uint32_t grid = (uint32_t)std::max<size_t>(1, std::min<size_t>((units + 255) / 256, (size_t)ctx->sm_count * 8));
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

int make_tp_reduce(hb_ctx* ctx, uint32_t n, uint32_t out, uint32_t world, uint32_t rank, bool staged, hb_kernel** res) {
    *res = nullptr;
    if (n == 0 || n % 8 != 0) return fail(ctx, HB_UNSUPPORTED, "tp_reduce: n a positive multiple of 8");
    if (out != HB_OUT_BF16 && out != HB_OUT_RESIDUAL) return fail(ctx, HB_UNSUPPORTED, "tp_reduce: output Bf16 or Residual");
    if (world < 1 || world > TP_MAX_WORLD || rank >= world) return fail(ctx, HB_UNSUPPORTED, "tp_reduce: 1..8 ranks");
    auto k = std::make_unique<TpReduce>();
    k->n = n;
    k->out = out;
    k->world = world;
    k->rank = rank;
    k->staged = staged;
    k->kind = 14;
    k->nargs = 2;
    k->name = std::string(staged ? "tp_sum_" : "tp_reduce_") + std::to_string(n) + "_" + out_tag(out) + "_r" + std::to_string(rank) + "of" + std::to_string(world);
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

extern "C" int hb_tp_sum_get(hb_ctx* ctx, uint32_t n, uint32_t out, uint32_t world, uint32_t rank, hb_kernel** res) {
    if (!ctx || !res) return hb::fail(ctx, HB_INVALID, "hb_tp_sum_get: bad argument");
    try {
        hb::bind(ctx);
        return hb::make_tp_reduce(ctx, n, out, world, rank, true, res);
    } catch (const std::exception& e) {
        return hb::fail(ctx, HB_BACKEND, e.what());
    }
}
