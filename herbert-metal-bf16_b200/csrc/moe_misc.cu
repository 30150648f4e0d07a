// The small kernels around the GEMMs: SwiGLU over rows, the MoE route (softmax + top-k),
// the row gather and the weighted combine.
// All are memory- or latency-bound CUDA-core kernels; results are bit-exact restatements
// of the reference's arithmetic (citations per kernel).
#include <algorithm>

#include "hb_internal.hpp"
#include "tc05.cuh"

namespace hb {

// ------------------------------------------------------------- swiglu_rows
// h[r][c] = bf16(g*sigmoid(g)*u), g = gu[r][c], u = gu[r][n + c]
// (reference src/metal/prefill.rs:2790-2818; src/metal/qwen_kernels.rs:2087 over expert rows).
__global__ void swiglu_rows_kernel(const uint16_t* __restrict__ gu, uint16_t* __restrict__ h, uint32_t m, uint32_t n, uint32_t vec) {
    griddep_wait();
    griddep_launch_dependents();
    if (vec) {
        const uint32_t n8 = n / 8;
        const size_t total = (size_t)m * n8;
        for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
            const uint32_t r = (uint32_t)(i / n8), c = (uint32_t)(i % n8);
            const uint4 g = *reinterpret_cast<const uint4*>(gu + (size_t)r * 2 * n + c * 8);
            const uint4 u = *reinterpret_cast<const uint4*>(gu + (size_t)r * 2 * n + n + c * 8);
            const uint32_t gw[4] = {g.x, g.y, g.z, g.w}, uw[4] = {u.x, u.y, u.z, u.w};
            uint32_t o[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint32_t lo = swiglu_bf16(bf16_to_f32(gw[j] & 0xffffu), bf16_to_f32(uw[j] & 0xffffu));
                const uint32_t hi = swiglu_bf16(bf16_to_f32(gw[j] >> 16), bf16_to_f32(uw[j] >> 16));
                o[j] = lo | (hi << 16);
            }
            *reinterpret_cast<uint4*>(h + (size_t)r * n + c * 8) = make_uint4(o[0], o[1], o[2], o[3]);
        }
    } else {
        const size_t total = (size_t)m * n;
        for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
            const uint32_t r = (uint32_t)(i / n), c = (uint32_t)(i % n);
            h[i] = (uint16_t)swiglu_bf16(bf16_to_f32(gu[(size_t)r * 2 * n + c]), bf16_to_f32(gu[(size_t)r * 2 * n + n + c]));
        }
    }
}

// ------------------------------------------------------------------- route
// One block of `experts` threads per row (reference src/metal/qwen_kernels.rs:1802-1878):
// softmax of the bf16 scores in f32 (max, exp, sum = 32-lane butterfly sums folded warp by
// warp in order, divide), top_k rounds of "largest value, lowest index on a tie", weights
// p/sum(p_top) with the sum taken best-first, rounded to bf16, written in increasing expert order.
// One warp per row: lane l holds experts l, 32 + l, 64 + l, ... so the butterfly over element g of every lane is
// the 32-lane sum of experts [32g, 32g + 32) - the same partial sums, folded in the same order, as a block of
// `experts` threads would make.
constexpr int ROUTE_WARPS = 8;
template <int MAXK, int NPL>  // NPL: values per lane = experts / 32 rounded up to a power of two
__global__ void __launch_bounds__(ROUTE_WARPS * 32) route_topk_kernel(const uint16_t* __restrict__ scores, uint32_t* __restrict__ route, uint32_t rows,
                                                                      uint32_t experts, uint32_t top_k) {
    __shared__ float vals_s[ROUTE_WARPS][MAXK];
    __shared__ uint32_t chosen_s[ROUTE_WARPS][MAXK];
    griddep_wait();  // (an overlapped launch: the scores may come from the kernel before this one)
    griddep_launch_dependents();
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t row = blockIdx.x * ROUTE_WARPS + warp;
    if (row >= rows) return;
    const uint32_t npl = experts >> 5;  // values per lane in use, <= NPL
    float* vals = vals_s[warp];
    uint32_t* chosen = chosen_s[warp];
    float p[NPL];
    float mx = -3.4e38f;
#pragma unroll
    for (int g = 0; g < NPL; ++g) {
        p[g] = 0.f;
        if ((uint32_t)g < npl) {
            p[g] = bf16_to_f32(scores[(size_t)row * experts + 32 * g + lane]);
            mx = fmaxf(mx, p[g]);
        }
    }
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
    float sum = 0.f;
#pragma unroll
    for (int g = 0; g < NPL; ++g) {
        if ((uint32_t)g < npl) {
            p[g] = exp_f32(__fsub_rn(p[g], mx));
            float part = p[g];
#pragma unroll
            for (int off = 16; off >= 1; off >>= 1) part = __fadd_rn(part, __shfl_xor_sync(0xffffffffu, part, off));
            sum = g == 0 ? part : __fadd_rn(sum, part);
        }
    }
#pragma unroll
    for (int g = 0; g < NPL; ++g)
        if ((uint32_t)g < npl) p[g] = __fdiv_rn(p[g], sum);
    for (uint32_t t = 0; t < top_k; ++t) {
        float bv = p[0];
        uint32_t bi = lane;
#pragma unroll
        for (int g = 1; g < NPL; ++g)
            if ((uint32_t)g < npl && p[g] > bv) { bv = p[g]; bi = 32 * g + lane; }  // strict >: the lowest index of a lane's ties
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, off);
            const uint32_t oi = __shfl_xor_sync(0xffffffffu, bi, off);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        if (lane == 0) { vals[t] = bv; chosen[t] = bi; }
        if ((bi & 31u) == lane) {
#pragma unroll
            for (int g = 0; g < NPL; ++g)
                if ((uint32_t)g == (bi >> 5)) p[g] = -1.0f;
        }
    }
    __syncwarp();
    for (uint32_t e = lane; e < top_k; e += 32) {
        float total = 0.0f;
        for (uint32_t j = 0; j < top_k; ++j) total = __fadd_rn(total, vals[j]);
        const float w = round_bf16(__fdiv_rn(vals[e], total));
        uint32_t rank = 0;
        for (uint32_t j = 0; j < top_k; ++j)
            if (j != e && chosen[j] < chosen[e]) rank++;
        uint32_t* r = route + (size_t)row * 2 * top_k;
        r[rank] = chosen[e];
        r[top_k + rank] = __float_as_uint(w);
    }
}

// -------------------------------------------------------------- moe_gather
// XS[p] = X[list[p] / top_k] (reference src/metal/prefill.rs:579).
__global__ void moe_gather_kernel(const uint4* __restrict__ x, const uint32_t* __restrict__ list, uint4* __restrict__ xs, uint32_t pairs, uint32_t h8, uint32_t top_k) {
    const size_t total = (size_t)pairs * h8;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const uint32_t p = (uint32_t)(i / h8), c = (uint32_t)(i % h8);
        xs[i] = x[(size_t)(list[p] / top_k) * h8 + c];
    }
}

// ---------------------------------------------------------- experts_matvec
// The projections of the top_k routed experts of every row, one matvec per (row, slot) (reference
// src/metal/qwen_kernels.rs:1880-1990; the engine's moe.grouped = 0 and its decode step): slot s of row r (g = r * top_k
// + s) multiplies the rows of expert route[r][s] in W ([experts * n][k]) with the input at r * x_row + s * x_stride
// (x_stride 0: every slot of a row the same input) and writes y[g * n ..] in bf16. The arithmetic is the matvec's: 32
// lanes stride K by chunks of 8, an f32 FMA chain per lane, the xor-butterfly sum, one rounding. A warp per R rows of W.
template <int R>
__global__ void __launch_bounds__(256) experts_matvec_kernel(const uint4* __restrict__ w, const uint4* __restrict__ x, uint16_t* __restrict__ y,
                                                             const uint32_t* __restrict__ route, uint32_t pairs, uint32_t n, uint32_t k8, uint32_t top_k,
                                                             uint32_t x_row8, uint32_t x_stride8) {
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t groups = (n + R - 1) / R;                 // row groups of one slot
    const size_t total = (size_t)pairs * groups;
    for (size_t item = (size_t)blockIdx.x * 8 + warp; item < total; item += (size_t)gridDim.x * 8) {
        const uint32_t g = (uint32_t)(item / groups), row0 = (uint32_t)(item % groups) * R;
        const uint32_t token = g / top_k, s_in = g % top_k;
        const uint32_t expert = route[(size_t)token * 2 * top_k + s_in];
        const uint4* xs = x + (size_t)token * x_row8 + (size_t)s_in * x_stride8;
        const uint4* base[R];
#pragma unroll
        for (int r = 0; r < R; ++r) base[r] = w + ((size_t)expert * n + min(row0 + r, n - 1)) * k8;  // rows past the end read the last row
        float acc[R];
#pragma unroll
        for (int r = 0; r < R; ++r) acc[r] = 0.f;
        for (uint32_t c = lane; c < k8; c += 32) {
            const uint4 xv = __ldg(xs + c);
            const uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const uint4 wv = __ldg(base[r] + c);
                const uint32_t ww[4] = {wv.x, wv.y, wv.z, wv.w};
                float a = acc[r];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    a = __fmaf_rn(__uint_as_float(ww[j] << 16), __uint_as_float(xw[j] << 16), a);
                    a = __fmaf_rn(__uint_as_float(ww[j] & 0xffff0000u), __uint_as_float(xw[j] & 0xffff0000u), a);
                }
                acc[r] = a;
            }
        }
#pragma unroll
        for (int r = 0; r < R; ++r) {
            float a = acc[r];
#pragma unroll
            for (int off = 16; off >= 1; off >>= 1) a += __shfl_xor_sync(0xffffffffu, a, off);
            if (lane == 0 && row0 + r < n) y[(size_t)g * n + row0 + r] = (uint16_t)f32_to_bf16(a);
        }
    }
}

// ------------------------------------------------------------- moe_combine
// out[r][i] over the slots in route order: acc = bf16(acc + bf16(y*w)) (reference
// src/metal/qwen_kernels.rs:2119-2161), or with F32SUM an f32 FMA chain rounded once.
template <bool F32SUM>
__global__ void moe_combine_kernel(const uint16_t* __restrict__ y, const uint32_t* __restrict__ route, uint16_t* __restrict__ out, uint32_t rows, uint32_t d,
                                   uint32_t top_k) {
    griddep_wait();
    griddep_launch_dependents();
    const uint32_t d8 = d / 8;
    const size_t total = (size_t)rows * d8;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const uint32_t row = (uint32_t)(i / d8), c = (uint32_t)(i % d8);
        float acc[8];        // F32SUM: the running sums
        uint32_t accp[4];    // otherwise: the running bf16 values, two per word
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = 0.f;
#pragma unroll
        for (int j = 0; j < 4; ++j) accp[j] = 0u;
        // slots in batches of eight: all of a batch's loads are issued before the first is used (the slot chain
        // itself is sequential by contract, the loads need not be)
        for (uint32_t s0 = 0; s0 < top_k; s0 += 8) {
            uint4 v[8];
            float w[8];
#pragma unroll
            for (int b = 0; b < 8; ++b) {
                const uint32_t s = min(s0 + b, top_k - 1);
                v[b] = __ldcs(reinterpret_cast<const uint4*>(y + ((size_t)row * top_k + s) * d + c * 8));
                w[b] = __uint_as_float(route[(size_t)row * 2 * top_k + top_k + s]);
            }
#pragma unroll
            for (int b = 0; b < 8; ++b) {
                if (s0 + b < top_k) {
                    const uint32_t vw[4] = {v[b].x, v[b].y, v[b].z, v[b].w};
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const float lo = __uint_as_float(vw[j] << 16), hi = __uint_as_float(vw[j] & 0xffff0000u);
                        if (F32SUM) {
                            acc[2 * j] = __fmaf_rn(lo, w[b], acc[2 * j]);
                            acc[2 * j + 1] = __fmaf_rn(hi, w[b], acc[2 * j + 1]);
                        } else {
                            // bf16(y * w), then bf16(acc + that): both roundings by the paired hardware conversion
                            const uint32_t t = f32x2_to_bf16x2(__fmul_rn(lo, w[b]), __fmul_rn(hi, w[b]));
                            accp[j] = f32x2_to_bf16x2(__fadd_rn(__uint_as_float(accp[j] << 16), __uint_as_float(t << 16)),
                                                      __fadd_rn(__uint_as_float(accp[j] & 0xffff0000u), __uint_as_float(t & 0xffff0000u)));
                        }
                    }
                }
            }
        }
        uint32_t o[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) o[j] = F32SUM ? f32x2_to_bf16x2(acc[2 * j], acc[2 * j + 1]) : accp[j];
        *reinterpret_cast<uint4*>(out + (size_t)row * d + c * 8) = make_uint4(o[0], o[1], o[2], o[3]);
    }
}

// ------------------------------------------------------------------ host side

namespace {

inline uint32_t grid_for(hb_ctx* ctx, size_t items, int threads) {
    size_t blocks = (items + threads - 1) / threads;
    return (uint32_t)std::max<size_t>(1, std::min<size_t>(blocks, (size_t)ctx->sm_count * 16));
}

struct SwigluRows : hb_kernel {
    uint32_t n = 0;
    int launch(hb_ctx* ctx, const hb_range* a, int na, uint32_t m) override {
        if (na != 2) return fail(ctx, HB_INVALID, name + ": bindings are gate_up, h");
        if (m == 0) return fail(ctx, HB_INVALID, name + ": m = 0");
        if (!range_ok(a[0], (size_t)m * 2 * n * 2) || !range_ok(a[1], (size_t)m * n * 2)) return fail(ctx, HB_INVALID, name + ": a bound range is too small");
        const uint32_t vec = (n % 8 == 0 && ((reinterpret_cast<uintptr_t>(a[0].ptr) | reinterpret_cast<uintptr_t>(a[1].ptr)) & 15u) == 0) ? 1u : 0u;
        const size_t items = vec ? (size_t)m * (n / 8) : (size_t)m * n;
        HB_CUDA(ctx, launch_kernel(ctx, true, swiglu_rows_kernel, dim3(grid_for(ctx, items, 256)), dim3(256), 0, static_cast<const uint16_t*>(a[0].ptr), static_cast<uint16_t*>(a[1].ptr), m, n, vec));
        HB_CUDA(ctx, cudaGetLastError());
        ctx->launches++;
        return HB_OK;
    }
};

struct Route : hb_kernel {
    uint32_t experts = 0, top_k = 0;
    int launch(hb_ctx* ctx, const hb_range* a, int na, uint32_t m) override {
        if (na != 2) return fail(ctx, HB_INVALID, name + ": bindings are scores, route");
        if (m == 0) return fail(ctx, HB_INVALID, name + ": m = 0");
        if (!range_ok(a[0], (size_t)m * experts * 2) || !range_ok(a[1], (size_t)m * 2 * top_k * 4)) return fail(ctx, HB_INVALID, name + ": a bound range is too small");
        const uint32_t grid = (m + ROUTE_WARPS - 1) / ROUTE_WARPS, npl = experts / 32;
        const uint16_t* sc = static_cast<const uint16_t*>(a[0].ptr);
        uint32_t* rt = static_cast<uint32_t*>(a[1].ptr);
        if (npl <= 1) HB_CUDA(ctx, launch_kernel(ctx, true, route_topk_kernel<64, 1>, dim3(grid), dim3(ROUTE_WARPS * 32), 0, sc, rt, m, experts, top_k));
        else if (npl <= 2) HB_CUDA(ctx, launch_kernel(ctx, true, route_topk_kernel<64, 2>, dim3(grid), dim3(ROUTE_WARPS * 32), 0, sc, rt, m, experts, top_k));
        else if (npl <= 4) HB_CUDA(ctx, launch_kernel(ctx, true, route_topk_kernel<64, 4>, dim3(grid), dim3(ROUTE_WARPS * 32), 0, sc, rt, m, experts, top_k));
        else if (npl <= 8) HB_CUDA(ctx, launch_kernel(ctx, true, route_topk_kernel<64, 8>, dim3(grid), dim3(ROUTE_WARPS * 32), 0, sc, rt, m, experts, top_k));
        else if (npl <= 16) HB_CUDA(ctx, launch_kernel(ctx, true, route_topk_kernel<64, 16>, dim3(grid), dim3(ROUTE_WARPS * 32), 0, sc, rt, m, experts, top_k));
        else HB_CUDA(ctx, launch_kernel(ctx, true, route_topk_kernel<64, 32>, dim3(grid), dim3(ROUTE_WARPS * 32), 0, sc, rt, m, experts, top_k));
        HB_CUDA(ctx, cudaGetLastError());
        ctx->launches++;
        return HB_OK;
    }
};

struct MoeGather : hb_kernel {
    uint32_t h = 0, top_k = 0;
    int launch(hb_ctx* ctx, const hb_range* a, int na, uint32_t m) override {
        if (na != 3) return fail(ctx, HB_INVALID, name + ": bindings are X, list, XS");
        if (m == 0) return fail(ctx, HB_INVALID, name + ": m = 0");
        const uint32_t pairs = m * top_k;
        if (!range_ok(a[0], (size_t)m * h * 2) || !range_ok(a[1], (size_t)pairs * 4) || !range_ok(a[2], (size_t)pairs * h * 2))
            return fail(ctx, HB_INVALID, name + ": a bound range is too small");
        if ((reinterpret_cast<uintptr_t>(a[0].ptr) | reinterpret_cast<uintptr_t>(a[2].ptr)) & 15u) return fail(ctx, HB_INVALID, name + ": X and XS must be 16-byte aligned");
        moe_gather_kernel<<<grid_for(ctx, (size_t)pairs * (h / 8), 256), 256, 0, ctx->stream>>>(static_cast<const uint4*>(a[0].ptr), static_cast<const uint32_t*>(a[1].ptr),
                                                                                                 static_cast<uint4*>(a[2].ptr), pairs, h / 8, top_k);
        HB_CUDA(ctx, cudaGetLastError());
        ctx->launches++;
        return HB_OK;
    }
};

struct ExpertsMatvec : hb_kernel {
    uint32_t k = 0, n = 0, top_k = 0, experts = 0, x_row = 0, x_stride = 0, rows = 0;
    int launch(hb_ctx* ctx, const hb_range* a, int na, uint32_t m) override {
        if (na != 4) return fail(ctx, HB_INVALID, name + ": bindings are W, x, y, route");
        if (m == 0) return fail(ctx, HB_INVALID, name + ": m = 0");
        const uint32_t pairs = m * top_k;
        const size_t xbytes = ((size_t)(m - 1) * x_row + (size_t)(top_k - 1) * x_stride + k) * 2;
        if (!range_ok(a[0], (size_t)experts * n * k * 2) || !range_ok(a[1], xbytes) || !range_ok(a[2], (size_t)pairs * n * 2) || !range_ok(a[3], (size_t)m * 2 * top_k * 4))
            return fail(ctx, HB_INVALID, name + ": a bound range is too small");
        if ((reinterpret_cast<uintptr_t>(a[0].ptr) | reinterpret_cast<uintptr_t>(a[1].ptr)) & 15u) return fail(ctx, HB_INVALID, name + ": W and x must be 16-byte aligned");
        const size_t items = (size_t)pairs * ((n + rows - 1) / rows);
        const uint32_t grid = (uint32_t)std::max<size_t>(1, std::min<size_t>((items + 7) / 8, (size_t)ctx->sm_count * 16));
        auto go = [&](auto fn) {
            fn<<<grid, 256, 0, ctx->stream>>>(static_cast<const uint4*>(a[0].ptr), static_cast<const uint4*>(a[1].ptr), static_cast<uint16_t*>(a[2].ptr),
                                              static_cast<const uint32_t*>(a[3].ptr), pairs, n, k / 8, top_k, x_row / 8, x_stride / 8);
        };
        switch (rows) {
            case 1: go(experts_matvec_kernel<1>); break;
            case 2: go(experts_matvec_kernel<2>); break;
            case 4: go(experts_matvec_kernel<4>); break;
            default: go(experts_matvec_kernel<8>); break;
        }
        HB_CUDA(ctx, cudaGetLastError());
        ctx->launches++;
        return HB_OK;
    }
};

struct MoeCombine : hb_kernel {
    uint32_t d = 0, top_k = 0, f32_sum = 0;
    int launch(hb_ctx* ctx, const hb_range* a, int na, uint32_t m) override {
        if (na != 3) return fail(ctx, HB_INVALID, name + ": bindings are y, route, out");
        if (m == 0) return fail(ctx, HB_INVALID, name + ": m = 0");
        if (!range_ok(a[0], (size_t)m * top_k * d * 2) || !range_ok(a[1], (size_t)m * 2 * top_k * 4) || !range_ok(a[2], (size_t)m * d * 2))
            return fail(ctx, HB_INVALID, name + ": a bound range is too small");
        if ((reinterpret_cast<uintptr_t>(a[0].ptr) | reinterpret_cast<uintptr_t>(a[2].ptr)) & 15u) return fail(ctx, HB_INVALID, name + ": y and out must be 16-byte aligned");
        const uint32_t grid = grid_for(ctx, (size_t)m * (d / 8), 256);
        HB_CUDA(ctx, launch_kernel(ctx, true, f32_sum ? moe_combine_kernel<true> : moe_combine_kernel<false>, dim3(grid), dim3(256), 0, static_cast<const uint16_t*>(a[0].ptr),
                                   static_cast<const uint32_t*>(a[1].ptr), static_cast<uint16_t*>(a[2].ptr), m, d, top_k));
        ctx->launches++;
        return HB_OK;
    }
};

}  // namespace

int make_swiglu_rows(hb_ctx* ctx, uint32_t n, hb_kernel** out) {
    *out = nullptr;
    if (n == 0) return fail(ctx, HB_INVALID, "swiglu_rows: n = 0");
    auto k = std::make_unique<SwigluRows>();
    k->n = n;
    k->kind = 3;
    k->nargs = 2;
    k->name = "swiglu_rows_" + std::to_string(n);
    *out = intern(ctx, std::move(k));
    return HB_OK;
}

int make_route(hb_ctx* ctx, uint32_t experts, uint32_t top_k, hb_kernel** out) {
    *out = nullptr;
    // the reference's own bound: experts a multiple of the simdgroup, <= 1024 (qwen_kernels.rs:1803)
    if (experts == 0 || experts % 32 != 0 || experts > 1024 || top_k < 1 || top_k > experts || top_k > 64)
        return fail(ctx, HB_UNSUPPORTED, "route: experts a multiple of 32 up to 1024, 1 <= top_k <= min(experts, 64)");
    auto k = std::make_unique<Route>();
    k->experts = experts;
    k->top_k = top_k;
    k->kind = 4;
    k->nargs = 2;
    k->name = "route_qwen_" + std::to_string(experts) + "_k" + std::to_string(top_k);
    *out = intern(ctx, std::move(k));
    return HB_OK;
}

int make_moe_gather(hb_ctx* ctx, uint32_t h, uint32_t top_k, hb_kernel** out) {
    *out = nullptr;
    if (h == 0 || h % 8 != 0 || top_k == 0) return fail(ctx, HB_UNSUPPORTED, "moe_gather: h a positive multiple of 8, top_k positive");
    auto k = std::make_unique<MoeGather>();
    k->h = h;
    k->top_k = top_k;
    k->kind = 6;
    k->nargs = 3;
    k->name = "moe_gather_" + std::to_string(h) + "_k" + std::to_string(top_k);
    *out = intern(ctx, std::move(k));
    return HB_OK;
}

int make_experts_matvec(hb_ctx* ctx, uint32_t k, uint32_t n, uint32_t top_k, uint32_t experts, uint32_t x_row, uint32_t x_stride, uint32_t rows, hb_kernel** out) {
    *out = nullptr;
    if (k == 0 || n == 0 || top_k == 0 || experts == 0) return fail(ctx, HB_INVALID, "experts_matvec: k, n, top_k and experts must be positive");
    if (k % 8 != 0 || x_row % 8 != 0 || x_stride % 8 != 0)  // the reference's own assertion (qwen_kernels.rs:1887)
        return fail(ctx, HB_UNSUPPORTED, "experts_matvec: K = " + std::to_string(k) + ", x row " + std::to_string(x_row) + ", x stride " + std::to_string(x_stride) + ": not multiples of 8");
    if (rows == 0) rows = 2;
    if (rows != 1 && rows != 2 && rows != 4 && rows != 8) return fail(ctx, HB_UNSUPPORTED, "experts_matvec: rows per warp must be 1, 2, 4 or 8");
    auto km = std::make_unique<ExpertsMatvec>();
    km->k = k;
    km->n = n;
    km->top_k = top_k;
    km->experts = experts;
    km->x_row = x_row;
    km->x_stride = x_stride;
    km->rows = rows;
    km->kind = 19;
    km->nargs = 4;
    km->name = "experts_matvec_" + std::to_string(k) + "x" + std::to_string(n) + "_k" + std::to_string(top_k) + "_e" + std::to_string(experts) + "_x" + std::to_string(x_row) + "_" +
               std::to_string(x_stride) + "_r" + std::to_string(rows);
    *out = intern(ctx, std::move(km));
    return HB_OK;
}

int make_moe_combine(hb_ctx* ctx, uint32_t d, uint32_t top_k, uint32_t f32_sum, hb_kernel** out) {
    *out = nullptr;
    if (d == 0 || d % 8 != 0 || top_k == 0) return fail(ctx, HB_UNSUPPORTED, "moe_combine: d a positive multiple of 8, top_k positive");
    auto k = std::make_unique<MoeCombine>();
    k->d = d;
    k->top_k = top_k;
    k->f32_sum = f32_sum;
    k->kind = 7;
    k->nargs = 3;
    k->name = "moe_combine_" + std::to_string(d) + "_k" + std::to_string(top_k) + (f32_sum ? "_f32" : "");
    *out = intern(ctx, std::move(k));
    return HB_OK;
}

}  // namespace hb
