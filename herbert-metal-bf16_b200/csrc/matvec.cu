// Decode matvec y[r][n] = out(W[n][k] . x[r][k]) for 1..8 activation rows.
//
// Counterpart of the reference's matvec / matvec_split (src/metal/kernels.rs:146-214,
// :502-981). HBM-bound: W is read once with 128-bit non-caching loads, every lane keeps
// an f32 FMA chain per (W row, activation row), a warp reduces R consecutive W rows
// sharing the x loads (the reference's `rows` axis), sums cross the warp by an xor
// butterfly and, with `split`, the K range is cut across the warps of a block and the
// partial sums folded in a fixed order (kernels.rs:916-928). CUDA cores only.
#include <algorithm>

#include "hb_internal.hpp"
#include "tc05.cuh"

namespace hb {

struct MatvecParams {
    const uint4* w;
    const uint4* x;
    void* y;
    uint32_t n;        // rows of W
    uint32_t n_out;    // outputs per activation row (n, or n/2 for SWIGLU)
    uint32_t k8;       // 16-byte chunks per row
    uint32_t m;        // activation rows in use
    uint32_t split;    // warps sharing one row group
    uint32_t groups;   // row groups in all
    // fused argmax over the outputs (Out::Bf16 only): see argmax_fold in tc05.cuh
    unsigned long long* keys;  // [rows][ARGMAX_SLOTS]
    uint32_t* counter;
    uint32_t* index;           // [rows]
    uint32_t store_y;          // 0: the index only
};

__device__ __forceinline__ uint4 ldg_stream(const uint4* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.L2::128B.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

constexpr int MV_THREADS = 256;
constexpr int MV_WARPS = MV_THREADS / 32;

template <int M, int R, int OUT, bool ARGMAX = false>
__global__ void __launch_bounds__(MV_THREADS) matvec_kernel(const MatvecParams p) {
    __shared__ float part[MV_WARPS][R * M];
    __shared__ unsigned long long best_s[ARGMAX ? MV_WARPS : 1][M];
    unsigned long long best[M];
#pragma unroll
    for (int i = 0; i < M; ++i) best[i] = 0ull;
    griddep_launch_dependents();
    griddep_wait();  // x comes from the kernel before this one
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t split = p.split;
    const uint32_t slots = MV_WARPS / split;  // row groups a block works on at a time
    const uint32_t slot = warp / split, piece = warp % split;
    const uint32_t per = (p.k8 + split - 1) / split;
    const uint32_t c_begin = piece * per, c_end = min(p.k8, c_begin + per);

    for (uint32_t g0 = blockIdx.x * slots; g0 < p.groups; g0 += gridDim.x * slots) {
        const uint32_t group = g0 + slot;
        const bool live = group < p.groups;
        float acc[R][M];
#pragma unroll
        for (int r = 0; r < R; ++r)
#pragma unroll
            for (int i = 0; i < M; ++i) acc[r][i] = 0.f;
        uint32_t rows[R];
        if (live) {
            // The W rows of this group. SWIGLU: R/2 gate rows and their up rows (kernels.rs:934-944).
#pragma unroll
            for (int r = 0; r < R; ++r) {
                uint32_t row;
                if constexpr (OUT == HB_OUT_SWIGLU) row = (r < R / 2) ? group * (R / 2) + r : p.n_out + group * (R / 2) + (r - R / 2);
                else row = group * R + r;
                rows[r] = min(row, p.n - 1);  // rows past the end read the last row and are not written
            }
            for (uint32_t c = c_begin + lane; c < c_end; c += 32) {
                uint4 wv[R];
#pragma unroll
                for (int r = 0; r < R; ++r) wv[r] = ldg_stream(p.w + (size_t)rows[r] * p.k8 + c);
#pragma unroll
                for (int i = 0; i < M; ++i) {
                    if ((uint32_t)i < p.m) {
                        const uint4 xv = __ldg(p.x + (size_t)i * p.k8 + c);
                        const uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
                        for (int r = 0; r < R; ++r) {
                            const uint32_t ww[4] = {wv[r].x, wv[r].y, wv[r].z, wv[r].w};
                            float a = acc[r][i];
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                a = __fmaf_rn(__uint_as_float(ww[j] << 16), __uint_as_float(xw[j] << 16), a);
                                a = __fmaf_rn(__uint_as_float(ww[j] & 0xffff0000u), __uint_as_float(xw[j] & 0xffff0000u), a);
                            }
                            acc[r][i] = a;
                        }
                    }
                }
            }
#pragma unroll
            for (int r = 0; r < R; ++r)
#pragma unroll
                for (int i = 0; i < M; ++i) {
                    float a = acc[r][i];
#pragma unroll
                    for (int off = 16; off >= 1; off >>= 1) a += __shfl_xor_sync(0xffffffffu, a, off);
                    acc[r][i] = a;
                }
        }
        if (split > 1) {
            if (live && lane == 0) {
#pragma unroll
                for (int r = 0; r < R; ++r)
#pragma unroll
                    for (int i = 0; i < M; ++i) part[warp][r * M + i] = acc[r][i];
            }
            __syncthreads();
            if (live && piece == 0 && lane == 0) {
#pragma unroll
                for (int r = 0; r < R; ++r)
#pragma unroll
                    for (int i = 0; i < M; ++i) {
                        float a = acc[r][i];
                        for (uint32_t s = 1; s < split; ++s) a += part[warp + s][r * M + i];
                        acc[r][i] = a;
                    }
            }
        }
        if (live && piece == 0 && lane == 0) {
            if constexpr (OUT == HB_OUT_SWIGLU) {
#pragma unroll
                for (int r = 0; r < R / 2; ++r) {
                    const uint32_t col = group * (R / 2) + r;
                    if (col < p.n_out) {
#pragma unroll
                        for (int i = 0; i < M; ++i)
                            if ((uint32_t)i < p.m)
                                reinterpret_cast<uint16_t*>(p.y)[(size_t)i * p.n_out + col] =
                                    (uint16_t)swiglu_bf16(round_bf16(acc[r][i]), round_bf16(acc[r + R / 2][i]));
                    }
                }
            } else {
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    const uint32_t col = group * R + r;
                    if (col < p.n) {
#pragma unroll
                        for (int i = 0; i < M; ++i) {
                            if ((uint32_t)i < p.m) {
                                const size_t at = (size_t)i * p.n + col;
                                if constexpr (OUT == HB_OUT_F32) reinterpret_cast<float*>(p.y)[at] = acc[r][i];
                                else if constexpr (OUT == HB_OUT_BF16) {
                                    const uint32_t h = f32_to_bf16(acc[r][i]);
                                    if (!ARGMAX || p.store_y) reinterpret_cast<uint16_t*>(p.y)[at] = (uint16_t)h;
                                    if constexpr (ARGMAX) {
                                        const unsigned long long key = argmax_key(h, col);
                                        best[i] = key > best[i] ? key : best[i];
                                    }
                                } else {
                                    uint16_t* y = reinterpret_cast<uint16_t*>(p.y) + at;
                                    *y = (uint16_t)f32_to_bf16(__fadd_rn(bf16_to_f32(*y), round_bf16(acc[r][i])));
                                }
                            }
                        }
                    }
                }
            }
        }
        if (split > 1) __syncthreads();  // `part` is reused by the next group
    }
    if constexpr (ARGMAX) {
        // lane 0 of every warp holds the best of the outputs it wrote; fold the block, then the grid
        if (lane == 0) {
#pragma unroll
            for (int i = 0; i < M; ++i) best_s[warp][i] = best[i];
        }
        __syncthreads();
        if (threadIdx.x < M) {
            unsigned long long b = best_s[0][threadIdx.x];
            for (int w = 1; w < MV_WARPS; ++w) b = best_s[w][threadIdx.x] > b ? best_s[w][threadIdx.x] : b;
            best_s[0][threadIdx.x] = b;
        }
        __syncthreads();
        argmax_fold(best_s[0], p.m, p.keys, p.counter, p.index, gridDim.x);
    }
}

namespace {

typedef void (*mv_fn)(const MatvecParams);

template <int M, int R>
mv_fn mv_out(uint32_t out, bool argmax) {
    if (argmax) return out == HB_OUT_BF16 ? matvec_kernel<M, R, HB_OUT_BF16, true> : nullptr;
    switch (out) {
        case HB_OUT_BF16: return matvec_kernel<M, R, HB_OUT_BF16>;
        case HB_OUT_F32: return matvec_kernel<M, R, HB_OUT_F32>;
        case HB_OUT_RESIDUAL: return matvec_kernel<M, R, HB_OUT_RESIDUAL>;
        case HB_OUT_SWIGLU:
            if constexpr (R >= 2) return matvec_kernel<M, R, HB_OUT_SWIGLU>;
            else return nullptr;
    }
    return nullptr;
}
template <int M>
mv_fn mv_rows(uint32_t r, uint32_t out, bool argmax) {
    switch (r) {
        case 1: return mv_out<M, 1>(out, argmax);
        case 2: return mv_out<M, 2>(out, argmax);
        case 4: return mv_out<M, 4>(out, argmax);
        case 8: return mv_out<M, 8>(out, argmax);
    }
    return nullptr;
}
mv_fn mv_pick(uint32_t mcap, uint32_t r, uint32_t out, bool argmax) {
    switch (mcap) {
        case 1: return mv_rows<1>(r, out, argmax);
        case 2: return mv_rows<2>(r, out, argmax);
        case 4: return mv_rows<4>(r, out, argmax);
        case 8: return mv_rows<8>(r, out, argmax);
    }
    return nullptr;
}

struct Matvec : hb_kernel {
    hb_matvec_desc d{};
    mv_fn fn = nullptr;
    int blocks_per_sm = 1;

    unsigned long long* keys = nullptr;
    uint32_t* counter = nullptr;

    int launch(hb_ctx* ctx, const hb_range* a, int na, uint32_t m) override {
        if (na != (d.argmax ? 4 : 3)) return fail(ctx, HB_INVALID, name + (d.argmax ? ": bindings are W, x, y, index" : ": bindings are W, x, y"));
        if (m == 0 || m > d.rows_max) return fail(ctx, HB_INVALID, name + ": m outside 1.." + std::to_string(d.rows_max));
        if (d.argmax && !range_ok(a[3], (size_t)m * 4)) return fail(ctx, HB_INVALID, name + ": the index range is too small");
        const uint32_t n_out = d.out == HB_OUT_SWIGLU ? d.n / 2 : d.n;
        const size_t ybytes = (size_t)m * n_out * (d.out == HB_OUT_F32 ? 4 : 2);
        if (!range_ok(a[0], (size_t)d.n * d.k * 2) || !range_ok(a[1], (size_t)m * d.k * 2) || !range_ok(a[2], ybytes))
            return fail(ctx, HB_INVALID, name + ": a bound range is too small");
        if ((reinterpret_cast<uintptr_t>(a[0].ptr) | reinterpret_cast<uintptr_t>(a[1].ptr)) & 15u)
            return fail(ctx, HB_INVALID, name + ": W and x must be 16-byte aligned");
        MatvecParams p{};
        p.w = static_cast<const uint4*>(a[0].ptr);
        p.x = static_cast<const uint4*>(a[1].ptr);
        p.y = a[2].ptr;
        p.n = d.n;
        p.n_out = n_out;
        p.k8 = d.k / 8;
        p.m = m;
        p.split = d.split;
        p.keys = keys;
        p.counter = counter;
        p.index = d.argmax ? static_cast<uint32_t*>(a[3].ptr) : nullptr;
        p.store_y = d.argmax == 2 ? 0u : 1u;
        const uint32_t rows_per_group = d.out == HB_OUT_SWIGLU ? d.rows_per_warp / 2 : d.rows_per_warp;
        p.groups = (n_out + rows_per_group - 1) / rows_per_group;
        const uint32_t slots = MV_WARPS / d.split;
        uint32_t grid = (p.groups + slots - 1) / slots;
        if (d.persist) grid = std::min<uint32_t>(grid, (uint32_t)(ctx->sm_count * blocks_per_sm));
        HB_CUDA(ctx, launch_kernel(ctx, true, fn, dim3(grid), dim3(MV_THREADS), 0, p));
        ctx->launches++;
        return HB_OK;
    }
};

}  // namespace

int make_matvec_xs(hb_ctx* ctx, const hb_matvec_desc* d, hb_kernel** out);
int make_matvec_skinny(hb_ctx* ctx, const hb_matvec_desc* d, hb_kernel** out);

int make_matvec(hb_ctx* ctx, const hb_matvec_desc* d, hb_kernel** out) {
    *out = nullptr;
    if (d->k == 0 || d->n == 0) return fail(ctx, HB_INVALID, "matvec: k and n must be positive");
    if (d->k % 8 != 0) return fail(ctx, HB_UNSUPPORTED, "matvec: K = " + std::to_string(d->k) + " is not a multiple of 8");
    if (d->out > HB_OUT_SWIGLU) return fail(ctx, HB_INVALID, "matvec: unknown output mode");
    if (d->tensor_core) return make_matvec_skinny(ctx, d, out);
    if (d->x_stationary) return make_matvec_xs(ctx, d, out);
    if (d->rows_max < 1 || d->rows_max > 8) return fail(ctx, HB_UNSUPPORTED, "matvec: 1..8 activation rows");
    if (d->out > HB_OUT_SWIGLU) return fail(ctx, HB_INVALID, "matvec: unknown output mode");
    const uint32_t r = d->rows_per_warp ? d->rows_per_warp : 2;
    const uint32_t split = d->split ? d->split : 1;
    if (r != 1 && r != 2 && r != 4 && r != 8) return fail(ctx, HB_UNSUPPORTED, "matvec: rows_per_warp must be 1, 2, 4 or 8");
    if (split != 1 && split != 2 && split != 4) return fail(ctx, HB_UNSUPPORTED, "matvec: split must be 1, 2 or 4");
    if (d->out == HB_OUT_SWIGLU && (r < 2 || d->n % 2 != 0)) return fail(ctx, HB_UNSUPPORTED, "matvec: the SwiGLU form pairs gate and up rows (rows_per_warp >= 2, even n)");
    uint32_t mcap = 1;
    while (mcap < d->rows_max) mcap *= 2;
    if (d->argmax > 2) return fail(ctx, HB_INVALID, "matvec: argmax is 0, 1 (logits and index) or 2 (index only)");
    if (d->argmax && d->out != HB_OUT_BF16) return fail(ctx, HB_UNSUPPORTED, "matvec: the fused argmax is over bf16 outputs (Out::Bf16)");
    mv_fn fn = mv_pick(mcap, r, d->out, d->argmax != 0);
    if (!fn) return fail(ctx, HB_UNSUPPORTED, "matvec: form not built");
    auto k = std::make_unique<Matvec>();
    k->d = *d;
    k->d.rows_per_warp = r;
    k->d.split = split;
    k->d.rows_max = mcap;
    if (d->argmax) k->d.persist = 1;  // the fold at the end of a block costs a round trip: few long-lived blocks, not thousands
    k->fn = fn;
    k->kind = 2;
    k->nargs = d->argmax ? 4 : 3;
    char nm[160];
    snprintf(nm, sizeof nm, "matvec_%ux%u_%s_m%u_r%u%s%s%s", d->k, d->n, out_tag(d->out), mcap, r,
             split > 1 ? (std::string("_s") + std::to_string(split)).c_str() : "", k->d.persist ? "_p" : "",
             d->argmax == 1 ? "_argmax" : d->argmax == 2 ? "_argmaxonly" : "");
    k->name = nm;
    if (hb_kernel* have = find(ctx, k->name)) {
        *out = have;
        return HB_OK;
    }
    if (d->argmax) {
        void* pk = nullptr;
        int st = hb_alloc(ctx, (size_t)mcap * ARGMAX_SLOTS * 8 + 16, &pk);  // zeroed: the keys, then the counter
        if (st != HB_OK) return st;
        k->keys = static_cast<unsigned long long*>(pk);
        k->counter = reinterpret_cast<uint32_t*>(k->keys + (size_t)mcap * ARGMAX_SLOTS);
    }
    int occ = 1;
    cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, reinterpret_cast<const void*>(fn), MV_THREADS, 0);
    k->blocks_per_sm = std::max(occ, 1);
    *out = intern(ctx, std::move(k));
    return HB_OK;
}

}  // namespace hb
