// Decode matvec for 2..8 activation rows, activation-stationary form.
//
// With several activation rows the plain matvec kernel (matvec.cu) is bound by the integer pipe: it widens
// the activations from bf16 again for every W chunk. Here K is split across the 256 threads of a persistent
// block; a thread owns the same 16-byte chunk columns for every W row, so its slice of the activations is
// widened ONCE into f32 registers. The inner loop per W chunk is then one 128-bit load, eight widenings and
// 8 x M fused multiply-adds. A group of R rows of W is reduced at a time: the R x M partial sums of a thread
// cross the warp by a transposing butterfly (31 shuffles for 32 values instead of 5 per value), the eight warps
// fold through shared memory in warp order, and threads 0..R*M-1 apply the output mode and store. The next
// group's W chunks are already in flight while a group is reduced. Same contract as matvec.cu (reference
// src/metal/kernels.rs:146-234): f32 accumulation of exact products, one rounding to nearest even.
#include <algorithm>

#include "hb_internal.hpp"
#include "tc05.cuh"

namespace hb {

struct MatvecXsParams {
    const uint4* w;
    const uint4* x;
    void* y;
    uint32_t n, n_out, k8, m, groups;
};

constexpr int XS_THREADS = 256;
constexpr int XS_WARPS = XS_THREADS / 32;

__device__ __forceinline__ uint4 ldg_stream_xs(const uint4* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.L2::128B.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

__device__ __forceinline__ void widen8(const uint4& v, float (&f)[8]) {
    f[0] = __uint_as_float(v.x << 16); f[1] = __uint_as_float(v.x & 0xffff0000u);
    f[2] = __uint_as_float(v.y << 16); f[3] = __uint_as_float(v.y & 0xffff0000u);
    f[4] = __uint_as_float(v.z << 16); f[5] = __uint_as_float(v.z & 0xffff0000u);
    f[6] = __uint_as_float(v.w << 16); f[7] = __uint_as_float(v.w & 0xffff0000u);
}

// Two f32 in one 64-bit register, and the packed fused multiply-add of sm_100 (two FMAs per instruction): the
// accumulators are kept as (sum over even elements, sum over odd elements) and folded once at the end.
__device__ __forceinline__ uint64_t pack2(uint32_t lo, uint32_t hi) {
    uint64_t d;
    asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "r"(lo), "r"(hi));
    return d;
}
__device__ __forceinline__ uint64_t ffma2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ float fold2(uint64_t v) {
    uint32_t lo, hi;
    asm("mov.b64 {%0, %1}, %2;" : "=r"(lo), "=r"(hi) : "l"(v));
    return __fadd_rn(__uint_as_float(lo), __uint_as_float(hi));
}
// The four (even, odd) pairs of a 16-byte chunk of bf16, widened.
__device__ __forceinline__ void widen_pairs(const uint4& v, uint64_t (&p)[4]) {
    p[0] = pack2(v.x << 16, v.x & 0xffff0000u);
    p[1] = pack2(v.y << 16, v.y & 0xffff0000u);
    p[2] = pack2(v.z << 16, v.z & 0xffff0000u);
    p[3] = pack2(v.w << 16, v.w & 0xffff0000u);
}

// Sums V values per lane across the 32 lanes. On return v[g] (g < max(V/32, 1)) of lane l holds the warp sum of
// value index g*32 + l (V >= 32) or l >> (5 - log2 V) (V < 32, every lane of a run of 32/V lanes the same sum).
template <int V>
__device__ __forceinline__ void warp_transpose_sum(float (&v)[V], uint32_t lane) {
    if constexpr (V >= 32) {
#pragma unroll
        for (int g = 0; g < V / 32; ++g) {
#pragma unroll
            for (int off = 16; off >= 1; off >>= 1) {
                const bool upper = (lane & off) != 0;
#pragma unroll
                for (int i = 0; i < off; ++i) {
                    const float send = upper ? v[g * 32 + i] : v[g * 32 + i + off];
                    const float keep = upper ? v[g * 32 + i + off] : v[g * 32 + i];
                    v[g * 32 + i] = keep + __shfl_xor_sync(0xffffffffu, send, off);
                }
            }
            v[g] = v[g * 32];
        }
    } else {
        int cnt = V / 2;
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) {
            if (cnt >= 1) {
                const bool upper = (lane & off) != 0;
#pragma unroll
                for (int i = 0; i < V / 2; ++i) {
                    if (i < cnt) {
                        const float send = upper ? v[i] : v[i + cnt];
                        const float keep = upper ? v[i + cnt] : v[i];
                        v[i] = keep + __shfl_xor_sync(0xffffffffu, send, off);
                    }
                }
                cnt >>= 1;
            } else {
                v[0] += __shfl_xor_sync(0xffffffffu, v[0], off);
            }
        }
    }
}

template <int M, int R, int CPT, int OUT>
__global__ void __launch_bounds__(XS_THREADS, 1) matvec_xs_kernel(const MatvecXsParams p) {
    constexpr int V = R * M;
    constexpr int LOG2V = V >= 32 ? 5 : (V == 16 ? 4 : (V == 8 ? 3 : (V == 4 ? 2 : 1)));
    constexpr int RG = OUT == HB_OUT_SWIGLU ? R / 2 : R;  // output columns per group
    __shared__ float red[2][XS_WARPS][V];
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

    // this thread's slice of the activations, widened once
    uint64_t xf[M][CPT][4];
#pragma unroll
    for (int j = 0; j < CPT; ++j) {
        const uint32_t c = tid + j * XS_THREADS;
#pragma unroll
        for (int i = 0; i < M; ++i) {
            uint4 v = make_uint4(0, 0, 0, 0);
            if (c < p.k8 && (uint32_t)i < p.m) v = __ldg(p.x + (size_t)i * p.k8 + c);
            widen_pairs(v, xf[i][j]);
        }
    }

    auto row_of = [&](uint32_t group, int r) -> uint32_t {
        uint32_t row;
        if constexpr (OUT == HB_OUT_SWIGLU) row = (r < R / 2) ? group * (R / 2) + r : p.n_out + group * (R / 2) + (r - R / 2);
        else row = group * R + r;
        return min(row, p.n - 1);  // rows past the end read the last row and are not written
    };
    auto load_group = [&](uint32_t group, uint4 (&wv)[R][CPT]) {
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const uint4* base = p.w + (size_t)row_of(group, r) * p.k8;
#pragma unroll
            for (int j = 0; j < CPT; ++j) {
                const uint32_t c = tid + j * XS_THREADS;
                wv[r][j] = c < p.k8 ? ldg_stream_xs(base + c) : make_uint4(0, 0, 0, 0);
            }
        }
    };

    uint4 wv[R][CPT], wn[R][CPT];
    uint32_t buf = 0;
    if (blockIdx.x < p.groups) load_group(blockIdx.x, wv);
    for (uint32_t g = blockIdx.x; g < p.groups; g += gridDim.x) {
        const uint32_t next = g + gridDim.x;
        if (next < p.groups) load_group(next, wn);
        uint64_t acc2[V];
#pragma unroll
        for (int i = 0; i < V; ++i) acc2[i] = 0ull;
#pragma unroll
        for (int r = 0; r < R; ++r)
#pragma unroll
            for (int j = 0; j < CPT; ++j) {
                uint64_t wp[4];
                widen_pairs(wv[r][j], wp);
#pragma unroll
                for (int i = 0; i < M; ++i)
#pragma unroll
                    for (int e = 0; e < 4; ++e) acc2[r * M + i] = ffma2(wp[e], xf[i][j][e], acc2[r * M + i]);
            }
        float acc[V];
#pragma unroll
        for (int i = 0; i < V; ++i) acc[i] = fold2(acc2[i]);
        warp_transpose_sum<V>(acc, lane);
        if constexpr (V >= 32) {
#pragma unroll
            for (int q = 0; q < V / 32; ++q) red[buf][warp][q * 32 + lane] = acc[q];
        } else {
            if ((lane & ((1u << (5 - LOG2V)) - 1u)) == 0) red[buf][warp][lane >> (5 - LOG2V)] = acc[0];
        }
        __syncthreads();
        constexpr int FIN = OUT == HB_OUT_SWIGLU ? V / 2 : V;
        if (tid < (uint32_t)FIN) {
            float s = red[buf][0][tid];
#pragma unroll
            for (int w = 1; w < XS_WARPS; ++w) s += red[buf][w][tid];
            const uint32_t r = tid / M, i = tid % M;
            const uint32_t col = g * RG + r;
            if (col < p.n_out && i < p.m) {
                const size_t at = (size_t)i * p.n_out + col;
                if constexpr (OUT == HB_OUT_SWIGLU) {
                    float u = red[buf][0][tid + V / 2];
#pragma unroll
                    for (int w = 1; w < XS_WARPS; ++w) u += red[buf][w][tid + V / 2];
                    reinterpret_cast<uint16_t*>(p.y)[at] = (uint16_t)swiglu_bf16(round_bf16(s), round_bf16(u));
                } else if constexpr (OUT == HB_OUT_F32) {
                    reinterpret_cast<float*>(p.y)[at] = s;
                } else if constexpr (OUT == HB_OUT_BF16) {
                    reinterpret_cast<uint16_t*>(p.y)[at] = (uint16_t)f32_to_bf16(s);
                } else {
                    uint16_t* y = reinterpret_cast<uint16_t*>(p.y) + at;
                    *y = (uint16_t)f32_to_bf16(__fadd_rn(bf16_to_f32(*y), round_bf16(s)));
                }
            }
        }
        buf ^= 1u;
#pragma unroll
        for (int r = 0; r < R; ++r)
#pragma unroll
            for (int j = 0; j < CPT; ++j) wv[r][j] = wn[r][j];
    }
}

namespace {

typedef void (*xs_fn)(const MatvecXsParams);

template <int M, int R, int CPT>
xs_fn xs_out(uint32_t out) {
    switch (out) {
        case HB_OUT_BF16: return matvec_xs_kernel<M, R, CPT, HB_OUT_BF16>;
        case HB_OUT_F32: return matvec_xs_kernel<M, R, CPT, HB_OUT_F32>;
        case HB_OUT_RESIDUAL: return matvec_xs_kernel<M, R, CPT, HB_OUT_RESIDUAL>;
        case HB_OUT_SWIGLU: return matvec_xs_kernel<M, R, CPT, HB_OUT_SWIGLU>;
    }
    return nullptr;
}
template <int M, int R>
xs_fn xs_cpt(uint32_t cpt, uint32_t out) {
    // the activation slice must fit the register file: M * CPT * 8 floats per thread, at most 128
    if (cpt == 1) return xs_out<M, R, 1>(out);
    if constexpr (M * 2 <= 16) if (cpt == 2) return xs_out<M, R, 2>(out);
    if constexpr (M * 4 <= 16) if (cpt <= 4) return xs_out<M, R, 4>(out);
    return nullptr;
}
template <int M>
xs_fn xs_rows(uint32_t r, uint32_t cpt, uint32_t out) {
    if (r == 2) return xs_cpt<M, 2>(cpt, out);
    if (r == 4) return xs_cpt<M, 4>(cpt, out);
    return nullptr;
}

struct MatvecXs : hb_kernel {
    hb_matvec_desc d{};
    xs_fn fn = nullptr;
    int blocks_per_sm = 1;

    int launch(hb_ctx* ctx, const hb_range* a, int na, uint32_t m) override {
        if (na != 3) return fail(ctx, HB_INVALID, name + ": bindings are W, x, y");
        if (m == 0 || m > d.rows_max) return fail(ctx, HB_INVALID, name + ": m outside 1.." + std::to_string(d.rows_max));
        const uint32_t n_out = d.out == HB_OUT_SWIGLU ? d.n / 2 : d.n;
        const size_t ybytes = (size_t)m * n_out * (d.out == HB_OUT_F32 ? 4 : 2);
        if (!range_ok(a[0], (size_t)d.n * d.k * 2) || !range_ok(a[1], (size_t)m * d.k * 2) || !range_ok(a[2], ybytes))
            return fail(ctx, HB_INVALID, name + ": a bound range is too small");
        if ((reinterpret_cast<uintptr_t>(a[0].ptr) | reinterpret_cast<uintptr_t>(a[1].ptr)) & 15u)
            return fail(ctx, HB_INVALID, name + ": W and x must be 16-byte aligned");
        MatvecXsParams p{};
        p.w = static_cast<const uint4*>(a[0].ptr);
        p.x = static_cast<const uint4*>(a[1].ptr);
        p.y = a[2].ptr;
        p.n = d.n;
        p.n_out = n_out;
        p.k8 = d.k / 8;
        p.m = m;
        const uint32_t rg = d.out == HB_OUT_SWIGLU ? d.rows_per_warp / 2 : d.rows_per_warp;
        p.groups = (n_out + rg - 1) / rg;
        const uint32_t grid = std::min<uint32_t>(p.groups, (uint32_t)(ctx->sm_count * blocks_per_sm));
        fn<<<grid, XS_THREADS, 0, ctx->stream>>>(p);
        HB_CUDA(ctx, cudaGetLastError());
        ctx->launches++;
        return HB_OK;
    }
};

}  // namespace

int make_matvec_xs(hb_ctx* ctx, const hb_matvec_desc* d, hb_kernel** out) {
    *out = nullptr;
    if (d->rows_max < 2 || d->rows_max > 8) return fail(ctx, HB_UNSUPPORTED, "matvec (activation-stationary): 2..8 activation rows");
    const uint32_t r = d->rows_per_warp ? d->rows_per_warp : 2;
    if (r != 2 && r != 4) return fail(ctx, HB_UNSUPPORTED, "matvec (activation-stationary): 2 or 4 rows of W per group");
    if (d->out == HB_OUT_SWIGLU && d->n % 2 != 0) return fail(ctx, HB_UNSUPPORTED, "matvec: the SwiGLU form needs an even n");
    uint32_t mcap = 2;
    while (mcap < d->rows_max) mcap *= 2;
    const uint32_t k8 = d->k / 8;
    uint32_t cpt = (k8 + XS_THREADS - 1) / XS_THREADS;
    if (cpt == 3) cpt = 4;
    xs_fn fn = nullptr;
    if (cpt <= 4) fn = mcap == 2 ? xs_rows<2>(r, cpt, d->out) : mcap == 4 ? xs_rows<4>(r, cpt, d->out) : xs_rows<8>(r, cpt, d->out);
    if (!fn)
        return fail(ctx, HB_UNSUPPORTED, "matvec (activation-stationary): K = " + std::to_string(d->k) + " at " + std::to_string(mcap) +
                                             " rows does not fit the register file (K * rows <= 32768)");
    auto k = std::make_unique<MatvecXs>();
    k->d = *d;
    k->d.rows_per_warp = r;
    k->d.rows_max = mcap;
    k->fn = fn;
    k->kind = 2;
    k->nargs = 3;
    char nm[160];
    snprintf(nm, sizeof nm, "matvec_%ux%u_%s_m%u_x%u", d->k, d->n, out_tag(d->out), mcap, r);
    k->name = nm;
    if (hb_kernel* have = find(ctx, k->name)) {
        *out = have;
        return HB_OK;
    }
    int occ = 1;
    cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, reinterpret_cast<const void*>(fn), XS_THREADS, 0);
    k->blocks_per_sm = std::max(occ, 1);
    *out = intern(ctx, std::move(k));
    return HB_OK;
}

}  // namespace hb
