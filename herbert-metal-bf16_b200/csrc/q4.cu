// Q4_0 weights (reference src/metal/q4.rs:7-24): per block of 32 weights along k one 16-byte group of nibbles and one
// f16 scale d, w = d * q with q in -8..7 (two's complement nibble; byte b of word i holds weight 8i + b low and
// 8i + 4 + b high). 4.5 bits per weight: the decode product streams 3.6 times fewer bytes than bf16.
//   dequant_q4  (src/metal/kernels.rs:1074-1102): W as bf16 [n][k], each value bf16(d * q) - what the reference's
//               prefill GEMM stages from Q4 weights (prefill.rs:1058-1076), so dequant + the bf16 GEMM gives its bits.
//   matvec_q4   (src/metal/kernels.rs:526-632): y = out(W . x), one activation row. A warp per R rows of W, the lanes
//               stride over the blocks; per block an FMA chain of q * x in the reference's element order, then
//               acc = fma(d, part, acc); the lanes summed by the xor butterfly: the reference's bits.
//   matmul_q4   (src/metal/kernels.rs:983-1071): the same for the 1..8 rows of a short block, each block of weights
//               decoded once and applied to every row; each row's sum in matvec_q4's order, so the decode step's bits.
// The nibbles become numbers without an integer-to-float conversion. In dequant_q4 a byte b placed in the low byte
// of 0x4B000000 is the float 8388608 + b. In the products two nibbles at a time become a pair of f16: a nibble v at
// bits 0..3 of 0x6400 is the f16 1024 + v, at bits 4..7 it is 1024 + 16 v; one packed f16 operation takes the bias
// off (exactly: these are small integers) and the widening to f32 runs on the FMA pipe, so the logic pipe spends
// 6 operations per 8 weights instead of 13.
#include <algorithm>

#include <cuda_fp16.h>

#include "hb_internal.hpp"
#include "tc05.cuh"

namespace hb {

__device__ __forceinline__ float q4_byte_to_q(uint32_t bytes, uint32_t sel) {
    // byte `sel` of `bytes` (a nibble xor 8, 0..15) -> that value minus 8, exactly
    return __uint_as_float(__byte_perm(bytes, 0x4B000000u, 0x7650u + sel)) - 8388616.0f;
}

__global__ void __launch_bounds__(256) dequant_q4_kernel(const uint4* __restrict__ w, const uint16_t* __restrict__ sc, uint4* __restrict__ out, uint32_t blocks) {
    for (uint32_t g = blockIdx.x * blockDim.x + threadIdx.x; g < blocks; g += gridDim.x * blockDim.x) {
        const uint4 wv = w[g];
        const float d = __half2float(__ushort_as_half(sc[g]));
        const uint32_t ww[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t lo = (ww[i] & 0x0F0F0F0Fu) ^ 0x08080808u, hi = ((ww[i] >> 4) & 0x0F0F0F0Fu) ^ 0x08080808u;
            uint32_t o[4];
            // weights 8i + 0..3 are the low nibbles of bytes 0..3, weights 8i + 4..7 the high ones
            o[0] = f32x2_to_bf16x2(__fmul_rn(d, q4_byte_to_q(lo, 0)), __fmul_rn(d, q4_byte_to_q(lo, 1)));
            o[1] = f32x2_to_bf16x2(__fmul_rn(d, q4_byte_to_q(lo, 2)), __fmul_rn(d, q4_byte_to_q(lo, 3)));
            o[2] = f32x2_to_bf16x2(__fmul_rn(d, q4_byte_to_q(hi, 0)), __fmul_rn(d, q4_byte_to_q(hi, 1)));
            o[3] = f32x2_to_bf16x2(__fmul_rn(d, q4_byte_to_q(hi, 2)), __fmul_rn(d, q4_byte_to_q(hi, 3)));
            out[(size_t)g * 4 + i] = make_uint4(o[0], o[1], o[2], o[3]);
        }
    }
}

// The eight weights of word `ww` of a block as four f16 pairs: h[0] = (w0, w2), h[1] = (w4, w6), h[2] = (w1, w3),
// h[3] = (w5, w7), where w_j is weight 8i + j of the block: q_j in -8..7, or with PLUS8 q_j + 8 in 0..15.
template <bool PLUS8>
__device__ __forceinline__ void q4_decode_word(uint32_t ww, __half2 (&h)[4]) {
    const uint32_t wx = ww ^ 0x88888888u, w8 = wx >> 8;
    const __half2 lo_bias = __float2half2_rn(PLUS8 ? 1024.f : 1032.f), hi_bias = __float2half2_rn(PLUS8 ? -64.f : -72.f);
    const __half2 sixteenth = __float2half2_rn(0.0625f);
    auto as_h2 = [](uint32_t v) { return *reinterpret_cast<__half2*>(&v); };
    h[0] = __hsub2(as_h2((wx & 0x000F000Fu) | 0x64006400u), lo_bias);
    h[1] = __hfma2(as_h2((wx & 0x00F000F0u) | 0x64006400u), sixteenth, hi_bias);
    h[2] = __hsub2(as_h2((w8 & 0x000F000Fu) | 0x64006400u), lo_bias);
    h[3] = __hfma2(as_h2((w8 & 0x00F000F0u) | 0x64006400u), sixteenth, hi_bias);
}
// weight j (0..7) of a decoded word, as f32
__device__ __forceinline__ float q4_elem(const __half2 (&h)[4], int j) {
    const int idx = (j >= 4 ? 1 : 0) + ((j & 1) ? 2 : 0);
    return (j & 2) ? __high2float(h[idx]) : __low2float(h[idx]);
}

// Two IEEE f32 operations in one instruction (two rows of W share every activation, so their chains go side by side).
__device__ __forceinline__ uint64_t q4_pack2(uint32_t lo, uint32_t hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(lo), "r"(hi));
    return r;
}
__device__ __forceinline__ uint64_t q4_ffma2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}

struct MatvecQ4Params {
    const uint4* w;
    const uint16_t* sc;
    const uint4* x;
    void* y;
    uint32_t n, nblk, groups;
    uint32_t split;  // warps sharing the blocks of one row group: block b to warp (b / 32) % split (matvec_q4_split, kernels.rs:472-500)
};

constexpr int Q4_THREADS = 256;
constexpr int Q4_WARPS = Q4_THREADS / 32;

// MASKS: the order of sums of the reference's matvec_q4s ("llama.cpp's masks", src/metal/kernels.rs:455-462,
// 1387-1424): per block sx = x_0 + ... + x_31 in order, part = fma(q_e + 8, x_e, part) over e = 8i + j, j = 0..7 (the low
// nibbles of bytes 0..3, then the high ones), part = fma(-8, sx, part). The reference multiplies the nibble taken in
// place (q + 8)·2^s by x·2^-s: the same product exactly (powers of two), so the same bits, without the scaling.
template <int R, int OUT, bool MASKS>
__global__ void __launch_bounds__(Q4_THREADS) matvec_q4_kernel(const MatvecQ4Params p) {
    // x staged in shared memory once per CTA, the four 16-byte chunks of a block xor-swizzled by the block's number:
    // the 32 lanes read 32 different blocks (64 bytes apart), which straight from L1 costs 16 wavefronts a load
    extern __shared__ uint4 q4_xs[];
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    griddep_launch_dependents();
    griddep_wait();  // x comes from the kernel before this one
    for (uint32_t j = threadIdx.x; j < p.nblk * 4; j += Q4_THREADS) q4_xs[(j & ~3u) + ((j & 3u) ^ ((j >> 3) & 3u))] = __ldg(p.x + j);
    __syncthreads();
    __shared__ float red[Q4_WARPS][R];
    const uint32_t split = p.split, slots = Q4_WARPS / split, slot = warp / split, piece = warp % split;
    for (uint32_t g0 = blockIdx.x * slots; g0 < p.groups; g0 += gridDim.x * slots) {
        const uint32_t group = min(g0 + slot, p.groups - 1);  // a slot past the end repeats the last group and writes nothing
        const bool live = g0 + slot < p.groups;
        size_t base[R];
#pragma unroll
        for (int r = 0; r < R; ++r) base[r] = (size_t)min(group * R + r, p.n - 1) * p.nblk;  // rows past the end read the last row
        float acc[R];
#pragma unroll
        for (int r = 0; r < R; ++r) acc[r] = 0.f;
        for (uint32_t b = lane + 32u * piece; b < p.nblk; b += 32u * split) {
            uint4 wv[R];
            uint16_t dh[R];
#pragma unroll
            for (int r = 0; r < R; ++r) {
                wv[r] = __ldcs(p.w + base[r] + b);
                dh[r] = __ldcs(p.sc + base[r] + b);
            }
            // the 32 activations of the block, in order
            float xs[32];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const uint4 xv = q4_xs[b * 4 + ((uint32_t)i ^ ((b >> 1) & 3u))];
                const uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    xs[8 * i + 2 * c] = __uint_as_float(xw[c] << 16);
                    xs[8 * i + 2 * c + 1] = __uint_as_float(xw[c] & 0xffff0000u);
                }
            }
            float sx = 0.f;
            if constexpr (MASKS) {
                sx = xs[0];
#pragma unroll
                for (int e = 1; e < 32; ++e) sx = __fadd_rn(sx, xs[e]);
            }
            // step t of a word's eight is weight j of the word:
            //   plain: weight byte, then 4 + byte, byte by byte; masks: the four low nibbles, then the four high
            auto elem_of = [](int t) { return MASKS ? t : ((t & 1) ? 4 : 0) + (t >> 1); };
            if constexpr (R == 1) {
                const uint32_t ww[4] = {wv[0].x, wv[0].y, wv[0].z, wv[0].w};
                float part = 0.f;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    __half2 h[4];
                    q4_decode_word<MASKS>(ww[i], h);
#pragma unroll
                    for (int t = 0; t < 8; ++t) {
                        const int j = elem_of(t);
                        part = __fmaf_rn(q4_elem(h, j), xs[8 * i + j], part);
                    }
                }
                if constexpr (MASKS) part = __fmaf_rn(-8.0f, sx, part);
                acc[0] = __fmaf_rn(__half2float(__ushort_as_half(dh[0])), part, acc[0]);
            } else {
                // rows in pairs: the two chains of a pair run as the two halves of packed f32x2 operations (each half
                // is the same IEEE operation as the scalar one, in the same order)
#pragma unroll
                for (int r = 0; r < R; r += 2) {
                    const uint32_t wa[4] = {wv[r].x, wv[r].y, wv[r].z, wv[r].w}, wb[4] = {wv[r + 1].x, wv[r + 1].y, wv[r + 1].z, wv[r + 1].w};
                    uint64_t part2 = 0ull;
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        __half2 ha[4], hb_[4];
                        q4_decode_word<MASKS>(wa[i], ha);
                        q4_decode_word<MASKS>(wb[i], hb_);
#pragma unroll
                        for (int t = 0; t < 8; ++t) {
                            const int j = elem_of(t);
                            const uint32_t xe = __float_as_uint(xs[8 * i + j]);
                            part2 = q4_ffma2(q4_pack2(__float_as_uint(q4_elem(ha, j)), __float_as_uint(q4_elem(hb_, j))), q4_pack2(xe, xe), part2);
                        }
                    }
                    uint32_t pa, pb;
                    asm("mov.b64 {%0, %1}, %2;" : "=r"(pa), "=r"(pb) : "l"(part2));
                    float fa = __uint_as_float(pa), fb = __uint_as_float(pb);
                    if constexpr (MASKS) {
                        fa = __fmaf_rn(-8.0f, sx, fa);
                        fb = __fmaf_rn(-8.0f, sx, fb);
                    }
                    acc[r] = __fmaf_rn(__half2float(__ushort_as_half(dh[r])), fa, acc[r]);
                    acc[r + 1] = __fmaf_rn(__half2float(__ushort_as_half(dh[r + 1])), fb, acc[r + 1]);
                }
            }
        }
#pragma unroll
        for (int r = 0; r < R; ++r) {
            float a = acc[r];
#pragma unroll
            for (int off = 16; off >= 1; off >>= 1) a = __fadd_rn(a, __shfl_xor_sync(0xffffffffu, a, off));
            acc[r] = a;
        }
        if (split > 1) {  // the row's sum: its `split` partials in warp order (kernels.rs:916-928)
            if (lane == 0) {
#pragma unroll
                for (int r = 0; r < R; ++r) red[warp][r] = acc[r];
            }
            __syncthreads();
            if (piece == 0 && lane == 0) {
#pragma unroll
                for (int r = 0; r < R; ++r)
                    for (uint32_t s2 = 1; s2 < split; ++s2) acc[r] = __fadd_rn(acc[r], red[warp + s2][r]);
            }
        }
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const float a = acc[r];
            const uint32_t row = group * R + r;
            if (live && piece == 0 && lane == 0 && row < p.n) {
                if constexpr (OUT == HB_OUT_F32) reinterpret_cast<float*>(p.y)[row] = a;
                else if constexpr (OUT == HB_OUT_BF16) reinterpret_cast<uint16_t*>(p.y)[row] = (uint16_t)f32_to_bf16(a);
                else {
                    uint16_t* y = reinterpret_cast<uint16_t*>(p.y) + row;
                    *y = (uint16_t)f32_to_bf16(__fadd_rn(bf16_to_f32(*y), round_bf16(a)));
                }
            }
        }
        if (split > 1) __syncthreads();  // `red` is read by the head before the next group writes it
    }
}

// ---------------------------------------------------------------- matmul_q4: 1..8 activation rows

struct MatmulQ4Params {
    const uint4* w;
    const uint16_t* sc;
    const uint16_t* x;
    uint16_t* y;
    uint32_t n, nblk, groups, m, ldx, ldy;
};

// A warp per R rows of W, the lanes over the blocks as in matvec_q4; a block's weights are decoded once and meet the
// rows of X two at a time: rows 2p and 2p + 1 are the halves of packed f32x2 chains (MP pairs; with an odd m the last
// pair's second half repeats the last row and is not stored). X is staged in shared memory once per CTA (bf16,
// [row][16-byte chunk], the four chunks of a block xor-swizzled by the block's number so that the 32 lanes - each on
// its own block, 64 bytes apart - spread over all the banks).
template <int R, int MP>
__global__ void __launch_bounds__(Q4_THREADS, 2) matmul_q4_kernel(const MatmulQ4Params p) {
    extern __shared__ uint4 q4_xs[];
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t chunks = p.nblk * 4;
    griddep_launch_dependents();
    griddep_wait();  // X comes from the kernel before this one
    for (uint32_t c = threadIdx.x; c < 2 * MP * chunks; c += Q4_THREADS) {
        const uint32_t r = c / chunks, j = c - r * chunks, b = j >> 2, i = j & 3;
        const uint32_t src = min(r, p.m - 1);
        q4_xs[r * chunks + b * 4 + (i ^ ((b >> 1) & 3u))] = __ldg(reinterpret_cast<const uint4*>(p.x + (size_t)src * p.ldx) + j);
    }
    __syncthreads();
    for (uint32_t group = blockIdx.x * Q4_WARPS + warp; group < p.groups; group += gridDim.x * Q4_WARPS) {
        size_t base[R];
#pragma unroll
        for (int r = 0; r < R; ++r) base[r] = (size_t)min(group * R + r, p.n - 1) * p.nblk;  // rows past the end read the last row
        uint64_t acc[R][MP];
#pragma unroll
        for (int r = 0; r < R; ++r)
#pragma unroll
            for (int q = 0; q < MP; ++q) acc[r][q] = 0ull;
        for (uint32_t b = lane; b < p.nblk; b += 32) {
            uint4 wv[R];
            uint16_t dh[R];
#pragma unroll
            for (int r = 0; r < R; ++r) {
                wv[r] = __ldcs(p.w + base[r] + b);
                dh[r] = __ldcs(p.sc + base[r] + b);
            }
            uint64_t part[R][MP];
#pragma unroll
            for (int r = 0; r < R; ++r)
#pragma unroll
                for (int q = 0; q < MP; ++q) part[r][q] = 0ull;
            const uint32_t sw = (b >> 1) & 3u;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                // the eight activations of this word's weights, of every row: raw bf16 pairs
                uint4 xv[2 * MP];
#pragma unroll
                for (int r = 0; r < 2 * MP; ++r) xv[r] = q4_xs[r * chunks + b * 4 + ((uint32_t)i ^ sw)];
                __half2 h[R][4];
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    const uint32_t ww = i == 0 ? wv[r].x : i == 1 ? wv[r].y : i == 2 ? wv[r].z : wv[r].w;
                    q4_decode_word<false>(ww, h[r]);
                }
#pragma unroll
                for (int t = 0; t < 8; ++t) {
                    const int j = ((t & 1) ? 4 : 0) + (t >> 1);  // weight `byte`, then 4 + byte, byte by byte
                    uint64_t x2[MP];
#pragma unroll
                    for (int q = 0; q < MP; ++q) {
                        const uint4 &a = xv[2 * q], &c = xv[2 * q + 1];
                        const uint32_t wa = (j >> 1) == 0 ? a.x : (j >> 1) == 1 ? a.y : (j >> 1) == 2 ? a.z : a.w;
                        const uint32_t wc = (j >> 1) == 0 ? c.x : (j >> 1) == 1 ? c.y : (j >> 1) == 2 ? c.z : c.w;
                        x2[q] = (j & 1) ? q4_pack2(wa & 0xffff0000u, wc & 0xffff0000u) : q4_pack2(wa << 16, wc << 16);
                    }
#pragma unroll
                    for (int r = 0; r < R; ++r) {
                        const uint32_t qf = __float_as_uint(q4_elem(h[r], j));
                        const uint64_t q2 = q4_pack2(qf, qf);
#pragma unroll
                        for (int q = 0; q < MP; ++q) part[r][q] = q4_ffma2(q2, x2[q], part[r][q]);
                    }
                }
            }
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const uint32_t d = __float_as_uint(__half2float(__ushort_as_half(dh[r])));
                const uint64_t d2 = q4_pack2(d, d);
#pragma unroll
                for (int q = 0; q < MP; ++q) acc[r][q] = q4_ffma2(d2, part[r][q], acc[r][q]);
            }
        }
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const uint32_t row = group * R + r;
#pragma unroll
            for (int q = 0; q < MP; ++q) {
                uint32_t ua, ub;
                asm("mov.b64 {%0, %1}, %2;" : "=r"(ua), "=r"(ub) : "l"(acc[r][q]));
                float a = __uint_as_float(ua), c = __uint_as_float(ub);
#pragma unroll
                for (int off = 16; off >= 1; off >>= 1) {
                    a = __fadd_rn(a, __shfl_xor_sync(0xffffffffu, a, off));
                    c = __fadd_rn(c, __shfl_xor_sync(0xffffffffu, c, off));
                }
                if (lane == 0 && row < p.n) {
                    if ((uint32_t)(2 * q) < p.m) p.y[(size_t)(2 * q) * p.ldy + row] = (uint16_t)f32_to_bf16(a);
                    if ((uint32_t)(2 * q + 1) < p.m) p.y[(size_t)(2 * q + 1) * p.ldy + row] = (uint16_t)f32_to_bf16(c);
                }
            }
        }
    }
}

namespace {

struct DequantQ4 : hb_kernel {
    uint32_t k = 0, n = 0;
    int launch(hb_ctx* ctx, const hb_range* a, int na, uint32_t m) override {
        (void)m;
        if (na != 3) return fail(ctx, HB_INVALID, name + ": bindings are W (nibbles), scales (f16), out (bf16)");
        const size_t blocks = (size_t)n * (k / 32);
        if (!range_ok(a[0], blocks * 16) || !range_ok(a[1], blocks * 2) || !range_ok(a[2], blocks * 64)) return fail(ctx, HB_INVALID, name + ": a bound range is too small");
        if ((reinterpret_cast<uintptr_t>(a[0].ptr) | reinterpret_cast<uintptr_t>(a[2].ptr)) & 15u) return fail(ctx, HB_INVALID, name + ": W and out must be 16-byte aligned");
        const uint32_t grid = (uint32_t)std::max<size_t>(1, std::min<size_t>((blocks + 255) / 256, (size_t)ctx->sm_count * 16));
        dequant_q4_kernel<<<grid, 256, 0, ctx->stream>>>(static_cast<const uint4*>(a[0].ptr), static_cast<const uint16_t*>(a[1].ptr), static_cast<uint4*>(a[2].ptr), (uint32_t)blocks);
        HB_CUDA(ctx, cudaGetLastError());
        ctx->launches++;
        return HB_OK;
    }
};

typedef void (*q4_fn)(const MatvecQ4Params);

template <int R, bool MASKS>
q4_fn q4_out(uint32_t out) {
    switch (out) {
        case HB_OUT_BF16: return matvec_q4_kernel<R, HB_OUT_BF16, MASKS>;
        case HB_OUT_F32: return matvec_q4_kernel<R, HB_OUT_F32, MASKS>;
        case HB_OUT_RESIDUAL: return matvec_q4_kernel<R, HB_OUT_RESIDUAL, MASKS>;
    }
    return nullptr;
}
template <bool MASKS>
q4_fn q4_rows(uint32_t rows, uint32_t out) {
    return rows == 1 ? q4_out<1, MASKS>(out) : rows == 2 ? q4_out<2, MASKS>(out) : rows == 4 ? q4_out<4, MASKS>(out) : nullptr;
}

struct MatvecQ4 : hb_kernel {
    uint32_t k = 0, n = 0, out = 0, rows = 0, split = 1, persist = 0;
    q4_fn fn = nullptr;
    int launch(hb_ctx* ctx, const hb_range* a, int na, uint32_t m) override {
        if (na != 4) return fail(ctx, HB_INVALID, name + ": bindings are W (nibbles), x, y, scales (f16)");
        if (m != 1) return fail(ctx, HB_INVALID, name + ": one activation row");
        const size_t blocks = (size_t)n * (k / 32);
        if (!range_ok(a[0], blocks * 16) || !range_ok(a[1], (size_t)k * 2) || !range_ok(a[2], (size_t)n * (out == HB_OUT_F32 ? 4 : 2)) || !range_ok(a[3], blocks * 2))
            return fail(ctx, HB_INVALID, name + ": a bound range is too small");
        if ((reinterpret_cast<uintptr_t>(a[0].ptr) | reinterpret_cast<uintptr_t>(a[1].ptr)) & 15u) return fail(ctx, HB_INVALID, name + ": W and x must be 16-byte aligned");
        MatvecQ4Params p{};
        p.w = static_cast<const uint4*>(a[0].ptr);
        p.x = static_cast<const uint4*>(a[1].ptr);
        p.y = a[2].ptr;
        p.sc = static_cast<const uint16_t*>(a[3].ptr);
        p.n = n;
        p.nblk = k / 32;
        p.groups = (n + rows - 1) / rows;
        p.split = split;
        const uint32_t slots = Q4_WARPS / split;
        // persist > 0: only that many blocks, each taking one row group after another (mv.persist); else as many as there are
        // row groups, up to eight a multiprocessor
        const uint32_t want = (p.groups + slots - 1) / slots;
        const uint32_t grid = std::max(1u, std::min<uint32_t>(want, persist ? persist : (uint32_t)ctx->sm_count * 8));
        HB_CUDA(ctx, launch_kernel(ctx, true, fn, dim3(grid), dim3(Q4_THREADS), (size_t)k * 2, p));
        ctx->launches++;
        return HB_OK;
    }
};

typedef void (*q4mm_fn)(const MatmulQ4Params);

struct MatmulQ4 : hb_kernel {
    uint32_t k = 0, n = 0, m = 0, ldx = 0, ldy = 0, rows = 0, ctas_per_sm = 1;
    size_t smem = 0;
    q4mm_fn fn = nullptr;
    int launch(hb_ctx* ctx, const hb_range* a, int na, uint32_t m_now) override {
        if (na != 4) return fail(ctx, HB_INVALID, name + ": bindings are W (nibbles), X, Y, scales (f16)");
        if (m_now != m) return fail(ctx, HB_INVALID, name + ": built for " + std::to_string(m) + " rows");
        const size_t blocks = (size_t)n * (k / 32);
        if (!range_ok(a[0], blocks * 16) || !range_ok(a[1], ((size_t)(m - 1) * ldx + k) * 2) || !range_ok(a[2], ((size_t)(m - 1) * ldy + n) * 2) || !range_ok(a[3], blocks * 2))
            return fail(ctx, HB_INVALID, name + ": a bound range is too small");
        if ((reinterpret_cast<uintptr_t>(a[0].ptr) | reinterpret_cast<uintptr_t>(a[1].ptr)) & 15u) return fail(ctx, HB_INVALID, name + ": W and X must be 16-byte aligned");
        MatmulQ4Params p{};
        p.w = static_cast<const uint4*>(a[0].ptr);
        p.x = static_cast<const uint16_t*>(a[1].ptr);
        p.y = static_cast<uint16_t*>(a[2].ptr);
        p.sc = static_cast<const uint16_t*>(a[3].ptr);
        p.n = n;
        p.nblk = k / 32;
        p.groups = (n + rows - 1) / rows;
        p.m = m;
        p.ldx = ldx;
        p.ldy = ldy;
        const uint32_t grid = std::max(1u, std::min<uint32_t>((p.groups + Q4_WARPS - 1) / Q4_WARPS, (uint32_t)ctx->sm_count * ctas_per_sm));
        HB_CUDA(ctx, launch_kernel(ctx, true, fn, dim3(grid), dim3(Q4_THREADS), smem, p));
        ctx->launches++;
        return HB_OK;
    }
};

}  // namespace

int make_dequant_q4(hb_ctx* ctx, uint32_t k, uint32_t n, hb_kernel** out) {
    *out = nullptr;
    if (k == 0 || n == 0 || k % 32 != 0) return fail(ctx, HB_UNSUPPORTED, "Q4: K = " + std::to_string(k) + " is not a multiple of 32");
    auto kn = std::make_unique<DequantQ4>();
    kn->k = k;
    kn->n = n;
    kn->kind = 19;
    kn->nargs = 3;
    kn->name = "dequant_q4_" + std::to_string(k) + "x" + std::to_string(n);
    *out = intern(ctx, std::move(kn));
    return HB_OK;
}

int make_matvec_q4(hb_ctx* ctx, uint32_t k, uint32_t n, uint32_t out_mode, uint32_t rows, uint32_t masks, uint32_t split, uint32_t persist, hb_kernel** out) {
    *out = nullptr;
    if (k == 0 || n == 0 || k % 32 != 0) return fail(ctx, HB_UNSUPPORTED, "Q4: K = " + std::to_string(k) + " is not a multiple of 32");
    if (rows == 0) rows = 2;
    if (split == 0) split = 1;
    if (split != 1 && split != 2 && split != 4 && split != 8) return fail(ctx, HB_UNSUPPORTED, "matvec_q4: split must be 1, 2, 4 or 8 (it divides the eight warps of a block)");
    q4_fn fn = masks ? q4_rows<true>(rows, out_mode) : q4_rows<false>(rows, out_mode);
    if (!fn) return fail(ctx, HB_UNSUPPORTED, "matvec_q4: rows per warp 1, 2 or 4; output Bf16, F32 or Residual");
    if ((size_t)k * 2 > ctx->smem_optin) return fail(ctx, HB_UNSUPPORTED, "matvec_q4: a row of K = " + std::to_string(k) + " does not fit in shared memory");
    auto kn = std::make_unique<MatvecQ4>();
    kn->k = k;
    kn->n = n;
    kn->out = out_mode;
    kn->rows = rows;
    kn->split = split;
    kn->persist = persist;
    kn->fn = fn;
    kn->kind = 20;
    kn->nargs = 4;
    kn->name = std::string(masks ? "matvec_q4s_" : "matvec_q4_") + std::to_string(k) + "x" + std::to_string(n) + "_" + out_tag(out_mode) + "_r" + std::to_string(rows) +
               (split > 1 ? "_s" + std::to_string(split) : "") + (persist ? "_p" + std::to_string(persist) : "");
    if (hb_kernel* have = find(ctx, kn->name)) {
        *out = have;
        return HB_OK;
    }
    if ((size_t)k * 2 > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(reinterpret_cast<const void*>(fn), cudaFuncAttributeMaxDynamicSharedMemorySize, (int)ctx->smem_optin);
        if (e != cudaSuccess) return cuda_fail(ctx, e, "cudaFuncSetAttribute(max dynamic shared memory)");
    }
    *out = intern(ctx, std::move(kn));
    return HB_OK;
}

int make_matmul_q4(hb_ctx* ctx, uint32_t k, uint32_t n, uint32_t m, uint32_t ldx, uint32_t ldy, hb_kernel** out) {
    *out = nullptr;
    if (k == 0 || n == 0 || k % 32 != 0 || ldx % 8 != 0) return fail(ctx, HB_UNSUPPORTED, "Q4 block: K = " + std::to_string(k) + ", ldx = " + std::to_string(ldx) + " (K in blocks of 32, rows of X on 16-byte boundaries)");
    if (m == 0 || m > 8) return fail(ctx, HB_UNSUPPORTED, "matmul_q4: 1 to 8 rows (longer blocks go through dequant_q4 and the GEMM)");
    if (ldx < k || ldy < n) return fail(ctx, HB_INVALID, "matmul_q4: ldx < k or ldy < n");
    const uint32_t mp = (m + 1) / 2;
    // four rows of W per warp while the accumulators fit comfortably, two with three or four pairs of rows of X
    const uint32_t rows = mp <= 2 ? 4 : 2;
    q4mm_fn fn = mp == 1 ? matmul_q4_kernel<4, 1> : mp == 2 ? matmul_q4_kernel<4, 2> : mp == 3 ? matmul_q4_kernel<2, 3> : matmul_q4_kernel<2, 4>;
    const size_t smem = (size_t)2 * mp * k * 2;
    if (smem > ctx->smem_optin) return fail(ctx, HB_UNSUPPORTED, "matmul_q4: " + std::to_string(2 * mp) + " rows of K = " + std::to_string(k) + " do not fit in shared memory");
    auto kn = std::make_unique<MatmulQ4>();
    kn->k = k;
    kn->n = n;
    kn->m = m;
    kn->ldx = ldx;
    kn->ldy = ldy;
    kn->rows = rows;
    kn->smem = smem;
    kn->ctas_per_sm = (uint32_t)std::max<size_t>(1, std::min<size_t>(2, (size_t)(ctx->smem_optin + 1024) / (smem + 1024)));
    kn->fn = fn;
    kn->kind = 21;
    kn->nargs = 4;
    kn->name = "matmul_q4_" + std::to_string(k) + "x" + std::to_string(n) + "_m" + std::to_string(m) + "_x" + std::to_string(ldx) + "_y" + std::to_string(ldy);
    if (hb_kernel* have = find(ctx, kn->name)) {
        *out = have;
        return HB_OK;
    }
    cudaError_t e = cudaFuncSetAttribute(reinterpret_cast<const void*>(fn), cudaFuncAttributeMaxDynamicSharedMemorySize, (int)ctx->smem_optin);
    if (e != cudaSuccess) return cuda_fail(ctx, e, "cudaFuncSetAttribute(max dynamic shared memory)");
    *out = intern(ctx, std::move(kn));
    return HB_OK;
}

}  // namespace hb

extern "C" {

int hb_dequant_q4_get(hb_ctx* ctx, uint32_t k, uint32_t n, hb_kernel** out) {
    if (!ctx || !out) return hb::fail(ctx, HB_INVALID, "hb_dequant_q4_get: bad argument");
    try {
        hb::bind(ctx);
        return hb::make_dequant_q4(ctx, k, n, out);
    } catch (const std::exception& e) {
        return hb::fail(ctx, HB_BACKEND, e.what());
    }
}

int hb_matvec_q4_get(hb_ctx* ctx, uint32_t k, uint32_t n, uint32_t out_mode, uint32_t rows_per_warp, uint32_t masks, hb_kernel** out) {
    if (!ctx || !out) return hb::fail(ctx, HB_INVALID, "hb_matvec_q4_get: bad argument");
    try {
        hb::bind(ctx);
        return hb::make_matvec_q4(ctx, k, n, out_mode, rows_per_warp, masks, 1, 0, out);
    } catch (const std::exception& e) {
        return hb::fail(ctx, HB_BACKEND, e.what());
    }
}

int hb_matvec_q4_split_get(hb_ctx* ctx, uint32_t k, uint32_t n, uint32_t out_mode, uint32_t rows_per_warp, uint32_t masks, uint32_t split, uint32_t persist,
                           hb_kernel** out) {
    if (!ctx || !out) return hb::fail(ctx, HB_INVALID, "hb_matvec_q4_split_get: bad argument");
    try {
        hb::bind(ctx);
        return hb::make_matvec_q4(ctx, k, n, out_mode, rows_per_warp, masks, split, persist, out);
    } catch (const std::exception& e) {
        return hb::fail(ctx, HB_BACKEND, e.what());
    }
}

int hb_matmul_q4_get(hb_ctx* ctx, uint32_t k, uint32_t n, uint32_t m, uint32_t ldx, uint32_t ldy, hb_kernel** out) {
    if (!ctx || !out) return hb::fail(ctx, HB_INVALID, "hb_matmul_q4_get: bad argument");
    try {
        hb::bind(ctx);
        return hb::make_matmul_q4(ctx, k, n, m, ldx, ldy, out);
    } catch (const std::exception& e) {
        return hb::fail(ctx, HB_BACKEND, e.what());
    }
}

}  // extern "C"
