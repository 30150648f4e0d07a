// Q4_0 weights (reference src/metal/q4.rs:7-24): per block of 32 weights along k one 16-byte group of nibbles and one
// f16 scale d, w = d * q with q in -8..7 (two's complement nibble; byte b of word i holds weight 8i + b low and
// 8i + 4 + b high). 4.5 bits per weight: the decode product streams 3.6 times fewer bytes than bf16.
//   dequant_q4  (src/metal/kernels.rs:1074-1102): W as bf16 [n][k], each value bf16(d * q) - what the reference's
//               prefill GEMM stages from Q4 weights (prefill.rs:1058-1076), so dequant + the bf16 GEMM gives its bits.
//   matvec_q4   (src/metal/kernels.rs:526-632): y = out(W . x), one activation row. A warp per R rows of W, the lanes
//               stride over the blocks; per block an FMA chain of q * x in the reference's element order, then
//               acc = fma(d, part, acc); the lanes summed by the xor butterfly: the reference's bits.
// The nibbles become floats without an integer-to-float conversion: a byte b placed in the low byte of 0x4B000000
// is the float 8388608 + b, so (that) - 8388616 is exactly (b ^ 8's value) - 8 once the bytes were xored with 8.
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
__device__ __forceinline__ uint64_t q4_fadd2(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}

struct MatvecQ4Params {
    const uint4* w;
    const uint16_t* sc;
    const uint4* x;
    void* y;
    uint32_t n, nblk, groups;
};

constexpr int Q4_THREADS = 256;
constexpr int Q4_WARPS = Q4_THREADS / 32;

// MASKS: the order of sums of the reference's matvec_q4s ("llama.cpp's masks", src/metal/kernels.rs:455-462,
// 1387-1424): per block sx = x_0 + ... + x_31 in order, part = fma(q_e + 8, x_e, part) over e = 8i + j, j = 0..7 (the low
// nibbles of bytes 0..3, then the high ones), part = fma(-8, sx, part). The reference multiplies the nibble taken in
// place (q + 8)·2^s by x·2^-s: the same product exactly (powers of two), so the same bits, without the scaling.
template <int R, int OUT, bool MASKS>
__global__ void __launch_bounds__(Q4_THREADS) matvec_q4_kernel(const MatvecQ4Params p) {
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    griddep_launch_dependents();
    griddep_wait();  // x comes from the kernel before this one
    for (uint32_t group = blockIdx.x * Q4_WARPS + warp; group < p.groups; group += gridDim.x * Q4_WARPS) {
        size_t base[R];
#pragma unroll
        for (int r = 0; r < R; ++r) base[r] = (size_t)min(group * R + r, p.n - 1) * p.nblk;  // rows past the end read the last row
        float acc[R];
#pragma unroll
        for (int r = 0; r < R; ++r) acc[r] = 0.f;
        for (uint32_t b = lane; b < p.nblk; b += 32) {
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
                const uint4 xv = __ldg(p.x + (size_t)b * 4 + i);
                const uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    xs[8 * i + 2 * c] = __uint_as_float(xw[c] << 16);
                    xs[8 * i + 2 * c + 1] = __uint_as_float(xw[c] & 0xffff0000u);
                }
            }
            // what is subtracted from the byte-in-0x4B000000 float: 8388608 + 8 gives q, 8388608 gives q + 8
            constexpr float MAGIC = MASKS ? -8388608.0f : -8388616.0f;
            float sx = 0.f;
            if constexpr (MASKS) {
                sx = xs[0];
#pragma unroll
                for (int e = 1; e < 32; ++e) sx = __fadd_rn(sx, xs[e]);
            }
            // step t of a word's eight: which nibble (low or high) of which byte, and which activation
            //   plain: weight 8i + byte, then 8i + 4 + byte, byte by byte; masks: the four low nibbles, then the four high
            auto nib_of = [](int t, bool& high, int& byte) {
                if (MASKS) { high = t >= 4; byte = t & 3; }
                else { high = (t & 1) != 0; byte = t >> 1; }
            };
            if constexpr (R == 1) {
                const uint32_t ww[4] = {wv[0].x, wv[0].y, wv[0].z, wv[0].w};
                float part = 0.f;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const uint32_t lo = (ww[i] & 0x0F0F0F0Fu) ^ 0x08080808u, hi = ((ww[i] >> 4) & 0x0F0F0F0Fu) ^ 0x08080808u;
#pragma unroll
                    for (int t = 0; t < 8; ++t) {
                        bool high;
                        int byte;
                        nib_of(t, high, byte);
                        const float q = __fadd_rn(__uint_as_float(__byte_perm(high ? hi : lo, 0x4B000000u, 0x7650u + byte)), MAGIC);
                        part = __fmaf_rn(q, xs[8 * i + (high ? 4 : 0) + byte], part);
                    }
                }
                if constexpr (MASKS) part = __fmaf_rn(-8.0f, sx, part);
                acc[0] = __fmaf_rn(__half2float(__ushort_as_half(dh[0])), part, acc[0]);
            } else {
                // rows in pairs: the two chains of a pair run as the two halves of packed f32x2 operations (each half
                // is the same IEEE operation as the scalar one, in the same order)
                const uint64_t minus = q4_pack2(__float_as_uint(MAGIC), __float_as_uint(MAGIC));
#pragma unroll
                for (int r = 0; r < R; r += 2) {
                    const uint32_t wa[4] = {wv[r].x, wv[r].y, wv[r].z, wv[r].w}, wb[4] = {wv[r + 1].x, wv[r + 1].y, wv[r + 1].z, wv[r + 1].w};
                    uint64_t part2 = 0ull;
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const uint32_t lo_a = (wa[i] & 0x0F0F0F0Fu) ^ 0x08080808u, hi_a = ((wa[i] >> 4) & 0x0F0F0F0Fu) ^ 0x08080808u;
                        const uint32_t lo_b = (wb[i] & 0x0F0F0F0Fu) ^ 0x08080808u, hi_b = ((wb[i] >> 4) & 0x0F0F0F0Fu) ^ 0x08080808u;
#pragma unroll
                        for (int t = 0; t < 8; ++t) {
                            bool high;
                            int byte;
                            nib_of(t, high, byte);
                            const uint32_t xe = __float_as_uint(xs[8 * i + (high ? 4 : 0) + byte]);
                            const uint64_t q2 = q4_fadd2(q4_pack2(__byte_perm(high ? hi_a : lo_a, 0x4B000000u, 0x7650u + byte),
                                                                  __byte_perm(high ? hi_b : lo_b, 0x4B000000u, 0x7650u + byte)), minus);
                            part2 = q4_ffma2(q2, q4_pack2(xe, xe), part2);
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
            const uint32_t row = group * R + r;
            if (lane == 0 && row < p.n) {
                if constexpr (OUT == HB_OUT_F32) reinterpret_cast<float*>(p.y)[row] = a;
                else if constexpr (OUT == HB_OUT_BF16) reinterpret_cast<uint16_t*>(p.y)[row] = (uint16_t)f32_to_bf16(a);
                else {
                    uint16_t* y = reinterpret_cast<uint16_t*>(p.y) + row;
                    *y = (uint16_t)f32_to_bf16(__fadd_rn(bf16_to_f32(*y), round_bf16(a)));
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
    uint32_t k = 0, n = 0, out = 0, rows = 0;
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
        const uint32_t grid = std::max(1u, std::min<uint32_t>((p.groups + Q4_WARPS - 1) / Q4_WARPS, (uint32_t)ctx->sm_count * 8));
        HB_CUDA(ctx, launch_kernel(ctx, true, fn, dim3(grid), dim3(Q4_THREADS), 0, p));
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

int make_matvec_q4(hb_ctx* ctx, uint32_t k, uint32_t n, uint32_t out_mode, uint32_t rows, uint32_t masks, hb_kernel** out) {
    *out = nullptr;
    if (k == 0 || n == 0 || k % 32 != 0) return fail(ctx, HB_UNSUPPORTED, "Q4: K = " + std::to_string(k) + " is not a multiple of 32");
    if (rows == 0) rows = 2;
    q4_fn fn = masks ? q4_rows<true>(rows, out_mode) : q4_rows<false>(rows, out_mode);
    if (!fn) return fail(ctx, HB_UNSUPPORTED, "matvec_q4: rows per warp 1, 2 or 4; output Bf16, F32 or Residual");
    auto kn = std::make_unique<MatvecQ4>();
    kn->k = k;
    kn->n = n;
    kn->out = out_mode;
    kn->rows = rows;
    kn->fn = fn;
    kn->kind = 20;
    kn->nargs = 4;
    kn->name = std::string(masks ? "matvec_q4s_" : "matvec_q4_") + std::to_string(k) + "x" + std::to_string(n) + "_" + out_tag(out_mode) + "_r" + std::to_string(rows);
    *out = intern(ctx, std::move(kn));
    return HB_OK;
}

}  // namespace hb

extern "C" {

int hb_dequant_q4_get(hb_ctx* ctx, uint32_t k, uint32_t n, hb_kernel** out) {
    if (!ctx || !out) return hb::fail(ctx, HB_INVALID, "hb_dequant_q4_get: bad argument");
    try {
        return hb::make_dequant_q4(ctx, k, n, out);
    } catch (const std::exception& e) {
        return hb::fail(ctx, HB_BACKEND, e.what());
    }
}

int hb_matvec_q4_get(hb_ctx* ctx, uint32_t k, uint32_t n, uint32_t out_mode, uint32_t rows_per_warp, uint32_t masks, hb_kernel** out) {
    if (!ctx || !out) return hb::fail(ctx, HB_INVALID, "hb_matvec_q4_get: bad argument");
    try {
        return hb::make_matvec_q4(ctx, k, n, out_mode, rows_per_warp, masks, out);
    } catch (const std::exception& e) {
        return hb::fail(ctx, HB_BACKEND, e.what());
    }
}

}  // extern "C"
