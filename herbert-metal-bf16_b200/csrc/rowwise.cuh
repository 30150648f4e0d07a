// Row-wise helpers shared by the kernels that sum over a row in the reference's order: a group of 256 (virtual)
// lanes, lane l an FMA chain over elements l, l + 256, ..., the 32 lanes of a simdgroup summed by the xor butterfly,
// the 8 partials folded in order (reference src/msl/mod.rs:716-756).
#pragma once

#include "hb_internal.hpp"
#include "tc05.cuh"

namespace hb {

constexpr int ROW_THREADS = 256;

// The group's sum of one f32 per thread, in the reference's order. `part` is shared scratch of 9 floats.
__device__ __forceinline__ float group_sum256(float v, float* part) {
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, off));
    if (lane == 0) part[warp] = v;
    __syncthreads();
    if (threadIdx.x == 0) {
        float acc = part[0];
#pragma unroll
        for (int g = 1; g < 8; ++g) acc = __fadd_rn(acc, part[g]);
        part[8] = acc;
    }
    __syncthreads();
    const float r = part[8];
    __syncthreads();  // the scratch can be reused right after
    return r;
}

// Copies a row of d bf16 into shared memory (16-byte pieces when the row allows).
__device__ __forceinline__ void stage_row(uint16_t* dst, const uint16_t* src, uint32_t d, bool vec) {
    if (vec) {
        for (uint32_t i = threadIdx.x; i < d / 8; i += ROW_THREADS) reinterpret_cast<uint4*>(dst)[i] = reinterpret_cast<const uint4*>(src)[i];
    } else {
        for (uint32_t i = threadIdx.x; i < d; i += ROW_THREADS) dst[i] = src[i];
    }
}

// RMSNorm of `rows` (at most MAXR) rows of d elements (d a multiple of 8) by all threads of the block, whatever their
// number (a multiple of 32, at most 256): the sums in rmsnorm_rows' order (each warp plays the simdgroups w, w + warps,
// ... of the reference's group of 256), y = bf16((x * inv) * (w [+ 1])), inv = 1 / sqrt(sum(x^2) * (1/d) + eps)
// (reference src/metal/kernels.rs:355-442, norm_into). x: rows ldx apart; dst (shared or global memory): rows d apart;
// part: shared scratch of MAXR * 9 floats. Ends with a __syncthreads().
template <int MAXR>
__device__ __forceinline__ void norm_rows_into(const uint16_t* __restrict__ x, size_t ldx, const uint16_t* __restrict__ w, uint32_t rows, uint32_t d, float eps,
                                               bool plus_one, uint16_t* dst, float* part) {
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    for (uint32_t vw = warp; vw < 8; vw += nwarps) {
        float acc[MAXR];
#pragma unroll
        for (int r = 0; r < MAXR; ++r) acc[r] = 0.f;
        for (uint32_t i = vw * 32 + lane; i < d; i += 256) {
#pragma unroll
            for (int r = 0; r < MAXR; ++r) {
                if ((uint32_t)r < rows) {
                    const float v = bf16_to_f32(x[(size_t)r * ldx + i]);
                    acc[r] = __fmaf_rn(v, v, acc[r]);
                }
            }
        }
#pragma unroll
        for (int r = 0; r < MAXR; ++r) {
            float v = acc[r];
#pragma unroll
            for (int off = 16; off >= 1; off >>= 1) v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, off));
            if (lane == 0) part[r * 9 + vw] = v;
        }
    }
    __syncthreads();
    if (threadIdx.x < rows) {
        float a = part[threadIdx.x * 9];
#pragma unroll
        for (int g = 1; g < 8; ++g) a = __fadd_rn(a, part[threadIdx.x * 9 + g]);
        part[threadIdx.x * 9 + 8] = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fmul_rn(a, 1.0f / (float)d), eps)));
    }
    __syncthreads();
    const uint32_t d8 = d / 8;
    for (uint32_t i = threadIdx.x; i < rows * d8; i += blockDim.x) {
        const uint32_t r = i / d8, c = i - r * d8;
        const float inv = part[r * 9 + 8];
        const uint4 xv = *reinterpret_cast<const uint4*>(x + (size_t)r * ldx + c * 8);
        const uint4 wv = *reinterpret_cast<const uint4*>(w + c * 8);
        const uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w}, ww[4] = {wv.x, wv.y, wv.z, wv.w};
        uint32_t o[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            float w0 = __uint_as_float(ww[j] << 16), w1 = __uint_as_float(ww[j] & 0xffff0000u);
            if (plus_one) { w0 = __fadd_rn(w0, 1.0f); w1 = __fadd_rn(w1, 1.0f); }
            const float n0 = __fmul_rn(__uint_as_float(xw[j] << 16), inv), n1 = __fmul_rn(__uint_as_float(xw[j] & 0xffff0000u), inv);
            o[j] = f32x2_to_bf16x2(__fmul_rn(n0, w0), __fmul_rn(n1, w1));
        }
        *reinterpret_cast<uint4*>(dst + (size_t)r * d + c * 8) = make_uint4(o[0], o[1], o[2], o[3]);
    }
    __syncthreads();
}

}  // namespace hb
