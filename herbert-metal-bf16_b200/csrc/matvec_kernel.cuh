// The decode matvec's kernel template and launch parameters, shared by the translation units that instantiate it
// (matvec.cu: x as it is bound; matvec_fused_x.cu: x made inside the kernel from the residual stream or from
// [gate | up], the reference's XSrc::Norm and XSrc::Swiglu, src/metal/kernels.rs:236-252).
#pragma once

#include <algorithm>

#include "hb_internal.hpp"
#include "rowwise.cuh"
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
    // x made inside the kernel (XSRC != 0): the weights of the norm, its eps, whether 1 is added to them
    const uint16_t* norm_w;
    float eps;
    uint32_t plus_one;
};

// What the x binding holds (reference enum XSrc, src/metal/kernels.rs:236-252).
enum : int { XSRC_PLAIN = 0, XSRC_NORM = 1, XSRC_SWIGLU = 2 };

__device__ __forceinline__ uint4 ldg_stream(const uint4* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.L2::128B.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

constexpr int MV_THREADS = 256;
constexpr int MV_WARPS = MV_THREADS / 32;

// XSRC_NORM: x is the residual stream and the projection's input is its RMSNorm; XSRC_SWIGLU: x is [gate (k) | up (k)]
// and the input is bf16(g * sigmoid(g) * u). Every block first makes its input rows in shared memory (the norm's sums
// in rmsnorm_rows' order, the SwiGLU as swiglu_rows computes it: the same bits as the separate kernels) and reads
// them from there: one launch less, and no round trip of the rows through memory.
template <int M, int R, int OUT, bool ARGMAX = false, int XSRC = XSRC_PLAIN>
__global__ void __launch_bounds__(MV_THREADS) matvec_kernel(const MatvecParams p) {
    __shared__ float part[MV_WARPS][R * M];
    extern __shared__ uint4 xs_dyn[];  // XSRC != 0: the input rows, [M][k] bf16
    __shared__ unsigned long long best_s[ARGMAX ? MV_WARPS : 1][M];
    unsigned long long best[M];
#pragma unroll
    for (int i = 0; i < M; ++i) best[i] = 0ull;
    griddep_launch_dependents();
    griddep_wait();  // x comes from the kernel before this one
    if constexpr (XSRC == XSRC_NORM) {
        __shared__ float npart[M * 9];
        norm_rows_into<M>(reinterpret_cast<const uint16_t*>(p.x), (size_t)p.k8 * 8, p.norm_w, p.m, p.k8 * 8, p.eps, p.plus_one != 0, reinterpret_cast<uint16_t*>(xs_dyn), npart);
    } else if constexpr (XSRC == XSRC_SWIGLU) {
        for (uint32_t i = threadIdx.x; i < p.m * p.k8; i += MV_THREADS) {
            const uint32_t r = i / p.k8, c = i - r * p.k8;
            const uint4 gv = __ldg(p.x + (size_t)r * 2 * p.k8 + c), uv = __ldg(p.x + (size_t)r * 2 * p.k8 + p.k8 + c);
            const uint32_t gw[4] = {gv.x, gv.y, gv.z, gv.w}, uw[4] = {uv.x, uv.y, uv.z, uv.w};
            uint32_t o[4];
#pragma unroll
            for (int j = 0; j < 4; ++j)
                o[j] = swiglu_bf16(__uint_as_float(gw[j] << 16), __uint_as_float(uw[j] << 16)) |
                       (swiglu_bf16(__uint_as_float(gw[j] & 0xffff0000u), __uint_as_float(uw[j] & 0xffff0000u)) << 16);
            xs_dyn[i] = make_uint4(o[0], o[1], o[2], o[3]);
        }
        __syncthreads();
    }
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
                        const uint4 xv = XSRC == XSRC_PLAIN ? __ldg(p.x + (size_t)i * p.k8 + c) : xs_dyn[(size_t)i * p.k8 + c];
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

}  // namespace hb
