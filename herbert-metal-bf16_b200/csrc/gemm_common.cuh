// Shared by the dense prefill GEMM kernels: launch parameters, tile constants, barrier block and the
// epilogue that applies the output mode to 32 consecutive accumulator columns of one row
// (reference src/metal/kernels.rs:217-234, src/metal/prefill.rs:1200-1230).
#pragma once

#include "hb_internal.hpp"
#include "tc05.cuh"

namespace hb {

struct GemmParams {
    void* y;
    uint32_t m, n_w;      // rows of X, rows of W
    uint32_t n_out;       // columns (and row stride) of Y
    uint32_t k_blocks;    // ceil(k / 64)
    uint32_t tiles_m, tiles_n, num_tiles;
    uint32_t stages;
    uint32_t m_first;
    uint32_t vec_ok;      // Y rows allow 16-byte accesses
    uint32_t* status;
    // Out::F32 only: Y cut into blocks of shard_rows rows, block b stored at address y_shards[b] (a device array);
    // the blocks may be other GPUs' memory (a row-parallel projection pushes each block of its partial product
    // to the rank that will sum it). Null: Y is one array at y.
    const uint64_t* y_shards;
    uint32_t shard_rows;
    // y_shards with the rows dealt in groups (hb_gemm_desc.y_group_rows): group_rows = G, group_part = G / P rows of
    // every group per block; 0 = contiguous blocks of shard_rows rows
    uint32_t group_rows, group_part;
    // y_signal: where to tell the summing ranks that a group of rows is complete
    const uint64_t* flag_table;  // [world] -> u32[world][TP_MAX_GROUPS] on every rank
    uint32_t* ctl;               // this rank's control words: [0] steps completed, [TP_CTL_GROUP0 + g] arrivals of group g
    uint32_t world, rank;
    // split_k = S > 1 (the CTA-pair form): a work item is (tile, one of S equal slices of K); the slices of a tile hand a
    // running f32 sum from one to the next through `partial` and the last applies the output mode.
    // partial: [tiles][2][4] blocks of 32 x 256 f32; split_counters: [tiles][2][4], slices done, zero between launches.
    uint32_t split_k;
    float* partial;
    uint32_t* split_counters;
};

constexpr uint32_t TP_MAX_GROUPS = 64;   // HB_TP_MAX_GROUPS
constexpr uint32_t TP_CTL_DONE = 1;      // of ctl: blocks of the summing kernel that have finished
constexpr uint32_t TP_CTL_GROUP0 = 8;    // of ctl: first of the per-group arrival counters

// Where row `row` of a Y in row blocks lives: the block's base address and the row inside the block.
__device__ __forceinline__ float* shard_row(const GemmParams& p, uint32_t row) {
    uint32_t block, local;
    if (p.group_rows) {
        const uint32_t g = row / p.group_rows, in = row % p.group_rows;
        block = in / p.group_part;
        local = g * p.group_part + in % p.group_part;
    } else {
        block = row / p.shard_rows;
        local = row % p.shard_rows;
    }
    return reinterpret_cast<float*>(p.y_shards[block]) + (size_t)local * p.n_out;
}

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int A_BYTES = BM * BK * 2;
constexpr int MAX_STAGES = 10;
constexpr int GEMM_THREADS = 192;

struct __align__(8) GemmBarriers {
    uint64_t full[MAX_STAGES];
    uint64_t empty[MAX_STAGES];
    uint64_t tmem_full[2];
    uint64_t tmem_empty[2];
    uint32_t tmem_base;
    uint32_t abort;
};

// Stores 32 consecutive outputs of one row. v[] are the f32 accumulators (or for SWIGLU the
// gate accumulators, u[] the up ones).
template <int OUT>
__device__ __forceinline__ void store_chunk(const GemmParams& p, uint32_t row, uint32_t col0, const uint32_t (&v)[32], const uint32_t (&u)[32]) {
    if (row >= p.m || col0 >= p.n_out) return;
    const uint32_t ncols = min(32u, p.n_out - col0);
    if constexpr (OUT == HB_OUT_F32) {
        float* y = p.y_shards ? shard_row(p, row) + col0 : reinterpret_cast<float*>(p.y) + (size_t)row * p.n_out + col0;
        if (ncols == 32 && p.vec_ok) {
#pragma unroll
            for (int i = 0; i < 8; ++i)
                reinterpret_cast<uint4*>(y)[i] = make_uint4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
        } else {
            for (uint32_t i = 0; i < ncols; ++i) y[i] = __uint_as_float(v[i]);
        }
    } else {
        uint16_t* y = reinterpret_cast<uint16_t*>(p.y) + (size_t)row * p.n_out + col0;
        uint32_t o[32];
        if constexpr (OUT == HB_OUT_BF16) {
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = f32_to_bf16(__uint_as_float(v[i]));
        } else if constexpr (OUT == HB_OUT_SWIGLU) {
#pragma unroll
            for (int i = 0; i < 32; ++i)
                o[i] = swiglu_bf16(round_bf16(__uint_as_float(v[i])), round_bf16(__uint_as_float(u[i])));
        } else {  // RESIDUAL: y = bf16(f32(y_old) + f32(bf16(acc)))
            uint32_t old[32];
            if (ncols == 32 && p.vec_ok) {
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    uint4 q = reinterpret_cast<const uint4*>(y)[i];
                    uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        old[8 * i + 2 * j] = w[j] & 0xffffu;
                        old[8 * i + 2 * j + 1] = w[j] >> 16;
                    }
                }
            } else {
#pragma unroll
                for (int i = 0; i < 32; ++i) old[i] = (uint32_t)i < ncols ? y[i] : 0u;
            }
#pragma unroll
            for (int i = 0; i < 32; ++i)
                o[i] = f32_to_bf16(__fadd_rn(bf16_to_f32(old[i]), round_bf16(__uint_as_float(v[i]))));
        }
        if (ncols == 32 && p.vec_ok) {
#pragma unroll
            for (int i = 0; i < 4; ++i)
                reinterpret_cast<uint4*>(y)[i] = make_uint4(o[8 * i] | (o[8 * i + 1] << 16), o[8 * i + 2] | (o[8 * i + 3] << 16),
                                                            o[8 * i + 4] | (o[8 * i + 5] << 16), o[8 * i + 6] | (o[8 * i + 7] << 16));
        } else {
#pragma unroll
            for (int i = 0; i < 32; ++i)
                if ((uint32_t)i < ncols) y[i] = (uint16_t)o[i];
        }
    }
}

// Out::F32 into row blocks that may be other GPUs' memory: the 32 rows x 32 columns a warp holds (one row per lane)
// go through 4 KB of the warp's shared memory and leave as whole 128-byte row segments, four rows per store
// instruction. Stored lane by lane they would be 32 separate 16-byte writes per instruction, which NVLink carries
// one small packet each. `scratch` is the shared-memory address of the warp's 4 KB (16-byte chunks, xor-swizzled).
__device__ __forceinline__ void store_chunk_f32_blocks(const GemmParams& p, uint32_t row0, uint32_t col0, const uint32_t (&v)[32], uint32_t scratch) {
    const uint32_t lane = threadIdx.x & 31u;
#pragma unroll
    for (uint32_t j = 0; j < 8; ++j)
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(scratch + ((lane * 8u + (j ^ (lane & 7u))) << 4)), "r"(v[4 * j]), "r"(v[4 * j + 1]),
                     "r"(v[4 * j + 2]), "r"(v[4 * j + 3])
                     : "memory");
    __syncwarp();
    const uint32_t c = lane & 7u;
#pragma unroll
    for (uint32_t i = 0; i < 8; ++i) {
        const uint32_t r = 4u * i + (lane >> 3);
        uint4 q;
        asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(q.x), "=r"(q.y), "=r"(q.z), "=r"(q.w) : "r"(scratch + ((r * 8u + (c ^ (r & 7u))) << 4)));
        const uint32_t row = row0 + r, col = col0 + 4u * c;
        if (row < p.m && col < p.n_out) {
            float* y = shard_row(p, row) + col;
            if (p.vec_ok && col + 4u <= p.n_out) {
                *reinterpret_cast<uint4*>(y) = q;
            } else {
                const uint32_t w[4] = {q.x, q.y, q.z, q.w};
                for (uint32_t e = 0; e < 4u && col + e < p.n_out; ++e) y[e] = __uint_as_float(w[e]);
            }
        }
    }
    __syncwarp();
}

}  // namespace hb
