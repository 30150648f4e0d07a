// Decode-time products with a few activation rows (1..64) on the tensor cores: Y[m][n] = out(X[m][k] . W[n][k]^T).
//
// The reference's matvec (src/metal/kernels.rs:146-214, 502-981) multiplies one activation row; its multi-row twin
// exists only for Q4 weights (kernels.rs:990). With 4 or 8 rows a CUDA-core kernel spends 4 or 8 FMAs per weight
// element and becomes issue-bound long before HBM is busy. Here the weights are the 128-row operand of tcgen05.mma
// and the activation rows its narrow N side (16, 32 or 64 columns, rows past m zero-filled by TMA): the arithmetic
// is free and the kernel is a pure weight stream - 16 KB TMA boxes of W into a ring of up to 12 stages, 2..8 KB of
// X beside each. One persistent CTA per SM:
//   warp 0    TMA producer;   warp 1    MMA issuer (TMEM: two accumulator sets, so an epilogue overlaps the next item);
//   warps 2-5 epilogue: TMEM lane = output feature, TMEM column = activation row.
// Work is dealt in one of two ways. Whole blocks: a CTA takes 128 features over all of K, block after block (best
// when n / 128 is many times the SM count). Balanced: the (feature block, 64-element k-block) units are cut into one
// contiguous range per CTA, all equal, so every SM streams the same number of bytes whatever n is; a block shared by
// several CTAs gets its f32 partials through scratch: each contributor stores its partial and bumps a counter, and
// whichever arrives last adds the partials in K order (the same order whoever is last) and applies the output
// mode (src/metal/kernels.rs:217-234). Nobody waits for anybody: no spin, only the bounded pipeline waits.
#include <algorithm>
#include <cstring>
#include <vector>

#include "hb_internal.hpp"
#include "rowwise.cuh"
#include "tc05.cuh"

namespace hb {

constexpr int SK_THREADS = 192;
constexpr int SK_MAX_STAGES = 12;
constexpr int SK_A_BYTES = 128 * 64 * 2;
constexpr int SK_SEG_CACHE = 32;

// A CTA's piece of work: k-blocks [kb0, kb1) of feature block fb. With nslots > 1 the block is shared: this CTA is
// contributor number `slot` of `nslots`, in the order of the K ranges.
struct SkinnySeg {
    uint32_t fb, kb0, kb1, slot, nslots;
};

struct SkinnyParams {
    void* y;
    uint32_t m, n_out;
    uint32_t k_blocks, feat_blocks, stages;
    uint32_t block_rows;  // W rows (output features) per feature block: 128, or fewer so that the blocks fill whole waves of CTAs
    uint32_t balanced;    // 0: a CTA takes whole feature blocks; 1: the (feature block, k-block) units are dealt evenly
    uint32_t maxslots;    // balanced: the most CTAs that share one feature block
    float* scratch;       // balanced: [feat_blocks][maxslots][NACC * NP][128]
    uint32_t* counters;   // balanced: [feat_blocks][4], zero between launches
    uint32_t* status;
    const uint32_t* seg_start;   // [grid + 1]: where each CTA's segments begin in `segs` (worked out on the host once)
    const SkinnySeg* segs;
    // NORM: the input rows are the RMSNorm of x_raw [m][k], made by every CTA into xn (which the X descriptor covers)
    const uint16_t* x_raw;
    const uint16_t* norm_w;
    uint16_t* xn;
    uint32_t k, plus_one;
    float eps;
};

__host__ __device__ __forceinline__ uint32_t skinny_cta_of(uint64_t u, uint64_t units, uint32_t grid) {
    uint32_t c = (uint32_t)(((u + 1) * grid - 1) / units);
    while (c > 0 && (uint64_t)c * units / grid > u) --c;
    while (c + 1 < grid && (uint64_t)(c + 1) * units / grid <= u) ++c;
    return c;
}

// Segment i of CTA `cta`; returns the number of segments (out may be null).
__host__ __device__ __forceinline__ uint32_t skinny_seg(const SkinnyParams& p, uint32_t cta, uint32_t grid, uint32_t i, SkinnySeg* out) {
    const uint32_t KB = p.k_blocks;
    if (!p.balanced) {
        const uint32_t n = cta < p.feat_blocks ? (p.feat_blocks - cta + grid - 1) / grid : 0;
        if (out && i < n) *out = SkinnySeg{cta + i * grid, 0, KB, 0, 1};
        return n;
    }
    const uint64_t units = (uint64_t)p.feat_blocks * KB;
    const uint64_t u0 = (uint64_t)cta * units / grid, u1 = (uint64_t)(cta + 1) * units / grid;
    if (u1 <= u0) return 0;
    const uint32_t fb0 = (uint32_t)(u0 / KB), fb1 = (uint32_t)((u1 - 1) / KB);
    const uint32_t n = fb1 - fb0 + 1;
    if (out && i < n) {
        const uint32_t fb = fb0 + i;
        out->fb = fb;
        out->kb0 = i == 0 ? (uint32_t)(u0 - (uint64_t)fb0 * KB) : 0;
        const uint64_t rest = u1 - (uint64_t)fb * KB;
        out->kb1 = rest < KB ? (uint32_t)rest : KB;
        const uint32_t c_first = skinny_cta_of((uint64_t)fb * KB, units, grid), c_last = skinny_cta_of((uint64_t)(fb + 1) * KB - 1, units, grid);
        out->slot = cta - c_first;
        out->nslots = c_last - c_first + 1;
    }
    return n;
}

struct __align__(8) SkinnyBarriers {
    uint64_t full[SK_MAX_STAGES];
    uint64_t empty[SK_MAX_STAGES];
    uint64_t tmem_full[2];
    uint64_t tmem_empty[2];
    uint32_t tmem_base;
};

template <int NP>
__device__ __forceinline__ void skinny_ld(uint32_t taddr, uint32_t (&v)[NP]) {
    if constexpr (NP == 16) {
        tmem_ld_32x16(taddr, v);
    } else if constexpr (NP == 32) {
        tmem_ld_32x32(taddr, v);
    } else {
        uint32_t a[32], b[32];
        tmem_ld_32x32(taddr, a);
        tmem_ld_32x32(taddr + 32, b);
#pragma unroll
        for (int i = 0; i < 32; ++i) { v[i] = a[i]; v[32 + i] = b[i]; }
    }
}

// One output element of row j, feature f: the output mode applied to the finished sums.
template <int OUT>
__device__ __forceinline__ void skinny_store(const SkinnyParams& p, uint32_t j, uint32_t f, float g, float u) {
    if constexpr (OUT == HB_OUT_F32) {
        reinterpret_cast<float*>(p.y)[(size_t)j * p.n_out + f] = g;
    } else {
        uint16_t* y = reinterpret_cast<uint16_t*>(p.y) + (size_t)j * p.n_out + f;
        uint32_t o;
        if constexpr (OUT == HB_OUT_BF16) o = f32_to_bf16(g);
        else if constexpr (OUT == HB_OUT_SWIGLU) o = swiglu_bf16(round_bf16(g), round_bf16(u));
        else o = f32_to_bf16(__fadd_rn(bf16_to_f32(*y), round_bf16(g)));
        *y = (uint16_t)o;
    }
}

// NORM (the reference's XSrc::Norm, src/metal/kernels.rs:236-252, 355-442): x is the residual stream. Every CTA makes
// the normalised rows itself (rmsnorm_rows' sums in their order, so the same bits as the separate kernel) and writes
// them to one scratch array the X descriptor covers; all CTAs write the same values, and a CTA's TMA reads follow its
// own writes. The first weight boxes are in flight before that starts.
template <int OUT, int NP, int KPS, bool NORM = false>
__global__ void __launch_bounds__(SK_THREADS, 1)
gemm_skinny_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x, const SkinnyParams p) {
    constexpr int NACC = OUT == HB_OUT_SWIGLU ? 2 : 1;
    constexpr int A_STAGE = NACC * SK_A_BYTES;
    constexpr int B_BYTES = NP * 128;
    constexpr int KB_BYTES = A_STAGE + B_BYTES;       // one 64-element k-block of W and X
    constexpr int STAGE_BYTES = KPS * KB_BYTES;       // a stage holds KPS neighbouring k-blocks: longer runs per W row in DRAM
    constexpr uint32_t SET_COLS = NACC * NP;
    constexpr uint32_t TMEM_COLS = 2 * SET_COLS < 32 ? 32 : 2 * SET_COLS;
    constexpr uint32_t IDESC = umma_idesc_bf16(128, NP);

    extern __shared__ uint8_t smem_raw[];
    __shared__ SkinnyBarriers bars;
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t S = p.stages;

    // this CTA's segments. Whole feature blocks per CTA: block c, c + grid, ... over all of K, worked out here. Balanced
    // units: the table made on the host when the kernel object was made (it depends on n, k and the grid only); the
    // first SK_SEG_CACHE entries are copied to shared memory for the three roles.
    __shared__ SkinnySeg segs_s[SK_SEG_CACHE];
    const bool table = p.balanced != 0;
    const uint32_t seg0 = table ? p.seg_start[blockIdx.x] : 0u;
    const uint32_t n_segs = table ? p.seg_start[blockIdx.x + 1] - seg0
                                  : (blockIdx.x < p.feat_blocks ? (p.feat_blocks - blockIdx.x + gridDim.x - 1) / gridDim.x : 0u);
    auto seg_at = [&](uint32_t i, SkinnySeg* out) {
        if (!table) *out = SkinnySeg{blockIdx.x + i * gridDim.x, 0u, p.k_blocks, 0u, 1u};
        else *out = i < (uint32_t)SK_SEG_CACHE ? segs_s[i] : p.segs[seg0 + i];
    };
    // The stage fills of this CTA, in order. The first S of them find their stage free; their weight boxes do
    // not depend on the kernel before this one on the stream, so they are issued first (pass 0), then the
    // predecessor is waited for, then their activation boxes follow (pass 1) and the rest of the fills (pass 2).
    auto walk = [&](int pass) -> bool {
        uint32_t s = 0, ph = 0, fill = 0;
        for (uint32_t i = 0; i < n_segs; ++i) {
            SkinnySeg sg;
            seg_at(i, &sg);
            const uint32_t fb = sg.fb, kb0 = sg.kb0, kb1 = sg.kb1;
            const int row_w0 = (int)(fb * p.block_rows);
            const int row_w1 = (int)(p.n_out + fb * p.block_rows);  // SWIGLU: the up rows of the same features
            for (uint32_t kb = kb0; kb < kb1; kb += KPS, ++fill) {
                const bool early = fill < S;
                if (pass != 2 && !early) return true;
                const bool do_w = pass == 0 || (pass == 2 && !early), do_x = pass == 1 || (pass == 2 && !early);
                if (pass == 2 && !early && !mbar_wait(smem_u32(&bars.empty[s]), ph ^ 1u)) {
                    report(p.status, ST_WAIT_TIMEOUT, WHERE_EMPTY, s);
                    return false;
                }
                const uint32_t full = smem_u32(&bars.full[s]);
                const uint32_t nkb = min((uint32_t)KPS, kb1 - kb);
                // (a W box is block_rows rows; the rest of its 128-row slot is never written, and the rows of the
                // accumulator that come from it are never read)
                if (do_w) mbar_arrive_expect_tx(full, nkb * (NACC * p.block_rows * 128u + B_BYTES));
#pragma unroll
                for (uint32_t j = 0; j < (uint32_t)KPS; ++j) {
                    if (j < nkb) {
                        const uint32_t dst = smem_base + s * STAGE_BYTES + j * KB_BYTES;
                        if (do_w) {
                            tma_load_2d(dst, &tm_w, full, (int)((kb + j) * 64), row_w0);
                            if (NACC == 2) tma_load_2d(dst + SK_A_BYTES, &tm_w, full, (int)((kb + j) * 64), row_w1);
                        }
                        if (do_x) tma_load_2d(dst + A_STAGE, &tm_x, full, (int)((kb + j) * 64), 0);
                    }
                }
                if (++s == S) { s = 0; ph ^= 1u; }
            }
        }
        return true;
    };
    // Set-up. Thread 0 makes the barriers and, where nothing else is needed to know this CTA's work (whole blocks, no
    // fused norm), requests the weight boxes of the first fills at once: before tensor memory is allocated and before
    // the first block-wide barrier (a weight stream of 100 MB is 15 us long: every microsecond before its first byte counts).
    bool early_w = false;
    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < S; ++s) {
            mbar_init(smem_u32(&bars.full[s]), 1);
            mbar_init(smem_u32(&bars.empty[s]), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(smem_u32(&bars.tmem_full[a]), 1);
            mbar_init(smem_u32(&bars.tmem_empty[a]), 4);
        }
        fence_mbar_init();
        fence_proxy_async();
        if (!table && !NORM) {
            tma_prefetch_desc(&tm_w);
            tma_prefetch_desc(&tm_x);
            walk(0);
            early_w = true;
        }
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(&bars.tmem_base), TMEM_COLS);
        tmem_relinquish();
    }
    if (table && threadIdx.x < min(n_segs, (uint32_t)SK_SEG_CACHE)) segs_s[threadIdx.x] = p.segs[seg0 + threadIdx.x];
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = bars.tmem_base;
    griddep_launch_dependents();

    if constexpr (NORM) {
        if (warp == 0 && lane == 0) {
            tma_prefetch_desc(&tm_w);
            tma_prefetch_desc(&tm_x);
            walk(0);
        }
        griddep_wait();
        __shared__ float npart[NP * 9];
        norm_rows_into<NP>(p.x_raw, p.k, p.norm_w, p.m, p.k, p.eps, p.plus_one != 0, p.xn, npart);
        // written through the generic proxy, read by TMA
        __threadfence();
        asm volatile("fence.proxy.async;" ::: "memory");
        __syncthreads();
    }
    if (warp == 0) {
        if (lane == 0) {
            if constexpr (!NORM) {
                if (!early_w) {
                    tma_prefetch_desc(&tm_w);
                    tma_prefetch_desc(&tm_x);
                    walk(0);
                }
                griddep_wait();
            }
            walk(1);
            walk(2);
        }
    } else if (warp == 1) {
        if (lane == 0) {
            uint32_t s = 0, ph = 0, it = 0;
            bool ok = true;
            for (; ok && it < n_segs; ++it) {
                SkinnySeg sg;
                seg_at(it, &sg);
                const uint32_t kb0 = sg.kb0, kb1 = sg.kb1;
                const uint32_t acc = it & 1u, acc_ph = (it >> 1) & 1u;
                if (!mbar_wait(smem_u32(&bars.tmem_empty[acc]), acc_ph ^ 1u)) {
                    report(p.status, ST_WAIT_TIMEOUT, WHERE_TMEM_EMPTY, acc);
                    break;
                }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * SET_COLS;
                for (uint32_t kb = kb0; kb < kb1; kb += KPS) {
                    if (!mbar_wait(smem_u32(&bars.full[s]), ph)) {
                        report(p.status, ST_WAIT_TIMEOUT, WHERE_FULL, s);
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t nkb = min((uint32_t)KPS, kb1 - kb);
#pragma unroll
                    for (uint32_t i = 0; i < (uint32_t)KPS; ++i) {
                        if (i < nkb) {
                            const uint32_t a_addr = smem_base + s * STAGE_BYTES + i * KB_BYTES;
                            const uint64_t a_desc = umma_desc_sw128(a_addr);
                            const uint64_t b_desc = umma_desc_sw128(a_addr + A_STAGE);
#pragma unroll
                            for (uint32_t k4 = 0; k4 < 4; ++k4) {
                                const uint32_t accum = (kb + i != kb0 || k4 != 0) ? 1u : 0u;
                                umma_bf16(d_tmem, a_desc + 2 * k4, b_desc + 2 * k4, IDESC, accum);
                                if (NACC == 2) umma_bf16(d_tmem + NP, umma_desc_sw128(a_addr + SK_A_BYTES) + 2 * k4, b_desc + 2 * k4, IDESC, accum);
                            }
                        }
                    }
                    umma_commit(smem_u32(&bars.empty[s]));
                    if (++s == S) { s = 0; ph ^= 1u; }
                }
                if (ok) umma_commit(smem_u32(&bars.tmem_full[acc]));
            }
        }
    } else {
        const uint32_t q = (uint32_t)warp & 3u;
        uint32_t it = 0;
        griddep_wait();  // Y may be read (residual) or still be in use by the kernel before this one
        for (; it < n_segs; ++it) {
            SkinnySeg sg;
            seg_at(it, &sg);
            const uint32_t fb = sg.fb;
            const uint32_t acc = it & 1u, acc_ph = (it >> 1) & 1u;
            const bool got = mbar_wait(smem_u32(&bars.tmem_full[acc]), acc_ph);
            if (!__all_sync(0xffffffffu, got)) {
                if (lane == 0) report(p.status, ST_WAIT_TIMEOUT, WHERE_TMEM_FULL, acc);
                break;
            }
            tc_fence_after();
            const uint32_t t_addr = tmem_base + ((q * 32u) << 16) + acc * SET_COLS;
            uint32_t g[NP], u[NP];
            skinny_ld<NP>(t_addr, g);
            if (NACC == 2) skinny_ld<NP>(t_addr + NP, u);
            tmem_ld_wait();
            // the accumulator is in registers: the MMA warp may have the set back
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&bars.tmem_empty[acc]));
            const uint32_t f = fb * p.block_rows + q * 32 + lane;
            if (sg.nslots == 1) {
                if (q * 32 + lane < p.block_rows && f < p.n_out) {
#pragma unroll
                    for (int j = 0; j < NP; ++j)
                        if ((uint32_t)j < p.m) skinny_store<OUT>(p, j, f, __uint_as_float(g[j]), NACC == 2 ? __uint_as_float(u[j]) : 0.f);
                }
                continue;
            }
            // this CTA's partial of the block: [set row a * NP + j][128 features], this warp's 32 features of each row
            float* mine = p.scratch + ((size_t)fb * p.maxslots + sg.slot) * (NACC * NP) * 128 + q * 32 + lane;
#pragma unroll
            for (int j = 0; j < NP; ++j) {
                if ((uint32_t)j < p.m) {
                    mine[(size_t)j * 128] = __uint_as_float(g[j]);
                    if (NACC == 2) mine[(size_t)(NP + j) * 128] = __uint_as_float(u[j]);
                }
            }
            __threadfence();
            __syncwarp();
            uint32_t arrived = 0;
            if (lane == 0) arrived = atomicAdd(&p.counters[fb * 4 + q], 1u);
            arrived = __shfl_sync(0xffffffffu, arrived, 0);
            if (arrived + 1 != sg.nslots) continue;
            // last of this feature quarter: every contributor's partial is in memory; add them in K order
            __threadfence();
            if (lane == 0) p.counters[fb * 4 + q] = 0;
            const float* part = p.scratch + (size_t)fb * p.maxslots * (NACC * NP) * 128 + q * 32 + lane;
            // contributor by contributor (the order of the sum), all rows of one at once (independent loads in flight)
            float sg_[NP], su[NACC == 2 ? NP : 1];
#pragma unroll
            for (int j = 0; j < NP; ++j) {
                sg_[j] = 0.f;
                if (NACC == 2) su[j] = 0.f;
            }
            // contributors in batches: all loads of a batch are in flight together, the additions follow in K order
            constexpr uint32_t BATCH = NP <= 16 ? 4 : NP <= 32 ? 2 : 1;
            for (uint32_t k0 = 0; k0 < sg.nslots; k0 += BATCH) {
                float a[BATCH][NP], b[BATCH][NACC == 2 ? NP : 1];
#pragma unroll
                for (uint32_t u = 0; u < BATCH; ++u) {
                    const bool live = k0 + u < sg.nslots;
                    const float* src = part + (size_t)(k0 + u) * (NACC * NP) * 128;
#pragma unroll
                    for (int j = 0; j < NP; ++j) {
                        a[u][j] = live && (uint32_t)j < p.m ? __ldcg(src + (size_t)j * 128) : 0.f;
                        if (NACC == 2) b[u][j] = live && (uint32_t)j < p.m ? __ldcg(src + (size_t)(NP + j) * 128) : 0.f;
                    }
                }
#pragma unroll
                for (uint32_t u = 0; u < BATCH; ++u) {
                    if (k0 + u < sg.nslots) {
                        const bool first = k0 + u == 0;
#pragma unroll
                        for (int j = 0; j < NP; ++j) {
                            sg_[j] = first ? a[u][j] : __fadd_rn(sg_[j], a[u][j]);
                            if (NACC == 2) su[j] = first ? b[u][j] : __fadd_rn(su[j], b[u][j]);
                        }
                    }
                }
            }
            if (f < p.n_out) {
#pragma unroll
                for (int j = 0; j < NP; ++j)
                    if ((uint32_t)j < p.m) skinny_store<OUT>(p, j, f, sg_[j], NACC == 2 ? su[j] : 0.f);
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
}

// ------------------------------------------------------------------ host side

namespace {

typedef void (*skinny_fn)(const CUtensorMap, const CUtensorMap, const SkinnyParams);

template <int NP, int KPS, bool NORM = false>
skinny_fn skinny_pick_out(uint32_t out) {
    switch (out) {
        case HB_OUT_BF16: return gemm_skinny_kernel<HB_OUT_BF16, NP, KPS, NORM>;
        case HB_OUT_F32: return gemm_skinny_kernel<HB_OUT_F32, NP, KPS, NORM>;
        case HB_OUT_RESIDUAL: return gemm_skinny_kernel<HB_OUT_RESIDUAL, NP, KPS, NORM>;
        case HB_OUT_SWIGLU: return gemm_skinny_kernel<HB_OUT_SWIGLU, NP, KPS, NORM>;
    }
    return nullptr;
}

template <int NP>
skinny_fn skinny_pick_kps(uint32_t out, uint32_t kps) {
    return kps == 1 ? skinny_pick_out<NP, 1>(out) : kps == 2 ? skinny_pick_out<NP, 2>(out) : skinny_pick_out<NP, 4>(out);
}
// the fused norm: at most 16 activation rows
skinny_fn skinny_pick_norm(uint32_t out, uint32_t kps) {
    return kps == 1 ? skinny_pick_out<16, 1, true>(out) : kps == 2 ? skinny_pick_out<16, 2, true>(out) : skinny_pick_out<16, 4, true>(out);
}

struct SkinnyGemm : hb_kernel {
    uint32_t k = 0, n = 0, out = 0, rows_max = 0, np = 0, balanced = 0, maxslots = 1, grid_balanced = 0, stages = 0, block_rows = 128;
    skinny_fn fn = nullptr;
    size_t smem = 0;
    float* scratch = nullptr;
    uint32_t* counters = nullptr;
    uint32_t* seg_start = nullptr;
    SkinnySeg* segs = nullptr;
    bool norm = false;         // x is the residual stream: the rows are normalised inside the kernel
    uint16_t* xn = nullptr;    // norm: [np][k], what the X descriptor covers
    float eps = 0.f;
    uint32_t plus_one = 0;
    const void* last_w = nullptr;
    const void* last_x = nullptr;
    uint32_t last_m = 0;
    CUtensorMap tm_w{}, tm_x{};

    int launch(hb_ctx* ctx, const hb_range* a, int na, uint32_t m) override {
        if (na != (norm ? 4 : 3)) return fail(ctx, HB_INVALID, name + (norm ? ": bindings are W, x, y, norm_w" : ": bindings are W, x, y"));
        if (norm && (!range_ok(a[3], (size_t)k * 2) || ((reinterpret_cast<uintptr_t>(a[3].ptr) | reinterpret_cast<uintptr_t>(a[1].ptr)) & 15u)))
            return fail(ctx, HB_INVALID, name + ": norm_w is too small, or x or norm_w is not 16-byte aligned");
        if (m == 0 || m > rows_max) return fail(ctx, HB_INVALID, name + ": m = " + std::to_string(m) + " outside 1.." + std::to_string(rows_max));
        const uint32_t n_out = out == HB_OUT_SWIGLU ? n / 2 : n;
        if (!range_ok(a[0], (size_t)n * k * 2) || !range_ok(a[1], (size_t)m * k * 2) || !range_ok(a[2], (size_t)m * n_out * (out == HB_OUT_F32 ? 4 : 2)))
            return fail(ctx, HB_INVALID, name + ": a bound range is too small for " + std::to_string(m) + " rows");
        if (a[0].ptr != last_w || a[1].ptr != last_x || m != last_m) {
            int r = make_tmap_bf16(ctx, &tm_w, a[0].ptr, n, k, block_rows);
            if (r != HB_OK) return r;
            if ((r = make_tmap_bf16(ctx, &tm_x, norm ? static_cast<const void*>(xn) : a[1].ptr, m, k, np)) != HB_OK) return r;
            last_w = a[0].ptr;
            last_x = a[1].ptr;
            last_m = m;
        }
        SkinnyParams p{};
        p.y = a[2].ptr;
        p.m = m;
        p.n_out = n_out;
        p.k_blocks = (k + 63) / 64;
        p.feat_blocks = (n_out + block_rows - 1) / block_rows;
        p.block_rows = block_rows;
        p.balanced = balanced;
        p.maxslots = maxslots;
        p.stages = stages;
        p.scratch = scratch;
        p.counters = counters;
        p.seg_start = seg_start;
        p.segs = segs;
        p.status = ctx->status_dev;
        if (norm) {
            p.x_raw = static_cast<const uint16_t*>(a[1].ptr);
            p.norm_w = static_cast<const uint16_t*>(a[3].ptr);
            p.xn = xn;
            p.k = k;
            p.eps = eps;
            p.plus_one = plus_one;
        }
        const uint32_t grid = balanced ? grid_balanced : std::min<uint32_t>(p.feat_blocks, (uint32_t)ctx->sm_count);
        HB_CUDA(ctx, launch_kernel(ctx, true, fn, dim3(grid), dim3(SK_THREADS), smem, tm_w, tm_x, p));
        ctx->launches++;
        return HB_OK;
    }
};

}  // namespace

// d->tensor_core: 1 = whole feature blocks of 128 rows per CTA, 2 = balanced units, 3 = whole feature blocks of as many
// rows (at most 128) as make the blocks fill whole waves of CTAs: a block's box of W rows is what one SM pulls, and one
// SM takes in 60-76 GB/s, so 96 blocks of 128 rows on 148 SMs cannot stream at the HBM rate where 147 blocks of 84 can.
int make_matvec_skinny(hb_ctx* ctx, const hb_matvec_desc* d, hb_kernel** out) {
    *out = nullptr;
    if (d->k == 0 || d->n == 0 || d->rows_max == 0) return fail(ctx, HB_INVALID, "matvec (tensor core): k, n and rows_max must be positive");
    if (d->k % 8 != 0) return fail(ctx, HB_UNSUPPORTED, "matvec (tensor core): k must be a multiple of 8 (16-byte rows for TMA)");
    if (d->rows_max > 64) return fail(ctx, HB_UNSUPPORTED, "matvec (tensor core): at most 64 activation rows (the prefill GEMM takes over)");
    if (d->out > HB_OUT_SWIGLU) return fail(ctx, HB_INVALID, "matvec: unknown output mode");
    if (d->out == HB_OUT_SWIGLU && d->n % 2 != 0) return fail(ctx, HB_INVALID, "matvec: the SwiGLU form needs an even n ([gate | up])");
    if (d->tensor_core > 3) return fail(ctx, HB_UNSUPPORTED, "matvec (tensor core): 1 = whole feature blocks, 2 = balanced units, 3 = feature blocks sized to the grid");
    const uint32_t balanced = d->tensor_core == 2 ? 1u : 0u;
    const uint32_t k_blocks = (d->k + 63) / 64;
    const uint32_t np = d->rows_max <= 16 ? 16 : d->rows_max <= 32 ? 32 : 64;
    const uint32_t kps = d->split == 2 ? 2u : d->split == 4 ? 4u : 1u;  // k-blocks per pipeline stage
    if (d->x_src == HB_X_SWIGLU) return fail(ctx, HB_UNSUPPORTED, "matvec (tensor core): the SwiGLU of [gate | up] as input is built for the CUDA-core form");
    const bool norm = d->x_src == HB_X_NORM;
    if (norm && np != 16) return fail(ctx, HB_UNSUPPORTED, "matvec (tensor core): the fused norm is built for at most 16 activation rows");
    skinny_fn fn = norm ? skinny_pick_norm(d->out, kps)
                        : np == 16 ? skinny_pick_kps<16>(d->out, kps) : np == 32 ? skinny_pick_kps<32>(d->out, kps) : skinny_pick_kps<64>(d->out, kps);
    const uint32_t nacc = d->out == HB_OUT_SWIGLU ? 2 : 1;
    uint32_t block_rows = 128;
    if (d->tensor_core == 3) {
        const uint32_t n_out = d->out == HB_OUT_SWIGLU ? d->n / 2 : d->n, sms = (uint32_t)ctx->sm_count;
        const uint32_t waves = (n_out + sms * 128 - 1) / (sms * 128);
        block_rows = std::min(128u, std::max(8u, (n_out + sms * waves - 1) / (sms * waves)));
    }
    const size_t stage_bytes = ((size_t)nacc * SK_A_BYTES + np * 128) * kps;
    const size_t budget = std::min<size_t>(ctx->smem_optin, 227 * 1024) - 3072;  // alignment slack, barriers, the segment table
    uint32_t stages = (uint32_t)std::min<size_t>(budget / stage_bytes, SK_MAX_STAGES);
    if (stages < 2) return fail(ctx, HB_UNSUPPORTED, "matvec (tensor core): the pipeline does not fit in shared memory");
    // `persist` caps the pipeline depth: with half the shared memory or less, the CTAs of two kernels that follow one
    // another on the stream fit on an SM together, and with overlapped launches the second streams its first
    // weights while the first drains
    if (d->persist >= 2) stages = std::min(stages, d->persist);
    auto k = std::make_unique<SkinnyGemm>();
    k->k = d->k;
    k->n = d->n;
    k->out = d->out;
    k->rows_max = np;  // the kernel is built for a padded row count: any m up to it
    k->np = np;
    k->balanced = balanced;
    k->block_rows = block_rows;
    k->stages = stages;
    k->fn = fn;
    k->smem = stages * stage_bytes + 1024;
    k->kind = 2;
    k->nargs = norm ? 4 : 3;
    k->norm = norm;
    char nm[200], xtag[48] = "";
    if (norm) {
        memcpy(&k->eps, &d->norm_eps_bits, 4);
        k->plus_one = d->norm_plus_one;
        snprintf(xtag, sizeof xtag, "_nrm%08x%s", d->norm_eps_bits, d->norm_plus_one ? "p1" : "");
    }
    char btag[16] = "blk";
    if (d->tensor_core == 3) snprintf(btag, sizeof btag, "fit%u", block_rows);
    snprintf(nm, sizeof nm, "matvec_tc_%ux%u_%s_m%u_%s_s%ux%u%s", d->k, d->n, out_tag(d->out), np, balanced ? "bal" : btag, stages, kps, xtag);
    k->name = nm;
    if (hb_kernel* have = find(ctx, k->name)) {
        *out = have;
        return HB_OK;
    }
    if (norm) {
        void* xs = nullptr;
        int r = hb_alloc(ctx, (size_t)np * d->k * 2, &xs);
        if (r != HB_OK) return r;
        k->xn = static_cast<uint16_t*>(xs);
    }
    if (balanced) {
        const uint32_t n_out = d->out == HB_OUT_SWIGLU ? d->n / 2 : d->n;
        const uint64_t feat_blocks = (n_out + 127) / 128;
        const uint64_t units = feat_blocks * k_blocks;
        const uint32_t grid = (uint32_t)std::min<uint64_t>(units, (uint64_t)ctx->sm_count);
        // a block of k_blocks units overlaps at most ceil(k_blocks / floor(units / grid)) + 1 ranges
        const uint64_t per = std::max<uint64_t>(units / grid, 1);
        k->grid_balanced = grid;
        k->maxslots = (uint32_t)std::min<uint64_t>((k_blocks + per - 1) / per + 1, grid);
        void* sc = nullptr;
        void* cn = nullptr;
        int r = hb_alloc(ctx, feat_blocks * k->maxslots * nacc * np * 128 * sizeof(float), &sc);
        if (r != HB_OK) return r;
        if ((r = hb_alloc(ctx, feat_blocks * 4 * sizeof(uint32_t), &cn)) != HB_OK) return r;
        zero_on_failure(ctx, cn, feat_blocks * 4 * sizeof(uint32_t));  // arrival counters: the last arriver resets them
        k->scratch = static_cast<float*>(sc);
        k->counters = static_cast<uint32_t*>(cn);
    }
    {   // the segment table: what every CTA of the (fixed) grid works on
        const uint32_t n_out = d->out == HB_OUT_SWIGLU ? d->n / 2 : d->n;
        SkinnyParams tp{};
        tp.k_blocks = k_blocks;
        tp.feat_blocks = (n_out + block_rows - 1) / block_rows;
        tp.balanced = balanced;
        const uint32_t grid = balanced ? k->grid_balanced : std::min<uint32_t>(tp.feat_blocks, (uint32_t)ctx->sm_count);
        std::vector<uint32_t> start(grid + 1, 0);
        std::vector<SkinnySeg> all;
        for (uint32_t c = 0; c < grid; ++c) {
            const uint32_t ns = skinny_seg(tp, c, grid, 0, nullptr);
            for (uint32_t i = 0; i < ns; ++i) {
                SkinnySeg sg{};
                skinny_seg(tp, c, grid, i, &sg);
                all.push_back(sg);
            }
            start[c + 1] = (uint32_t)all.size();
        }
        void* ds = nullptr;
        void* da = nullptr;
        int r = hb_alloc(ctx, start.size() * 4, &ds);
        if (r != HB_OK) return r;
        if ((r = hb_alloc(ctx, std::max<size_t>(all.size(), 1) * sizeof(SkinnySeg), &da)) != HB_OK) return r;
        if ((r = hb_upload(ctx, ds, start.data(), start.size() * 4)) != HB_OK) return r;
        if (!all.empty() && (r = hb_upload(ctx, da, all.data(), all.size() * sizeof(SkinnySeg))) != HB_OK) return r;
        k->seg_start = static_cast<uint32_t*>(ds);
        k->segs = static_cast<SkinnySeg*>(da);
    }
    cudaError_t e = cudaFuncSetAttribute(reinterpret_cast<const void*>(fn), cudaFuncAttributeMaxDynamicSharedMemorySize, (int)ctx->smem_optin - 2048);
    if (e != cudaSuccess) return cuda_fail(ctx, e, "cudaFuncSetAttribute(max dynamic shared memory)");
    // all of the SM's L1/shared array as shared memory, whatever one CTA asks for: with a capped pipeline two CTAs
    // (of two consecutive kernels) must fit side by side
    e = cudaFuncSetAttribute(reinterpret_cast<const void*>(fn), cudaFuncAttributePreferredSharedMemoryCarveout, (int)cudaSharedmemCarveoutMaxShared);
    if (e != cudaSuccess) return cuda_fail(ctx, e, "cudaFuncSetAttribute(shared memory carveout)");
    *out = intern(ctx, std::move(k));
    return HB_OK;
}

}  // namespace hb
