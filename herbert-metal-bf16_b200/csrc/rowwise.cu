// The row-wise kernels on either side of the matrix products: RMSNorm of the rows that feed a projection, argmax
// over the logits a projection produced, and the end of the sparse MoE block. All three are bit-exact restatements
// of the reference's arithmetic, including the order of its sums: a group of 256 threads, thread l an FMA chain over
// elements l, l + 256, ..., the 32 lanes of a simdgroup summed (xor butterfly), the 8 partials folded in order by
// thread 0 (reference src/msl/mod.rs:716-756). They are memory-bound: a row is staged in shared memory with 16-byte
// loads so that the lane-strided chains read it from there.
#include <algorithm>

#include "rowwise.cuh"

namespace hb {

// ----------------------------------------------------------------- rmsnorm_rows
// y = bf16((x * inv) * (w [+ 1])), inv = 1 / sqrt(sum(x^2) * (1/d) + eps) (reference src/metal/prefill.rs:70-117;
// the decode twin src/metal/kernels.rs:355-442 makes the same sums).
__global__ void __launch_bounds__(ROW_THREADS) rmsnorm_rows_kernel(const uint16_t* __restrict__ x, const uint16_t* __restrict__ w, uint16_t* __restrict__ y,
                                                                   uint32_t rows, uint32_t d, float inv_d, float eps, uint32_t plus_one, uint32_t vec) {
    extern __shared__ uint16_t row_s[];
    __shared__ float part[9];
    griddep_launch_dependents();
    griddep_wait();
    for (uint32_t row = blockIdx.x; row < rows; row += gridDim.x) {
        const uint16_t* xr = x + (size_t)row * d;
        stage_row(row_s, xr, d, vec);
        __syncthreads();
        float acc = 0.f;
        for (uint32_t i = threadIdx.x; i < d; i += ROW_THREADS) {
            const float v = bf16_to_f32(row_s[i]);
            acc = __fmaf_rn(v, v, acc);
        }
        const float ss = group_sum256(acc, part);
        const float inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fmul_rn(ss, inv_d), eps)));
        uint16_t* yr = y + (size_t)row * d;
        if (vec) {
            for (uint32_t i = threadIdx.x; i < d / 8; i += ROW_THREADS) {
                const uint4 xv = reinterpret_cast<const uint4*>(row_s)[i];
                const uint4 wv = reinterpret_cast<const uint4*>(w)[i];
                const uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w}, ww[4] = {wv.x, wv.y, wv.z, wv.w};
                uint32_t o[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    float w0 = __uint_as_float(ww[j] << 16), w1 = __uint_as_float(ww[j] & 0xffff0000u);
                    if (plus_one) { w0 = __fadd_rn(w0, 1.0f); w1 = __fadd_rn(w1, 1.0f); }
                    const float n0 = __fmul_rn(__uint_as_float(xw[j] << 16), inv), n1 = __fmul_rn(__uint_as_float(xw[j] & 0xffff0000u), inv);
                    o[j] = f32x2_to_bf16x2(__fmul_rn(n0, w0), __fmul_rn(n1, w1));
                }
                reinterpret_cast<uint4*>(yr)[i] = make_uint4(o[0], o[1], o[2], o[3]);
            }
        } else {
            for (uint32_t i = threadIdx.x; i < d; i += ROW_THREADS) {
                float wf = bf16_to_f32(w[i]);
                if (plus_one) wf = __fadd_rn(wf, 1.0f);
                yr[i] = (uint16_t)f32_to_bf16(__fmul_rn(__fmul_rn(bf16_to_f32(row_s[i]), inv), wf));
            }
        }
        __syncthreads();  // the staged row is read out before the next one overwrites it
    }
}

// ---------------------------------------------------------------------- moe_out
// g = bf16(sigmoid(bf16(xn . gate))), x = bf16(x + bf16(experts + bf16(g * shared))) in place
// (reference src/metal/qwen_kernels.rs:2163-2214).
__global__ void __launch_bounds__(ROW_THREADS) moe_out_kernel(const uint16_t* __restrict__ xn, const uint16_t* __restrict__ gate, const uint16_t* __restrict__ ex,
                                                              const uint16_t* __restrict__ sh, uint16_t* __restrict__ x, uint32_t rows, uint32_t d, uint32_t vec) {
    extern __shared__ uint16_t row_s[];
    __shared__ float part[9];
    for (uint32_t row = blockIdx.x; row < rows; row += gridDim.x) {
        const size_t base = (size_t)row * d;
        stage_row(row_s, xn + base, d, vec);
        __syncthreads();
        float acc = 0.f;
        for (uint32_t i = threadIdx.x; i < d; i += ROW_THREADS) acc = __fmaf_rn(bf16_to_f32(row_s[i]), bf16_to_f32(gate[i]), acc);
        const float logit = round_bf16(group_sum256(acc, part));
        const float g = round_bf16(sigmoid_f32(logit));
        if (vec) {
            for (uint32_t i = threadIdx.x; i < d / 8; i += ROW_THREADS) {
                const uint4 sv = reinterpret_cast<const uint4*>(sh + base)[i], ev = reinterpret_cast<const uint4*>(ex + base)[i];
                const uint4 xv = reinterpret_cast<const uint4*>(x + base)[i];
                const uint32_t sw[4] = {sv.x, sv.y, sv.z, sv.w}, ew[4] = {ev.x, ev.y, ev.z, ev.w}, xw[4] = {xv.x, xv.y, xv.z, xv.w};
                uint32_t o[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const uint32_t s = f32x2_to_bf16x2(__fmul_rn(g, __uint_as_float(sw[j] << 16)), __fmul_rn(g, __uint_as_float(sw[j] & 0xffff0000u)));
                    const uint32_t t = f32x2_to_bf16x2(__fadd_rn(__uint_as_float(ew[j] << 16), __uint_as_float(s << 16)),
                                                       __fadd_rn(__uint_as_float(ew[j] & 0xffff0000u), __uint_as_float(s & 0xffff0000u)));
                    o[j] = f32x2_to_bf16x2(__fadd_rn(__uint_as_float(xw[j] << 16), __uint_as_float(t << 16)),
                                           __fadd_rn(__uint_as_float(xw[j] & 0xffff0000u), __uint_as_float(t & 0xffff0000u)));
                }
                reinterpret_cast<uint4*>(x + base)[i] = make_uint4(o[0], o[1], o[2], o[3]);
            }
        } else {
            for (uint32_t i = threadIdx.x; i < d; i += ROW_THREADS) {
                const float s = round_bf16(__fmul_rn(g, bf16_to_f32(sh[base + i])));
                const float o = round_bf16(__fadd_rn(bf16_to_f32(ex[base + i]), s));
                x[base + i] = (uint16_t)f32_to_bf16(__fadd_rn(bf16_to_f32(x[base + i]), o));
            }
        }
        __syncthreads();
    }
}

// ------------------------------------------------------------------ argmax_rows
// Index of the largest bf16 logit of each row, the first index on a tie (reference src/metal/kernels.rs:1461-1565:
// a pass over chunks of 4096 and a final pass). "Largest, then lowest index" does not depend on the order in which
// candidates meet, so one kernel does both passes: every block folds its chunk into a 64-bit key
// (order-preserving value bits | inverted index), the keys meet in an atomic max per row, and the block that
// finishes last turns the keys into indices and clears them for the next launch. A logit wins only if it is
// greater than -inf (the reference's compare is v > best from -inf): NaN and -inf never win, and a row without a
// winner gives 0xffffffff. -0 and +0 compare equal, as there.
constexpr uint32_t ARGMAX_CHUNK = 4096;

__global__ void __launch_bounds__(ROW_THREADS) argmax_rows_kernel(const uint16_t* __restrict__ logits, uint32_t* __restrict__ idx, unsigned long long* keys,
                                                                  uint32_t* counter, uint32_t rows, uint32_t n, uint32_t chunks) {
    __shared__ unsigned long long best_s[ROW_THREADS / 32];
    __shared__ uint32_t last_s;
    const uint32_t row = blockIdx.y, chunk = blockIdx.x;
    const uint32_t i0 = chunk * ARGMAX_CHUNK, i1 = min(n, i0 + ARGMAX_CHUNK);
    const uint16_t* lr = logits + (size_t)row * n;
    unsigned long long best = 0ull;
    for (uint32_t i = i0 + threadIdx.x; i < i1; i += ROW_THREADS) {
        const unsigned long long k = argmax_key(lr[i], i);
        best = k > best ? k : best;
    }
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) {
        const unsigned long long o = __shfl_xor_sync(0xffffffffu, best, off);
        best = o > best ? o : best;
    }
    if ((threadIdx.x & 31) == 0) best_s[threadIdx.x >> 5] = best;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int g = 1; g < ROW_THREADS / 32; ++g) best = best_s[g] > best ? best_s[g] : best;
        if (best) atomicMax(&keys[row], best);
        __threadfence();
        last_s = atomicAdd(counter, 1u) == chunks * rows - 1 ? 1u : 0u;
    }
    __syncthreads();
    if (last_s) {
        __threadfence();
        for (uint32_t r = threadIdx.x; r < rows; r += ROW_THREADS) {
            const unsigned long long k = atomicExch(&keys[r], 0ull);
            idx[r] = argmax_index_of(k);
        }
        if (threadIdx.x == 0) *counter = 0u;
    }
}

namespace {

inline uint32_t row_grid(hb_ctx* ctx, uint32_t rows) { return std::max(1u, std::min<uint32_t>(rows, (uint32_t)ctx->sm_count * 8)); }

struct RmsNorm : hb_kernel {
    uint32_t d = 0, plus_one = 0;
    float eps = 0.f;
    int launch(hb_ctx* ctx, const hb_range* a, int na, uint32_t m) override {
        if (na != 3) return fail(ctx, HB_INVALID, name + ": bindings are x, w, y");
        if (m == 0) return fail(ctx, HB_INVALID, name + ": m = 0");
        if (!range_ok(a[0], (size_t)m * d * 2) || !range_ok(a[1], (size_t)d * 2) || !range_ok(a[2], (size_t)m * d * 2))
            return fail(ctx, HB_INVALID, name + ": a bound range is too small");
        const uintptr_t al = reinterpret_cast<uintptr_t>(a[0].ptr) | reinterpret_cast<uintptr_t>(a[1].ptr) | reinterpret_cast<uintptr_t>(a[2].ptr);
        const uint32_t vec = (d % 8 == 0 && (al & 15u) == 0) ? 1u : 0u;
        HB_CUDA(ctx, launch_kernel(ctx, true, rmsnorm_rows_kernel, dim3(row_grid(ctx, m)), dim3(ROW_THREADS), (size_t)d * 2 + 16, static_cast<const uint16_t*>(a[0].ptr),
                                   static_cast<const uint16_t*>(a[1].ptr), static_cast<uint16_t*>(a[2].ptr), m, d, 1.0f / (float)d, eps, plus_one, vec));
        ctx->launches++;
        return HB_OK;
    }
};

struct MoeOut : hb_kernel {
    uint32_t d = 0;
    int launch(hb_ctx* ctx, const hb_range* a, int na, uint32_t m) override {
        if (na != 5) return fail(ctx, HB_INVALID, name + ": bindings are xn, gate, experts, shared, x");
        if (m == 0) return fail(ctx, HB_INVALID, name + ": m = 0");
        const size_t rb = (size_t)m * d * 2;
        if (!range_ok(a[0], rb) || !range_ok(a[1], (size_t)d * 2) || !range_ok(a[2], rb) || !range_ok(a[3], rb) || !range_ok(a[4], rb))
            return fail(ctx, HB_INVALID, name + ": a bound range is too small");
        uintptr_t al = 0;
        for (int i = 0; i < 5; ++i) al |= reinterpret_cast<uintptr_t>(a[i].ptr);
        const uint32_t vec = (d % 8 == 0 && (al & 15u) == 0) ? 1u : 0u;
        moe_out_kernel<<<row_grid(ctx, m), ROW_THREADS, (size_t)d * 2 + 16, ctx->stream>>>(static_cast<const uint16_t*>(a[0].ptr), static_cast<const uint16_t*>(a[1].ptr),
                                                                                          static_cast<const uint16_t*>(a[2].ptr), static_cast<const uint16_t*>(a[3].ptr),
                                                                                          static_cast<uint16_t*>(a[4].ptr), m, d, vec);
        HB_CUDA(ctx, cudaGetLastError());
        ctx->launches++;
        return HB_OK;
    }
};

struct ArgmaxRows : hb_kernel {
    uint32_t n = 0, rows_max = 0;
    unsigned long long* keys = nullptr;
    uint32_t* counter = nullptr;
    int launch(hb_ctx* ctx, const hb_range* a, int na, uint32_t m) override {
        if (na != 2) return fail(ctx, HB_INVALID, name + ": bindings are logits, index");
        if (m == 0 || m > rows_max) return fail(ctx, HB_INVALID, name + ": m outside 1.." + std::to_string(rows_max));
        if (!range_ok(a[0], (size_t)m * n * 2) || !range_ok(a[1], (size_t)m * 4)) return fail(ctx, HB_INVALID, name + ": a bound range is too small");
        const uint32_t chunks = (n + ARGMAX_CHUNK - 1) / ARGMAX_CHUNK;
        argmax_rows_kernel<<<dim3(chunks, m), ROW_THREADS, 0, ctx->stream>>>(static_cast<const uint16_t*>(a[0].ptr), static_cast<uint32_t*>(a[1].ptr), keys, counter, m, n, chunks);
        HB_CUDA(ctx, cudaGetLastError());
        ctx->launches++;
        return HB_OK;
    }
};

}  // namespace

int make_rmsnorm(hb_ctx* ctx, uint32_t d, float eps, uint32_t plus_one, hb_kernel** out) {
    *out = nullptr;
    if (d == 0 || d > 65536) return fail(ctx, HB_UNSUPPORTED, "rmsnorm_rows: 1..65536 columns");
    if (!(eps >= 0.f)) return fail(ctx, HB_INVALID, "rmsnorm_rows: eps must not be negative");
    auto k = std::make_unique<RmsNorm>();
    k->d = d;
    k->eps = eps;
    k->plus_one = plus_one ? 1u : 0u;
    k->kind = 16;
    k->nargs = 3;
    char nm[96];
    uint32_t eb;
    memcpy(&eb, &eps, 4);
    snprintf(nm, sizeof nm, "rmsnorm_rows_%u%s_e%08x", d, plus_one ? "_p1" : "", eb);
    k->name = nm;
    if (hb_kernel* have = find(ctx, k->name)) {
        *out = have;
        return HB_OK;
    }
    if ((size_t)d * 2 + 16 > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(reinterpret_cast<const void*>(rmsnorm_rows_kernel), cudaFuncAttributeMaxDynamicSharedMemorySize, 132 * 1024);
        if (e != cudaSuccess) return cuda_fail(ctx, e, "cudaFuncSetAttribute(max dynamic shared memory)");
    }
    *out = intern(ctx, std::move(k));
    return HB_OK;
}

int make_moe_out(hb_ctx* ctx, uint32_t d, hb_kernel** out) {
    *out = nullptr;
    if (d == 0 || d > 65536) return fail(ctx, HB_UNSUPPORTED, "moe_out: 1..65536 columns");
    auto k = std::make_unique<MoeOut>();
    k->d = d;
    k->kind = 17;
    k->nargs = 5;
    k->name = "moe_out_" + std::to_string(d);
    if (hb_kernel* have = find(ctx, k->name)) {
        *out = have;
        return HB_OK;
    }
    if ((size_t)d * 2 + 16 > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(reinterpret_cast<const void*>(moe_out_kernel), cudaFuncAttributeMaxDynamicSharedMemorySize, 132 * 1024);
        if (e != cudaSuccess) return cuda_fail(ctx, e, "cudaFuncSetAttribute(max dynamic shared memory)");
    }
    *out = intern(ctx, std::move(k));
    return HB_OK;
}

int make_argmax(hb_ctx* ctx, uint32_t n, uint32_t rows_max, hb_kernel** out) {
    *out = nullptr;
    if (n == 0 || rows_max == 0 || rows_max > 65535) return fail(ctx, HB_UNSUPPORTED, "argmax_rows: n positive, 1..65535 rows");
    auto k = std::make_unique<ArgmaxRows>();
    k->n = n;
    k->rows_max = rows_max;
    k->kind = 18;
    k->nargs = 2;
    k->name = "argmax_rows_" + std::to_string(n) + "_r" + std::to_string(rows_max);
    if (hb_kernel* have = find(ctx, k->name)) {
        *out = have;
        return HB_OK;
    }
    void* p = nullptr;
    int r = hb_alloc(ctx, (size_t)rows_max * 8 + 16, &p);  // zeroed: the keys, then the counter
    if (r != HB_OK) return r;
    zero_on_failure(ctx, p, (size_t)rows_max * 8 + 16);
    k->keys = static_cast<unsigned long long*>(p);
    k->counter = reinterpret_cast<uint32_t*>(k->keys + rows_max);
    *out = intern(ctx, std::move(k));
    return HB_OK;
}

}  // namespace hb

extern "C" {

int hb_rmsnorm_get(hb_ctx* ctx, uint32_t d, float eps, uint32_t plus_one, hb_kernel** out) {
    if (!ctx || !out) return hb::fail(ctx, HB_INVALID, "hb_rmsnorm_get: bad argument");
    try {
        hb::bind(ctx);
        return hb::make_rmsnorm(ctx, d, eps, plus_one, out);
    } catch (const std::exception& e) {
        return hb::fail(ctx, HB_BACKEND, e.what());
    }
}

int hb_moe_out_get(hb_ctx* ctx, uint32_t d, hb_kernel** out) {
    if (!ctx || !out) return hb::fail(ctx, HB_INVALID, "hb_moe_out_get: bad argument");
    try {
        hb::bind(ctx);
        return hb::make_moe_out(ctx, d, out);
    } catch (const std::exception& e) {
        return hb::fail(ctx, HB_BACKEND, e.what());
    }
}

int hb_argmax_get(hb_ctx* ctx, uint32_t n, uint32_t rows_max, hb_kernel** out) {
    if (!ctx || !out) return hb::fail(ctx, HB_INVALID, "hb_argmax_get: bad argument");
    try {
        hb::bind(ctx);
        return hb::make_argmax(ctx, n, rows_max, out);
    } catch (const std::exception& e) {
        return hb::fail(ctx, HB_BACKEND, e.what());
    }
}

}  // extern "C"
