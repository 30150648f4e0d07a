// Decode matvec y[r][n] = out(W[n][k] . x[r][k]) for 1..8 activation rows.
//
// Counterpart of the reference's matvec / matvec_split (src/metal/kernels.rs:146-214,
// :502-981). HBM-bound: W is read once with 128-bit non-caching loads, every lane keeps
// an f32 FMA chain per (W row, activation row), a warp reduces R consecutive W rows
// sharing the x loads (the reference's `rows` axis), sums cross the warp by an xor
// butterfly and, with `split`, the K range is cut across the warps of a block and the
// partial sums folded in a fixed order (kernels.rs:916-928). CUDA cores only.
#include <cstring>

#include "matvec_kernel.cuh"

namespace hb {

typedef void (*mv_fn)(const MatvecParams);

namespace {

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
    size_t smem = 0;  // x_src != 0: the input rows made in the kernel

    unsigned long long* keys = nullptr;
    uint32_t* counter = nullptr;

    int launch(hb_ctx* ctx, const hb_range* a, int na, uint32_t m) override {
        const bool norm = d.x_src == HB_X_NORM;
        if (na != 3 + (norm ? 1 : 0) + (d.argmax ? 1 : 0))
            return fail(ctx, HB_INVALID, name + (norm ? ": bindings are W, x, y, norm_w" : d.argmax ? ": bindings are W, x, y, index" : ": bindings are W, x, y"));
        if (m == 0 || m > d.rows_max) return fail(ctx, HB_INVALID, name + ": m outside 1.." + std::to_string(d.rows_max));
        if (d.argmax && !range_ok(a[3], (size_t)m * 4)) return fail(ctx, HB_INVALID, name + ": the index range is too small");
        if (norm && (!range_ok(a[3], (size_t)d.k * 2) || (reinterpret_cast<uintptr_t>(a[3].ptr) & 15u)))
            return fail(ctx, HB_INVALID, name + ": norm_w is too small or not 16-byte aligned");
        const uint32_t n_out = d.out == HB_OUT_SWIGLU ? d.n / 2 : d.n;
        const size_t ybytes = (size_t)m * n_out * (d.out == HB_OUT_F32 ? 4 : 2);
        const size_t xbytes = (size_t)m * d.k * 2 * (d.x_src == HB_X_SWIGLU ? 2 : 1);  // XSrc::Swiglu: rows of [gate | up]
        if (!range_ok(a[0], (size_t)d.n * d.k * 2) || !range_ok(a[1], xbytes) || !range_ok(a[2], ybytes))
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
        if (norm) {
            p.norm_w = static_cast<const uint16_t*>(a[3].ptr);
            memcpy(&p.eps, &d.norm_eps_bits, 4);
            p.plus_one = d.norm_plus_one;
        }
        const uint32_t rows_per_group = d.out == HB_OUT_SWIGLU ? d.rows_per_warp / 2 : d.rows_per_warp;
        p.groups = (n_out + rows_per_group - 1) / rows_per_group;
        const uint32_t slots = MV_WARPS / d.split;
        uint32_t grid = (p.groups + slots - 1) / slots;
        if (d.persist) grid = std::min<uint32_t>(grid, (uint32_t)(ctx->sm_count * blocks_per_sm));
        HB_CUDA(ctx, launch_kernel(ctx, true, fn, dim3(grid), dim3(MV_THREADS), smem, p));
        ctx->launches++;
        return HB_OK;
    }
};

}  // namespace

mv_fn mv_pick_fused_x(uint32_t mcap, uint32_t r, uint32_t out, uint32_t x_src);  // matvec_fused_x.cu
int make_matvec_xs(hb_ctx* ctx, const hb_matvec_desc* d, hb_kernel** out);
int make_matvec_skinny(hb_ctx* ctx, const hb_matvec_desc* d, hb_kernel** out);

int make_matvec(hb_ctx* ctx, const hb_matvec_desc* d, hb_kernel** out) {
    *out = nullptr;
    if (d->k == 0 || d->n == 0) return fail(ctx, HB_INVALID, "matvec: k and n must be positive");
    if (d->k % 8 != 0) return fail(ctx, HB_UNSUPPORTED, "matvec: K = " + std::to_string(d->k) + " is not a multiple of 8");
    if (d->out > HB_OUT_SWIGLU) return fail(ctx, HB_INVALID, "matvec: unknown output mode");
    if (d->x_src > HB_X_SWIGLU) return fail(ctx, HB_INVALID, "matvec: x_src is 0 (x), 1 (RMSNorm of x) or 2 (SwiGLU of [gate | up])");
    if (d->x_src == HB_X_NORM && (d->k % 256 != 0 || d->k / 256 > 32))
        return fail(ctx, HB_UNSUPPORTED, "matvec: the fused norm is built for k a multiple of 256, at most 8192 (the reference's condition, src/metal/qwen.rs:1604)");
    if (d->tensor_core) return make_matvec_skinny(ctx, d, out);
    if (d->x_src && d->x_stationary) return fail(ctx, HB_UNSUPPORTED, "matvec: the activation-stationary form takes x as it is");
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
    if (d->x_src && d->argmax) return fail(ctx, HB_UNSUPPORTED, "matvec: the fused argmax takes x as it is");
    const size_t smem = d->x_src ? (size_t)mcap * d->k * 2 : 0;
    if (smem > 96 * 1024) return fail(ctx, HB_UNSUPPORTED, "matvec: the rows made in the kernel do not fit in shared memory (rows * k * 2 <= 96 KiB)");
    mv_fn fn = d->x_src ? mv_pick_fused_x(mcap, r, d->out, d->x_src) : mv_pick(mcap, r, d->out, d->argmax != 0);
    if (!fn) return fail(ctx, HB_UNSUPPORTED, "matvec: form not built");
    auto k = std::make_unique<Matvec>();
    k->d = *d;
    k->d.rows_per_warp = r;
    k->d.split = split;
    k->d.rows_max = mcap;
    if (d->argmax) k->d.persist = 1;  // the fold at the end of a block costs a round trip: few long-lived blocks, not thousands
    k->fn = fn;
    k->smem = smem;
    k->kind = 2;
    k->nargs = 3 + (d->argmax ? 1 : 0) + (d->x_src == HB_X_NORM ? 1 : 0);
    char nm[200];
    std::string xtag;  // the reference's x_tag (src/metal/kernels.rs:286-293); the norm's constants are part of the kernel
    if (d->x_src == HB_X_NORM) {
        char t[48];
        snprintf(t, sizeof t, "_nrm%08x%s", d->norm_eps_bits, d->norm_plus_one ? "p1" : "");
        xtag = t;
    } else if (d->x_src == HB_X_SWIGLU) {
        xtag = "_swi";
    }
    snprintf(nm, sizeof nm, "matvec_%ux%u_%s_m%u_r%u%s%s%s%s", d->k, d->n, out_tag(d->out), mcap, r,
             split > 1 ? (std::string("_s") + std::to_string(split)).c_str() : "", k->d.persist ? "_p" : "",
             d->argmax == 1 ? "_argmax" : d->argmax == 2 ? "_argmaxonly" : "", xtag.c_str());
    k->name = nm;
    if (hb_kernel* have = find(ctx, k->name)) {
        *out = have;
        return HB_OK;
    }
    if (d->argmax) {
        void* pk = nullptr;
        int st = hb_alloc(ctx, (size_t)mcap * ARGMAX_SLOTS * 8 + 16, &pk);  // zeroed: the keys, then the counter
        if (st != HB_OK) return st;
        zero_on_failure(ctx, pk, (size_t)mcap * ARGMAX_SLOTS * 8 + 16);
        k->keys = static_cast<unsigned long long*>(pk);
        k->counter = reinterpret_cast<uint32_t*>(k->keys + (size_t)mcap * ARGMAX_SLOTS);
    }
    if (smem > 32 * 1024) {  // with the kernel's static shared memory the default limit of 48 KiB is near
        cudaError_t e = cudaFuncSetAttribute(reinterpret_cast<const void*>(fn), cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
        if (e != cudaSuccess) return cuda_fail(ctx, e, "cudaFuncSetAttribute(max dynamic shared memory)");
    }
    int occ = 1;
    cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, reinterpret_cast<const void*>(fn), MV_THREADS, smem);
    k->blocks_per_sm = std::max(occ, 1);
    *out = intern(ctx, std::move(k));
    return HB_OK;
}

}  // namespace hb
