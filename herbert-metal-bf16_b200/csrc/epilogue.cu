// The output modes applied to an f32 accumulator array that was finished outside a GEMM: the
// row-parallel down projection of a tensor-parallel FFN sums f32 partial products across GPUs and
// only then rounds (once) and adds the residual. Same arithmetic as the GEMM's epilogue
// (reference src/metal/kernels.rs:217-234, src/metal/prefill.rs:1200-1230).
#include <algorithm>

#include "hb_internal.hpp"
#include "tc05.cuh"

namespace hb {

template <int OUT>
__global__ void epilogue_kernel(const float* __restrict__ acc, uint16_t* __restrict__ y, size_t count4) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < count4; i += (size_t)gridDim.x * blockDim.x) {
        const float4 a = reinterpret_cast<const float4*>(acc)[i];
        const float v[4] = {a.x, a.y, a.z, a.w};
        uint32_t o[4];
        if (OUT == HB_OUT_RESIDUAL) {
            const uint2 old = reinterpret_cast<const uint2*>(y)[i];
            const uint32_t ov[4] = {old.x & 0xffffu, old.x >> 16, old.y & 0xffffu, old.y >> 16};
#pragma unroll
            for (int j = 0; j < 4; ++j) o[j] = f32_to_bf16(__fadd_rn(bf16_to_f32(ov[j]), round_bf16(v[j])));
        } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) o[j] = f32_to_bf16(v[j]);
        }
        reinterpret_cast<uint2*>(y)[i] = make_uint2(o[0] | (o[1] << 16), o[2] | (o[3] << 16));
    }
}

namespace {
struct Epilogue : hb_kernel {
    uint32_t n = 0, out = 0;
    int launch(hb_ctx* ctx, const hb_range* a, int na, uint32_t m) override {
        if (na != 2) return fail(ctx, HB_INVALID, name + ": bindings are acc (f32), y (bf16)");
        if (m == 0) return fail(ctx, HB_INVALID, name + ": m = 0");
        const size_t count = (size_t)m * n;
        if (!range_ok(a[0], count * 4) || !range_ok(a[1], count * 2)) return fail(ctx, HB_INVALID, name + ": a bound range is too small");
        if ((reinterpret_cast<uintptr_t>(a[0].ptr) & 15u) || (reinterpret_cast<uintptr_t>(a[1].ptr) & 7u))
            return fail(ctx, HB_INVALID, name + ": acc must be 16-byte and y 8-byte aligned");
        const size_t count4 = count / 4;
        const uint32_t grid = (uint32_t)std::max<size_t>(1, std::min<size_t>((count4 + 255) / 256, (size_t)ctx->sm_count * 16));
        if (out == HB_OUT_RESIDUAL)
            epilogue_kernel<HB_OUT_RESIDUAL><<<grid, 256, 0, ctx->stream>>>(static_cast<const float*>(a[0].ptr), static_cast<uint16_t*>(a[1].ptr), count4);
        else
            epilogue_kernel<HB_OUT_BF16><<<grid, 256, 0, ctx->stream>>>(static_cast<const float*>(a[0].ptr), static_cast<uint16_t*>(a[1].ptr), count4);
        HB_CUDA(ctx, cudaGetLastError());
        ctx->launches++;
        return HB_OK;
    }
};
}  // namespace

int make_epilogue(hb_ctx* ctx, uint32_t n, uint32_t out, hb_kernel** res) {
    *res = nullptr;
    if (n == 0 || n % 4 != 0) return fail(ctx, HB_UNSUPPORTED, "epilogue: n a positive multiple of 4");
    if (out != HB_OUT_BF16 && out != HB_OUT_RESIDUAL) return fail(ctx, HB_UNSUPPORTED, "epilogue: output Bf16 or Residual");
    auto k = std::make_unique<Epilogue>();
    k->n = n;
    k->out = out;
    k->kind = 9;
    k->nargs = 2;
    k->name = std::string("epilogue_") + std::to_string(n) + "_" + out_tag(out);
    *res = intern(ctx, std::move(k));
    return HB_OK;
}

}  // namespace hb

extern "C" int hb_epilogue_get(hb_ctx* ctx, uint32_t n, uint32_t out, hb_kernel** res) {
    if (!ctx || !res) return hb::fail(ctx, HB_INVALID, "hb_epilogue_get: bad argument");
    try {
        return hb::make_epilogue(ctx, n, out, res);
    } catch (const std::exception& e) {
        return hb::fail(ctx, HB_BACKEND, e.what());
    }
}
