// The decode matvec with its input made inside the kernel: the RMSNorm of the residual stream (the reference's
// XSrc::Norm, src/metal/kernels.rs:236-252, 355-442; engine switch dec.fnorm, src/metal/qwen.rs:224-228, 1603) or the
// SwiGLU of [gate | up] (XSrc::Swiglu; dec.fswi). The kernel template is matvec_kernel.cuh's; these are its
// instantiations for 2 and 4 weight rows per warp (a translation unit of their own: they compile beside matvec.cu).
#include "matvec_kernel.cuh"

namespace hb {

typedef void (*mv_fn)(const MatvecParams);

namespace {

template <int M, int R, int XSRC>
mv_fn fx_out(uint32_t out) {
    switch (out) {
        case HB_OUT_BF16: return matvec_kernel<M, R, HB_OUT_BF16, false, XSRC>;
        case HB_OUT_F32: return matvec_kernel<M, R, HB_OUT_F32, false, XSRC>;
        case HB_OUT_RESIDUAL: return matvec_kernel<M, R, HB_OUT_RESIDUAL, false, XSRC>;
        case HB_OUT_SWIGLU: return matvec_kernel<M, R, HB_OUT_SWIGLU, false, XSRC>;
    }
    return nullptr;
}
template <int M, int XSRC>
mv_fn fx_rows(uint32_t r, uint32_t out) {
    return r == 2 ? fx_out<M, 2, XSRC>(out) : r == 4 ? fx_out<M, 4, XSRC>(out) : nullptr;
}
template <int XSRC>
mv_fn fx_m(uint32_t mcap, uint32_t r, uint32_t out) {
    switch (mcap) {
        case 1: return fx_rows<1, XSRC>(r, out);
        case 2: return fx_rows<2, XSRC>(r, out);
        case 4: return fx_rows<4, XSRC>(r, out);
        case 8: return fx_rows<8, XSRC>(r, out);
    }
    return nullptr;
}

}  // namespace

mv_fn mv_pick_fused_x(uint32_t mcap, uint32_t r, uint32_t out, uint32_t x_src) {
    return x_src == HB_X_NORM ? fx_m<XSRC_NORM>(mcap, r, out) : x_src == HB_X_SWIGLU ? fx_m<XSRC_SWIGLU>(mcap, r, out) : nullptr;
}

}  // namespace hb
