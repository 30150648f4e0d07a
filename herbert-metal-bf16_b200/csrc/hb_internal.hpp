// Internal C++ side of the C ABI declared in include/hb200.h: the context, the
// kernel objects behind hb_kernel handles, error plumbing and launch helpers.
#pragma once

#include <cstdint>
#include <cstdio>
#include <map>
#include <memory>
#include <string>
#include <vector>

#include <cuda.h>
#include <cuda_runtime.h>

#include "../../include/hb200.h"

struct hb_kernel {
    std::string name;
    int kind = 0;  // HB_KIND_*
    int nargs = 0;
    // false for a kernel whose launches would differ by a host-side counter (replaying a recorded launch would repeat
    // it); none of the kernels built today needs one
    bool replayable = true;
    virtual ~hb_kernel() = default;
    // Validates the bound ranges for `m` rows and enqueues the kernel on ctx->stream.
    virtual int launch(hb_ctx* ctx, const hb_range* args, int nargs, uint32_t m) = 0;
};

typedef CUresult (*hb_encode_tiled_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                       const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                       CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

struct hb_ctx {
    int device = 0;
    int sm_count = 0;
    size_t smem_optin = 0;
    std::string device_name;
    cudaStream_t stream = nullptr;
    bool own_stream = false;
    cudaEvent_t ev0 = nullptr, ev1 = nullptr;
    cudaStream_t copy_lane[2] = {nullptr, nullptr};  // upload, download: made on first use
    std::vector<void*> host_allocs;
    bool overlap_launches = false;  // kernels that know how to wait for their predecessor are launched ahead of its end
    uint32_t peer_wait_ms = 5000;  // bound of a barrier's wait for the other GPUs
    std::vector<void*> ipc_opened;  // peers' allocations mapped into this process
    uint32_t* status_dev = nullptr;  // 8 words, see tc05.cuh
    std::string err;
    std::vector<void*> allocs;
    size_t allocated = 0;
    size_t alloc_limit = 0;  // 0 = none; a test hook to provoke HB_OOM without exhausting a GPU
    hb_encode_tiled_fn encode = nullptr;
    std::map<std::string, std::unique_ptr<hb_kernel>> kernels;  // by name: one object per distinct kernel
    uint64_t launches = 0;  // kernels enqueued through this context
    // scratch of the stream-K GEMM: f32 partial tiles [sm_count][128][256] and their flags, made on first use
    float* sk_scratch = nullptr;
    uint32_t* sk_flags = nullptr;
    // Counters and flags that kernels leave at zero when they end normally (arrival counters of the split forms, the
    // argmax fold's keys, the stream-K flags): a launch that gave up on a bounded wait may leave them set, so they are
    // all cleared when the failure is reported (check_status). Registered by whoever allocates them.
    std::vector<std::pair<void*, size_t>> zero_on_failure;
    // scratch of the split-K CTA-pair GEMM: f32 partial tiles and their arrival counters, grown on demand
    float* splitk_partial = nullptr;
    size_t splitk_partial_bytes = 0;
    uint32_t* splitk_counters = nullptr;
    size_t splitk_counter_bytes = 0;
};

namespace hb {

int fail(hb_ctx* ctx, int code, const std::string& msg);
// Makes the context's device the calling thread's current one (a process may hold contexts on several devices).
inline void bind(hb_ctx* ctx) {
    int cur = -1;
    if (cudaGetDevice(&cur) != cudaSuccess || cur != ctx->device) cudaSetDevice(ctx->device);
}
int cuda_fail(hb_ctx* ctx, cudaError_t e, const char* what);
#define HB_CUDA(ctx, call)                                        \
    do {                                                          \
        cudaError_t e__ = (call);                                 \
        if (e__ != cudaSuccess) return hb::cuda_fail(ctx, e__, #call); \
    } while (0)

// A 2-D bf16 row-major tensor [rows][cols] as a TMA descriptor with a box of
// box_rows x 64 elements in the 128-byte swizzle. Rows or columns past the
// extents read as zero.
int make_tmap_bf16(hb_ctx* ctx, CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows);

// Reads the device status words; turns a kernel-side failure into an error.
int check_status(hb_ctx* ctx);

inline bool range_ok(const hb_range& r, size_t need) { return r.ptr != nullptr && r.size >= need; }
inline void zero_on_failure(hb_ctx* ctx, void* p, size_t bytes) { ctx->zero_on_failure.emplace_back(p, bytes); }

// Factories (one translation unit per kernel family).
int make_gemm(hb_ctx* ctx, const hb_gemm_desc* d, hb_kernel** out);
int make_matvec(hb_ctx* ctx, const hb_matvec_desc* d, hb_kernel** out);
int make_swiglu_rows(hb_ctx* ctx, uint32_t n, hb_kernel** out);
int make_route(hb_ctx* ctx, uint32_t experts, uint32_t top_k, hb_kernel** out);
int make_moe_sort(hb_ctx* ctx, uint32_t experts, uint32_t top_k, uint32_t rows_max, uint32_t bm, hb_kernel** out);
int make_moe_gather(hb_ctx* ctx, uint32_t h, uint32_t top_k, hb_kernel** out);
int make_moe_combine(hb_ctx* ctx, uint32_t d, uint32_t top_k, uint32_t f32_sum, hb_kernel** out);
int make_ep_move(hb_ctx* ctx, bool ret, uint32_t h, uint32_t top_k, uint32_t experts, uint32_t world, uint32_t rank, uint32_t cap, hb_kernel** out, bool direct = false);
int make_ep_plan(hb_ctx* ctx, uint32_t experts, uint32_t world, uint32_t rank, uint32_t bm, uint32_t cap, hb_kernel** out, bool direct = false);
int make_experts_matvec(hb_ctx* ctx, uint32_t k, uint32_t n, uint32_t top_k, uint32_t experts, uint32_t x_row, uint32_t x_stride, uint32_t rows, hb_kernel** out);
int make_ep_combine(hb_ctx* ctx, uint32_t h, uint32_t top_k, uint32_t world, hb_kernel** out, bool sync = false, uint32_t rank = 0);

// Launches `fn`; with `waits_itself` (the kernel calls griddep_wait before it touches its predecessor's data) and the
// context's overlap switch on, with programmatic stream serialization.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_kernel(hb_ctx* ctx, bool waits_itself, void (*fn)(KArgs...), dim3 grid, dim3 block, size_t smem, Args&&... args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    if (waits_itself && ctx->overlap_launches) {
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
    }
    return cudaLaunchKernelEx(&cfg, fn, static_cast<KArgs>(args)...);
}

// Registers `k` under its name (or returns the existing object of that name).
hb_kernel* intern(hb_ctx* ctx, std::unique_ptr<hb_kernel> k);
hb_kernel* find(hb_ctx* ctx, const std::string& name);

const char* out_tag(uint32_t out);

}  // namespace hb
