// Device layer of the C ABI: context, buffers, copies, launches, timing.
// Takes the place of the reference's src/metal/gpu.rs for the matrix-multiply path.
#include <algorithm>
#include <cstring>
#include <mutex>
#include <new>

#include "hb_internal.hpp"

namespace {
thread_local std::string g_open_error;  // message of a failed hb_open (no context yet)
}

namespace hb {

int fail(hb_ctx* ctx, int code, const std::string& msg) {
    if (ctx) ctx->err = msg;
    else g_open_error = msg;
    return code;
}

int cuda_fail(hb_ctx* ctx, cudaError_t e, const char* what) {
    return fail(ctx, e == cudaErrorMemoryAllocation ? HB_OOM : HB_BACKEND,
                std::string("cuda: ") + cudaGetErrorString(e) + " (" + what + ")");
}

const char* out_tag(uint32_t out) {
    switch (out) {
        case HB_OUT_BF16: return "bf16";
        case HB_OUT_F32: return "f32";
        case HB_OUT_RESIDUAL: return "res";
        case HB_OUT_SWIGLU: return "swiglu";
    }
    return "?";
}

int make_tmap_bf16(hb_ctx* ctx, CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows) {
    if (!ctx->encode) return fail(ctx, HB_BACKEND, "cuTensorMapEncodeTiled is not available from this driver");
    if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0 || (cols * 2) % 16 != 0)
        return fail(ctx, HB_INVALID, "a TMA operand needs a 16-byte aligned base and a row length that is a multiple of 8 elements");
    if (box_rows == 0 || box_rows > 256) return fail(ctx, HB_INVALID, "TMA box rows out of range");
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {cols * 2};
    cuuint32_t box[2] = {64, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = ctx->encode(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(ctx, HB_BACKEND, "cuTensorMapEncodeTiled failed with CUresult " + std::to_string((int)r));
    return HB_OK;
}

int check_status(hb_ctx* ctx) {
    uint32_t st[8];
    HB_CUDA(ctx, cudaMemcpyAsync(st, ctx->status_dev, sizeof st, cudaMemcpyDeviceToHost, ctx->stream));
    HB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    if (st[0] != 0) {
        char msg[160];
        if (st[0] == 2) snprintf(msg, sizeof msg, "kernel status 2: block %u read a table that does not fit its buffers (%u against %u)", st[1], st[2], st[3]);
        else snprintf(msg, sizeof msg, "kernel status %u: block %u gave up waiting at point %u (detail %u)", st[0], st[1], st[2], st[3]);
        cudaMemsetAsync(ctx->status_dev, 0, sizeof st, ctx->stream);
        // a launch that gave up may have left flags of partial tiles or arrival counters set: clear them for the next launch
        for (const auto& z : ctx->zero_on_failure) cudaMemsetAsync(z.first, 0, z.second, ctx->stream);
        cudaStreamSynchronize(ctx->stream);
        return fail(ctx, HB_KERNEL, msg);
    }
    return HB_OK;
}

hb_kernel* intern(hb_ctx* ctx, std::unique_ptr<hb_kernel> k) {
    auto it = ctx->kernels.find(k->name);
    if (it != ctx->kernels.end()) return it->second.get();
    hb_kernel* raw = k.get();
    ctx->kernels.emplace(raw->name, std::move(k));
    return raw;
}

hb_kernel* find(hb_ctx* ctx, const std::string& name) {
    auto it = ctx->kernels.find(name);
    return it == ctx->kernels.end() ? nullptr : it->second.get();
}

}  // namespace hb

using hb::fail;

#define HB_GUARD_BEGIN try {
#define HB_GUARD_BIND(ctx) try { hb::bind(ctx);
#define HB_GUARD_END(ctx)                                                        \
    }                                                                            \
    catch (const std::exception& e) { return hb::fail(ctx, HB_BACKEND, e.what()); } \
    catch (...) { return hb::fail(ctx, HB_BACKEND, "unknown exception"); }

extern "C" {

int hb_open(int device, hb_ctx** out) {
    if (!out) return fail(nullptr, HB_INVALID, "hb_open: out is null");
    *out = nullptr;
    HB_GUARD_BEGIN
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess || count == 0)
        return fail(nullptr, HB_BACKEND, std::string("no CUDA device: ") + (e != cudaSuccess ? cudaGetErrorString(e) : "device count is 0") +
                                             " (this library has no CPU path)");
    if (device < 0 || device >= count) return fail(nullptr, HB_INVALID, "hb_open: no such device");
    cudaDeviceProp prop;
    if ((e = cudaGetDeviceProperties(&prop, device)) != cudaSuccess) return hb::cuda_fail(nullptr, e, "cudaGetDeviceProperties");
    if (prop.major != 10)
        return fail(nullptr, HB_BACKEND, std::string("device ") + prop.name + " is sm_" + std::to_string(prop.major) + std::to_string(prop.minor) +
                                             "; these kernels are built for sm_100a only");
    if ((e = cudaSetDevice(device)) != cudaSuccess) return hb::cuda_fail(nullptr, e, "cudaSetDevice");
    auto ctx = std::make_unique<hb_ctx>();
    ctx->device = device;
    ctx->sm_count = prop.multiProcessorCount;
    ctx->smem_optin = prop.sharedMemPerBlockOptin;
    ctx->device_name = prop.name;
    auto undo = [&](cudaError_t err, const char* what) {  // a half-made context: give back what exists
        if (ctx->status_dev) cudaFree(ctx->status_dev);
        if (ctx->ev0) cudaEventDestroy(ctx->ev0);
        if (ctx->ev1) cudaEventDestroy(ctx->ev1);
        if (ctx->stream) cudaStreamDestroy(ctx->stream);
        return hb::cuda_fail(nullptr, err, what);
    };
    if ((e = cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking)) != cudaSuccess) return undo(e, "cudaStreamCreate");
    ctx->own_stream = true;
    if ((e = cudaEventCreate(&ctx->ev0)) != cudaSuccess || (e = cudaEventCreate(&ctx->ev1)) != cudaSuccess) return undo(e, "cudaEventCreate");
    if ((e = cudaMalloc(&ctx->status_dev, 8 * sizeof(uint32_t))) != cudaSuccess) return undo(e, "cudaMalloc(status)");
    if ((e = cudaMemset(ctx->status_dev, 0, 8 * sizeof(uint32_t))) != cudaSuccess) return undo(e, "cudaMemset(status)");
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
        ctx->encode = reinterpret_cast<hb_encode_tiled_fn>(fn);
    *out = ctx.release();
    return HB_OK;
    HB_GUARD_END(nullptr)
}

int hb_close(hb_ctx* ctx) {
    if (!ctx) return HB_OK;
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    ctx->kernels.clear();
    for (void* p : ctx->allocs) cudaFree(p);
    cudaFree(ctx->status_dev);
    cudaEventDestroy(ctx->ev0);
    cudaEventDestroy(ctx->ev1);
    for (cudaStream_t& c : ctx->copy_lane)
        if (c) {
            cudaStreamSynchronize(c);
            cudaStreamDestroy(c);
        }
    for (void* p : ctx->host_allocs) cudaFreeHost(p);
    for (void* p : ctx->ipc_opened) cudaIpcCloseMemHandle(p);
    if (ctx->own_stream) cudaStreamDestroy(ctx->stream);
    delete ctx;
    return HB_OK;
}

const char* hb_last_error(const hb_ctx* ctx) { return ctx ? ctx->err.c_str() : g_open_error.c_str(); }

int hb_describe(hb_ctx* ctx, char* buf, size_t len) {
    if (!ctx || !buf || len == 0) return fail(ctx, HB_INVALID, "hb_describe: bad argument");
    snprintf(buf, len, "%s, %d SMs, %zu KiB shared memory per block, device %d", ctx->device_name.c_str(), ctx->sm_count,
             ctx->smem_optin / 1024, ctx->device);
    return HB_OK;
}

int hb_set_stream(hb_ctx* ctx, void* cuda_stream) {
    if (!ctx) return HB_INVALID;
    if (ctx->own_stream) {
        cudaStreamSynchronize(ctx->stream);
        cudaStreamDestroy(ctx->stream);
        ctx->own_stream = false;
    }
    if (cuda_stream) {
        ctx->stream = static_cast<cudaStream_t>(cuda_stream);
    } else {
        HB_CUDA(ctx, cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking));
        ctx->own_stream = true;
    }
    return HB_OK;
}

int hb_set_alloc_limit(hb_ctx* ctx, size_t bytes) {
    if (!ctx) return HB_INVALID;
    ctx->alloc_limit = bytes;
    return HB_OK;
}

int hb_alloc(hb_ctx* ctx, size_t bytes, void** dptr) {
    if (!ctx || !dptr) return fail(ctx, HB_INVALID, "hb_alloc: bad argument");
    hb::bind(ctx);
    *dptr = nullptr;
    if (bytes == 0) return fail(ctx, HB_INVALID, "hb_alloc: zero bytes");
    if (ctx->alloc_limit && ctx->allocated + bytes > ctx->alloc_limit)
        return fail(ctx, HB_OOM, "hb_alloc: " + std::to_string(bytes) + " bytes over the context's limit of " + std::to_string(ctx->alloc_limit));
    void* p = nullptr;
    HB_CUDA(ctx, cudaMalloc(&p, bytes));
    cudaError_t e = cudaMemsetAsync(p, 0, bytes, ctx->stream);
    if (e != cudaSuccess) {
        cudaFree(p);
        return hb::cuda_fail(ctx, e, "cudaMemsetAsync");
    }
    ctx->allocs.push_back(p);
    ctx->allocated += bytes;
    *dptr = p;
    return HB_OK;
}

int hb_upload(hb_ctx* ctx, void* dst, const void* src, size_t bytes) {
    if (!ctx || !dst || !src) return fail(ctx, HB_INVALID, "hb_upload: bad argument");
    hb::bind(ctx);
    HB_CUDA(ctx, cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, ctx->stream));
    HB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return HB_OK;
}

int hb_download(hb_ctx* ctx, void* dst, const void* src, size_t bytes) {
    if (!ctx || !dst || !src) return fail(ctx, HB_INVALID, "hb_download: bad argument");
    hb::bind(ctx);
    HB_CUDA(ctx, cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, ctx->stream));
    HB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return hb::check_status(ctx);
}

// ---- peer memory ------------------------------------------------------------------------------
int hb_ipc_export(hb_ctx* ctx, void* dptr, void* handle64) {
    if (!ctx || !dptr || !handle64) return fail(ctx, HB_INVALID, "hb_ipc_export: bad argument");
    hb::bind(ctx);
    static_assert(sizeof(cudaIpcMemHandle_t) == HB_IPC_HANDLE_BYTES, "handle size");
    if (std::find(ctx->allocs.begin(), ctx->allocs.end(), dptr) == ctx->allocs.end())
        return fail(ctx, HB_INVALID, "hb_ipc_export: not the start of an hb_alloc allocation");
    cudaIpcMemHandle_t h;
    HB_CUDA(ctx, cudaIpcGetMemHandle(&h, dptr));
    memcpy(handle64, &h, sizeof h);
    return HB_OK;
}

int hb_ipc_open(hb_ctx* ctx, const void* handle64, void** dptr) {
    if (!ctx || !handle64 || !dptr) return fail(ctx, HB_INVALID, "hb_ipc_open: bad argument");
    hb::bind(ctx);
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, sizeof h);
    void* p = nullptr;
    HB_CUDA(ctx, cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
    ctx->ipc_opened.push_back(p);
    *dptr = p;
    return HB_OK;
}

int hb_ipc_close(hb_ctx* ctx, void* dptr) {
    if (!ctx || !dptr) return HB_OK;
    hb::bind(ctx);
    for (size_t i = 0; i < ctx->ipc_opened.size(); ++i)
        if (ctx->ipc_opened[i] == dptr) {
            ctx->ipc_opened.erase(ctx->ipc_opened.begin() + i);
            HB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
            HB_CUDA(ctx, cudaIpcCloseMemHandle(dptr));
            return HB_OK;
        }
    return fail(ctx, HB_INVALID, "hb_ipc_close: not a pointer of hb_ipc_open");
}

// ---- copy lanes -------------------------------------------------------------------------------
struct hb_event {
    cudaEvent_t ev = nullptr;
};

namespace {
int lane_stream(hb_ctx* ctx, int lane, cudaStream_t* out) {
    if (lane == HB_LANE_KERNELS) {
        *out = ctx->stream;
        return HB_OK;
    }
    if (lane != HB_LANE_UPLOAD && lane != HB_LANE_DOWNLOAD) return fail(ctx, HB_INVALID, "no such lane");
    cudaStream_t& c = ctx->copy_lane[lane - 1];
    if (!c) HB_CUDA(ctx, cudaStreamCreateWithFlags(&c, cudaStreamNonBlocking));
    *out = c;
    return HB_OK;
}
}  // namespace

int hb_event_new(hb_ctx* ctx, hb_event** out) {
    if (!ctx || !out) return fail(ctx, HB_INVALID, "hb_event_new: bad argument");
    hb::bind(ctx);  // an event belongs to the device that is current when it is made
    auto* e = new (std::nothrow) hb_event;
    if (!e) return fail(ctx, HB_OOM, "hb_event_new: out of memory");
    cudaError_t st = cudaEventCreateWithFlags(&e->ev, cudaEventDisableTiming);
    if (st != cudaSuccess) {
        delete e;
        return hb::cuda_fail(ctx, st, "cudaEventCreateWithFlags");
    }
    *out = e;
    return HB_OK;
}

int hb_event_free(hb_ctx* ctx, hb_event* ev) {
    if (!ev) return HB_OK;
    if (ctx) hb::bind(ctx);
    cudaEventDestroy(ev->ev);
    delete ev;
    return HB_OK;
}

int hb_lane_record(hb_ctx* ctx, int lane, hb_event* ev) {
    if (!ctx || !ev) return fail(ctx, HB_INVALID, "hb_lane_record: bad argument");
    hb::bind(ctx);
    cudaStream_t s;
    int r = lane_stream(ctx, lane, &s);
    if (r != HB_OK) return r;
    HB_CUDA(ctx, cudaEventRecord(ev->ev, s));
    return HB_OK;
}

int hb_lane_wait(hb_ctx* ctx, int lane, const hb_event* ev) {
    if (!ctx || !ev) return fail(ctx, HB_INVALID, "hb_lane_wait: bad argument");
    hb::bind(ctx);
    cudaStream_t s;
    int r = lane_stream(ctx, lane, &s);
    if (r != HB_OK) return r;
    HB_CUDA(ctx, cudaStreamWaitEvent(s, ev->ev, 0));
    return HB_OK;
}

int hb_event_sync(hb_ctx* ctx, const hb_event* ev) {
    if (!ctx || !ev) return fail(ctx, HB_INVALID, "hb_event_sync: bad argument");
    hb::bind(ctx);
    HB_CUDA(ctx, cudaEventSynchronize(ev->ev));
    return HB_OK;
}

int hb_upload_async(hb_ctx* ctx, void* dst, const void* src, size_t bytes) {
    if (!ctx || !dst || !src) return fail(ctx, HB_INVALID, "hb_upload_async: bad argument");
    hb::bind(ctx);
    cudaStream_t s;
    int r = lane_stream(ctx, HB_LANE_UPLOAD, &s);
    if (r != HB_OK) return r;
    HB_CUDA(ctx, cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, s));
    return HB_OK;
}

int hb_download_async(hb_ctx* ctx, void* dst, const void* src, size_t bytes) {
    if (!ctx || !dst || !src) return fail(ctx, HB_INVALID, "hb_download_async: bad argument");
    hb::bind(ctx);
    cudaStream_t s;
    int r = lane_stream(ctx, HB_LANE_DOWNLOAD, &s);
    if (r != HB_OK) return r;
    HB_CUDA(ctx, cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, s));
    return HB_OK;
}

int hb_host_alloc(hb_ctx* ctx, size_t bytes, void** host_ptr) {
    if (!ctx || !host_ptr || bytes == 0) return fail(ctx, HB_INVALID, "hb_host_alloc: bad argument");
    void* p = nullptr;
    cudaError_t st = cudaHostAlloc(&p, bytes, cudaHostAllocDefault);
    if (st != cudaSuccess) {
        cudaGetLastError();
        return fail(ctx, HB_OOM, std::string("hb_host_alloc: ") + cudaGetErrorString(st));
    }
    ctx->host_allocs.push_back(p);
    *host_ptr = p;
    return HB_OK;
}

int hb_host_free(hb_ctx* ctx, void* host_ptr) {
    if (!ctx || !host_ptr) return HB_OK;
    for (size_t i = 0; i < ctx->host_allocs.size(); ++i)
        if (ctx->host_allocs[i] == host_ptr) {
            ctx->host_allocs.erase(ctx->host_allocs.begin() + i);
            HB_CUDA(ctx, cudaFreeHost(host_ptr));
            return HB_OK;
        }
    return fail(ctx, HB_INVALID, "hb_host_free: not a pointer of hb_host_alloc");
}

int hb_memset(hb_ctx* ctx, void* dst, int value, size_t bytes) {
    if (!ctx || !dst) return fail(ctx, HB_INVALID, "hb_memset: bad argument");
    hb::bind(ctx);
    HB_CUDA(ctx, cudaMemsetAsync(dst, value, bytes, ctx->stream));
    return HB_OK;
}

int hb_sync(hb_ctx* ctx) {
    if (!ctx) return HB_INVALID;
    hb::bind(ctx);
    HB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return hb::check_status(ctx);
}

uint64_t hb_launch_count(const hb_ctx* ctx) { return ctx ? ctx->launches : 0; }

const char* hb_kernel_name(const hb_kernel* k) { return k ? k->name.c_str() : ""; }

int hb_launch(hb_ctx* ctx, const hb_kernel* k, const hb_range* args, int nargs, uint32_t m) {
    if (!ctx || !k || !args) return fail(ctx, HB_INVALID, "hb_launch: bad argument");
    HB_GUARD_BIND(ctx)
    int r = const_cast<hb_kernel*>(k)->launch(ctx, args, nargs, m);
    return r;
    HB_GUARD_END(ctx)
}

int hb_run(hb_ctx* ctx, const hb_op* ops, int nops) {
    if (!ctx || (!ops && nops > 0)) return fail(ctx, HB_INVALID, "hb_run: bad argument");
    for (int i = 0; i < nops; ++i) {
        int r = hb_launch(ctx, ops[i].kernel, ops[i].args, ops[i].nargs, ops[i].m);
        if (r != HB_OK) return r;
    }
    return HB_OK;
}

int hb_time(hb_ctx* ctx, const hb_op* ops, int nops, int reps, double* gpu_seconds) {
    if (!ctx || !gpu_seconds || reps < 1) return fail(ctx, HB_INVALID, "hb_time: bad argument");
    hb::bind(ctx);
    HB_CUDA(ctx, cudaEventRecord(ctx->ev0, ctx->stream));
    for (int r = 0; r < reps; ++r) {
        int s = hb_run(ctx, ops, nops);
        if (s != HB_OK) return s;
    }
    HB_CUDA(ctx, cudaEventRecord(ctx->ev1, ctx->stream));
    HB_CUDA(ctx, cudaEventSynchronize(ctx->ev1));
    float ms = 0.f;
    HB_CUDA(ctx, cudaEventElapsedTime(&ms, ctx->ev0, ctx->ev1));
    *gpu_seconds = (double)ms * 1e-3;
    return hb::check_status(ctx);
}

int hb_set_launch_overlap(hb_ctx* ctx, int on) {
    if (!ctx) return HB_INVALID;
    ctx->overlap_launches = on != 0;
    return HB_OK;
}

// ---- recorded sequences ------------------------------------------------------------------------
struct hb_graph {
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
    uint64_t kernels = 0;
};

int hb_graph_record(hb_ctx* ctx, const hb_op* ops, int nops, hb_graph** out) {
    if (!ctx || !ops || nops < 1 || !out) return fail(ctx, HB_INVALID, "hb_graph_record: bad argument");
    hb::bind(ctx);
    *out = nullptr;
    for (int i = 0; i < nops; ++i) {
        if (!ops[i].kernel) return fail(ctx, HB_INVALID, "hb_graph_record: an op without a kernel");
        if (!ops[i].kernel->replayable) return fail(ctx, HB_UNSUPPORTED, "hb_graph_record: " + ops[i].kernel->name + " cannot be replayed (its launches carry a counter)");
    }
    HB_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    const uint64_t before = ctx->launches;
    HB_CUDA(ctx, cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal));
    int st = hb_run(ctx, ops, nops);
    const std::string why = st != HB_OK ? ctx->err : std::string();  // the failing launch's message, before anything overwrites it
    cudaGraph_t g = nullptr;
    cudaError_t e = cudaStreamEndCapture(ctx->stream, &g);
    const uint64_t recorded = ctx->launches - before;
    ctx->launches = before;  // recording enqueues nothing
    if (st != HB_OK || e != cudaSuccess) {
        if (g) cudaGraphDestroy(g);
        cudaGetLastError();  // a capture that was invalidated leaves a sticky error behind
        if (st != HB_OK) return fail(ctx, st, why);
        return hb::cuda_fail(ctx, e, "cudaStreamEndCapture");
    }
    auto* hg = new (std::nothrow) hb_graph;
    if (!hg) {
        cudaGraphDestroy(g);
        return fail(ctx, HB_OOM, "hb_graph_record: out of memory");
    }
    hg->graph = g;
    hg->kernels = recorded;
    e = cudaGraphInstantiate(&hg->exec, g, 0);
    if (e != cudaSuccess) {
        cudaGraphDestroy(g);
        delete hg;
        return hb::cuda_fail(ctx, e, "cudaGraphInstantiate");
    }
    *out = hg;
    return HB_OK;
}

int hb_graph_launch(hb_ctx* ctx, hb_graph* g) {
    if (!ctx || !g) return fail(ctx, HB_INVALID, "hb_graph_launch: bad argument");
    hb::bind(ctx);
    HB_CUDA(ctx, cudaGraphLaunch(g->exec, ctx->stream));
    ctx->launches += g->kernels;
    return HB_OK;
}

int hb_graph_time(hb_ctx* ctx, hb_graph* g, int reps, double* gpu_seconds) {
    if (!ctx || !g || !gpu_seconds || reps < 1) return fail(ctx, HB_INVALID, "hb_graph_time: bad argument");
    hb::bind(ctx);
    HB_CUDA(ctx, cudaEventRecord(ctx->ev0, ctx->stream));
    for (int r = 0; r < reps; ++r) {
        HB_CUDA(ctx, cudaGraphLaunch(g->exec, ctx->stream));
        ctx->launches += g->kernels;
    }
    HB_CUDA(ctx, cudaEventRecord(ctx->ev1, ctx->stream));
    HB_CUDA(ctx, cudaEventSynchronize(ctx->ev1));
    float ms = 0.f;
    HB_CUDA(ctx, cudaEventElapsedTime(&ms, ctx->ev0, ctx->ev1));
    *gpu_seconds = (double)ms * 1e-3;
    return hb::check_status(ctx);
}

int hb_graph_free(hb_ctx* ctx, hb_graph* g) {
    if (!g) return HB_OK;
    if (ctx) {
        hb::bind(ctx);
        cudaStreamSynchronize(ctx->stream);
    }
    if (g->exec) cudaGraphExecDestroy(g->exec);
    if (g->graph) cudaGraphDestroy(g->graph);
    delete g;
    return HB_OK;
}

int hb_gemm_get(hb_ctx* ctx, const hb_gemm_desc* d, hb_kernel** out) {
    if (!ctx || !d || !out) return fail(ctx, HB_INVALID, "hb_gemm_get: bad argument");
    HB_GUARD_BIND(ctx)
    return hb::make_gemm(ctx, d, out);
    HB_GUARD_END(ctx)
}
int hb_matvec_get(hb_ctx* ctx, const hb_matvec_desc* d, hb_kernel** out) {
    if (!ctx || !d || !out) return fail(ctx, HB_INVALID, "hb_matvec_get: bad argument");
    HB_GUARD_BIND(ctx)
    return hb::make_matvec(ctx, d, out);
    HB_GUARD_END(ctx)
}
int hb_swiglu_get(hb_ctx* ctx, uint32_t n, hb_kernel** out) {
    if (!ctx || !out) return fail(ctx, HB_INVALID, "hb_swiglu_get: bad argument");
    HB_GUARD_BIND(ctx)
    return hb::make_swiglu_rows(ctx, n, out);
    HB_GUARD_END(ctx)
}
int hb_route_get(hb_ctx* ctx, uint32_t experts, uint32_t top_k, hb_kernel** out) {
    if (!ctx || !out) return fail(ctx, HB_INVALID, "hb_route_get: bad argument");
    HB_GUARD_BIND(ctx)
    return hb::make_route(ctx, experts, top_k, out);
    HB_GUARD_END(ctx)
}
int hb_moe_sort_get(hb_ctx* ctx, uint32_t experts, uint32_t top_k, uint32_t rows_max, uint32_t bm, hb_kernel** out) {
    if (!ctx || !out) return fail(ctx, HB_INVALID, "hb_moe_sort_get: bad argument");
    HB_GUARD_BIND(ctx)
    return hb::make_moe_sort(ctx, experts, top_k, rows_max, bm, out);
    HB_GUARD_END(ctx)
}
uint32_t hb_moe_tiles(uint32_t rows_max, uint32_t top_k, uint32_t experts, uint32_t bm) {
    if (bm == 0) return 0;
    return (rows_max * top_k + bm - 1) / bm + experts;
}
int hb_moe_gather_get(hb_ctx* ctx, uint32_t h, uint32_t top_k, hb_kernel** out) {
    if (!ctx || !out) return fail(ctx, HB_INVALID, "hb_moe_gather_get: bad argument");
    HB_GUARD_BIND(ctx)
    return hb::make_moe_gather(ctx, h, top_k, out);
    HB_GUARD_END(ctx)
}
int hb_ep_dispatch_get(hb_ctx* ctx, uint32_t h, uint32_t top_k, uint32_t experts, uint32_t world, uint32_t rank, uint32_t cap, hb_kernel** out) {
    if (!ctx || !out) return fail(ctx, HB_INVALID, "hb_ep_dispatch_get: bad argument");
    HB_GUARD_BIND(ctx)
    return hb::make_ep_move(ctx, false, h, top_k, experts, world, rank, cap, out);
    HB_GUARD_END(ctx)
}
int hb_ep_return_get(hb_ctx* ctx, uint32_t h, uint32_t top_k, uint32_t experts, uint32_t world, uint32_t rank, uint32_t cap, hb_kernel** out) {
    if (!ctx || !out) return fail(ctx, HB_INVALID, "hb_ep_return_get: bad argument");
    HB_GUARD_BIND(ctx)
    return hb::make_ep_move(ctx, true, h, top_k, experts, world, rank, cap, out);
    HB_GUARD_END(ctx)
}
int hb_ep_plan_get(hb_ctx* ctx, uint32_t experts, uint32_t world, uint32_t rank, uint32_t bm, uint32_t cap, hb_kernel** out) {
    if (!ctx || !out) return fail(ctx, HB_INVALID, "hb_ep_plan_get: bad argument");
    HB_GUARD_BIND(ctx)
    return hb::make_ep_plan(ctx, experts, world, rank, bm, cap, out);
    HB_GUARD_END(ctx)
}
int hb_ep_dispatch_direct_get(hb_ctx* ctx, uint32_t h, uint32_t top_k, uint32_t experts, uint32_t world, uint32_t rank, uint32_t cap, hb_kernel** out) {
    if (!ctx || !out) return fail(ctx, HB_INVALID, "hb_ep_dispatch_direct_get: bad argument");
    HB_GUARD_BIND(ctx)
    return hb::make_ep_move(ctx, false, h, top_k, experts, world, rank, cap, out, true);
    HB_GUARD_END(ctx)
}
int hb_ep_plan_direct_get(hb_ctx* ctx, uint32_t experts, uint32_t world, uint32_t rank, uint32_t bm, uint32_t cap, hb_kernel** out) {
    if (!ctx || !out) return fail(ctx, HB_INVALID, "hb_ep_plan_direct_get: bad argument");
    HB_GUARD_BIND(ctx)
    return hb::make_ep_plan(ctx, experts, world, rank, bm, cap, out, true);
    HB_GUARD_END(ctx)
}
int hb_experts_matvec_get(hb_ctx* ctx, uint32_t k, uint32_t n, uint32_t top_k, uint32_t experts, uint32_t x_row, uint32_t x_stride, uint32_t rows_per_warp, hb_kernel** out) {
    if (!ctx || !out) return fail(ctx, HB_INVALID, "hb_experts_matvec_get: bad argument");
    HB_GUARD_BIND(ctx)
    return hb::make_experts_matvec(ctx, k, n, top_k, experts, x_row, x_stride, rows_per_warp, out);
    HB_GUARD_END(ctx)
}
int hb_ep_combine_get(hb_ctx* ctx, uint32_t h, uint32_t top_k, uint32_t world, hb_kernel** out) {
    if (!ctx || !out) return fail(ctx, HB_INVALID, "hb_ep_combine_get: bad argument");
    HB_GUARD_BIND(ctx)
    return hb::make_ep_combine(ctx, h, top_k, world, out);
    HB_GUARD_END(ctx)
}
int hb_ep_combine_sync_get(hb_ctx* ctx, uint32_t h, uint32_t top_k, uint32_t world, uint32_t rank, hb_kernel** out) {
    if (!ctx || !out) return fail(ctx, HB_INVALID, "hb_ep_combine_sync_get: bad argument");
    HB_GUARD_BIND(ctx)
    return hb::make_ep_combine(ctx, h, top_k, world, out, true, rank);
    HB_GUARD_END(ctx)
}
int hb_moe_combine_get(hb_ctx* ctx, uint32_t d, uint32_t top_k, uint32_t f32_sum, hb_kernel** out) {
    if (!ctx || !out) return fail(ctx, HB_INVALID, "hb_moe_combine_get: bad argument");
    HB_GUARD_BIND(ctx)
    return hb::make_moe_combine(ctx, d, top_k, f32_sum, out);
    HB_GUARD_END(ctx)
}

}  // extern "C"
