// sm_100a primitives used by the GEMM kernels: mbarrier, TMA (cp.async.bulk.tensor),
// tcgen05 (tensor memory allocation, MMA, commit, load) and the shared-memory /
// instruction descriptors they take. Inline PTX only; no library headers.
#pragma once

#include <cstdint>
#include <cuda.h>
#include <cuda_runtime.h>

namespace hb {

// ---------------------------------------------------------------- numerics

// Exact widening of a bf16 held in the low 16 bits.
__host__ __device__ __forceinline__ float bf16_to_f32(uint32_t h) {
#ifdef __CUDA_ARCH__
    return __uint_as_float(h << 16);
#else
    union { uint32_t u; float f; } v;
    v.u = h << 16;
    return v.f;
#endif
}

// Round to nearest even: the engine's rule is the integer form (bits + 0x7fff + lsb) >> 16 with no NaN special
// case (reference src/core/bf16.rs:13-23, src/msl/mod.rs:1333-1345). On the device the hardware conversion does the
// same for every value that is not a NaN (zeros, subnormals, the carry into the exponent and into infinity
// included; a test walks the bit patterns), in one instruction instead of five; NaN inputs are outside the contract.
__host__ __device__ __forceinline__ uint32_t f32_to_bf16(float f) {
#ifdef __CUDA_ARCH__
    uint16_t r;
    asm("cvt.rn.bf16.f32 %0, %1;" : "=h"(r) : "f"(f));
    return r;
#else
    union { uint32_t u; float f; } v;
    v.f = f;
    uint32_t bits = v.u;
    return ((bits + 0x7fffu + ((bits >> 16) & 1u)) >> 16) & 0xffffu;
#endif
}

// Two values at once, `lo` into the low half of the result.
__device__ __forceinline__ uint32_t f32x2_to_bf16x2(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}

__device__ __forceinline__ float round_bf16(float f) { return bf16_to_f32(f32_to_bf16(f)); }

// e^x as a fixed sequence of IEEE f32 operations (range reduction by ln 2, a
// degree-6 polynomial evaluated with fused multiply-adds, exponent insertion in
// two exact steps). Every rounding is explicit, so the compiler cannot contract
// or reorder it and a host implementation of the same sequence gives the same
// bits. Max error below 1 ulp on [-87, 88].
__device__ __forceinline__ float exp_f32(float x) {
    if (x != x) return x;
    if (x > 88.72283f) return __int_as_float(0x7f800000);
    if (x < -103.98f) return 0.0f;
    const float LOG2E = 1.44269504088896341f;
    const float LN2_HI = 0.693359375f;
    const float LN2_LO = -2.12194440e-4f;
    float n = rintf(__fmul_rn(x, LOG2E));
    float r = __fmaf_rn(n, -LN2_HI, x);
    r = __fmaf_rn(n, -LN2_LO, r);
    float p = 1.9875691500e-4f;
    p = __fmaf_rn(p, r, 1.3981999507e-3f);
    p = __fmaf_rn(p, r, 8.3334519073e-3f);
    p = __fmaf_rn(p, r, 4.1665795894e-2f);
    p = __fmaf_rn(p, r, 1.6666665459e-1f);
    p = __fmaf_rn(p, r, 5.0000001201e-1f);
    float r2 = __fmul_rn(r, r);
    p = __fmaf_rn(p, r2, r);
    p = __fadd_rn(p, 1.0f);
    int k = (int)n;
    int k1 = k / 2, k2 = k - k1;
    float s1 = __int_as_float((k1 + 127) << 23);
    float s2 = __int_as_float((k2 + 127) << 23);
    return __fmul_rn(__fmul_rn(p, s1), s2);
}

// 1/(1+e^-x) (reference src/msl/mod.rs:885-891), IEEE division.
__device__ __forceinline__ float sigmoid_f32(float x) {
    float e = exp_f32(-x);
    float d = __fadd_rn(1.0f, e);
    return __fdiv_rn(1.0f, d);
}

// bf16(g*sigmoid(g)*u) of two bf16-valued floats, in the order s, g*s, (g*s)*u
// (reference src/metal/prefill.rs:811-813, :2790-2818).
__device__ __forceinline__ uint32_t swiglu_bf16(float g, float u) {
    float s = sigmoid_f32(g);
    float gs = __fmul_rn(g, s);
    return f32_to_bf16(__fmul_rn(gs, u));
}

// ------------------------------------------------- overlapped launches
// A kernel launched with programmatic stream serialization may start while its predecessor on the stream is still
// running; griddep_wait() is where it stops until the predecessor has completed and its memory is visible. What
// comes before the wait must not touch anything the predecessor writes (prefetching weights is fine). A kernel
// calls griddep_launch_dependents() early to let its successor start as SMs free up. Both are no-ops in a plain launch.
__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void griddep_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ----------------------------------------------------------------- argmax
// "The largest logit, the first index on a tie" (reference src/metal/kernels.rs:1461-1565) as the maximum of a
// 64-bit key: order-preserving value bits above the inverted index. The result does not depend on the order in
// which candidates meet. A logit is a candidate only if it is greater than -inf (the reference's compare is
// v > best, starting from -inf): NaN and -inf give key 0, and a row without a candidate gives index 0xffffffff.
// -0 and +0 compare equal, as there.
__device__ __forceinline__ unsigned long long argmax_key(uint32_t bf16_bits, uint32_t idx) {
    const float v = bf16_to_f32(bf16_bits);
    if (!(v > -INFINITY)) return 0ull;
    uint32_t b = __float_as_uint(v);
    if (b == 0x80000000u) b = 0u;
    const uint32_t ord = (b & 0x80000000u) ? ~b : (b | 0x80000000u);
    return ((unsigned long long)ord << 32) | (unsigned long long)(0xffffffffu - idx);
}
__device__ __forceinline__ uint32_t argmax_index_of(unsigned long long key) { return key ? 0xffffffffu - (uint32_t)(key & 0xffffffffull) : 0xffffffffu; }

// Folds one key per row from every block of a grid: block_best[r] (shared memory, r < rows) goes into one of
// ARGMAX_SLOTS global keys of the row (spread so that the atomics do not queue on one address); the block that
// arrives last reduces the slots, writes index[r] and clears keys and counter for the next launch. Call with all
// threads of the block; `arrivals` blocks call it.
constexpr uint32_t ARGMAX_SLOTS = 64;
__device__ __forceinline__ void argmax_fold(const unsigned long long* block_best, uint32_t rows, unsigned long long* keys, uint32_t* counter, uint32_t* index,
                                            uint32_t arrivals) {
    __shared__ uint32_t last_s;
    if (threadIdx.x < rows && block_best[threadIdx.x]) atomicMax(&keys[(size_t)threadIdx.x * ARGMAX_SLOTS + blockIdx.x % ARGMAX_SLOTS], block_best[threadIdx.x]);
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) last_s = atomicAdd(counter, 1u) == arrivals - 1 ? 1u : 0u;
    __syncthreads();
    if (!last_s) return;
    __threadfence();
    for (uint32_t r = threadIdx.x / 32; r < rows; r += blockDim.x / 32) {  // a warp per row
        unsigned long long b = 0ull;
        for (uint32_t sidx = threadIdx.x & 31; sidx < ARGMAX_SLOTS; sidx += 32) {
            const unsigned long long k = atomicExch(&keys[(size_t)r * ARGMAX_SLOTS + sidx], 0ull);
            b = k > b ? k : b;
        }
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) {
            const unsigned long long o = __shfl_xor_sync(0xffffffffu, b, off);
            b = o > b ? o : b;
        }
        if ((threadIdx.x & 31) == 0) index[r] = argmax_index_of(b);
    }
    if (threadIdx.x == 0) *counter = 0u;
}

// ----------------------------------------------------------------- status

// Words of the per-context device status buffer that kernels write on a failed
// bounded wait: [0] = code (0 ok), [1] = block, [2] = where, [3] = detail. ST_BAD_TABLE: a table
// the kernel read (row counts of an exchange) does not fit the buffers it was given; [2], [3] = the numbers.
enum : uint32_t { ST_OK = 0, ST_WAIT_TIMEOUT = 1, ST_BAD_TABLE = 2 };
enum : uint32_t { WHERE_EMPTY = 1, WHERE_FULL = 2, WHERE_TMEM_FULL = 3, WHERE_TMEM_EMPTY = 4, WHERE_PEER = 5 };

__device__ __forceinline__ void report(uint32_t* status, uint32_t code, uint32_t where, uint32_t detail) {
    if (atomicCAS(status, 0u, code) == 0u) {
        status[1] = blockIdx.x;
        status[2] = where;
        status[3] = detail;
    }
}

// Waits until a step number another GPU (or another kernel) stores with release semantics at system scope has reached
// `step`; gives up after `limit` SM cycles. What the writer stored before the number is visible after the wait.
__device__ __forceinline__ bool wait_for_step(const uint32_t* word, uint32_t step, long long limit) {
    const long long t0 = clock64();
    uint32_t v;
    while (true) {
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(word) : "memory");
        if ((int32_t)(v - step) >= 0) return true;
        if (clock64() - t0 > limit) return false;
        __nanosleep(64);
    }
}

// ---------------------------------------------------------------- mbarrier

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

// Wait with a time limit (about two seconds of SM clock): a mis-programmed
// pipeline ends with an error status instead of a hung GPU.
#ifndef HB_WAIT_LIMIT_CYCLES
#define HB_WAIT_LIMIT_CYCLES (4000000000ll)
#endif
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    if (mbar_try_wait(bar, parity)) return true;
    long long t0 = clock64();
    while (true) {
        for (int i = 0; i < 64; ++i)
            if (mbar_try_wait(bar, parity)) return true;
        if (clock64() - t0 > HB_WAIT_LIMIT_CYCLES) return false;
    }
}

// --------------------------------------------------------------------- TMA

__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* d) {
    asm volatile("prefetch.tensormap [%0];" ::"l"((uint64_t)d) : "memory");
}
// 2-D tiled load global -> shared, completion on an mbarrier of this CTA.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* d, uint32_t bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"((uint64_t)d), "r"(bar), "r"(x), "r"(y)
        : "memory");
}
// 2-D tiled store shared -> global (bulk async group).
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* d, uint32_t src, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                 ::"l"((uint64_t)d), "r"(src), "r"(x), "r"(y)
                 : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void tma_store_wait_read() {
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N>
__device__ __forceinline__ void tma_store_wait() {
    asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

// ----------------------------------------------------------------- tcgen05

__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// D[tmem] (+)= A[smem] * B[smem]^T, bf16 inputs, f32 accumulate, one CTA.
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// The mbarrier gets one arrival when every MMA issued so far by this thread is done.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// 32 lanes x 32 consecutive f32 columns: thread t of the warp gets lane (base lane + t).
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_32x16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
// The reverse of tmem_ld_32x32: thread t of the warp writes 32 consecutive f32 columns of lane (base lane + t).
__device__ __forceinline__ void tmem_st_32x32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]),
          "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]),
          "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// Untiled bulk copy global -> shared (16-byte aligned, size a multiple of 16), completion on an mbarrier.
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}

// Shared-memory matrix descriptor of a K-major bf16 tile whose rows are 128
// bytes (64 elements) in the 128-byte swizzle TMA writes: 8-row groups are
// 1024 bytes apart (stride byte offset), the leading byte offset is unused,
// descriptor version 1, layout type 2 (128-byte swizzle). The tile base must
// be 1024-byte aligned; stepping K by 16 elements adds 32 bytes to the start.
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)(1024u >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

// Instruction descriptor, kind::f16: f32 accumulator (bits 4-5 = 1), A and B
// bf16 (bits 7-9, 10-12 = 1), both K-major (bits 15, 16 = 0), N/8 at bit 17,
// M/16 at bit 24.
__host__ __device__ constexpr uint32_t umma_idesc_bf16(uint32_t m, uint32_t n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

}  // namespace hb
