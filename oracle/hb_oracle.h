/*
 * CPU oracle for the bf16 matrix-multiply path of herbert-metal-bf16.
 *
 * TEST INFRASTRUCTURE ONLY. This is a plain-C restatement of the arithmetic the
 * reference engine's kernels perform on this path; it is the checker that the
 * tests, the smoke run and the benchmark's CPU-baseline leg call. The product
 * (the CUDA library) never links or calls anything in this directory.
 *
 * Parity status: PARITY UNPINNED BY REFERENCE FIXTURES. The reference holds no
 * golden vector or known-answer test for its GEMM, matvec, route, sort or
 * combine kernels (its two bf16.rs unit tests cover f16 only), and its kernels
 * exist only as Metal shader text emitted at run time, which cannot execute
 * here. What pins this file is the arithmetic written in the reference source
 * (cited per function below) plus known-answer vectors derived by hand from
 * those rules (tests/golden/).
 *
 * Citations are path:line inside the reference project.
 */
#ifndef HB_ORACLE_H
#define HB_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Epilogue modes, src/metal/kernels.rs:30-42. */
enum { HBO_OUT_BF16 = 0, HBO_OUT_F32 = 1, HBO_OUT_RESIDUAL = 2, HBO_OUT_SWIGLU = 3 };

/* ---- scalar rules ------------------------------------------------------ */
/* src/core/bf16.rs:7-9 (exact widening) and :13-23 (round to nearest even on
 * the integer bits, no NaN special case; msl/mod.rs:1333-1345 is the same rule
 * written (bits + 0x7fff + lsb) >> 16). */
float hbo_bf16_to_f32(uint16_t h);
uint16_t hbo_f32_to_bf16(float v);
/* f rounded to bf16 and widened again, msl/mod.rs:1361-1372. */
float hbo_round_bf16(float v);
/* A double rounded ONCE to bf16 (round-to-odd to f32, then the rule above). */
uint16_t hbo_f64_to_bf16(double v);
/* e^x in f32. The reference calls the Metal library's exp with fast-math off
 * (src/metal/gpu.rs:128-130); its bits are the driver's. Here exp is a fixed
 * sequence of IEEE f32 operations (range reduction by ln2, degree-6 polynomial
 * with fused multiply-adds, exponent insertion) so that every implementation of
 * this contract gives the same bits. Max error 1 ulp over [-88, 88]. */
float hbo_expf(float x);
/* 1/(1+e^-x), msl/mod.rs:885-891. */
float hbo_sigmoid(float x);
/* bf16((g*sigmoid(g))*u) for bf16 g and u, prefill.rs:2790-2818, kernels.rs:256-261. */
uint16_t hbo_swiglu_one(uint16_t g, uint16_t u);

/* ---- dense product + epilogue ----------------------------------------- */
/* Y[m][n] = epilogue(sum_k X[m][k]*W[n][k]); X [M][K], W [N][K] bf16 row-major
 * (prefill.rs:6-7, :852-1301). `y` is bf16 [M][N] (BF16, RESIDUAL: read and
 * written), f32 [M][N] (F32) or bf16 [M][N/2] (SWIGLU: W rows 0..N/2 are the
 * gate, N/2..N the up, prefill.rs:784-789,811-818).
 * hbo_gemm_f64: dot products accumulated in f64, rounded once (the primary
 * oracle). hbo_gemm_f32: the engine's contract as a CPU kernel - f32
 * accumulation, one RNE - threaded with OpenMP; this is the timed CPU baseline.
 * Epilogues: prefill.rs:1200-1230, kernels.rs:217-234. */
void hbo_gemm_f64(const uint16_t* x, const uint16_t* w, void* y, int m, int n, int k, int out);
void hbo_gemm_f32(const uint16_t* x, const uint16_t* w, void* y, int m, int n, int k, int out);
/* The same, for selected rows only: row_ids[i] indexes X and Y rows. */
void hbo_gemm_f64_rows(const uint16_t* x, const uint16_t* w, void* y, const int* row_ids, int nrows, int n, int k, int out);
/* The matvec in the reference's own order (kernels.rs:146-214): 32 lanes
 * stride K by chunks of 8, an f32 FMA chain per lane, butterfly sum. M=1. */
void hbo_matvec_ref_order(const uint16_t* x, const uint16_t* w, uint16_t* y, int n, int k);
/* Unfused SwiGLU over [m][2n] -> [m][n], prefill.rs:2790-2818. */
void hbo_swiglu_rows(const uint16_t* gu, uint16_t* h, int m, int n);

/* ---- MoE --------------------------------------------------------------- */
/* qwen_kernels.rs:1802-1878. scores bf16 [rows][experts]; route u32
 * [rows][2*top_k]: experts in increasing order, then the f32 bits of their
 * bf16-rounded renormalised weights. Softmax sums: 32-lane butterfly sums
 * (xor 16,8,4,2,1), warps folded in order (msl/mod.rs:716-756). */
void hbo_route_topk(const uint16_t* scores, uint32_t* route, int rows, int experts, int top_k);
/* prefill.rs:1303-1442. list u32[rows*top_k]; tiles u32[1+3*max_tiles].
 * Returns the number of tiles. */
int hbo_moe_sort(const uint32_t* route, int rows, int experts, int top_k, int bm, uint32_t* list, uint32_t* tiles);
/* Expert gate/up over the sorted rows (prefill.rs:317-328,929-941): row p
 * reads X[list[p]/top_k], W rows e*2mi.., writes EGU[p] (bf16 [pairs][2mi]). */
void hbo_moe_gate_up(const uint16_t* x, const uint16_t* wgu, const uint32_t* list, const uint32_t* tiles, uint16_t* egu, int h, int mi, int top_k);
/* qwen_kernels.rs:2087: EHB[p][f] = swiglu(EGU[p][f], EGU[p][mi+f]). */
void hbo_swiglu_slots(const uint16_t* egu, uint16_t* ehb, int pairs, int mi);
/* Expert down with scatter (prefill.rs:1206-1209): EY[list[p]] = bf16(EHB[p] . Wd rows e*h..). */
void hbo_moe_down(const uint16_t* ehb, const uint16_t* wd, const uint32_t* list, const uint32_t* tiles, uint16_t* ey, int h, int mi);
/* qwen_kernels.rs:2119-2161: acc = bf16(acc + bf16(y*w)) over the slots. */
void hbo_moe_combine(const uint16_t* ey, const uint32_t* route, uint16_t* out, int rows, int d, int top_k);
/* The combine as an f32 sum (a variant some callers ask for; the reference rounds to bf16 at every step): out = bf16(sum_s y_s*w_s), f32 FMA chain in slot order. */
void hbo_moe_combine_f32(const uint16_t* ey, const uint32_t* route, uint16_t* out, int rows, int d, int top_k);

/* ---- the rows around the matrix products ------------------------------- */
/* prefill.rs:70-117 (rmsnorm_rows), kernels.rs:355-442 (norm_into, the same sums): per row of d, 256 lanes each an
 * FMA chain over i = lane, lane + 256, ...; the 32 lanes of a simdgroup summed (xor butterfly 16..1), the 8 partials
 * folded in order; inv = 1 / sqrt(ss * (1/d) + eps); y = bf16((x * inv) * (w [+ 1])). */
void hbo_rmsnorm_rows(const uint16_t* x, const uint16_t* w, uint16_t* y, int rows, int d, float eps, int plus_one);
/* kernels.rs:1461-1565 (argmax_partial + argmax_final): index of the largest bf16 logit of each row, the first
 * index on a tie; 0xffffffff when no logit is greater than -inf (NaN never wins: the compare is v > best). */
void hbo_argmax_rows(const uint16_t* logits, uint32_t* idx, int rows, int n);
/* qwen_kernels.rs:2163-2214 (moe_out): g = bf16(sigmoid(bf16(xn . gate))) with the dot product summed as in
 * rmsnorm_rows; x = bf16(x + bf16(experts + bf16(g * shared))), in place. */
void hbo_moe_out(const uint16_t* xn, const uint16_t* gate, const uint16_t* experts, const uint16_t* shared, uint16_t* x, int rows, int d);

/* ---- Q4_0 weights -------------------------------------------------------- */
/* src/metal/q4.rs:16-103 (quantize): W [n][k] bf16 -> per block of 32 along k a 16-byte word group and an f16 scale.
 * Byte b of word i of a block holds weight 8i + b in its low nibble and 8i + 4 + b in its high one, two's complement
 * (q in -8..7); d is the candidate m / c (m the value of largest magnitude, c in -8, 7, -7, ... -1 in that order) with
 * the least squared error, the first on a tie. data: n*k/2 bytes, scales: n*k/32 f16 bit patterns. */
void hbo_q4_quantize(const uint16_t* w, int n, int k, uint8_t* data, uint16_t* scales);
/* src/metal/kernels.rs:1074-1102, 1425-1450 (dequant_q4, q4_word_bf16): out[n][k] = bf16(d * q). */
void hbo_q4_dequant(const uint8_t* data, const uint16_t* scales, int n, int k, uint16_t* out);
/* src/metal/kernels.rs:526-632 (matvec_q4, rows = 1): lane l of 32 takes blocks l, l + 32, ...; per block an FMA chain
 * part = fma(q_e, x_e, part) over e in the order 8i + b, 8i + 4 + b (i, b = 0..3), then acc = fma(d, part, acc); the
 * lanes are summed by the xor butterfly; the output mode as for the matvec (y holds the old values for RESIDUAL). */
void hbo_matvec_q4(const uint8_t* data, const uint16_t* scales, const uint16_t* x, void* y, int n, int k, int out);
/* src/metal/kernels.rs:472-500, 896-928 (matvec_q4_split): the same with the blocks of a row shared by `split`
 * simdgroups (block b to simdgroup (b / 32) % split), each simdgroup's butterfly sum, the partials added in order. */
void hbo_matvec_q4_split(const uint8_t* data, const uint16_t* scales, const uint16_t* x, void* y, int n, int k, int out, int split);
/* src/metal/kernels.rs:983-1071 (matmul_q4): Y[r][.] = bf16(W . X[r]) for the m rows of a block, row r of X at r * ldx
 * and of Y at r * ldy (bf16 elements); each row's sum runs in matvec_q4's order, so a block gives the decode step's bits. */
void hbo_matmul_q4(const uint8_t* data, const uint16_t* scales, const uint16_t* x, uint16_t* y, int n, int k, int m, int ldx, int ldy);
/* src/metal/kernels.rs:455-462, 1387-1424 (matvec_q4s, "llama.cpp's masks"): the same product with the sums in another
 * order. Per block: sx = x_0 + x_1 + ... + x_31 (in order); every word xored with 0x88888888 (nibbles become q + 8);
 * part = fma(float(word & (15 << s_j)), x_e * 2^-s_j, part) over e = 8i + j, j = 0..7 (the low nibbles of bytes 0..3,
 * then the high ones); part = fma(-8, sx, part); acc = fma(d, part, acc). */
void hbo_matvec_q4s(const uint8_t* data, const uint16_t* scales, const uint16_t* x, void* y, int n, int k, int out);

/* ---- the selection loop's correctness rule ----------------------------- */
/* qwen.rs:2497-2543: scale = max(max|ref|,1e-6); err = max|ref-got|;
 * returns 1 (eligible) iff err <= scale/64 (NaN fails). f32_out selects the
 * element type of both arrays. */
int hbo_check_1_64(const void* ref, const void* got, size_t count, int f32_out, float* err, float* scale);

/* ---- seeded inputs ------------------------------------------------------ */
/* Counter-based: element i of tensor `tensor_id` under `seed` is
 * sigma * z, z = (sum of twelve 16-bit fields of three splitmix64 outputs -
 * 12*32767.5)/65536 (Irwin-Hall, variance 1), rounded to bf16. Integer and
 * exact-f64 arithmetic only, so any platform reproduces the bits. */
void hbo_fill_normal(uint16_t* dst, size_t count, uint64_t seed, uint64_t tensor_id, double sigma);
/* qwen.rs:2613-2626: xorshift32 (<<13, >>17, <<5), (s>>8)/2^23 - 1 in [-1,1),
 * rounded to bf16; returns the state after the last element. */
uint32_t hbo_fill_xorshift16(uint16_t* dst, size_t count, uint32_t seed);
/* herbert-metal-probe.rs:435-462: magnitudes 2^-6..2^-1 from the 64-bit LCG. */
void hbo_fill_random16(uint16_t* dst, size_t count, uint64_t seed);

/* ---- comparison helpers ------------------------------------------------- */
typedef struct {
    size_t count;       /* elements compared */
    size_t over_1ulp;   /* elements more than 1 bf16 ulp apart */
    size_t mismatched;  /* elements whose bits differ */
    uint32_t max_ulp;   /* largest distance in bf16 ulps */
    float max_abs_err;  /* largest |ref-got| */
    float max_abs_ref;  /* largest |ref| */
} hbo_cmp;
void hbo_compare_bf16(const uint16_t* ref, const uint16_t* got, size_t count, hbo_cmp* out);

int hbo_threads(void);

#ifdef __cplusplus
}
#endif
#endif
