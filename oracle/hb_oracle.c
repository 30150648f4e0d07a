/*
 * CPU oracle for the bf16 matrix-multiply path of herbert-metal-bf16.
 * TEST INFRASTRUCTURE ONLY - see hb_oracle.h for scope, citations and the
 * "parity unpinned" note. Build: make -C oracle  (gcc, -ffp-contract=off so
 * that no multiply-add is fused unless written as fmaf).
 */
#include "hb_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

/* ------------------------------------------------------------------ scalars */

static inline uint32_t f2u(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static inline float u2f(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }

float hbo_bf16_to_f32(uint16_t h) { return u2f((uint32_t)h << 16); }

/* src/core/bf16.rs:13-23: result = bits>>16, +1 when the round bit is set and
 * (sticky bits non-zero or the kept lsb is 1). */
uint16_t hbo_f32_to_bf16(float v) {
    uint32_t bits = f2u(v);
    uint32_t lsb = (bits >> 16) & 1u;
    uint32_t round_bit = (bits >> 15) & 1u;
    uint32_t sticky = bits & 0x7FFFu;
    uint32_t r = bits >> 16;
    if (round_bit == 1u && (sticky != 0u || lsb == 1u)) r += 1u;
    return (uint16_t)r;
}

float hbo_round_bf16(float v) { return hbo_bf16_to_f32(hbo_f32_to_bf16(v)); }

uint16_t hbo_f64_to_bf16(double v) {
    float f = (float)v; /* RNE */
    if ((double)f != v && isfinite(f)) {
        /* make it round-to-odd: truncate toward zero, then set the lsb */
        if (fabs((double)f) > fabs(v)) f = nextafterf(f, 0.0f);
        f = u2f(f2u(f) | 1u);
    }
    return hbo_f32_to_bf16(f);
}

static inline float pow2i(int j) { return u2f((uint32_t)(j + 127) << 23); }

float hbo_expf(float x) {
    if (x != x) return x;
    if (x > 88.72283f) return INFINITY;
    if (x < -103.98f) return 0.0f;
    const float LOG2E = 1.44269504088896341f;
    const float LN2_HI = 0.693359375f;
    const float LN2_LO = -2.12194440e-4f;
    float n = rintf(x * LOG2E);
    float r = fmaf(n, -LN2_HI, x);
    r = fmaf(n, -LN2_LO, r);
    float p = 1.9875691500e-4f;
    p = fmaf(p, r, 1.3981999507e-3f);
    p = fmaf(p, r, 8.3334519073e-3f);
    p = fmaf(p, r, 4.1665795894e-2f);
    p = fmaf(p, r, 1.6666665459e-1f);
    p = fmaf(p, r, 5.0000001201e-1f);
    float r2 = r * r;
    p = fmaf(p, r2, r);
    p = p + 1.0f;
    int k = (int)n;
    int k1 = k / 2, k2 = k - k1;
    return (p * pow2i(k1)) * pow2i(k2);
}

float hbo_sigmoid(float x) {
    float e = hbo_expf(-x);
    float d = 1.0f + e;
    return 1.0f / d;
}

static inline float swiglu_f(float g, float u) {
    float s = hbo_sigmoid(g);
    float gs = g * s;
    return gs * u;
}

uint16_t hbo_swiglu_one(uint16_t g, uint16_t u) {
    return hbo_f32_to_bf16(swiglu_f(hbo_bf16_to_f32(g), hbo_bf16_to_f32(u)));
}

/* ----------------------------------------------------------------- epilogue */

/* One output from an f32 accumulator, kernels.rs:217-234 / prefill.rs:1200-1230. */
static inline void store_out(void* y, size_t at, float acc, int out) {
    switch (out) {
    case HBO_OUT_F32: ((float*)y)[at] = acc; break;
    case HBO_OUT_BF16: ((uint16_t*)y)[at] = hbo_f32_to_bf16(acc); break;
    case HBO_OUT_RESIDUAL: {
        float r = hbo_round_bf16(acc);
        float old = hbo_bf16_to_f32(((uint16_t*)y)[at]);
        ((uint16_t*)y)[at] = hbo_f32_to_bf16(old + r);
    } break;
    default: break;
    }
}

/* The same from an f64 sum: the product is rounded ONCE to bf16 (or to f32 for
 * the F32 mode), then the mode's further f32 steps follow. */
static inline void store_out64(void* y, size_t at, double acc, int out) {
    switch (out) {
    case HBO_OUT_F32: ((float*)y)[at] = (float)acc; break;
    case HBO_OUT_BF16: ((uint16_t*)y)[at] = hbo_f64_to_bf16(acc); break;
    case HBO_OUT_RESIDUAL: {
        float r = hbo_bf16_to_f32(hbo_f64_to_bf16(acc));
        float old = hbo_bf16_to_f32(((uint16_t*)y)[at]);
        ((uint16_t*)y)[at] = hbo_f32_to_bf16(old + r);
    } break;
    default: break;
    }
}

static double dotdd(const double* a, const double* b, int k) {
    double s = 0.0;
#pragma omp simd reduction(+ : s)
    for (int i = 0; i < k; ++i) s += a[i] * b[i];
    return s;
}

void hbo_gemm_f64_rows(const uint16_t* x, const uint16_t* w, void* y, const int* row_ids, int nrows, int n, int k, int out) {
    int nout = out == HBO_OUT_SWIGLU ? n / 2 : n;
    /* the selected X rows widened once (exact) */
    double* xd = (double*)malloc((size_t)nrows * k * sizeof(double));
#pragma omp parallel for schedule(static)
    for (int i = 0; i < nrows; ++i) {
        int r = row_ids ? row_ids[i] : i;
        for (int j = 0; j < k; ++j) xd[(size_t)i * k + j] = (double)hbo_bf16_to_f32(x[(size_t)r * k + j]);
    }
#pragma omp parallel
    {
        double* wd = (double*)malloc((size_t)2 * k * sizeof(double));
#pragma omp for schedule(static)
        for (int c = 0; c < nout; ++c) {
            for (int j = 0; j < k; ++j) wd[j] = (double)hbo_bf16_to_f32(w[(size_t)c * k + j]);
            if (out == HBO_OUT_SWIGLU)
                for (int j = 0; j < k; ++j) wd[k + j] = (double)hbo_bf16_to_f32(w[(size_t)(nout + c) * k + j]);
            for (int i = 0; i < nrows; ++i) {
                int r = row_ids ? row_ids[i] : i;
                const double* xr = xd + (size_t)i * k;
                if (out == HBO_OUT_SWIGLU) {
                    uint16_t g = hbo_f64_to_bf16(dotdd(xr, wd, k));
                    uint16_t u = hbo_f64_to_bf16(dotdd(xr, wd + k, k));
                    ((uint16_t*)y)[(size_t)r * nout + c] = hbo_swiglu_one(g, u);
                } else {
                    store_out64(y, (size_t)r * n + c, dotdd(xr, wd, k), out);
                }
            }
        }
        free(wd);
    }
    free(xd);
}

void hbo_gemm_f64(const uint16_t* x, const uint16_t* w, void* y, int m, int n, int k, int out) {
    hbo_gemm_f64_rows(x, w, y, NULL, m, n, k, out);
}

/* f32-accumulate contract kernel (the timed CPU baseline): X widened once, four W rows widened
 * per step into a thread-local buffer and reused over every X row, 4x4 register block, the k loop
 * left to the compiler's vectoriser (partial sums per SIMD lane, folded at the end: an
 * accumulation order, as every GPU kernel has its own). */
static void widen(const uint16_t* s, float* d, size_t count) {
    for (size_t i = 0; i < count; ++i) d[i] = hbo_bf16_to_f32(s[i]);
}

void hbo_gemm_f32(const uint16_t* x, const uint16_t* w, void* y, int m, int n, int k, int out) {
    float* xf = (float*)malloc((size_t)m * k * sizeof(float));
#pragma omp parallel for schedule(static)
    for (int r = 0; r < m; ++r) widen(x + (size_t)r * k, xf + (size_t)r * k, (size_t)k);
    int nout = out == HBO_OUT_SWIGLU ? n / 2 : n;
    float* acc_all = NULL;
    if (out == HBO_OUT_SWIGLU) acc_all = (float*)malloc((size_t)m * n * sizeof(float));
    int nb = (n + 3) / 4;
#pragma omp parallel
    {
        float* wf = (float*)malloc((size_t)4 * k * sizeof(float));
#pragma omp for schedule(dynamic, 8)
        for (int cb = 0; cb < nb; ++cb) {
            int c0 = cb * 4;
            int cn = n - c0 < 4 ? n - c0 : 4;
            for (int j = 0; j < 4; ++j) widen(w + (size_t)(c0 + (j < cn ? j : 0)) * k, wf + (size_t)j * k, (size_t)k);
            const float *w0 = wf, *w1 = wf + k, *w2 = wf + 2 * (size_t)k, *w3 = wf + 3 * (size_t)k;
            for (int r0 = 0; r0 < m; r0 += 4) {
                int rn = m - r0 < 4 ? m - r0 : 4;
                const float* x0 = xf + (size_t)r0 * k;
                const float* x1 = xf + (size_t)(r0 + (rn > 1 ? 1 : 0)) * k;
                const float* x2 = xf + (size_t)(r0 + (rn > 2 ? 2 : 0)) * k;
                const float* x3 = xf + (size_t)(r0 + (rn > 3 ? 3 : 0)) * k;
                float a00 = 0, a01 = 0, a02 = 0, a03 = 0, a10 = 0, a11 = 0, a12 = 0, a13 = 0;
                float a20 = 0, a21 = 0, a22 = 0, a23 = 0, a30 = 0, a31 = 0, a32 = 0, a33 = 0;
#pragma omp simd reduction(+ : a00, a01, a02, a03, a10, a11, a12, a13, a20, a21, a22, a23, a30, a31, a32, a33)
                for (int i = 0; i < k; ++i) {
                    float b0 = w0[i], b1 = w1[i], b2 = w2[i], b3 = w3[i];
                    float v0 = x0[i], v1 = x1[i], v2 = x2[i], v3 = x3[i];
                    a00 += v0 * b0; a01 += v0 * b1; a02 += v0 * b2; a03 += v0 * b3;
                    a10 += v1 * b0; a11 += v1 * b1; a12 += v1 * b2; a13 += v1 * b3;
                    a20 += v2 * b0; a21 += v2 * b1; a22 += v2 * b2; a23 += v2 * b3;
                    a30 += v3 * b0; a31 += v3 * b1; a32 += v3 * b2; a33 += v3 * b3;
                }
                float a[4][4] = {{a00, a01, a02, a03}, {a10, a11, a12, a13}, {a20, a21, a22, a23}, {a30, a31, a32, a33}};
                for (int i = 0; i < rn; ++i)
                    for (int j = 0; j < cn; ++j) {
                        size_t at = (size_t)(r0 + i) * n + (c0 + j);
                        if (out == HBO_OUT_SWIGLU) acc_all[at] = a[i][j];
                        else store_out(y, at, a[i][j], out);
                    }
            }
        }
        free(wf);
    }
    if (out == HBO_OUT_SWIGLU) {
#pragma omp parallel for schedule(static)
        for (int r = 0; r < m; ++r)
            for (int c = 0; c < nout; ++c) {
                uint16_t g = hbo_f32_to_bf16(acc_all[(size_t)r * n + c]);
                uint16_t u = hbo_f32_to_bf16(acc_all[(size_t)r * n + nout + c]);
                ((uint16_t*)y)[(size_t)r * nout + c] = hbo_swiglu_one(g, u);
            }
        free(acc_all);
    }
    free(xf);
}

/* kernels.rs:146-214 with a 32-lane simdgroup: lane l takes chunks l, l+32, ..
 * of 8 bf16; inside a chunk the FMAs run lo, hi of each 32-bit word in order;
 * simd_sum is taken as the xor butterfly 16,8,4,2,1. */
void hbo_matvec_ref_order(const uint16_t* x, const uint16_t* w, uint16_t* y, int n, int k) {
    int chunks = k / 8;
#pragma omp parallel for schedule(static)
    for (int row = 0; row < n; ++row) {
        float lane[32];
        for (int l = 0; l < 32; ++l) {
            float a = 0.0f;
            for (int c = l; c < chunks; c += 32)
                for (int i = 0; i < 8; ++i)
                    a = fmaf(hbo_bf16_to_f32(w[(size_t)row * k + c * 8 + i]), hbo_bf16_to_f32(x[c * 8 + i]), a);
            lane[l] = a;
        }
        for (int off = 16; off >= 1; off >>= 1) {
            float t[32];
            for (int l = 0; l < 32; ++l) t[l] = lane[l] + lane[l ^ off];
            memcpy(lane, t, sizeof t);
        }
        y[row] = hbo_f32_to_bf16(lane[0]);
    }
}

void hbo_swiglu_rows(const uint16_t* gu, uint16_t* h, int m, int n) {
#pragma omp parallel for schedule(static)
    for (int r = 0; r < m; ++r)
        for (int c = 0; c < n; ++c)
            h[(size_t)r * n + c] = hbo_swiglu_one(gu[(size_t)r * 2 * n + c], gu[(size_t)r * 2 * n + n + c]);
}

/* ---------------------------------------------------------------------- MoE */

static float butterfly_sum32(const float* v) {
    float a[32], t[32];
    memcpy(a, v, sizeof a);
    for (int off = 16; off >= 1; off >>= 1) {
        for (int l = 0; l < 32; ++l) t[l] = a[l] + a[l ^ off];
        memcpy(a, t, sizeof a);
    }
    return a[0];
}

void hbo_route_topk(const uint16_t* scores, uint32_t* route, int rows, int experts, int top_k) {
#pragma omp parallel for schedule(static)
    for (int row = 0; row < rows; ++row) {
        float* p = (float*)malloc(sizeof(float) * (size_t)experts);
        const uint16_t* s = scores + (size_t)row * experts;
        float mx = hbo_bf16_to_f32(s[0]);
        for (int e = 1; e < experts; ++e) mx = fmaxf(mx, hbo_bf16_to_f32(s[e]));
        for (int e = 0; e < experts; ++e) p[e] = hbo_expf(hbo_bf16_to_f32(s[e]) - mx);
        float sum = butterfly_sum32(p);
        for (int g = 1; g < experts / 32; ++g) sum = sum + butterfly_sum32(p + 32 * g);
        for (int e = 0; e < experts; ++e) p[e] = p[e] / sum;
        uint32_t chosen[64];
        float vals[64];
        for (int t = 0; t < top_k; ++t) {
            float best = -2.0f;
            uint32_t idx = 0;
            for (int e = 0; e < experts; ++e)
                if (p[e] > best) { best = p[e]; idx = (uint32_t)e; }
            p[idx] = -1.0f;
            chosen[t] = idx;
            vals[t] = best;
        }
        float total = 0.0f;
        for (int t = 0; t < top_k; ++t) total = total + vals[t];
        uint32_t* r = route + (size_t)row * 2 * top_k;
        for (int i = 0; i < top_k; ++i) {
            float wgt = hbo_round_bf16(vals[i] / total);
            int rank = 0;
            for (int j = 0; j < top_k; ++j)
                if (j != i && chosen[j] < chosen[i]) rank++;
            r[rank] = chosen[i];
            r[top_k + rank] = f2u(wgt);
        }
        free(p);
    }
}

int hbo_moe_sort(const uint32_t* route, int rows, int experts, int top_k, int bm, uint32_t* list, uint32_t* tiles) {
    int pairs = rows * top_k;
    uint32_t* cnt = (uint32_t*)calloc((size_t)experts + 1, sizeof(uint32_t));
    uint32_t* off = (uint32_t*)calloc((size_t)experts + 1, sizeof(uint32_t));
    for (int i = 0; i < pairs; ++i) cnt[route[(size_t)(i / top_k) * 2 * top_k + (i % top_k)]]++;
    uint32_t total = 0, nt = 0;
    for (int e = 0; e < experts; ++e) {
        uint32_t c = cnt[e], start = total;
        off[e] = start;
        for (uint32_t j = 0; j < c; j += (uint32_t)bm) {
            tiles[1 + 3 * nt] = (uint32_t)e;
            tiles[2 + 3 * nt] = start + j;
            tiles[3 + 3 * nt] = c - j > (uint32_t)bm ? (uint32_t)bm : c - j;
            nt++;
        }
        total += c;
    }
    tiles[0] = nt;
    for (int i = 0; i < pairs; ++i) {
        uint32_t e = route[(size_t)(i / top_k) * 2 * top_k + (i % top_k)];
        list[off[e]++] = (uint32_t)i;
    }
    free(cnt);
    free(off);
    return (int)nt;
}

void hbo_moe_gate_up(const uint16_t* x, const uint16_t* wgu, const uint32_t* list, const uint32_t* tiles, uint16_t* egu, int h, int mi, int top_k) {
    int nt = (int)tiles[0];
#pragma omp parallel for schedule(dynamic, 1)
    for (int t = 0; t < nt; ++t) {
        uint32_t e = tiles[1 + 3 * t], start = tiles[2 + 3 * t], rows = tiles[3 + 3 * t];
        double* xd = (double*)malloc(((size_t)rows + 1) * h * sizeof(double));
        double* wd = xd + (size_t)rows * h;
        for (uint32_t i = 0; i < rows; ++i) {
            const uint16_t* xr = x + (size_t)(list[start + i] / (uint32_t)top_k) * h;
            for (int j = 0; j < h; ++j) xd[(size_t)i * h + j] = (double)hbo_bf16_to_f32(xr[j]);
        }
        for (int j = 0; j < 2 * mi; ++j) {
            const uint16_t* wr = wgu + ((size_t)e * 2 * mi + j) * h;
            for (int i = 0; i < h; ++i) wd[i] = (double)hbo_bf16_to_f32(wr[i]);
            for (uint32_t i = 0; i < rows; ++i)
                egu[(size_t)(start + i) * 2 * mi + j] = hbo_f64_to_bf16(dotdd(xd + (size_t)i * h, wd, h));
        }
        free(xd);
    }
}

void hbo_swiglu_slots(const uint16_t* egu, uint16_t* ehb, int pairs, int mi) {
    hbo_swiglu_rows(egu, ehb, pairs, mi);
}

void hbo_moe_down(const uint16_t* ehb, const uint16_t* wd, const uint32_t* list, const uint32_t* tiles, uint16_t* ey, int h, int mi) {
    int nt = (int)tiles[0];
#pragma omp parallel for schedule(dynamic, 1)
    for (int t = 0; t < nt; ++t) {
        uint32_t e = tiles[1 + 3 * t], start = tiles[2 + 3 * t], rows = tiles[3 + 3 * t];
        double* xd = (double*)malloc(((size_t)rows + 1) * mi * sizeof(double));
        double* wr = xd + (size_t)rows * mi;
        for (uint32_t i = 0; i < rows; ++i)
            for (int j = 0; j < mi; ++j) xd[(size_t)i * mi + j] = (double)hbo_bf16_to_f32(ehb[(size_t)(start + i) * mi + j]);
        for (int c = 0; c < h; ++c) {
            const uint16_t* w = wd + ((size_t)e * h + c) * mi;
            for (int j = 0; j < mi; ++j) wr[j] = (double)hbo_bf16_to_f32(w[j]);
            for (uint32_t i = 0; i < rows; ++i)
                ey[(size_t)list[start + i] * h + c] = hbo_f64_to_bf16(dotdd(xd + (size_t)i * mi, wr, mi));
        }
        free(xd);
    }
}

void hbo_moe_combine(const uint16_t* ey, const uint32_t* route, uint16_t* out, int rows, int d, int top_k) {
#pragma omp parallel for schedule(static)
    for (int row = 0; row < rows; ++row)
        for (int i = 0; i < d; ++i) {
            float acc = 0.0f;
            for (int s = 0; s < top_k; ++s) {
                float yf = hbo_bf16_to_f32(ey[((size_t)row * top_k + s) * d + i]);
                float wf = u2f(route[(size_t)row * 2 * top_k + top_k + s]);
                float c = hbo_round_bf16(yf * wf);
                acc = hbo_round_bf16(acc + c);
            }
            out[(size_t)row * d + i] = hbo_f32_to_bf16(acc);
        }
}

void hbo_moe_combine_f32(const uint16_t* ey, const uint32_t* route, uint16_t* out, int rows, int d, int top_k) {
#pragma omp parallel for schedule(static)
    for (int row = 0; row < rows; ++row)
        for (int i = 0; i < d; ++i) {
            float acc = 0.0f;
            for (int s = 0; s < top_k; ++s) {
                float yf = hbo_bf16_to_f32(ey[((size_t)row * top_k + s) * d + i]);
                float wf = u2f(route[(size_t)row * 2 * top_k + top_k + s]);
                acc = fmaf(yf, wf, acc);
            }
            out[(size_t)row * d + i] = hbo_f32_to_bf16(acc);
        }
}

/* -------------------------------------------------- rows around the products */

/* The sum a 256-thread group makes of one f32 per thread (msl/mod.rs:716-756): simd_sum per simdgroup (taken as
 * the xor butterfly 16,8,4,2,1, as everywhere in this file), thread 0 folds the 8 partials in order. */
static float group_sum256(const float* lane_vals) {
    float acc = butterfly_sum32(lane_vals);
    for (int g = 1; g < 8; ++g) acc = acc + butterfly_sum32(lane_vals + 32 * g);
    return acc;
}

void hbo_rmsnorm_rows(const uint16_t* x, const uint16_t* w, uint16_t* y, int rows, int d, float eps, int plus_one) {
    const float inv_d = 1.0f / (float)d;
#pragma omp parallel for schedule(static)
    for (int r = 0; r < rows; ++r) {
        const uint16_t* xr = x + (size_t)r * d;
        float lanes[256];
        for (int l = 0; l < 256; ++l) {
            float a = 0.0f;
            for (int i = l; i < d; i += 256) {
                float v = hbo_bf16_to_f32(xr[i]);
                a = fmaf(v, v, a);
            }
            lanes[l] = a;
        }
        float ss = group_sum256(lanes);
        float mm = ss * inv_d;
        mm = mm + eps;
        float inv = 1.0f / sqrtf(mm);
        for (int i = 0; i < d; ++i) {
            float wf = hbo_bf16_to_f32(w[i]);
            if (plus_one) wf = wf + 1.0f;
            float n = hbo_bf16_to_f32(xr[i]) * inv;
            y[(size_t)r * d + i] = hbo_f32_to_bf16(n * wf);
        }
    }
}

void hbo_argmax_rows(const uint16_t* logits, uint32_t* idx, int rows, int n) {
#pragma omp parallel for schedule(static)
    for (int r = 0; r < rows; ++r) {
        float best = -INFINITY;
        uint32_t best_i = 0xffffffffu;
        for (int i = 0; i < n; ++i) {
            float v = hbo_bf16_to_f32(logits[(size_t)r * n + i]);
            if (v > best) { best = v; best_i = (uint32_t)i; }
        }
        idx[r] = best_i;
    }
}

void hbo_moe_out(const uint16_t* xn, const uint16_t* gate, const uint16_t* experts, const uint16_t* shared, uint16_t* x, int rows, int d) {
#pragma omp parallel for schedule(static)
    for (int r = 0; r < rows; ++r) {
        const size_t base = (size_t)r * d;
        float lanes[256];
        for (int l = 0; l < 256; ++l) {
            float a = 0.0f;
            for (int i = l; i < d; i += 256) a = fmaf(hbo_bf16_to_f32(xn[base + i]), hbo_bf16_to_f32(gate[i]), a);
            lanes[l] = a;
        }
        float logit = hbo_round_bf16(group_sum256(lanes));
        float g = hbo_round_bf16(hbo_sigmoid(logit));
        for (int i = 0; i < d; ++i) {
            float s = hbo_round_bf16(g * hbo_bf16_to_f32(shared[base + i]));
            float o = hbo_round_bf16(hbo_bf16_to_f32(experts[base + i]) + s);
            x[base + i] = hbo_f32_to_bf16(hbo_bf16_to_f32(x[base + i]) + o);
        }
    }
}

/* ------------------------------------------------------------- Q4_0 weights */

static inline float f16_bits_to_f32(uint16_t h) {
    _Float16 v;
    memcpy(&v, &h, 2);
    return (float)v;
}
static inline uint16_t f32_to_f16_bits(float f) {
    _Float16 v = (_Float16)f; /* round to nearest even */
    uint16_t h;
    memcpy(&h, &v, 2);
    return h;
}

void hbo_q4_quantize(const uint16_t* w, int n, int k, uint8_t* data, uint16_t* scales) {
    static const int cands[15] = {-8, 7, -7, 6, -6, 5, -5, 4, -4, 3, -3, 2, -2, 1, -1};
    const int nblk = k / 32;
#pragma omp parallel for schedule(static)
    for (long blk = 0; blk < (long)n * nblk; ++blk) {
        float v[32];
        float m = 0.0f;
        for (int i = 0; i < 32; ++i) {
            v[i] = hbo_bf16_to_f32(w[(size_t)blk * 32 + i]);
            if (fabsf(v[i]) > fabsf(m)) m = v[i];
        }
        uint8_t q[32], best_q[32];
        double best_e = INFINITY;
        uint16_t best_d = 0;
        if (m != 0.0f) {
            for (int ci = 0; ci < 15; ++ci) {
                uint16_t dh = f32_to_f16_bits(m / (float)cands[ci]);
                float dq = f16_bits_to_f32(dh);
                if (dq == 0.0f || !isfinite(dq)) continue;
                float inv = 1.0f / dq;
                double e = 0.0;
                for (int i = 0; i < 32; ++i) {
                    float qi = roundf(v[i] * inv); /* half away from zero, as f32::round */
                    qi = qi < -8.0f ? -8.0f : qi > 7.0f ? 7.0f : qi;
                    q[i] = (uint8_t)((int)qi + 8);
                    double r = (double)(v[i] - dq * qi);
                    e += r * r;
                }
                if (e < best_e) {
                    best_e = e;
                    best_d = dh;
                    memcpy(best_q, q, 32);
                }
            }
        } else {
            best_e = 0.0;
            memset(best_q, 8, 32);
        }
        if (!isfinite(best_e)) memset(best_q, 8, 32); /* every candidate scale rounds to 0 in f16: zeros */
        for (int i = 0; i < 4; ++i)
            for (int b = 0; b < 4; ++b)
                data[(size_t)blk * 16 + 4 * i + b] = (uint8_t)(((best_q[8 * i + b] ^ 8) & 15) | (((best_q[8 * i + 4 + b] ^ 8) & 15) << 4));
        scales[blk] = best_d;
    }
}

/* weight e of a block: the nibble, two's complement */
static inline float q4_weight(const uint8_t* blk, int e) {
    int i = e / 8, j = e % 8;
    uint8_t byte = blk[4 * i + (j % 4)];
    uint8_t nib = j < 4 ? (byte & 15) : (byte >> 4);
    return (float)(nib ^ 8) - 8.0f;
}

void hbo_q4_dequant(const uint8_t* data, const uint16_t* scales, int n, int k, uint16_t* out) {
    const long nblk = (long)n * (k / 32);
#pragma omp parallel for schedule(static)
    for (long blk = 0; blk < nblk; ++blk) {
        float d = f16_bits_to_f32(scales[blk]);
        for (int e = 0; e < 32; ++e) out[(size_t)blk * 32 + e] = hbo_f32_to_bf16(d * q4_weight(data + (size_t)blk * 16, e));
    }
}

void hbo_matvec_q4(const uint8_t* data, const uint16_t* scales, const uint16_t* x, void* y, int n, int k, int out) {
    const int nblk = k / 32;
#pragma omp parallel for schedule(static)
    for (int row = 0; row < n; ++row) {
        float lane[32];
        for (int l = 0; l < 32; ++l) {
            float acc = 0.0f;
            for (int b = l; b < nblk; b += 32) {
                const uint8_t* blk = data + ((size_t)row * nblk + b) * 16;
                float part = 0.0f;
                for (int i = 0; i < 4; ++i)
                    for (int byte = 0; byte < 4; ++byte) {
                        int e0 = 8 * i + byte, e1 = 8 * i + 4 + byte;
                        part = fmaf(q4_weight(blk, e0), hbo_bf16_to_f32(x[b * 32 + e0]), part);
                        part = fmaf(q4_weight(blk, e1), hbo_bf16_to_f32(x[b * 32 + e1]), part);
                    }
                acc = fmaf(f16_bits_to_f32(scales[(size_t)row * nblk + b]), part, acc);
            }
            lane[l] = acc;
        }
        store_out(y, (size_t)row, butterfly_sum32(lane), out);
    }
}

/* src/metal/kernels.rs:472-500, 896-928 (matvec_q4_split): the blocks of a row shared by `split` simdgroups (block b to
 * simdgroup (b / 32) % split, lane b % 32), every simdgroup's lanes summed by the butterfly, the partials added in
 * simdgroup order. split = 1 is hbo_matvec_q4. */
void hbo_matvec_q4_split(const uint8_t* data, const uint16_t* scales, const uint16_t* x, void* y, int n, int k, int out, int split) {
    const int nblk = k / 32;
#pragma omp parallel for schedule(static)
    for (int row = 0; row < n; ++row) {
        float total = 0.0f;
        for (int sub = 0; sub < split; ++sub) {
            float lane[32];
            for (int l = 0; l < 32; ++l) {
                float acc = 0.0f;
                for (int b = l + 32 * sub; b < nblk; b += 32 * split) {
                    const uint8_t* blk = data + ((size_t)row * nblk + b) * 16;
                    float part = 0.0f;
                    for (int i = 0; i < 4; ++i)
                        for (int byte = 0; byte < 4; ++byte) {
                            int e0 = 8 * i + byte, e1 = 8 * i + 4 + byte;
                            part = fmaf(q4_weight(blk, e0), hbo_bf16_to_f32(x[b * 32 + e0]), part);
                            part = fmaf(q4_weight(blk, e1), hbo_bf16_to_f32(x[b * 32 + e1]), part);
                        }
                    acc = fmaf(f16_bits_to_f32(scales[(size_t)row * nblk + b]), part, acc);
                }
                lane[l] = acc;
            }
            const float s = butterfly_sum32(lane);
            total = sub == 0 ? s : total + s;
        }
        store_out(y, (size_t)row, total, out);
    }
}

/* src/metal/kernels.rs:983-1071 (matmul_q4): the m rows of a prefill block, each summed as matvec_q4 sums its one. */
void hbo_matmul_q4(const uint8_t* data, const uint16_t* scales, const uint16_t* x, uint16_t* y, int n, int k, int m, int ldx, int ldy) {
    uint16_t* row = (uint16_t*)malloc((size_t)n * sizeof(uint16_t));
    for (int r = 0; r < m; ++r) {
        hbo_matvec_q4(data, scales, x + (size_t)r * ldx, row, n, k, HBO_OUT_BF16);
        memcpy(y + (size_t)r * ldy, row, (size_t)n * sizeof(uint16_t));
    }
    free(row);
}

void hbo_matvec_q4s(const uint8_t* data, const uint16_t* scales, const uint16_t* x, void* y, int n, int k, int out) {
    const int nblk = k / 32;
#pragma omp parallel for schedule(static)
    for (int row = 0; row < n; ++row) {
        float lane[32];
        for (int l = 0; l < 32; ++l) {
            float acc = 0.0f;
            for (int b = l; b < nblk; b += 32) {
                float xs[32], scaled[32];
                for (int e = 0; e < 32; ++e) xs[e] = hbo_bf16_to_f32(x[b * 32 + e]);
                float sx = xs[0];
                for (int e = 1; e < 32; ++e) sx = sx + xs[e];
                for (int e = 0; e < 32; ++e) {
                    int jj = e % 8, shift = jj < 4 ? 8 * jj : 8 * (jj - 4) + 4;
                    scaled[e] = xs[e] * ldexpf(1.0f, -shift);
                }
                const uint8_t* blk = data + ((size_t)row * nblk + b) * 16;
                float part = 0.0f;
                for (int i = 0; i < 4; ++i) {
                    uint32_t ww;
                    memcpy(&ww, blk + 4 * i, 4);
                    ww ^= 0x88888888u;
                    for (int jj = 0; jj < 8; ++jj) {
                        int shift = jj < 4 ? 8 * jj : 8 * (jj - 4) + 4;
                        uint32_t v = ww & (15u << shift);
                        part = fmaf((float)v, scaled[8 * i + jj], part);
                    }
                }
                part = fmaf(-8.0f, sx, part);
                acc = fmaf(f16_bits_to_f32(scales[(size_t)row * nblk + b]), part, acc);
            }
            lane[l] = acc;
        }
        store_out(y, (size_t)row, butterfly_sum32(lane), out);
    }
}

/* -------------------------------------------------------------------- check */

int hbo_check_1_64(const void* ref, const void* got, size_t count, int f32_out, float* err_out, float* scale_out) {
    float scale = 0.0f, err = 0.0f;
    int nan_seen = 0;
    for (size_t i = 0; i < count; ++i) {
        float r = f32_out ? ((const float*)ref)[i] : hbo_bf16_to_f32(((const uint16_t*)ref)[i]);
        float g = f32_out ? ((const float*)got)[i] : hbo_bf16_to_f32(((const uint16_t*)got)[i]);
        /* Rust's f32::max ignores a NaN operand; a NaN difference must still fail. */
        float a = fabsf(r);
        if (a > scale) scale = a;
        float d = fabsf(r - g);
        if (d != d) nan_seen = 1;
        else if (d > err) err = d;
    }
    if (scale < 1e-6f) scale = 1e-6f;
    if (err_out) *err_out = nan_seen ? NAN : err;
    if (scale_out) *scale_out = scale;
    return (!nan_seen && err <= scale / 64.0f) ? 1 : 0;
}

/* ------------------------------------------------------------------- inputs */

static inline uint64_t splitmix64(uint64_t z) {
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

void hbo_fill_normal(uint16_t* dst, size_t count, uint64_t seed, uint64_t tensor_id, double sigma) {
#pragma omp parallel for schedule(static)
    for (size_t i = 0; i < count; ++i) {
        uint64_t base = seed ^ (tensor_id << 40) ^ (uint64_t)i;
        uint64_t sum = 0;
        for (uint64_t j = 0; j < 3; ++j) {
            uint64_t u = splitmix64(base * 3u + j);
            sum += (u & 0xFFFF) + ((u >> 16) & 0xFFFF) + ((u >> 32) & 0xFFFF) + ((u >> 48) & 0xFFFF);
        }
        double z = ((double)sum - 393210.0) / 65536.0; /* 12 * 32767.5 */
        dst[i] = hbo_f32_to_bf16((float)(z * sigma));
    }
}

uint32_t hbo_fill_xorshift16(uint16_t* dst, size_t count, uint32_t seed) {
    for (size_t i = 0; i < count; ++i) {
        seed ^= seed << 13;
        seed ^= seed >> 17;
        seed ^= seed << 5;
        dst[i] = hbo_f32_to_bf16((float)(seed >> 8) / (float)(1u << 23) - 1.0f);
    }
    return seed;
}

void hbo_fill_random16(uint16_t* dst, size_t count, uint64_t seed) {
    uint64_t s = seed;
    for (size_t i = 0; i < count; ++i) {
        s = s * 6364136223846793005ull + 1442695040888963407ull;
        uint32_t r = (uint32_t)(s >> 32);
        uint16_t sign = (uint16_t)(r >> 31);
        uint32_t e = 9 + ((r >> 24) & 7u) % 6u;
        dst[i] = (uint16_t)((sign << 15) | ((uint16_t)(e + 112) << 7) | (uint16_t)(r & 0x7f));
    }
}

/* --------------------------------------------------------------- comparison */

static inline int32_t bf16_ord(uint16_t b) {
    int32_t mag = b & 0x7FFF;
    return (b & 0x8000) ? -mag : mag;
}

void hbo_compare_bf16(const uint16_t* ref, const uint16_t* got, size_t count, hbo_cmp* out) {
    hbo_cmp c = {count, 0, 0, 0, 0.0f, 0.0f};
    for (size_t i = 0; i < count; ++i) {
        int32_t d = bf16_ord(ref[i]) - bf16_ord(got[i]);
        uint32_t ud = (uint32_t)(d < 0 ? -d : d);
        if (ref[i] != got[i]) c.mismatched++;
        if (ud > 1) c.over_1ulp++;
        if (ud > c.max_ulp) c.max_ulp = ud;
        float r = hbo_bf16_to_f32(ref[i]), g = hbo_bf16_to_f32(got[i]);
        float e = fabsf(r - g);
        if (e != e) { c.over_1ulp++; c.max_abs_err = NAN; }
        else if (!(c.max_abs_err != c.max_abs_err) && e > c.max_abs_err) c.max_abs_err = e;
        if (fabsf(r) > c.max_abs_ref) c.max_abs_ref = fabsf(r);
    }
    *out = c;
}

int hbo_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
