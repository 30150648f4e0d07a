// The load-time selection loop: candidates, the 1/64 correctness check, interleaved timing,
// cached picks. Restates QwenEngine::gemm, gate_up_pipes, expert_pipes, mv_full,
// check_candidates, pick_flagged, time_ops, autotune_inputs of the reference
// (src/metal/qwen.rs:2200-2315, :2148-2191, :2326-2386, :1311-1505, :2497-2543, :2547-2573,
// :2593, :2605-2626) on top of the device boundary (hb_gemm_get, hb_launch, hb_time, ...).
// The "[autotune] ..." lines keep the reference's formats: they are the observable
// behaviour of the loop.
#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstring>
#include <deque>
#include <functional>
#include <memory>

#include "../csrc/hb_internal.hpp"
#include "tune.hpp"

namespace {

// A kernel that runs another one and then scales its bf16 / f32 output by 1.25: the
// deliberately wrong candidate of hb_selector_inject_wrong.
__global__ void scale_output_kernel(void* y, size_t count, int f32_out) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += (size_t)gridDim.x * blockDim.x) {
        if (f32_out) {
            static_cast<float*>(y)[i] *= 1.25f;
        } else {
            uint16_t* p = static_cast<uint16_t*>(y) + i;
            float v = __uint_as_float((uint32_t)*p << 16) * 1.25f;
            *p = (uint16_t)(__float_as_uint(v) >> 16);
        }
    }
}

struct WrongKernel : hb_kernel {
    hb_kernel* inner = nullptr;
    uint32_t n_out = 0;
    bool f32 = false;
    int launch(hb_ctx* ctx, const hb_range* a, int na, uint32_t m) override {
        int r = inner->launch(ctx, a, na, m);
        if (r != HB_OK) return r;
        scale_output_kernel<<<ctx->sm_count * 4, 256, 0, ctx->stream>>>(a[2].ptr, (size_t)m * n_out, f32 ? 1 : 0);
        HB_CUDA(ctx, cudaGetLastError());
        ctx->launches++;
        return HB_OK;
    }
};

const char* out_debug(uint32_t out) {  // Rust's {:?} of enum Out
    switch (out) {
        case HB_OUT_BF16: return "Bf16";
        case HB_OUT_F32: return "F32";
        case HB_OUT_RESIDUAL: return "Residual";
        case HB_OUT_SWIGLU: return "Swiglu";
    }
    return "?";
}

// Rust's {:.3e}: mantissa with three decimals, exponent without padding or plus sign.
std::string fmt_e3(double v) {
    if (std::isnan(v)) return "NaN";
    if (std::isinf(v)) return v > 0 ? "inf" : "-inf";
    if (v == 0.0) return "0.000e0";
    int e = (int)std::floor(std::log10(std::fabs(v)));
    double mant = v / std::pow(10.0, e);
    char buf[64];
    snprintf(buf, sizeof buf, "%.3f", mant);
    if (std::fabs(atof(buf)) >= 10.0) {  // 9.9996 rounds up to 10.000
        e += 1;
        mant = v / std::pow(10.0, e);
        snprintf(buf, sizeof buf, "%.3f", mant);
    }
    return std::string(buf) + "e" + std::to_string(e);
}

struct Cand {
    std::string name;
    // Launch sequence; every op's m is replaced by the row count under test.
    std::vector<const hb_kernel*> kernels;
    std::vector<std::vector<hb_range>> ranges;
    std::vector<int> row_scale;  // m multiplier per op (top_k for ops over sorted expert rows), 0 = fixed m
    std::vector<uint32_t> fixed_m;
};

}  // namespace

struct hb_selector {
    hb_ctx* ctx = nullptr;
    hb_tune tune;
    std::string log;
    std::map<std::string, const hb_kernel*> gemm_pick;
    std::map<std::string, std::vector<const hb_kernel*>> gate_up_pick;
    std::map<std::string, const hb_kernel*> mv_pick;
    bool inject_wrong = false;
    double autotune_seconds = 0.0;
    bool timed_before = false;
    std::chrono::steady_clock::time_point last_timed;  // when a timed comparison last ended (heat, qwen.rs:2577)
};

namespace {

void say(hb_selector* s, const std::string& line) {
    fprintf(stderr, "%s\n", line.c_str());
    s->log += line;
    s->log += '\n';
}

std::vector<hb_op> ops_of(const Cand& c, uint32_t rows) {
    std::vector<hb_op> ops(c.kernels.size());
    for (size_t i = 0; i < ops.size(); ++i) {
        ops[i].kernel = c.kernels[i];
        ops[i].args = c.ranges[i].data();
        ops[i].nargs = (int)c.ranges[i].size();
        ops[i].m = c.row_scale[i] ? rows * (uint32_t)c.row_scale[i] : c.fixed_m[i];
    }
    return ops;
}

int time_ops(hb_selector* s, const Cand& c, uint32_t rows, int reps, double* sec) {
    auto ops = ops_of(c, rows);
    return hb_time(s->ctx, ops.data(), (int)ops.size(), reps, sec);
}

void add_op(Cand& c, const hb_kernel* k, std::vector<hb_range> r, int row_scale = 1, uint32_t fixed_m = 0) {
    c.kernels.push_back(k);
    c.ranges.push_back(std::move(r));
    c.row_scale.push_back(row_scale);
    c.fixed_m.push_back(fixed_m);
}

float widen(const void* p, size_t i, bool f32_out) {
    if (f32_out) return static_cast<const float*>(p)[i];
    uint32_t u = (uint32_t)static_cast<const uint16_t*>(p)[i] << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

// The rule of check_candidates (qwen.rs:2519-2531): scale = max(max|ref|, 1e-6), err = max|ref - got|,
// eligible iff err <= scale/64. Rust's f32::max drops a NaN operand, so a NaN difference would vanish
// from the fold; it is tracked apart and fails the candidate, which is what the reference's negated
// comparison is written for.
bool rule_1_64(const void* ref, const void* got, size_t count, bool f32_out, float* err_out, float* scale_out) {
    float scale = 0.f, err = 0.f;
    bool nan_seen = false;
    for (size_t i = 0; i < count; ++i) {
        const float r = widen(ref, i, f32_out), g = widen(got, i, f32_out);
        const float a = std::fabs(r);
        if (a > scale) scale = a;
        const float d = std::fabs(r - g);
        if (d != d) nan_seen = true;
        else if (d > err) err = d;
    }
    scale = std::max(scale, 1e-6f);
    if (err_out) *err_out = nan_seen ? NAN : err;
    if (scale_out) *scale_out = scale;
    return !nan_seen && err <= scale / 64.0f;
}

// check_candidates, qwen.rs:2497-2543. `out` is the output range all candidates write, `row_bytes` the bytes
// of one block row in it, `rows_scale` the output rows per block row (top_k for expert outputs).
int check_candidates(hb_selector* s, const std::string& what, const std::vector<Cand>& cands, std::vector<char>& eligible, hb_range out, size_t row_bytes,
                     bool f32_out, uint32_t m) {
    hb_ctx* ctx = s->ctx;
    const size_t full = std::min(out.size, (size_t)m * row_bytes);
    std::vector<uint8_t> before(full), ref(full), got(full);
    int r = hb_download(ctx, before.data(), out.ptr, full);
    if (r != HB_OK) return r;
    std::vector<std::string> wrong;
    const uint32_t partial = std::max<int64_t>((int64_t)m - m / 3 - 3, 1);
    for (uint32_t rows : {m, partial}) {
        const size_t used = std::min(full, (size_t)rows * row_bytes);
        double t;
        if ((r = hb_memset(ctx, out.ptr, 0, full)) != HB_OK) return r;
        if ((r = time_ops(s, cands[0], rows, 1, &t)) != HB_OK) return r;
        if ((r = hb_download(ctx, ref.data(), out.ptr, used)) != HB_OK) return r;
        for (size_t i = 1; i < cands.size(); ++i) {
            if (!eligible[i]) continue;
            if ((r = hb_memset(ctx, out.ptr, 0, full)) != HB_OK) return r;
            if ((r = time_ops(s, cands[i], rows, 1, &t)) != HB_OK) return r;
            if ((r = hb_download(ctx, got.data(), out.ptr, used)) != HB_OK) return r;
            float err, scale;
            if (!rule_1_64(ref.data(), got.data(), used / (f32_out ? 4 : 2), f32_out, &err, &scale)) {
                eligible[i] = 0;
                wrong.push_back(cands[i].name + " (" + std::to_string(rows) + " rows: max err " + fmt_e3(err) + " of " + fmt_e3(scale) + ")");
            }
        }
    }
    if ((r = hb_upload(ctx, out.ptr, before.data(), full)) != HB_OK) return r;
    if (!wrong.empty()) {
        std::string line = "[autotune] " + what + ": wrong against " + cands[0].name + ", never picked: ";
        for (size_t i = 0; i < wrong.size(); ++i) line += (i ? ", " : "") + wrong[i];
        say(s, line);
    }
    return HB_OK;
}

// heat, qwen.rs:2577-2590 (auto.heat, in ms): the GPU brought to its sustained regime before a timed comparison when it
// has been idle for more than 200 ms: the first candidate run back to back, about 50 ms a call, until auto.heat ms of
// GPU time. On a power-capped part the first candidate of a cold chip is otherwise timed at a higher clock than the rest.
int heat(hb_selector* s, const Cand& c, uint32_t m) {
    const double want = s->tune.get("auto.heat") * 1e-3;
    const auto now = std::chrono::steady_clock::now();
    if (want <= 0.0 || (s->timed_before && std::chrono::duration<double>(now - s->last_timed).count() < 0.2)) return HB_OK;
    double one = 0.0;
    int r = time_ops(s, c, m, 1, &one);
    if (r != HB_OK) return r;
    const int reps = (int)std::min(256.0, std::max(1.0, std::ceil(0.05 / std::max(one, 1e-6))));
    for (double t = 0.0; t < want;) {
        double dt;
        if ((r = time_ops(s, c, m, reps, &dt)) != HB_OK) return r;
        t += dt;
    }
    s->timed_before = true;
    s->last_timed = std::chrono::steady_clock::now();
    return HB_OK;
}

// pick_flagged, qwen.rs:2547-2573: warm the first candidate, reps sized to about 2 ms, five rounds with the
// candidates in turn, medians, the fastest eligible one; the others are timed and starred.
int pick_flagged(hb_selector* s, const std::string& what, const std::vector<Cand>& cands, const std::vector<char>& eligible, uint32_t m, size_t* best_out,
                 double* median_out) {
    int r;
    double one = 0.0;
    if ((r = heat(s, cands[0], m)) != HB_OK) return r;
    if ((r = time_ops(s, cands[0], m, 1, &one)) != HB_OK) return r;
    if ((r = time_ops(s, cands[0], m, 1, &one)) != HB_OK) return r;
    const int reps = (int)std::min(64.0, std::max(1.0, std::ceil(2e-3 / std::max(one, 1e-6))));
    std::vector<std::vector<double>> times(cands.size());
    for (int round = 0; round < 5; ++round)
        for (size_t i = 0; i < cands.size(); ++i) {
            double t;
            if ((r = time_ops(s, cands[i], m, reps, &t)) != HB_OK) return r;
            times[i].push_back(t / reps);
        }
    std::vector<double> med(cands.size());
    for (size_t i = 0; i < cands.size(); ++i) {
        std::sort(times[i].begin(), times[i].end());
        med[i] = times[i][times[i].size() / 2];
    }
    size_t best = cands.size();
    for (size_t i = 0; i < cands.size(); ++i)
        if (eligible[i] && (best == cands.size() || med[i] < med[best])) best = i;
    if (best == cands.size()) return hb::fail(s->ctx, HB_BACKEND, what + ": no eligible candidate");
    std::string line = "[autotune] " + what + ": ";
    for (size_t i = 0; i < cands.size(); ++i) {
        char buf[64];
        snprintf(buf, sizeof buf, " %.3f ms", med[i] * 1e3);
        line += (i ? ", " : "") + cands[i].name + (eligible[i] ? "" : "*") + buf;
    }
    line += " -> " + cands[best].name;
    say(s, line);
    for (auto& v : times)
        for (double t : v) s->autotune_seconds += t * reps;
    *best_out = best;
    if (median_out) *median_out = med[best];
    s->timed_before = true;
    s->last_timed = std::chrono::steady_clock::now();
    return HB_OK;
}

// The K splits worth timing for the CTA-pair form at m rows: those that bring the work items (tiles x slices) close to
// one, two, three or four whole waves of the SM pairs. None when the tiles alone fill a wave, or the block is long.
std::vector<uint32_t> pair_splits(hb_ctx* ctx, uint32_t m, uint32_t k, uint32_t n_out, uint32_t cols_per_tile) {
    std::vector<uint32_t> v;
    if (m > 1024) return v;
    const uint32_t tiles = ((m + 255) / 256) * ((n_out + cols_per_tile - 1) / cols_per_tile), pairs = (uint32_t)ctx->sm_count / 2, k_blocks = (k + 63) / 64;
    for (uint32_t waves = 1; waves <= 4; ++waves) {
        const uint32_t sp = pairs * waves / std::max(tiles, 1u);
        if (sp >= 2 && sp <= 16 && sp <= k_blocks && std::find(v.begin(), v.end(), sp) == v.end()) v.push_back(sp);
    }
    return v;
}

// gemm.tn names the columns of the reference's tile (16/32/64); the B200 tile has four times as many.
uint32_t tile_n_of_tn(uint32_t tn) { return tn >= 64 ? 256 : tn == 32 ? 128 : 64; }

int get_dense(hb_selector* s, uint32_t k, uint32_t n, uint32_t out, uint32_t tile_n, uint32_t stages, uint32_t m_first, uint32_t pair, uint32_t rows_max,
              hb_kernel** kern, uint32_t stream_k = 0, uint32_t split_k = 0) {
    hb_gemm_desc d{};
    d.stream_k = stream_k;
    d.split_k = split_k;
    d.k = k;
    d.n = n;
    d.out = out;
    d.rows_mode = HB_ROWS_DENSE;
    d.tile_n = tile_n;
    d.stages = stages;
    d.cta_pair = pair;
    d.m_first = m_first;
    d.rows_max = rows_max;
    return hb_gemm_get(s->ctx, &d, kern);
}

struct DenseForm {
    const char* name;
    uint32_t tile_n, pair, flip, stream_k;
};
// The first one is the production reference every other candidate is checked against (the role of
// "mma" in the reference's list, qwen.rs:2248).
const DenseForm kDenseForms[] = {
    {"t128x256", 256, 0, 0, 0}, {"t128x128", 128, 0, 0, 0}, {"t128x64", 64, 0, 0, 0},   {"t128x256n", 256, 0, 1, 0}, {"t128x128n", 128, 0, 1, 0},
    {"sk128x256", 256, 0, 0, 1}, {"sk128x128", 128, 0, 0, 1}, {"sk128x64", 64, 0, 0, 1}, {"pair256x256", 256, 1, 0, 0},
    {"pair256x192", 192, 1, 0, 0},
};

}  // namespace

extern "C" {

int hb_selector_new(hb_ctx* ctx, const hb_tune* tune, hb_selector** out) {
    if (!ctx || !tune || !out) return hb::fail(ctx, HB_INVALID, "hb_selector_new: bad argument");
    try {
        auto* s = new hb_selector();
        s->ctx = ctx;
        s->tune = *tune;
        *out = s;
        return HB_OK;
    } catch (...) {
        return hb::fail(ctx, HB_OOM, "hb_selector_new: out of memory");
    }
}

void hb_selector_free(hb_selector* s) { delete s; }

const char* hb_selector_log(const hb_selector* s) { return s ? s->log.c_str() : ""; }

int hb_selector_buckets(const hb_selector* s, uint32_t* buckets, int cap) {
    if (!s) return 0;
    const uint32_t block = s->tune.get("prefill.block");
    std::vector<uint32_t> b;
    if (s->tune.gemm_timed())
        for (uint32_t r = 64; r < block; r += 64) b.push_back(r);  // qwen.rs:1049-1052
    b.push_back(block);
    int n = 0;
    for (uint32_t v : b)
        if (buckets && n < cap) buckets[n++] = v;
    return (int)b.size();
}

int hb_selector_inject_wrong(hb_selector* s, int enable) {
    if (!s) return HB_INVALID;
    s->inject_wrong = enable != 0;
    return HB_OK;
}

int hb_fill_random16(hb_ctx* ctx, hb_range dst, uint32_t seed) {
    if (!ctx || !dst.ptr) return hb::fail(ctx, HB_INVALID, "hb_fill_random16: bad argument");
    try {
        std::vector<uint16_t> v(dst.size / 2);
        for (auto& h : v) {
            seed ^= seed << 13;
            seed ^= seed >> 17;
            seed ^= seed << 5;
            const float f = (float)(seed >> 8) / (float)(1u << 23) - 1.0f;
            uint32_t bits;
            memcpy(&bits, &f, 4);
            h = (uint16_t)((bits + 0x7fffu + ((bits >> 16) & 1u)) >> 16);
        }
        return hb_upload(ctx, dst.ptr, v.data(), v.size() * 2);
    } catch (...) {
        return hb::fail(ctx, HB_OOM, "hb_fill_random16: out of host memory");
    }
}

int hb_check_rule(const void* reference, const void* got, size_t count, int f32_out, int* eligible, float* err, float* scale) {
    if (!reference || !got || !eligible) return HB_INVALID;
    *eligible = rule_1_64(reference, got, count, f32_out != 0, err, scale) ? 1 : 0;
    return HB_OK;
}

int hb_select_gemm(hb_selector* s, uint32_t k, uint32_t n, uint32_t out, hb_range w, hb_range x, hb_range y, uint32_t m, const hb_kernel** picked) {
    if (!s || !picked) return HB_INVALID;
    hb_ctx* ctx = s->ctx;
    try {
        const hb_tune& t = s->tune;
        const uint32_t mf = t.get("gemm.mfirst") != 0 ? 1u : 0u;
        const uint32_t rows_max = std::max(m, t.get("prefill.block"));
        hb_kernel* kern = nullptr;
        int r;
        if (!t.gemm_timed()) {
            // The tune keys name the kernel (qwen.rs:2231-2236). On this hardware every form is the tensor-core
            // kernel: gemm.mma 0/1 -> the 128x256 tile with gemm.mform fewer pipeline stages than fit;
            // 2 -> the tile gemm.tn names; 3 -> the CTA-pair form.
            const uint32_t mma = t.get("gemm.mma");
            if (mma == 2) r = get_dense(s, k, n, out, tile_n_of_tn(t.get("gemm.tn")), 0, mf, 0, rows_max, &kern);
            else if (mma == 3) r = get_dense(s, k, n, out, 256, 0, mf, 1, rows_max, &kern);
            else {
                const uint32_t form = t.get("gemm.mform");
                r = get_dense(s, k, n, out, 256, form ? std::max<int>(2, 4 - (int)form) : 0, mf, 0, rows_max, &kern);
            }
            if (r != HB_OK) return r;
            *picked = kern;
            return HB_OK;
        }
        const std::string key = std::to_string(k) + "x" + std::to_string(n) + " " + out_debug(out) + ", " + std::to_string(m) + " rows";
        auto it = s->gemm_pick.find(key);
        if (it != s->gemm_pick.end() && !s->inject_wrong) {
            *picked = it->second;
            return HB_OK;
        }
        const std::string what = "gemm " + key;
        std::vector<Cand> cands;
        std::vector<char> eligible;
        for (const auto& f : kDenseForms) {
            r = get_dense(s, k, n, out, f.tile_n, 0, f.flip ? 1u - mf : mf, f.pair, rows_max, &kern, f.stream_k);
            if (r != HB_OK) {
                if (cands.empty()) return r;  // the production kernel itself does not build: an error, not a skipped candidate
                say(s, "[autotune] gemm " + key + ": " + f.name + " not built (" + hb_last_error(ctx) + ")");
                continue;
            }
            Cand c;
            c.name = f.name;
            add_op(c, kern, {w, x, y});
            cands.push_back(std::move(c));
            eligible.push_back(1);
        }
        // short blocks have too few 256 x 256 tiles for the SM pairs: the pair form with K cut into slices
        for (uint32_t sp : pair_splits(ctx, m, k, out == HB_OUT_SWIGLU ? n / 2 : n, out == HB_OUT_SWIGLU ? 128 : 256)) {
            if (get_dense(s, k, n, out, 256, 0, mf, 1, std::min(rows_max, 1024u), &kern, 0, sp) != HB_OK) continue;
            Cand c;
            c.name = "pair256x256k" + std::to_string(sp);
            add_op(c, kern, {w, x, y});
            cands.push_back(std::move(c));
            eligible.push_back(1);
        }
        // blocks of at most 64 rows are weight streams, not GEMMs (64 FLOP per weight byte): the decode kernel that
        // feeds the weights to the tensor cores as the wide operand takes the same bindings
        if (m <= 64) {
            struct SkForm { const char* name; uint32_t tc, kps; };
            // (K blocks per stage: four while the activation tile is small, two when it is 64 rows: at least three stages must fit)
            for (const SkForm& f : {SkForm{"stream", 1, m <= 16 ? 4u : 2u}, SkForm{"streamb", 2, m <= 16 ? 2u : 1u}, SkForm{"streamf", 3, m <= 16 ? 4u : 2u}}) {
                hb_matvec_desc d{};
                d.k = k;
                d.n = n;
                d.out = out;
                d.rows_max = m;
                d.tensor_core = f.tc;
                d.split = f.kps;
                if (hb_matvec_get(ctx, &d, &kern) != HB_OK) continue;
                Cand c;
                c.name = f.name;
                add_op(c, kern, {w, x, y});
                cands.push_back(std::move(c));
                eligible.push_back(1);
            }
        }
        if (s->inject_wrong) {
            auto wrong = std::make_unique<WrongKernel>();
            wrong->inner = const_cast<hb_kernel*>(cands[0].kernels[0]);
            wrong->n_out = out == HB_OUT_SWIGLU ? n / 2 : n;
            wrong->f32 = out == HB_OUT_F32;
            wrong->name = "wrong:" + wrong->inner->name;
            hb_kernel* wk = hb::intern(ctx, std::move(wrong));  // owned by the context like every kernel
            Cand c;
            c.name = "wrong";
            add_op(c, wk, {w, x, y});
            cands.push_back(std::move(c));
            eligible.push_back(1);
        }
        const uint32_t n_out = out == HB_OUT_SWIGLU ? n / 2 : n;
        const bool f32_out = out == HB_OUT_F32;
        if ((r = check_candidates(s, what, cands, eligible, y, (size_t)n_out * (f32_out ? 4 : 2), f32_out, m)) != HB_OK) return r;
        size_t best;
        if ((r = pick_flagged(s, what, cands, eligible, m, &best, nullptr)) != HB_OK) return r;
        s->gemm_pick[key] = cands[best].kernels[0];
        *picked = cands[best].kernels[0];
        return HB_OK;
    } catch (const std::exception& e) {
        return hb::fail(ctx, HB_BACKEND, e.what());
    }
}

int hb_select_gemm_q4(hb_selector* s, uint32_t k, uint32_t n, uint32_t out, hb_range wq, hb_range scales, hb_range w_bf16, hb_range x, hb_range y, uint32_t m,
                      const hb_kernel** kernels_out, int* nkernels) {
    if (!s || !kernels_out || !nkernels) return HB_INVALID;
    hb_ctx* ctx = s->ctx;
    try {
        const hb_tune& t = s->tune;
        const uint32_t mf = t.get("gemm.mfirst") != 0 ? 1u : 0u;
        const uint32_t rows_max = std::max(m, t.get("prefill.block"));
        const bool have_copy = w_bf16.ptr != nullptr;
        int r;
        auto fused = [&](uint32_t tile_n, hb_kernel** kern) { return hb_gemm_q4_get(ctx, k, n, out, tile_n, mf, rows_max, kern); };
        auto apart = [&](std::vector<const hb_kernel*>* ks) -> int {
            hb_kernel* dq = nullptr;
            int rr = hb_dequant_q4_get(ctx, k, n, &dq);
            if (rr != HB_OK) return rr;
            const hb_kernel* g = nullptr;
            // the decoded matrix must be there before bf16 candidates are checked and timed on it
            hb_range a[3] = {wq, scales, w_bf16};
            if ((rr = hb_launch(ctx, dq, a, 3, 1)) != HB_OK) return rr;
            if ((rr = hb_select_gemm(s, k, n, out, w_bf16, x, y, m, &g)) != HB_OK) return rr;
            *ks = {dq, g};
            return HB_OK;
        };
        std::vector<const hb_kernel*> ks;
        if (!t.gemm_timed() || !have_copy) {  // q4.fuse names the form (qwen.rs:2234); without a scratch copy only the fused form exists
            if (t.get("q4.fuse") == 1 || !have_copy) {
                hb_kernel* f = nullptr;
                if ((r = fused(256, &f)) != HB_OK) return r;
                ks = {f};
            } else if ((r = apart(&ks)) != HB_OK) {
                return r;
            }
        } else {
            const std::string key = std::to_string(k) + "x" + std::to_string(n) + " " + out_debug(out) + " q4, " + std::to_string(m) + " rows";
            auto it = s->gate_up_pick.find(key);
            if (it != s->gate_up_pick.end()) {
                ks = it->second;
            } else {
                std::vector<const hb_kernel*> ap;
                if ((r = apart(&ap)) != HB_OK) return r;
                std::vector<Cand> cands;
                Cand c0;
                c0.name = "dequant+gemm";
                add_op(c0, ap[0], {wq, scales, w_bf16}, 0, 1);
                add_op(c0, ap[1], {w_bf16, x, y});
                cands.push_back(std::move(c0));
                for (uint32_t tn : {256u, 128u}) {
                    hb_kernel* f = nullptr;
                    if (fused(tn, &f) != HB_OK) {
                        say(s, "[autotune] gemm " + key + ": fused128x" + std::to_string(tn) + " not built (" + hb_last_error(ctx) + ")");
                        continue;
                    }
                    Cand c;
                    c.name = "fused128x" + std::to_string(tn);
                    add_op(c, f, {wq, x, y, scales});
                    cands.push_back(std::move(c));
                }
                std::vector<char> eligible(cands.size(), 1);
                const uint32_t n_out = out == HB_OUT_SWIGLU ? n / 2 : n;
                const bool f32_out = out == HB_OUT_F32;
                const std::string what = "gemm " + key;
                if ((r = check_candidates(s, what, cands, eligible, y, (size_t)n_out * (f32_out ? 4 : 2), f32_out, m)) != HB_OK) return r;
                size_t best;
                if ((r = pick_flagged(s, what, cands, eligible, m, &best, nullptr)) != HB_OK) return r;
                ks = cands[best].kernels;
                s->gate_up_pick[key] = ks;
            }
        }
        for (size_t i = 0; i < ks.size(); ++i) kernels_out[i] = ks[i];
        *nkernels = (int)ks.size();
        return HB_OK;
    } catch (const std::exception& e) {
        return hb::fail(ctx, HB_BACKEND, e.what());
    }
}

int hb_select_gate_up(hb_selector* s, uint32_t k, uint32_t inter, hb_range w, hb_range x, hb_range gu, hb_range h, uint32_t m, const hb_kernel** kernels_out,
                      int* nkernels) {
    if (!s || !kernels_out || !nkernels) return HB_INVALID;
    hb_ctx* ctx = s->ctx;
    try {
        const hb_tune& t = s->tune;
        const uint32_t fswi = t.get("pf.fswi");
        const uint32_t mf = t.get("gemm.mfirst") != 0 ? 1u : 0u;
        const uint32_t rows_max = std::max(m, t.get("prefill.block"));
        int r;
        auto apart = [&](std::vector<const hb_kernel*>* ks) -> int {
            const hb_kernel* g = nullptr;
            int rr = hb_select_gemm(s, k, 2 * inter, HB_OUT_BF16, w, x, gu, m, &g);
            if (rr != HB_OK) return rr;
            hb_kernel* sw = nullptr;
            if ((rr = hb_swiglu_get(ctx, inter, &sw)) != HB_OK) return rr;
            *ks = {g, sw};
            return HB_OK;
        };
        std::vector<const hb_kernel*> ks;
        // pf.fswi: 0 apart, 1 fused, 2 timed (qwen.rs:233-235,2154-2191); the fused form needs K % 32 == 0.
        const bool can_fuse = k % 32 == 0;
        if (fswi == 0 || !can_fuse) {
            if ((r = apart(&ks)) != HB_OK) return r;
        } else if (fswi == 1 || !t.gemm_timed()) {
            hb_kernel* f = nullptr;
            if ((r = get_dense(s, k, 2 * inter, HB_OUT_SWIGLU, 256, 0, mf, t.get("gemm.mma") == 3 ? 1u : 0u, rows_max, &f)) != HB_OK) return r;
            ks = {f};
        } else {
            const std::string key = std::to_string(k) + "x" + std::to_string(2 * inter) + ", " + std::to_string(m) + " rows";
            auto it = s->gate_up_pick.find(key);
            if (it != s->gate_up_pick.end()) {
                ks = it->second;
            } else {
                std::vector<const hb_kernel*> ap;
                if ((r = apart(&ap)) != HB_OK) return r;
                std::vector<Cand> cands;
                std::vector<char> eligible;
                Cand c0;
                c0.name = "apart";
                add_op(c0, ap[0], {w, x, gu});
                add_op(c0, ap[1], {gu, h});
                cands.push_back(std::move(c0));
                eligible.push_back(1);
                for (uint32_t form = 0; form < 8; ++form) {
                    const uint32_t pair = form >= 6 ? 1u : 0u;
                    const uint32_t tn = pair ? (form == 6 ? 256u : 192u) : 256u >> (form % 3), sk = pair ? 0u : form / 3;
                    hb_kernel* f = nullptr;
                    const std::string name = pair ? "fusedpair256x" + std::to_string(tn) : std::string(sk ? "fusedsk128x" : "fused128x") + std::to_string(tn);
                    if (get_dense(s, k, 2 * inter, HB_OUT_SWIGLU, tn, 0, mf, pair, rows_max, &f, sk) != HB_OK) {
                        say(s, "[autotune] gate_up " + key + ": " + name + " not built (" + hb_last_error(ctx) + ")");
                        continue;
                    }
                    Cand c;
                    c.name = name;
                    add_op(c, f, {w, x, h});
                    cands.push_back(std::move(c));
                    eligible.push_back(1);
                }
                for (uint32_t sp : pair_splits(ctx, m, k, inter, 128)) {
                    hb_kernel* f = nullptr;
                    if (get_dense(s, k, 2 * inter, HB_OUT_SWIGLU, 256, 0, mf, 1, std::min(rows_max, 1024u), &f, 0, sp) != HB_OK) continue;
                    Cand c;
                    c.name = "fusedpair256x256k" + std::to_string(sp);
                    add_op(c, f, {w, x, h});
                    cands.push_back(std::move(c));
                    eligible.push_back(1);
                }
                if (m <= 64) {  // the weight-stream form with the SwiGLU epilogue (two weight tiles per step: two K blocks per stage)
                    for (uint32_t tc : {1u, 2u, 3u}) {
                        hb_matvec_desc d{};
                        d.k = k;
                        d.n = 2 * inter;
                        d.out = HB_OUT_SWIGLU;
                        d.rows_max = m;
                        d.tensor_core = tc;
                        d.split = 2;
                        hb_kernel* f = nullptr;
                        if (hb_matvec_get(ctx, &d, &f) != HB_OK) continue;
                        Cand c;
                        c.name = tc == 1 ? "fusedstream" : tc == 2 ? "fusedstreamb" : "fusedstreamf";
                        add_op(c, f, {w, x, h});
                        cands.push_back(std::move(c));
                        eligible.push_back(1);
                    }
                }
                const std::string what = "gate_up " + key;
                if ((r = check_candidates(s, what, cands, eligible, h, (size_t)inter * 2, false, m)) != HB_OK) return r;
                size_t best;
                if ((r = pick_flagged(s, what, cands, eligible, m, &best, nullptr)) != HB_OK) return r;
                ks = cands[best].kernels;
                s->gate_up_pick[key] = ks;
            }
        }
        for (size_t i = 0; i < ks.size(); ++i) kernels_out[i] = ks[i];
        *nkernels = (int)ks.size();
        return HB_OK;
    } catch (const std::exception& e) {
        return hb::fail(ctx, HB_BACKEND, e.what());
    }
}

int hb_select_matvec(hb_selector* s, uint32_t k, uint32_t n, uint32_t out, uint32_t rows, const hb_range* w_copies, int ncopies, hb_range x, hb_range y,
                     const hb_kernel** picked) {
    return hb_select_matvec_x(s, k, n, out, rows, HB_X_PLAIN, 0, 0, w_copies, ncopies, x, y, hb_range{nullptr, 0}, picked);
}

int hb_select_matvec_x(hb_selector* s, uint32_t k, uint32_t n, uint32_t out, uint32_t rows, uint32_t x_src, uint32_t norm_eps_bits, uint32_t norm_plus_one,
                       const hb_range* w_copies, int ncopies, hb_range x, hb_range y, hb_range norm_w, const hb_kernel** picked) {
    if (!s || !picked || !w_copies || ncopies < 1 || x_src > HB_X_SWIGLU) return HB_INVALID;
    hb_ctx* ctx = s->ctx;
    if (x_src == HB_X_NORM && !norm_w.ptr) return hb::fail(ctx, HB_INVALID, "hb_select_matvec_x: XSrc::Norm and its weights go together");  // qwen.rs:1332
    try {
        const hb_tune& t = s->tune;
        int r;
        // the bindings of a candidate: W, x, y and, with the norm made inside the kernel, its weights
        auto bind = [&](int copy) {
            std::vector<hb_range> b = {w_copies[copy], x, y};
            if (x_src == HB_X_NORM) b.push_back(norm_w);
            return b;
        };
        auto get = [&](uint32_t rpw, uint32_t split, uint32_t persist, hb_kernel** kern, uint32_t xs = 0, uint32_t tc = 0) {
            hb_matvec_desc d{};
            d.x_src = x_src;
            d.norm_eps_bits = norm_eps_bits;
            d.norm_plus_one = norm_plus_one;
            d.x_stationary = xs;
            d.tensor_core = tc;
            d.k = k;
            d.n = n;
            d.out = out;
            d.rows_max = rows;
            d.rows_per_warp = rpw;
            d.split = split;
            d.persist = persist;
            return hb_matvec_get(ctx, &d, kern);
        };
        hb_kernel* kern = nullptr;
        if (t.get("mv.auto") == 0) {  // the keys name the form (qwen.rs:1390-1402)
            const uint32_t rpw = out == HB_OUT_SWIGLU ? 2u : 2u;
            if ((r = get(rpw, std::max(1u, t.get("mv.split")), t.get("mv.persist") ? 1u : 0u, &kern)) != HB_OK) return r;
            *picked = kern;
            return HB_OK;
        }
        std::string key = std::to_string(k) + "x" + std::to_string(n) + " " + out_debug(out);
        if (x_src == HB_X_NORM) key += " norm";  // qwen.rs:1410
        if (x_src == HB_X_SWIGLU) key += " swiglu";
        if (rows > 1) key += ", " + std::to_string(rows) + " rows";
        if (!t.mv_persists.empty()) {
            key += " p[";
            for (size_t i = 0; i < t.mv_persists.size(); ++i) key += (i ? ", " : "") + std::to_string(t.mv_persists[i]);
            key += "]";
        }
        auto it = s->mv_pick.find(key);
        if (it != s->mv_pick.end()) {
            *picked = it->second;
            return HB_OK;
        }
        // Every candidate walks the same-shaped matrices in turn so that weights stream from memory
        // (mv.cold, qwen.rs:248-251,1177-1203); mv.cold=0 times on the first copy alone.
        const int copies = t.get("mv.cold") != 0 ? ncopies : 1;
        std::vector<uint32_t> splits = t.get("mv.splitauto") != 0 ? std::vector<uint32_t>{1, 2, 4} : std::vector<uint32_t>{1};
        std::vector<uint32_t> persists = {0};
        for (uint32_t p : t.mv_persists) persists.push_back(p);
        // an input made inside the kernel is made once per block: a grid of long-lived blocks is always a candidate
        if (x_src != HB_X_PLAIN && t.mv_persists.empty()) persists.push_back(1);
        std::vector<Cand> cands;
        for (uint32_t split : splits)
            for (uint32_t persist : persists)
                for (uint32_t rpw : {1u, 2u, 4u, 8u}) {
                    if (persist > 0 && rpw == 8) continue;          // qwen.rs:1453
                    if (out == HB_OUT_SWIGLU && rpw == 1) continue;  // a gate row and its up row at least
                    if (get(rpw, split, persist ? 1u : 0u, &kern) != HB_OK) continue;
                    Cand c;
                    c.name = "r" + std::to_string(rpw) + (split > 1 ? "k" + std::to_string(split) : "") + (persist ? "p" + std::to_string(persist) : "");
                    for (int i = 0; i < copies; ++i) add_op(c, kern, bind(i));
                    cands.push_back(std::move(c));
                }
        // with several activation rows: the forms that keep the activations widened in registers
        if (rows > 1 && x_src == HB_X_PLAIN)
            for (uint32_t rpw : {2u, 4u}) {
                if (get(rpw, 1, 1, &kern, 1) != HB_OK) continue;
                Cand c;
                c.name = "x" + std::to_string(rpw);
                for (int i = 0; i < copies; ++i) add_op(c, kern, bind(i));
                cands.push_back(std::move(c));
            }
        // the weight stream on the tensor cores: whole feature blocks per CTA or evenly dealt units, 2 or 4 K blocks
        // per pipeline stage
        {
            struct TcForm { const char* name; uint32_t ks, kps; };
            const uint32_t n_out = out == HB_OUT_SWIGLU ? n / 2 : n;
            (void)n_out;
            for (const TcForm& f : {TcForm{"tc", 1, 2}, TcForm{"tcw", 1, 4}, TcForm{"tcb", 2, 2}, TcForm{"tcbw", 2, 4}, TcForm{"tcf", 3, 2}, TcForm{"tcfw", 3, 4}}) {
                hb_matvec_desc d{};
                d.k = k;
                d.n = n;
                d.out = out;
                d.rows_max = rows;
                d.tensor_core = f.ks;
                d.split = f.kps;
                d.x_src = x_src;
                d.norm_eps_bits = norm_eps_bits;
                d.norm_plus_one = norm_plus_one;
                if (hb_matvec_get(ctx, &d, &kern) != HB_OK) continue;
                Cand c;
                c.name = f.name;
                for (int i = 0; i < copies; ++i) add_op(c, kern, bind(i));
                cands.push_back(std::move(c));
            }
        }
        if (cands.empty()) return hb::fail(ctx, HB_UNSUPPORTED, "matvec " + key + ": no form could be built");
        std::vector<char> eligible(cands.size(), 1);
        size_t best;
        if ((r = pick_flagged(s, "matvec " + key, cands, eligible, rows, &best, nullptr)) != HB_OK) return r;
        s->mv_pick[key] = cands[best].kernels[0];
        *picked = cands[best].kernels[0];
        return HB_OK;
    } catch (const std::exception& e) {
        return hb::fail(ctx, HB_BACKEND, e.what());
    }
}

// One axis of tune_step (src/metal/qwen.rs:3043-3170): the forms of the decode step that --tune does not fix are
// timed at load on the whole step, one axis after another. The caller records the step once per value of the axis;
// each is run twice to warm, then seven times, the median (ts[3]) kept; the first strictly fastest value wins.
int hb_select_axis(hb_selector* s, const char* axis, const char* key, const hb_op* const* variants, const int* nops, const uint32_t* values, int nvariants,
                   uint32_t position, uint32_t* best_value) {
    if (!s || !axis || !key || !variants || !nops || !values || nvariants < 1 || !best_value) return HB_INVALID;
    hb_ctx* ctx = s->ctx;
    try {
        const hb_tune& t = s->tune;
        // an axis whose key --tune gives keeps it (qwen.rs:3121-3123); dec.auto=0 times nothing
        if (t.was_given(key) || t.get("dec.auto") == 0) {
            *best_value = t.get(key);
            return HB_OK;
        }
        std::string line;
        double best = 1e300;
        uint32_t best_v = values[0];
        for (int v = 0; v < nvariants; ++v) {
            if (!variants[v] || nops[v] <= 0) {
                line += (line.empty() ? "" : ", ") + std::to_string(values[v]) + " unavailable";
                continue;
            }
            double sec;
            int r = hb_time(ctx, variants[v], nops[v], 2, &sec);
            if (r != HB_OK) return r;
            std::vector<double> ts(7);
            for (double& x : ts) {
                if ((r = hb_time(ctx, variants[v], nops[v], 1, &x)) != HB_OK) return r;
                s->autotune_seconds += x;
            }
            std::sort(ts.begin(), ts.end());
            char buf[64];
            snprintf(buf, sizeof buf, " %.3f ms", ts[3] * 1e3);
            line += (line.empty() ? "" : ", ") + std::to_string(values[v]) + buf;
            if (ts[3] < best) {
                best = ts[3];
                best_v = values[v];
            }
        }
        say(s, "[autotune] decode step at position " + std::to_string(position) + ", " + axis + ": " + line + " -> " + std::to_string(best_v));
        *best_value = best_v;
        return HB_OK;
    } catch (const std::exception& e) {
        return hb::fail(ctx, HB_BACKEND, e.what());
    }
}

int hb_select_experts(hb_selector* s, const hb_expert_io* io, hb_expert_pick* pick) {
    if (!s || !io || !pick) return HB_INVALID;
    hb_ctx* ctx = s->ctx;
    try {
        const hb_tune& t = s->tune;
        const uint32_t m = io->m, pairs = io->m * io->top_k;
        const uint32_t rows_max = std::max(m, t.get("prefill.block"));
        if (t.get("moe.grouped") == 0) {
            // moe.grouped = 0 (qwen.rs:2085-2088, 2725-2729): no sort, a matvec per (row, slot) against its expert's rows
            if (!io->egu.ptr) return hb::fail(ctx, HB_INVALID, "hb_select_experts: moe.grouped = 0 needs the [gate | up] rows (io.egu)");
            hb_kernel *gu = nullptr, *sw = nullptr, *dn = nullptr;
            int r0;
            if ((r0 = hb_experts_matvec_get(ctx, io->h, 2 * io->mi, io->top_k, io->experts, io->h, 0, 0, &gu)) != HB_OK) return r0;
            if ((r0 = hb_swiglu_get(ctx, io->mi, &sw)) != HB_OK) return r0;
            if ((r0 = hb_experts_matvec_get(ctx, io->mi, io->h, io->top_k, io->experts, io->top_k * io->mi, io->mi, 0, &dn)) != HB_OK) return r0;
            pick->bm = 0;
            pick->sort = nullptr;
            pick->gather = nullptr;
            pick->gate_up = gu;
            pick->swiglu = sw;
            pick->down = dn;
            return HB_OK;
        }
        std::vector<uint32_t> bms;
        if (t.moe_tile_set || !t.gemm_timed()) bms = {t.get("moe.tile")};  // qwen.rs:2352
        else bms = {16, 32, 64};
        auto expert_gemm = [&](uint32_t k, uint32_t n, uint32_t out, uint32_t mode, uint32_t bm, hb_kernel** kern, uint32_t merge = 0) {
            hb_gemm_desc d{};
            d.merge_runs = merge;
            d.k = k;
            d.n = n;
            d.out = out;
            d.rows_mode = mode;
            d.top_k = io->top_k;
            d.experts = io->experts;
            d.bm = bm;
            d.rows_max = rows_max;
            return hb_gemm_get(ctx, &d, kern);
        };
        double best_total = 0.0;
        bool have = false;
        int r;
        for (uint32_t bm : bms) {
            hb_kernel *sort = nullptr, *fused = nullptr, *down = nullptr;
            if ((r = hb_moe_sort_get(ctx, io->experts, io->top_k, rows_max, bm, &sort)) != HB_OK) return r;
            if ((r = expert_gemm(io->h, 2 * io->mi, HB_OUT_SWIGLU, HB_ROWS_GATHER, bm, &fused)) != HB_OK) return r;
            if ((r = expert_gemm(io->mi, io->h, HB_OUT_BF16, HB_ROWS_SCATTER, bm, &down)) != HB_OK) return r;
            const std::string tag = std::to_string(io->experts) + " experts, tiles of " + std::to_string(bm) + ", " + std::to_string(m) + " rows";
            // the sort (one form: the scan order is the contract; an atomic order would not be reproducible)
            Cand cs;
            cs.name = "scan";
            add_op(cs, sort, {io->route, io->list, io->tiles});
            double t_sort = 0.0;
            if (!t.gemm_timed()) {
                hb_range a[3] = {io->route, io->list, io->tiles};
                if ((r = hb_launch(ctx, sort, a, 3, m)) != HB_OK) return r;
                pick->bm = bm;
                pick->sort = sort;
                pick->gather = nullptr;
                pick->gate_up = fused;
                pick->swiglu = nullptr;
                pick->down = down;
                return hb_sync(ctx);
            }
            {
                std::vector<Cand> one;
                one.push_back(cs);
                std::vector<char> el = {1};
                size_t b;
                if ((r = pick_flagged(s, "experts sort " + tag, one, el, m, &b, &t_sort)) != HB_OK) return r;
            }
            // gate/up forms on the sorted route just produced
            std::vector<Cand> gu;
            Cand c0;
            c0.name = "fused";
            add_op(c0, fused, {io->wgu, io->x, io->ehb, io->list, io->tiles});
            gu.push_back(std::move(c0));
            hb_kernel *apart = nullptr, *swi = nullptr, *gather = nullptr, *sorted = nullptr;
            if (io->egu.ptr && expert_gemm(io->h, 2 * io->mi, HB_OUT_BF16, HB_ROWS_GATHER, bm, &apart) == HB_OK && hb_swiglu_get(ctx, io->mi, &swi) == HB_OK) {
                Cand c;
                c.name = "apart";
                add_op(c, apart, {io->wgu, io->x, io->egu, io->list, io->tiles});
                add_op(c, swi, {io->egu, io->ehb}, (int)io->top_k);
                gu.push_back(std::move(c));
            }
            if (io->xs.ptr && hb_moe_gather_get(ctx, io->h, io->top_k, &gather) == HB_OK &&
                expert_gemm(io->h, 2 * io->mi, HB_OUT_SWIGLU, HB_ROWS_SORTED, bm, &sorted) == HB_OK) {
                Cand c;
                c.name = "gather+fused";
                add_op(c, gather, {io->x, io->list, io->xs});
                add_op(c, sorted, {io->wgu, io->xs, io->ehb, io->list, io->tiles});
                gu.push_back(std::move(c));
            }
            hb_kernel *fused_m = nullptr, *sorted_m = nullptr, *down_m = nullptr;
            if (expert_gemm(io->h, 2 * io->mi, HB_OUT_SWIGLU, HB_ROWS_GATHER, bm, &fused_m, 1) == HB_OK) {
                Cand c;
                c.name = "fused+runs";
                add_op(c, fused_m, {io->wgu, io->x, io->ehb, io->list, io->tiles});
                gu.push_back(std::move(c));
            }
            if (io->xs.ptr && gather && expert_gemm(io->h, 2 * io->mi, HB_OUT_SWIGLU, HB_ROWS_SORTED, bm, &sorted_m, 1) == HB_OK) {
                Cand c;
                c.name = "gather+fused+runs";
                add_op(c, gather, {io->x, io->list, io->xs});
                add_op(c, sorted_m, {io->wgu, io->xs, io->ehb, io->list, io->tiles});
                gu.push_back(std::move(c));
            }
            std::vector<char> el(gu.size(), 1);
            // The partial-block pass of the check needs a route of that many rows: only the full block is sorted
            // here, so candidates are compared at m rows (rows past the sorted pairs are never written).
            {
                const size_t bytes = (size_t)pairs * io->mi * 2;
                std::vector<uint8_t> ref(bytes), got(bytes);
                double tt;
                if ((r = hb_memset(ctx, io->ehb.ptr, 0, bytes)) != HB_OK) return r;
                if ((r = time_ops(s, gu[0], m, 1, &tt)) != HB_OK) return r;
                if ((r = hb_download(ctx, ref.data(), io->ehb.ptr, bytes)) != HB_OK) return r;
                std::vector<std::string> wrong;
                for (size_t i = 1; i < gu.size(); ++i) {
                    if ((r = hb_memset(ctx, io->ehb.ptr, 0, bytes)) != HB_OK) return r;
                    if ((r = time_ops(s, gu[i], m, 1, &tt)) != HB_OK) return r;
                    if ((r = hb_download(ctx, got.data(), io->ehb.ptr, bytes)) != HB_OK) return r;
                    float err, scale;
                    if (!rule_1_64(ref.data(), got.data(), bytes / 2, false, &err, &scale)) {
                        el[i] = 0;
                        wrong.push_back(gu[i].name + " (" + std::to_string(m) + " rows: max err " + fmt_e3(err) + " of " + fmt_e3(scale) + ")");
                    }
                }
                if (!wrong.empty()) {
                    std::string line = "[autotune] experts gate_up " + tag + ": wrong against " + gu[0].name + ", never picked: ";
                    for (size_t i = 0; i < wrong.size(); ++i) line += (i ? ", " : "") + wrong[i];
                    say(s, line);
                }
            }
            size_t bgu;
            double t_gu = 0.0, t_down = 0.0;
            if ((r = pick_flagged(s, "experts gate_up " + tag, gu, el, m, &bgu, &t_gu)) != HB_OK) return r;
            // leave EHB as the picked form computes it, then time the down projection
            double tt;
            if ((r = time_ops(s, gu[bgu], m, 1, &tt)) != HB_OK) return r;
            std::vector<Cand> dn;
            Cand cd;
            cd.name = "scatter";
            add_op(cd, down, {io->wdown, io->ehb, io->ey, io->list, io->tiles});
            dn.push_back(std::move(cd));
            if (expert_gemm(io->mi, io->h, HB_OUT_BF16, HB_ROWS_SCATTER, bm, &down_m, 1) == HB_OK) {
                Cand c;
                c.name = "scatter+runs";
                add_op(c, down_m, {io->wdown, io->ehb, io->ey, io->list, io->tiles});
                dn.push_back(std::move(c));
            }
            std::vector<char> eld(dn.size(), 1);
            {   // the merged form against the per-tile form, on the EHB just made
                const size_t bytes = (size_t)pairs * io->h * 2;
                std::vector<uint8_t> ref(bytes), got(bytes);
                double tt;
                if ((r = hb_memset(ctx, io->ey.ptr, 0, bytes)) != HB_OK) return r;
                if ((r = time_ops(s, dn[0], m, 1, &tt)) != HB_OK) return r;
                if ((r = hb_download(ctx, ref.data(), io->ey.ptr, bytes)) != HB_OK) return r;
                for (size_t i = 1; i < dn.size(); ++i) {
                    if ((r = hb_memset(ctx, io->ey.ptr, 0, bytes)) != HB_OK) return r;
                    if ((r = time_ops(s, dn[i], m, 1, &tt)) != HB_OK) return r;
                    if ((r = hb_download(ctx, got.data(), io->ey.ptr, bytes)) != HB_OK) return r;
                    float err, scale;
                    if (!rule_1_64(ref.data(), got.data(), bytes / 2, false, &err, &scale)) {
                        eld[i] = 0;
                        say(s, "[autotune] experts down " + tag + ": wrong against " + dn[0].name + ", never picked: " + dn[i].name + " (" + std::to_string(m) +
                                   " rows: max err " + fmt_e3(err) + " of " + fmt_e3(scale) + ")");
                    }
                }
            }
            size_t bd;
            if ((r = pick_flagged(s, "experts down " + tag, dn, eld, m, &bd, &t_down)) != HB_OK) return r;
            const double total = t_sort + t_gu + t_down;
            if (!have || total < best_total) {
                have = true;
                best_total = total;
                pick->bm = bm;
                pick->sort = sort;
                const std::string& gn = gu[bgu].name;
                pick->gather = gn.rfind("gather+", 0) == 0 ? gather : nullptr;
                pick->gate_up = gn == "fused" ? fused : gn == "apart" ? apart : gn == "gather+fused" ? sorted : gn == "fused+runs" ? fused_m : sorted_m;
                pick->swiglu = gn == "apart" ? swi : nullptr;
                pick->down = dn[bd].name == "scatter" ? down : down_m;
            }
        }
        char buf[160];
        snprintf(buf, sizeof buf, "[autotune] experts %u rows: tiles of %u rows (sort + gate_up + down %.3f ms)", m, pick->bm, best_total * 1e3);
        say(s, buf);
        // the list and tile table must match the picked tile size
        hb_range a[3] = {io->route, io->list, io->tiles};
        if ((r = hb_launch(ctx, pick->sort, a, 3, m)) != HB_OK) return r;
        return hb_sync(ctx);
    } catch (const std::exception& e) {
        return hb::fail(ctx, HB_BACKEND, e.what());
    }
}

}  // extern "C"
