// The engine's --tune settings for the matrix-multiply path.
// Restates Tune / Tune::apply / Tune::summary of the reference (src/metal/qwen.rs:62-397):
// the same keys, defaults, side effects (a given gemm.mma / gemm.tn / gemm.mform turns the
// load-time timing off, qwen.rs:325-327) and error messages. Keys that steer parts of the
// engine outside this path (attention, DeltaNet, decode fusions) are parsed, range-checked
// where the reference checks them, and stored.
#include <algorithm>
#include <cstring>
#include <sstream>

#include "tune.hpp"

namespace {

struct KeyDefault {
    const char* key;
    uint32_t value;
};

// Defaults of Tune::default(), qwen.rs:279, in the order Tune::summary() prints them.
const KeyDefault kDefaults[] = {
    {"prefill.block", 2048}, {"rec.chunk", 4},   {"rec.pcols", 16},  {"rec.pslices", 16}, {"rec.vec", 0},      {"rec.pair", 0},
    {"rec.stage", 0},        {"conv.cols", 32},  {"sdpa.prefill", 1}, {"sdpa.bq", 16},    {"sdpa.bk", 16},     {"sdpa.mq", 0},
    {"sdpa.mk", 32},         {"sdpa.qreg", 0},   {"sdpa.kt", 0},     {"sdpa.msg", 8},     {"sdpa.auto", 1},    {"auto.heat", 0},
    {"gemm.simt", 1},        {"gemm.auto", 1},   {"gemm.mma", 1},    {"gemm.tn", 64},     {"gemm.mform", 0},   {"gemm.half", 1},
    {"gemm.mfirst", 1},      {"moe.grouped", 1}, {"moe.tile", 16},   {"q4.fuse", 0},      {"mv.auto", 1},      {"mv.masks", 0},
    {"mv.split", 1},         {"mv.splitauto", 1}, {"mv.persist", 0}, {"dec.sdpa", 32},    {"mv.cold", 1},      {"dec.swiglu", 0},
    {"dec.prep", 0},         {"dec.conc", 0},    {"dec.pf", 0},      {"dec.pfk", 0},      {"dec.auto", 1},     {"dec.gnorm", 0},
    {"dec.pfdn", 0},         {"dec.fnorm", 0},   {"dec.fswi", 0},    {"pf.fswi", 2},      {"dec.fdn", 0},      {"dec.frope", 0},
    {"dec.rec", 1},          {"dec.cols", 16},   {"dec.slices", 16}, {"dn.sscale", 0},    {"dn.oscale", 0},    {"dn.tscale", 0},
};

bool parse_u32(const std::string& s, uint32_t* out, std::string* why) {
    // Rust's u32::from_str: optional '+', decimal digits only, no overflow.
    if (s.empty()) {
        *why = "cannot parse integer from empty string";
        return false;
    }
    size_t i = s[0] == '+' ? 1 : 0;
    if (i == s.size()) {
        *why = "invalid digit found in string";
        return false;
    }
    uint64_t v = 0;
    for (; i < s.size(); ++i) {
        if (s[i] < '0' || s[i] > '9') {
            *why = "invalid digit found in string";
            return false;
        }
        v = v * 10 + (uint64_t)(s[i] - '0');
        if (v > 0xffffffffull) {
            *why = "number too large to fit in target type";
            return false;
        }
    }
    *out = (uint32_t)v;
    return true;
}

}  // namespace

hb_tune::hb_tune() {
    for (const auto& d : kDefaults) {
        order.push_back(d.key);
        values[d.key] = d.value;
    }
}

uint32_t hb_tune::get(const std::string& key) const {
    auto it = values.find(key);
    return it == values.end() ? 0 : it->second;
}

bool hb_tune::was_given(const std::string& key) const { return std::find(given.begin(), given.end(), key) != given.end(); }

bool hb_tune::gemm_timed() const { return get("gemm.auto") != 0 && !gemm_set; }

std::string hb_tune::apply(const std::string& list) {
    std::stringstream ss(list);
    std::string kv;
    while (std::getline(ss, kv, ',')) {
        if (kv.empty()) continue;
        const size_t eq = kv.find('=');
        if (eq == std::string::npos) return "--tune " + kv + ": key=value";
        const std::string key = kv.substr(0, eq), value = kv.substr(eq + 1);
        given.push_back(key);
        if (key == "mv.persists") {
            std::vector<uint32_t> v;
            std::stringstream ps(value);
            std::string item;
            while (std::getline(ps, item, '/')) {
                if (item.empty()) continue;
                uint32_t n;
                std::string why;
                if (!parse_u32(item, &n, &why)) return "--tune " + kv + ": " + why;
                v.push_back(n);
            }
            mv_persists = v;
            continue;
        }
        uint32_t n;
        std::string why;
        if (!parse_u32(value, &n, &why)) return "--tune " + kv + ": " + why;
        if (values.find(key) == values.end()) return "--tune " + key + ": unknown";
        if (key == "prefill.block") {
            values[key] = std::max(n, 1u);
            block_set = true;
        } else if (key == "sdpa.prefill") {
            values[key] = n;
            sdpa_set = true;
        } else if (key == "gemm.mma" || key == "gemm.tn" || key == "gemm.mform" || key == "q4.fuse") {
            values[key] = n;
            gemm_set = true;
        } else if (key == "moe.tile") {
            values[key] = n;
            moe_tile_set = true;
        } else if (key == "mv.masks" || key == "mv.split" || key == "mv.persist") {
            values[key] = n;
            values["mv.auto"] = 0;
        } else if (key == "dec.sdpa") {
            values[key] = std::min(n, 64u);
        } else {
            values[key] = n;
        }
    }
    auto v = [&](const char* k) { return get(k); };
    auto s = [](uint32_t x) { return std::to_string(x); };
    if (v("q4.fuse") > 1 || (v("q4.fuse") == 1 && v("gemm.mma") != 1)) return "--tune q4.fuse=" + s(v("q4.fuse")) + ": 0, or 1 with gemm.mma=1";
    const uint32_t tn = v("gemm.tn");
    if (v("gemm.mma") > 3 || !((tn == 16 || tn == 32 || tn == 64) || (v("gemm.mma") == 3 && tn == 128)) || v("gemm.mform") > 9)
        return "--tune gemm.mma=" + s(v("gemm.mma")) + " gemm.tn=" + s(tn) + " gemm.mform=" + s(v("gemm.mform")) +
               ": gemm.mma 0..2, gemm.tn 16, 32 or 64, gemm.mform 0..9";
    const uint32_t mt = v("moe.tile");
    if (mt != 16 && mt != 32 && mt != 64) return "--tune moe.tile=" + s(mt) + ": 16, 32 or 64";
    if (v("rec.chunk") > 4 || v("sdpa.prefill") > 7 || v("gemm.simt") < 1 || v("gemm.simt") > 2)
        return "--tune: rec.chunk 0..4, sdpa.prefill 0..7, gemm.simt 1..2";
    if (v("dn.sscale") > 15 || v("dn.oscale") > 15 || v("dn.tscale") > 15) return "--tune dn.sscale/oscale/tscale: 0..15";
    return "";
}

std::string hb_tune::summary() const {
    std::string out;
    for (const auto& key : order) {
        uint32_t val = get(key);
        // summary() prints the *effective* switches (qwen.rs:394): timing is off once a kernel was named.
        if (key == "gemm.auto") val = gemm_timed() ? 1 : 0;
        if (key == "sdpa.auto") val = (val != 0 && !sdpa_set) ? 1 : 0;
        if (!out.empty()) out += ' ';
        out += key + "=" + std::to_string(val);
        if (key == "mv.persist") {
            out += " mv.persists=[";
            for (size_t i = 0; i < mv_persists.size(); ++i) out += (i ? ", " : "") + std::to_string(mv_persists[i]);
            out += "]";
        }
    }
    return out;
}

extern "C" {

int hb_tune_new(hb_tune** out) {
    if (!out) return HB_INVALID;
    try {
        *out = new hb_tune();
    } catch (...) {
        *out = nullptr;
        return HB_OOM;
    }
    return HB_OK;
}

void hb_tune_free(hb_tune* t) { delete t; }

int hb_tune_apply(hb_tune* t, const char* list, char* err, size_t errlen) {
    if (!t || !list) return HB_INVALID;
    try {
        // Apply on a copy: a failed list leaves the settings as they were.
        hb_tune copy = *t;
        const std::string e = copy.apply(list);
        if (!e.empty()) {
            if (err && errlen) snprintf(err, errlen, "%s", e.c_str());
            return HB_INVALID;
        }
        *t = copy;
        if (err && errlen) err[0] = 0;
        return HB_OK;
    } catch (...) {
        return HB_BACKEND;
    }
}

int hb_tune_get(const hb_tune* t, const char* key, uint32_t* value) {
    if (!t || !key || !value) return HB_INVALID;
    auto it = t->values.find(key);
    if (it == t->values.end()) return HB_INVALID;
    *value = it->second;
    return HB_OK;
}

int hb_tune_summary(const hb_tune* t, char* buf, size_t len) {
    if (!t || !buf || !len) return HB_INVALID;
    snprintf(buf, len, "%s", t->summary().c_str());
    return HB_OK;
}

int hb_tune_gemm_timed(const hb_tune* t) { return t && t->gemm_timed() ? 1 : 0; }

}  // extern "C"
