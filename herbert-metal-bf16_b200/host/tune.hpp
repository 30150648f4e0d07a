// hb_tune: the --tune settings of the reference engine (src/metal/qwen.rs:62-397).
#pragma once

#include <cstdint>
#include <map>
#include <string>
#include <vector>

#include "../../include/hb200.h"

struct hb_tune {
    std::map<std::string, uint32_t> values;
    std::vector<std::string> order;    // the order Tune::summary prints
    std::vector<std::string> given;    // keys the user gave (qwen.rs:299)
    std::vector<uint32_t> mv_persists;
    bool gemm_set = false;     // gemm.mma / gemm.tn / gemm.mform / q4.fuse given: no timing (qwen.rs:325-327,333)
    bool block_set = false;    // prefill.block given (qwen.rs:306)
    bool moe_tile_set = false; // moe.tile given: only that tile is timed (qwen.rs:2352)
    bool sdpa_set = false;

    hb_tune();
    uint32_t get(const std::string& key) const;
    bool was_given(const std::string& key) const;
    bool gemm_timed() const;
    // Applies "k=v,k=v"; returns "" or the reference's error message.
    std::string apply(const std::string& list);
    std::string summary() const;
};
