// Internal data model shared by the host-side index compiler (builder.cpp) and the device engine (engine.cu).
#pragma once
#include <cstdint>
#include <string>
#include <vector>

#include "../../include/thrml_b200.h"

struct thrml_builder;

namespace thrml {

// Thread-local error slot behind thrml_last_error().
void set_error(const std::string& msg);
int32_t fail(int32_t code, const std::string& msg);

// RngKey::split (crates/thrml-samplers/src/rng.rs:19-41).
void rng_split(uint64_t key, int64_t n, uint64_t* out);

// One InteractionGroup as handed over by the caller (crates/thrml-core/src/interaction.rs:107-125).
struct GroupDesc {
    std::vector<int64_t> head;                // [rows]
    std::vector<std::vector<int64_t>> tails;  // [n_tails][rows]
    int32_t n_spin = 0;
    int32_t d1 = 1, d2 = 1;
    std::vector<float> w;  // [rows][d1][d2]
};

// One compiled (free block, interaction group) table — the per-block entries of BlockSamplingProgram
// (crates/thrml-samplers/src/program.rs:70-85).
struct SlotTable {
    int32_t k = 0;     // padded slot count = max number of rows in which a node of the block is head
    int32_t wdim = 1;  // d1*d2
    int32_t n_spin = 0;
    int32_t source_group = 0;
    std::vector<int32_t> rows;              // interaction_slices [n*k]
    std::vector<uint8_t> active;            // [n*k]
    std::vector<float> w;                   // [n*k*wdim]
    std::vector<std::vector<int32_t>> idx;  // [n_tails][n*k] global positions
    std::vector<int32_t> tail_sd;           // class (sd index) of each tail
    std::vector<int32_t> tail_is_cat;       // 1 when the tail block holds categorical nodes
};

struct BlockInfo {
    std::vector<int64_t> nodes;
    int32_t kind = 0;        // 0 spin, K categorical
    int32_t sd = 0;          // class (sd index)
    int64_t offset = 0;      // first global position inside its class
    int32_t superblock = 0;  // free blocks only
    int32_t sampler = 0;     // free blocks only
};

}  // namespace thrml

namespace thrml {
// Layout half of the index compilation (classes, sampling order, node positions, argument checks), on the host.
int32_t compile_layout(thrml_builder* b);
}  // namespace thrml

struct thrml_builder {
    std::vector<int32_t> kinds;
    std::vector<int32_t> dtype_order;
    std::vector<thrml::BlockInfo> free_blocks, clamped_blocks;
    std::vector<thrml::GroupDesc> groups;
    // compiled
    bool compiled = false;
    int32_t n_classes = 0;
    int32_t sd_spin = -1, sd_cat = -1;          // class index of the Bool / U8 TensorSpec, -1 if absent
    std::vector<int64_t> class_size;            // [n_classes]
    std::vector<int8_t> loc_sd;                 // per node, -1 = not in any block
    std::vector<int64_t> loc_pos;               // per node
    std::vector<std::vector<int32_t>> sampling_order;
    std::vector<std::vector<thrml::SlotTable>> tables;  // per free block
};
