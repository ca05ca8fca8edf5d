// Host side of libthrml_b200: RngKey splitting, input generators and the index compiler that turns blocks and
// interaction groups into the per-block slot tables the kernels consume.  No CUDA in this file.
#include <algorithm>
#include <cstring>
#include <numeric>

#include "tables.h"

namespace thrml {

static thread_local std::string g_last_error;
void set_error(const std::string& msg) { g_last_error = msg; }
int32_t fail(int32_t code, const std::string& msg) {
    g_last_error = msg;
    return code;
}

// ---------------------------------------------------------------------------------------------------------
// RngKey::split — crates/thrml-samplers/src/rng.rs:19-41.  The reference seeds rand_chacha's ChaCha8Rng with
// seed_from_u64: rand_core expands the u64 with a PCG32 generator into the 256-bit key; the generator then emits
// the ChaCha keystream (8 rounds, block counter from 0, stream 0) and next_u64 joins two 32-bit words, low first.
// ---------------------------------------------------------------------------------------------------------
namespace {
struct ChaCha8Stream {
    uint32_t key[8];
    uint64_t block = 0;
    uint32_t buf[16];
    int have = 0;

    explicit ChaCha8Stream(uint64_t seed) {
        uint64_t st = seed;
        for (uint32_t& word : key) {
            st = st * 6364136223846793005ull + 11634580027462260723ull;
            uint32_t xs = static_cast<uint32_t>(((st >> 18) ^ st) >> 27);
            uint32_t rot = static_cast<uint32_t>(st >> 59);
            word = (xs >> rot) | (xs << ((32u - rot) & 31u));
        }
    }
    static inline void quarter(uint32_t& a, uint32_t& b, uint32_t& c, uint32_t& d) {
        a += b; d ^= a; d = (d << 16) | (d >> 16);
        c += d; b ^= c; b = (b << 12) | (b >> 20);
        a += b; d ^= a; d = (d << 8) | (d >> 24);
        c += d; b ^= c; b = (b << 7) | (b >> 25);
    }
    void refill() {
        uint32_t in[16] = {0x61707865u, 0x3320646eu, 0x79622d32u, 0x6b206574u};
        std::memcpy(in + 4, key, sizeof(key));
        in[12] = static_cast<uint32_t>(block);
        in[13] = static_cast<uint32_t>(block >> 32);
        in[14] = in[15] = 0;
        uint32_t v[16];
        std::memcpy(v, in, sizeof(v));
        for (int dr = 0; dr < 4; ++dr) {  // 4 double rounds = 8 rounds
            quarter(v[0], v[4], v[8], v[12]);
            quarter(v[1], v[5], v[9], v[13]);
            quarter(v[2], v[6], v[10], v[14]);
            quarter(v[3], v[7], v[11], v[15]);
            quarter(v[0], v[5], v[10], v[15]);
            quarter(v[1], v[6], v[11], v[12]);
            quarter(v[2], v[7], v[8], v[13]);
            quarter(v[3], v[4], v[9], v[14]);
        }
        for (int i = 0; i < 16; ++i) buf[i] = v[i] + in[i];
        ++block;
        have = 16;
    }
    uint32_t next_u32() {
        if (have == 0) refill();
        return buf[16 - have--];
    }
    uint64_t next_u64() {
        uint64_t lo = next_u32();
        uint64_t hi = next_u32();
        return lo | (hi << 32);
    }
};
}  // namespace

void rng_split(uint64_t key, int64_t n, uint64_t* out) {
    if (n <= 0) return;
    if (n == 1) {  // rng.rs:24-26: a single split returns the key itself
        out[0] = key;
        return;
    }
    ChaCha8Stream s(key);
    for (int64_t i = 0; i < n; ++i) out[i] = s.next_u64();
}

}  // namespace thrml

using namespace thrml;

extern "C" {

const char* thrml_last_error(void) { return g_last_error.c_str(); }
const char* thrml_version(void) { return "thrml_b200 0.1 (sm_100a)"; }

int32_t thrml_rng_split(uint64_t key, int64_t n, uint64_t* out) {
    if (n < 0) return fail(THRML_ERR_INVALID_ARG, "split count must be non-negative");
    if (n > 0 && !out) return fail(THRML_ERR_INVALID_ARG, "null output");
    rng_split(key, n, out);
    return THRML_OK;
}

// ---------------------------------------------------------------------------------------------------------
// Generators.
// ---------------------------------------------------------------------------------------------------------
int32_t thrml_lattice_edges(int64_t side_len, int32_t torus, int64_t* side_out, int64_t* n_edges_out, int64_t* edges_out,
                            int32_t* colour_out) {
    if (side_len <= 0) return fail(THRML_ERR_INVALID_ARG, "side_len must be positive");
    const int64_t L = (side_len + 1) / 2 * 2;  // graph_utils.rs:184
    // Visiting cells in row-major order and emitting (right, down) neighbours gives pairs that are already unique
    // except on a torus of side 2, so collect, sort by (min,max) and deduplicate.
    std::vector<std::pair<int64_t, int64_t>> e;
    e.reserve(static_cast<size_t>(2 * L * L));
    for (int64_t r = 0; r < L; ++r)
        for (int64_t c = 0; c < L; ++c) {
            const int64_t here = r * L + c;
            int64_t down = -1, right = -1;
            if (r + 1 < L) down = (r + 1) * L + c; else if (torus) down = c;
            if (c + 1 < L) right = r * L + c + 1; else if (torus) right = r * L;
            if (down >= 0) e.emplace_back(std::min(here, down), std::max(here, down));
            if (right >= 0) e.emplace_back(std::min(here, right), std::max(here, right));
        }
    std::sort(e.begin(), e.end());
    e.erase(std::unique(e.begin(), e.end()), e.end());
    if (side_out) *side_out = L;
    if (n_edges_out) *n_edges_out = static_cast<int64_t>(e.size());
    if (edges_out)
        for (size_t i = 0; i < e.size(); ++i) {
            edges_out[2 * i] = e[i].first;
            edges_out[2 * i + 1] = e[i].second;
        }
    if (colour_out)
        for (int64_t r = 0; r < L; ++r)
            for (int64_t c = 0; c < L; ++c) colour_out[r * L + c] = static_cast<int32_t>((r + c) & 1);
    return THRML_OK;
}

int32_t thrml_greedy_coloring(int64_t n_nodes, int64_t n_edges, const int64_t* edges, int32_t* colour_out, int32_t* n_colours_out) {
    if (n_nodes < 0 || n_edges < 0 || !colour_out || (n_edges > 0 && !edges)) return fail(THRML_ERR_INVALID_ARG, "bad colouring arguments");
    // CSR adjacency
    std::vector<int64_t> ptr(static_cast<size_t>(n_nodes) + 1, 0);
    for (int64_t e = 0; e < 2 * n_edges; ++e) {
        if (edges[e] < 0 || edges[e] >= n_nodes) return fail(THRML_ERR_INVALID_ARG, "edge endpoint out of range");
        ++ptr[edges[e] + 1];
    }
    std::partial_sum(ptr.begin(), ptr.end(), ptr.begin());
    std::vector<int64_t> adj(static_cast<size_t>(2 * n_edges)), fill(ptr.begin(), ptr.end() - 1);
    for (int64_t e = 0; e < n_edges; ++e) {
        adj[fill[edges[2 * e]]++] = edges[2 * e + 1];
        adj[fill[edges[2 * e + 1]]++] = edges[2 * e];
    }
    std::fill(colour_out, colour_out + n_nodes, -1);
    int32_t n_col = 0;
    std::vector<uint8_t> taken;
    for (int64_t v = 0; v < n_nodes; ++v) {  // node index order, lib.rs:117
        const int64_t deg = ptr[v + 1] - ptr[v];
        taken.assign(static_cast<size_t>(deg) + 2, 0);
        for (int64_t q = ptr[v]; q < ptr[v + 1]; ++q) {
            const int32_t c = colour_out[adj[q]];
            if (c >= 0 && c <= deg) taken[c] = 1;
        }
        int32_t c = 0;
        while (taken[c]) ++c;  // smallest colour no coloured neighbour uses, lib.rs:132-141
        colour_out[v] = c;
        n_col = std::max(n_col, c + 1);
    }
    if (n_colours_out) *n_colours_out = n_col;
    return THRML_OK;
}

// ---------------------------------------------------------------------------------------------------------
// Builder.
// ---------------------------------------------------------------------------------------------------------
static int32_t validate_block(const thrml_builder* b, const int64_t* nodes, int64_t n) {
    if (n <= 0 || !nodes) return fail(THRML_ERR_INVALID_ARG, "Block cannot be empty");  // block.rs:12-14
    const int64_t total = static_cast<int64_t>(b->kinds.size());
    for (int64_t i = 0; i < n; ++i)
        if (nodes[i] < 0 || nodes[i] >= total) return fail(THRML_ERR_INVALID_ARG, "node id out of range");
    const int32_t kind0 = b->kinds[nodes[0]];
    for (int64_t i = 1; i < n; ++i)
        if (b->kinds[nodes[i]] != kind0) return fail(THRML_ERR_INVALID_ARG, "All nodes in a block must be of the same type");  // block.rs:17-19
    return THRML_OK;
}

int32_t thrml_builder_create(const int32_t* kinds, int64_t n_nodes, const int32_t* dtype_order, int32_t n_dtype_order, thrml_builder** out) {
    if (!out || n_nodes < 0 || (n_nodes > 0 && !kinds) || n_dtype_order < 0 || (n_dtype_order > 0 && !dtype_order))
        return fail(THRML_ERR_INVALID_ARG, "bad builder arguments");
    for (int64_t i = 0; i < n_nodes; ++i)
        if (kinds[i] < 0 || kinds[i] > 255) return fail(THRML_ERR_INVALID_ARG, "node kind must be 0 (spin) or a category count 1..255");
    auto* b = new thrml_builder();
    b->kinds.assign(kinds, kinds + n_nodes);
    b->dtype_order.assign(dtype_order, dtype_order + n_dtype_order);
    *out = b;
    return THRML_OK;
}
void thrml_builder_destroy(thrml_builder* b) { delete b; }

int32_t thrml_builder_add_free_block(thrml_builder* b, const int64_t* nodes, int64_t n, int32_t superblock, int32_t sampler_kind) {
    if (!b) return fail(THRML_ERR_INVALID_ARG, "null builder");
    if (int32_t rc = validate_block(b, nodes, n)) return rc;
    if (!b->free_blocks.empty() && superblock < b->free_blocks.back().superblock)
        return fail(THRML_ERR_INVALID_ARG, "superblock ids must be non-decreasing");
    if (sampler_kind != THRML_SAMPLER_SPIN_GIBBS && sampler_kind != THRML_SAMPLER_CATEGORICAL_GIBBS && sampler_kind != THRML_SAMPLER_SOFTMAX)
        return fail(THRML_ERR_INVALID_ARG, "unknown sampler kind");
    BlockInfo bi;
    bi.nodes.assign(nodes, nodes + n);
    bi.kind = b->kinds[nodes[0]];
    bi.superblock = superblock;
    bi.sampler = sampler_kind;
    b->free_blocks.push_back(std::move(bi));
    b->compiled = false;
    return THRML_OK;
}
int32_t thrml_builder_add_clamped_block(thrml_builder* b, const int64_t* nodes, int64_t n) {
    if (!b) return fail(THRML_ERR_INVALID_ARG, "null builder");
    if (int32_t rc = validate_block(b, nodes, n)) return rc;
    BlockInfo bi;
    bi.nodes.assign(nodes, nodes + n);
    bi.kind = b->kinds[nodes[0]];
    b->clamped_blocks.push_back(std::move(bi));
    b->compiled = false;
    return THRML_OK;
}

int32_t thrml_builder_add_interaction_group(thrml_builder* b, const int64_t* head, int64_t rows, const int64_t* tails, int32_t n_tails,
                                            int32_t n_spin, const float* w, int32_t d1, int32_t d2) {
    if (!b) return fail(THRML_ERR_INVALID_ARG, "null builder");
    if (n_tails < 0 || d1 < 1 || d2 < 1 || !w) return fail(THRML_ERR_INVALID_ARG, "bad interaction group arguments");
    if (int32_t rc = validate_block(b, head, rows)) return rc;
    GroupDesc g;
    g.head.assign(head, head + rows);
    for (int32_t t = 0; t < n_tails; ++t) {
        // interaction.rs:156-162: tails have the head's length (guaranteed by the [n_tails][rows] layout) and are Blocks
        if (int32_t rc = validate_block(b, tails + static_cast<int64_t>(t) * rows, rows)) return rc;
        g.tails.emplace_back(tails + static_cast<int64_t>(t) * rows, tails + static_cast<int64_t>(t + 1) * rows);
    }
    if (n_spin < 0 || n_spin > n_tails) return fail(THRML_ERR_INVALID_ARG, "n_spin cannot exceed number of tail blocks");  // interaction.rs:171-173
    for (int32_t t = 0; t < n_tails; ++t) {
        const bool is_cat = b->kinds[g.tails[t][0]] != 0;
        if (is_cat != (t >= n_spin)) return fail(THRML_ERR_INVALID_ARG, "the first n_spin tail node blocks must be spin blocks and the rest categorical");
    }
    g.n_spin = n_spin;
    g.d1 = d1;
    g.d2 = d2;
    g.w.assign(w, w + rows * d1 * d2);
    b->groups.push_back(std::move(g));
    b->compiled = false;
    return THRML_OK;
}

int32_t thrml_builder_add_discrete_factor(thrml_builder* b, const int64_t* spin_groups, int32_t n_spin_groups, const int64_t* cat_groups,
                                          int32_t n_cat_groups, int64_t rows, const float* w, int32_t d1, int32_t d2, int32_t* n_groups_out) {
    if (!b) return fail(THRML_ERR_INVALID_ARG, "null builder");
    if (n_spin_groups < 0 || n_cat_groups < 0 || n_spin_groups + n_cat_groups == 0)
        return fail(THRML_ERR_INVALID_ARG, "At least one node group must be provided");  // discrete_ebm.rs:309-311
    if (!w || d1 < 1 || d2 < 1) return fail(THRML_ERR_INVALID_ARG, "The leading dimension of weights must have the same length as the number of nodes in each node group");
    auto grp = [rows](const int64_t* base, int32_t g) { return base + static_cast<int64_t>(g) * rows; };
    for (int32_t g = 0; g < n_spin_groups; ++g) {
        if (int32_t rc = validate_block(b, grp(spin_groups, g), rows)) return rc;
        if (b->kinds[grp(spin_groups, g)[0]] != 0) return fail(THRML_ERR_INVALID_ARG, "spin node group holds non-spin nodes");
    }
    for (int32_t g = 0; g < n_cat_groups; ++g) {
        if (int32_t rc = validate_block(b, grp(cat_groups, g), rows)) return rc;
        if (b->kinds[grp(cat_groups, g)[0]] == 0) return fail(THRML_ERR_INVALID_ARG, "categorical node group holds spin nodes");
    }
    // discrete_ebm.rs:330-351: trailing unit dimensions do not count; one dimension per categorical group is needed.
    const int32_t effective = d2 > 1 ? 2 : (d1 > 1 ? 1 : 0);
    if (effective < n_cat_groups)
        return fail(THRML_ERR_INVALID_ARG, "The shape of the weight tensor must be [b, x_1, ..., x_k], where k is the length of categorical_node_groups");
    if (n_cat_groups > 2) return fail(THRML_ERR_UNSUPPORTED, "rank-3 weights carry at most two categorical groups");
    const int64_t wlen = rows * d1 * d2;
    int32_t made = 0;
    const int32_t n_total = n_spin_groups + n_cat_groups;
    if (n_spin_groups > 0) {
        // discrete_ebm.rs:391-453: a single merged group; heads = every spin group in turn, tails = the other spin groups in
        // order followed by every categorical group; the weights are repeated once per head group.
        GroupDesc g;
        g.tails.assign(static_cast<size_t>(n_total - 1), {});
        for (auto& t : g.tails) t.reserve(static_cast<size_t>(rows) * n_spin_groups);
        g.head.reserve(static_cast<size_t>(rows) * n_spin_groups);
        g.w.reserve(static_cast<size_t>(wlen) * n_spin_groups);
        for (int32_t h = 0; h < n_spin_groups; ++h) {
            g.head.insert(g.head.end(), grp(spin_groups, h), grp(spin_groups, h) + rows);
            int32_t slot = 0;
            for (int32_t o = 0; o < n_spin_groups; ++o)
                if (o != h) {
                    g.tails[slot].insert(g.tails[slot].end(), grp(spin_groups, o), grp(spin_groups, o) + rows);
                    ++slot;
                }
            for (int32_t c = 0; c < n_cat_groups; ++c)
                g.tails[n_spin_groups - 1 + c].insert(g.tails[n_spin_groups - 1 + c].end(), grp(cat_groups, c), grp(cat_groups, c) + rows);
            g.w.insert(g.w.end(), w, w + wlen);
        }
        g.n_spin = n_spin_groups - 1;
        g.d1 = d1;
        g.d2 = d2;
        b->groups.push_back(std::move(g));
        ++made;
    }
    for (int32_t h = 0; h < n_cat_groups; ++h) {
        // discrete_ebm.rs:456-507: head = categorical group h, tails = all spin groups then the other categorical groups;
        // the head's category axis is moved to position 1 (a transpose of the two trailing axes when h == 1).
        GroupDesc g;
        g.head.assign(grp(cat_groups, h), grp(cat_groups, h) + rows);
        for (int32_t s = 0; s < n_spin_groups; ++s) g.tails.emplace_back(grp(spin_groups, s), grp(spin_groups, s) + rows);
        for (int32_t o = 0; o < n_cat_groups; ++o)
            if (o != h) g.tails.emplace_back(grp(cat_groups, o), grp(cat_groups, o) + rows);
        g.n_spin = n_spin_groups;
        if (n_cat_groups == 1 || h == 0) {
            g.d1 = d1;
            g.d2 = d2;
            g.w.assign(w, w + wlen);
        } else {
            g.d1 = d2;
            g.d2 = d1;
            g.w.resize(static_cast<size_t>(wlen));
            const int64_t plane = static_cast<int64_t>(d1) * d2;
            for (int64_t r = 0; r < rows; ++r) {
                const float* src = w + r * plane;
                float* dst = g.w.data() + r * plane;
                for (int32_t q = 0; q < d2; ++q)
                    for (int32_t p = 0; p < d1; ++p) dst[q * d1 + p] = src[p * d2 + q];
            }
        }
        b->groups.push_back(std::move(g));
        ++made;
    }
    if (n_groups_out) *n_groups_out = made;
    b->compiled = false;
    return THRML_OK;
}

int32_t thrml_builder_add_ising(thrml_builder* b, const int64_t* nodes, int64_t n_nodes, const float* biases, const int64_t* edges, int64_t n_edges,
                                const float* weights, float beta) {
    if (!b) return fail(THRML_ERR_INVALID_ARG, "null builder");
    if (n_nodes > 0) {  // ising.rs:109-122
        std::vector<float> scaled(static_cast<size_t>(n_nodes));
        for (int64_t i = 0; i < n_nodes; ++i) scaled[i] = beta * biases[i];
        if (int32_t rc = thrml_builder_add_discrete_factor(b, nodes, 1, nullptr, 0, n_nodes, scaled.data(), 1, 1, nullptr)) return rc;
    }
    if (n_edges > 0) {  // ising.rs:125-140
        std::vector<int64_t> ends(static_cast<size_t>(2 * n_edges));
        std::vector<float> scaled(static_cast<size_t>(n_edges));
        for (int64_t e = 0; e < n_edges; ++e) {
            ends[e] = edges[2 * e];
            ends[n_edges + e] = edges[2 * e + 1];
            scaled[e] = beta * weights[e];
        }
        if (int32_t rc = thrml_builder_add_discrete_factor(b, ends.data(), 2, nullptr, 0, n_edges, scaled.data(), 1, 1, nullptr)) return rc;
    }
    return THRML_OK;
}

}  // extern "C"

// BlockGibbsSpec::new + BlockSpec::new (program.rs:28-64, blockspec.rs:15-66): classes, sampling order, node positions and the
// checks that do not depend on the slot tables.  O(nodes) host work shared by the host and the device table compilers.
int32_t thrml::compile_layout(thrml_builder* b) {
    if (!b) return fail(THRML_ERR_INVALID_ARG, "null builder");
    b->compiled = false;
    // --- classes: distinct TensorSpecs of node_shape_dtypes, first-seen order (blockspec.rs:19-28).  Spin -> Bool scalar,
    //     any Categorical -> U8 scalar (node.rs:60-73), so there are at most two.
    b->sd_spin = b->sd_cat = -1;
    b->n_classes = 0;
    for (int32_t kind : b->dtype_order) {
        int32_t& slot = (kind == 0) ? b->sd_spin : b->sd_cat;
        if (slot < 0) slot = b->n_classes++;
    }
    auto kind_known = [&](int32_t kind) { return std::find(b->dtype_order.begin(), b->dtype_order.end(), kind) != b->dtype_order.end(); };
    // --- BlockGibbsSpec::new (program.rs:33-47): sampling order = runs of equal superblock id.
    b->sampling_order.clear();
    for (size_t i = 0; i < b->free_blocks.size(); ++i) {
        if (i == 0 || b->free_blocks[i].superblock != b->free_blocks[i - 1].superblock) b->sampling_order.emplace_back();
        b->sampling_order.back().push_back(static_cast<int32_t>(i));
    }
    // --- BlockSpec::new (blockspec.rs:30-57): positions = running offset per class over free ++ clamped.
    const int64_t n_nodes = static_cast<int64_t>(b->kinds.size());
    b->class_size.assign(static_cast<size_t>(b->n_classes), 0);
    b->loc_sd.assign(static_cast<size_t>(n_nodes), -1);
    b->loc_pos.assign(static_cast<size_t>(n_nodes), 0);
    auto place = [&](BlockInfo& blk) -> int32_t {
        if (blk.nodes.empty()) return fail(THRML_ERR_INVALID_ARG, "Encountered an empty block in BlockSpec");
        if (!kind_known(blk.kind)) return fail(THRML_ERR_INVALID_ARG, "Node type not found in node_shape_dtypes");
        blk.sd = blk.kind == 0 ? b->sd_spin : b->sd_cat;
        blk.offset = b->class_size[blk.sd];
        b->class_size[blk.sd] += static_cast<int64_t>(blk.nodes.size());
        int64_t pos = blk.offset;
        for (int64_t nd : blk.nodes) {
            if (b->loc_sd[nd] >= 0) return fail(THRML_ERR_INVALID_ARG, "Node appears twice in blocks");
            b->loc_sd[nd] = static_cast<int8_t>(blk.sd);
            b->loc_pos[nd] = pos++;
        }
        return THRML_OK;
    };
    for (auto& blk : b->free_blocks)
        if (int32_t rc = place(blk)) return rc;
    for (auto& blk : b->clamped_blocks)
        if (int32_t rc = place(blk)) return rc;
    for (auto& blk : b->free_blocks) {
        const bool ok = (blk.sampler == THRML_SAMPLER_SPIN_GIBBS && blk.kind == 0) ||
                        ((blk.sampler == THRML_SAMPLER_CATEGORICAL_GIBBS || blk.sampler == THRML_SAMPLER_SOFTMAX) && blk.kind > 0);
        if (!ok) return fail(THRML_ERR_UNSUPPORTED, "sampler kind does not match the block's node type");
    }
    for (int64_t v : b->class_size)
        if (v > 0x7fffffffLL) return fail(THRML_ERR_UNSUPPORTED, "more than 2^31-1 nodes in one state class");
    // --- tails must live in the global state (program.rs:175-179 -> get_node_locations panics otherwise)
    for (const GroupDesc& g : b->groups)
        for (const auto& tail : g.tails)
            for (int64_t nd : tail)
                if (b->loc_sd[nd] < 0) return fail(THRML_ERR_INVALID_ARG, "Node not found in global location map");
    return THRML_OK;
}

extern "C" {

int32_t thrml_builder_compile(thrml_builder* b) {
    if (int32_t rc = thrml::compile_layout(b)) return rc;
    const int64_t n_nodes = static_cast<int64_t>(b->kinds.size());
    // --- head_node_map (program.rs:101-108) as a CSR over nodes: entries (group, row), ordered by group then row.
    std::vector<int64_t> hptr(static_cast<size_t>(n_nodes) + 1, 0);
    for (const GroupDesc& g : b->groups)
        for (int64_t nd : g.head) ++hptr[nd + 1];
    std::partial_sum(hptr.begin(), hptr.end(), hptr.begin());
    std::vector<int32_t> h_group(static_cast<size_t>(hptr.back()));
    std::vector<int64_t> h_row(static_cast<size_t>(hptr.back()));
    {
        std::vector<int64_t> cur(hptr.begin(), hptr.end() - 1);
        for (size_t gi = 0; gi < b->groups.size(); ++gi) {
            const auto& head = b->groups[gi].head;
            for (size_t r = 0; r < head.size(); ++r) {
                const int64_t at = cur[head[r]]++;
                h_group[at] = static_cast<int32_t>(gi);
                h_row[at] = static_cast<int64_t>(r);
            }
        }
    }
    // --- per free block: slot counts, then the tables (program.rs:114-134, 159-300).
    const size_t n_groups = b->groups.size();
    b->tables.assign(b->free_blocks.size(), {});
    std::vector<int32_t> kmax(n_groups), table_of(n_groups);
    for (size_t bi = 0; bi < b->free_blocks.size(); ++bi) {
        const BlockInfo& blk = b->free_blocks[bi];
        const size_t n = blk.nodes.size();
        std::fill(kmax.begin(), kmax.end(), 0);
        for (int64_t nd : blk.nodes) {
            int64_t q = hptr[nd];
            while (q < hptr[nd + 1]) {  // entries of one node are grouped by interaction group
                const int32_t g = h_group[q];
                int32_t cnt = 0;
                while (q < hptr[nd + 1] && h_group[q] == g) { ++cnt; ++q; }
                kmax[g] = std::max(kmax[g], cnt);
            }
        }
        auto& tabs = b->tables[bi];
        for (size_t gi = 0; gi < n_groups; ++gi) {
            table_of[gi] = -1;
            if (kmax[gi] == 0) continue;  // program.rs:166
            const GroupDesc& g = b->groups[gi];
            if (g.head.size() > 0x7fffffffULL) return fail(THRML_ERR_UNSUPPORTED, "interaction group with more than 2^31-1 rows");
            SlotTable t;
            t.k = kmax[gi];
            t.wdim = g.d1 * g.d2;
            t.n_spin = g.n_spin;
            t.source_group = static_cast<int32_t>(gi);
            const size_t nk = n * static_cast<size_t>(t.k);
            t.rows.assign(nk, 0);
            t.active.assign(nk, 0);
            t.w.assign(nk * t.wdim, 0.0f);
            t.idx.assign(g.tails.size(), std::vector<int32_t>(nk, 0));
            for (const auto& tail : g.tails) {
                const int32_t kind = b->kinds[tail[0]];
                t.tail_sd.push_back(kind == 0 ? b->sd_spin : b->sd_cat);
                t.tail_is_cat.push_back(kind != 0);
            }
            table_of[gi] = static_cast<int32_t>(tabs.size());
            tabs.push_back(std::move(t));
        }
        for (size_t j = 0; j < n; ++j) {
            const int64_t nd = blk.nodes[j];
            int64_t q = hptr[nd];
            while (q < hptr[nd + 1]) {
                const int32_t gi = h_group[q];
                SlotTable& t = tabs[table_of[gi]];
                const GroupDesc& g = b->groups[gi];
                int32_t slot = 0;
                for (; q < hptr[nd + 1] && h_group[q] == gi; ++q, ++slot) {
                    const size_t at = j * static_cast<size_t>(t.k) + slot;
                    const int64_t row = h_row[q];
                    t.rows[at] = static_cast<int32_t>(row);
                    t.active[at] = 1;
                    for (size_t tl = 0; tl < g.tails.size(); ++tl) t.idx[tl][at] = static_cast<int32_t>(b->loc_pos[g.tails[tl][row]]);
                }
            }
        }
        // weights: every slot (padded ones included, which point at row 0) copies its row — program.rs:216-235
        for (SlotTable& t : tabs) {
            const GroupDesc& g = b->groups[t.source_group];
            const size_t nk = n * static_cast<size_t>(t.k);
            if (t.wdim == 1) {
                for (size_t s = 0; s < nk; ++s) t.w[s] = g.w[t.rows[s]];
            } else {
                for (size_t s = 0; s < nk; ++s) std::memcpy(&t.w[s * t.wdim], &g.w[static_cast<size_t>(t.rows[s]) * t.wdim], sizeof(float) * t.wdim);
            }
        }
    }
    b->compiled = true;
    return THRML_OK;
}

// ---------------------------------------------------------------------------------------------------------
// Introspection.
// ---------------------------------------------------------------------------------------------------------
int32_t thrml_builder_counts(const thrml_builder* b, int32_t* n_free, int32_t* n_clamped, int32_t* n_groups_total, int32_t* n_classes) {
    if (!b) return fail(THRML_ERR_INVALID_ARG, "null builder");
    if (n_free) *n_free = static_cast<int32_t>(b->free_blocks.size());
    if (n_clamped) *n_clamped = static_cast<int32_t>(b->clamped_blocks.size());
    if (n_groups_total) *n_groups_total = static_cast<int32_t>(b->groups.size());
    if (n_classes) *n_classes = b->n_classes;
    return THRML_OK;
}
int32_t thrml_builder_node_location(const thrml_builder* b, int64_t node, int32_t* sd_index, int64_t* position) {
    if (!b || !b->compiled) return fail(THRML_ERR_INVALID_ARG, "builder is not compiled");
    if (node < 0 || node >= static_cast<int64_t>(b->kinds.size()) || b->loc_sd[node] < 0)
        return fail(THRML_ERR_INVALID_ARG, "Node not found in global location map");
    if (sd_index) *sd_index = b->loc_sd[node];
    if (position) *position = b->loc_pos[node];
    return THRML_OK;
}
int32_t thrml_builder_group_shape(const thrml_builder* b, int32_t g, int64_t* rows, int32_t* n_tails, int32_t* n_spin, int32_t* d1, int32_t* d2) {
    if (!b || g < 0 || g >= static_cast<int32_t>(b->groups.size())) return fail(THRML_ERR_INVALID_ARG, "group index out of range");
    const GroupDesc& G = b->groups[g];
    if (rows) *rows = static_cast<int64_t>(G.head.size());
    if (n_tails) *n_tails = static_cast<int32_t>(G.tails.size());
    if (n_spin) *n_spin = G.n_spin;
    if (d1) *d1 = G.d1;
    if (d2) *d2 = G.d2;
    return THRML_OK;
}
int32_t thrml_builder_group_data(const thrml_builder* b, int32_t g, int64_t* head, int64_t* tails, float* w) {
    if (!b || g < 0 || g >= static_cast<int32_t>(b->groups.size())) return fail(THRML_ERR_INVALID_ARG, "group index out of range");
    const GroupDesc& G = b->groups[g];
    const size_t rows = G.head.size();
    if (head) std::copy(G.head.begin(), G.head.end(), head);
    if (tails)
        for (size_t t = 0; t < G.tails.size(); ++t) std::copy(G.tails[t].begin(), G.tails[t].end(), tails + t * rows);
    if (w) std::copy(G.w.begin(), G.w.end(), w);
    return THRML_OK;
}
int32_t thrml_builder_block_tables(const thrml_builder* b, int32_t block, int32_t* n_tables, int64_t* n_nodes) {
    if (!b || !b->compiled) return fail(THRML_ERR_INVALID_ARG, "builder is not compiled");
    if (block < 0 || block >= static_cast<int32_t>(b->free_blocks.size())) return fail(THRML_ERR_INVALID_ARG, "block index out of range");
    if (n_tables) *n_tables = static_cast<int32_t>(b->tables[block].size());
    if (n_nodes) *n_nodes = static_cast<int64_t>(b->free_blocks[block].nodes.size());
    return THRML_OK;
}
static const SlotTable* find_table(const thrml_builder* b, int32_t block, int32_t t) {
    if (!b || !b->compiled || block < 0 || block >= static_cast<int32_t>(b->free_blocks.size())) return nullptr;
    if (t < 0 || t >= static_cast<int32_t>(b->tables[block].size())) return nullptr;
    return &b->tables[block][t];
}
int32_t thrml_builder_table_shape(const thrml_builder* b, int32_t block, int32_t t, int32_t* k, int32_t* wdim, int32_t* n_spin, int32_t* n_tails,
                                  int32_t* source_group) {
    const SlotTable* T = find_table(b, block, t);
    if (!T) return fail(THRML_ERR_INVALID_ARG, "table index out of range");
    if (k) *k = T->k;
    if (wdim) *wdim = T->wdim;
    if (n_spin) *n_spin = T->n_spin;
    if (n_tails) *n_tails = static_cast<int32_t>(T->idx.size());
    if (source_group) *source_group = T->source_group;
    return THRML_OK;
}
int32_t thrml_builder_table_data(const thrml_builder* b, int32_t block, int32_t t, int32_t* rows, uint8_t* active, float* w, int32_t* idx,
                                 int32_t* tail_sd) {
    const SlotTable* T = find_table(b, block, t);
    if (!T) return fail(THRML_ERR_INVALID_ARG, "table index out of range");
    const size_t nk = T->rows.size();
    if (rows) std::copy(T->rows.begin(), T->rows.end(), rows);
    if (active) std::copy(T->active.begin(), T->active.end(), active);
    if (w) std::copy(T->w.begin(), T->w.end(), w);
    if (idx)
        for (size_t tl = 0; tl < T->idx.size(); ++tl) std::copy(T->idx[tl].begin(), T->idx[tl].end(), idx + tl * nk);
    if (tail_sd) std::copy(T->tail_sd.begin(), T->tail_sd.end(), tail_sd);
    return THRML_OK;
}

}  // extern "C"
