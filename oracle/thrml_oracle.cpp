// thrml_oracle.cpp — CPU restatement of thrml-rs's block-Gibbs sampling path.
//
// TEST INFRASTRUCTURE ONLY.  This file is the checker the CUDA library is compared against (and the timed
// CPU baseline of the benchmark).  Nothing in the product may include, link or call it.
//
// It follows the reference's own Rust code, keeping its data representation: one f32 per node and chain
// (spins 0.0/1.0, categories as f32 indices), materialised [n,k] neighbour gathers, per-sample moment loop.
// Each function cites the reference file:line it restates (paths relative to the thrml-rs repository).
//
// Parity status.  Pinned by the reference's own known-answer tests: BlockSpec positions, spin_product,
// batch_gather, lattice edge counts, greedy colouring, categorical_sample with +-10 logits (see
// tests/test_oracle_kat.py for the list with file:line).  PARITY UNPINNED: the values RngKey::split returns
// (rand_chacha 0.3.1 ChaCha8Rng + rand_core 0.6.4 seed_from_u64 are third-party crates whose sources are not
// in the reference tree and no reference test fixes a value; the restatement below follows their published
// algorithms and is checked against the ChaCha8 zero-key keystream) and the random stream itself (the
// reference draws from Burn's global Tensor::random and never consumes an RngKey, so no reference test fixes a
// draw).  Draws are therefore compared either with injected noise or through this file's own counter-based
// stream, which is the engine's documented key -> noise mapping.
#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <map>
#include <string>
#include <thread>
#include <unordered_map>
#include <vector>

#define ORC_API extern "C" __attribute__((visibility("default")))

static thread_local std::string g_err;
static int fail(const std::string& m) {
    g_err = m;
    return -1;
}
ORC_API const char* orc_last_error() { return g_err.c_str(); }

// ------------------------------------------------------------------------------------------------
// RngKey::split — crates/thrml-samplers/src/rng.rs:19-51.
// ChaCha8Rng::seed_from_u64 (rand_core 0.6.4): the u64 is expanded to a 32-byte key with PCG32
// (multiplier 6364136223846793005, increment 11634580027462260723, XSH-RR output, state advanced before each
// output).  rand_chacha 0.3.1: ChaCha, 8 rounds, 64-bit block counter in words 12-13 starting at 0, stream id 0
// in words 14-15; next_u64 = two consecutive little-endian u32 words of the keystream, low word first.
// ------------------------------------------------------------------------------------------------
static inline uint32_t rotl32(uint32_t x, int r) { return (x << r) | (x >> (32 - r)); }
static inline uint32_t rotr32(uint32_t x, unsigned r) { r &= 31; return r ? ((x >> r) | (x << (32 - r))) : x; }

static void chacha_block(const uint32_t key[8], uint64_t counter, uint64_t stream, int rounds, uint32_t out[16]) {
    uint32_t s[16] = {0x61707865u, 0x3320646eu, 0x79622d32u, 0x6b206574u,
                      key[0], key[1], key[2], key[3], key[4], key[5], key[6], key[7],
                      (uint32_t)counter, (uint32_t)(counter >> 32), (uint32_t)stream, (uint32_t)(stream >> 32)};
    uint32_t x[16];
    memcpy(x, s, sizeof(x));
#define QR(a, b, c, d)                     \
    x[a] += x[b]; x[d] = rotl32(x[d] ^ x[a], 16); \
    x[c] += x[d]; x[b] = rotl32(x[b] ^ x[c], 12); \
    x[a] += x[b]; x[d] = rotl32(x[d] ^ x[a], 8);  \
    x[c] += x[d]; x[b] = rotl32(x[b] ^ x[c], 7);
    for (int i = 0; i < rounds; i += 2) {
        QR(0, 4, 8, 12) QR(1, 5, 9, 13) QR(2, 6, 10, 14) QR(3, 7, 11, 15)
        QR(0, 5, 10, 15) QR(1, 6, 11, 12) QR(2, 7, 8, 13) QR(3, 4, 9, 14)
    }
#undef QR
    for (int i = 0; i < 16; i++) out[i] = x[i] + s[i];
}

ORC_API void orc_chacha_block(const uint32_t* key8, uint64_t counter, uint64_t stream, int rounds, uint32_t* out16) {
    chacha_block(key8, counter, stream, rounds, out16);
}

static void seed_from_u64(uint64_t state, uint32_t key[8]) {
    const uint64_t MUL = 6364136223846793005ull, INC = 11634580027462260723ull;
    for (int i = 0; i < 8; i++) {
        state = state * MUL + INC;
        uint32_t xorshifted = (uint32_t)(((state >> 18) ^ state) >> 27);
        uint32_t rot = (uint32_t)(state >> 59);
        key[i] = rotr32(xorshifted, rot);
    }
}

ORC_API void orc_rng_split(uint64_t key, int64_t n, uint64_t* out) {
    if (n <= 0) return;
    if (n == 1) { out[0] = key; return; }  // rng.rs:24-26
    uint32_t k[8];
    seed_from_u64(key, k);
    uint32_t blk[16];
    uint64_t ctr = 0;
    int pos = 16;
    for (int64_t i = 0; i < n; i++) {
        uint32_t w[2];
        for (int j = 0; j < 2; j++) {
            if (pos == 16) { chacha_block(k, ctr++, 0, 8, blk); pos = 0; }
            w[j] = blk[pos++];
        }
        out[i] = (uint64_t)w[0] | ((uint64_t)w[1] << 32);
    }
}

// ------------------------------------------------------------------------------------------------
// The engine's key -> noise mapping (no reference counterpart: the reference never consumes its keys).
// Philox4x32-10 (Salmon et al. 2011), key = the block's RngKey, counter = (node in block, chain index, lane, tag).
// ------------------------------------------------------------------------------------------------
static const uint32_t TAG_SPIN = 0x5350494Eu, TAG_CAT = 0x43415447u, TAG_HINT = 0x48494E54u, TAG_RAND = 0x52414E44u;

static inline void philox4x32_10(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3, uint32_t k0, uint32_t k1, uint32_t out[4]) {
    for (int r = 0; r < 10; r++) {
        uint64_t p0 = (uint64_t)0xD2511F53u * c0, p1 = (uint64_t)0xCD9E8D57u * c2;
        uint32_t n0 = (uint32_t)(p1 >> 32) ^ c1 ^ k0, n1 = (uint32_t)p1, n2 = (uint32_t)(p0 >> 32) ^ c3 ^ k1, n3 = (uint32_t)p0;
        c0 = n0; c1 = n1; c2 = n2; c3 = n3;
        k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
    }
    out[0] = c0; out[1] = c1; out[2] = c2; out[3] = c3;
}
ORC_API void orc_philox(const uint32_t* ctr4, const uint32_t* key2, uint32_t* out4) {
    philox4x32_10(ctr4[0], ctr4[1], ctr4[2], ctr4[3], key2[0], key2[1], out4);
}
static inline float u24(uint32_t r) { return (float)(r >> 8) * 5.9604644775390625e-8f; }             // [0,1)
static inline float u23_open(uint32_t r) { return ((float)(r >> 9) + 0.5f) * 1.1920928955078125e-7f; }  // (0,1)

// Deterministic f32 exp / sigmoid / log: fixed sequences of IEEE-754 single operations (fmaf, *, +, /), so the
// same bits come out of any conforming CPU or GPU.  Checked against libm in tests/test_oracle_kat.py.
static inline float det_exp_nonpos(float t) {  // t <= 0
    if (t < -86.0f) return 0.0f;
    float n = rintf(t * 1.44269504088896341f);
    float r = fmaf(n, -0.693359375f, t);
    r = fmaf(n, 2.12194440e-4f, r);
    float z = r * r;
    float y = 1.9875691500e-4f;
    y = fmaf(y, r, 1.3981999507e-3f);
    y = fmaf(y, r, 8.3334519073e-3f);
    y = fmaf(y, r, 4.1665795894e-2f);
    y = fmaf(y, r, 1.6666665459e-1f);
    y = fmaf(y, r, 5.0000001201e-1f);
    y = fmaf(y, z, r);
    y = y + 1.0f;
    int32_t e = (int32_t)n + 127;  // n in [-124, 0]
    uint32_t bits = (uint32_t)e << 23;
    float s;
    memcpy(&s, &bits, 4);
    return y * s;
}
static inline float det_sigmoid(float x) {
    if (x >= 0.0f) {
        float e = det_exp_nonpos(-x);
        return 1.0f / (1.0f + e);
    }
    float e = det_exp_nonpos(x);
    return e / (1.0f + e);
}
static inline float det_log(float x) {  // x > 0, normal
    uint32_t bits;
    memcpy(&bits, &x, 4);
    int32_t e = (int32_t)((bits >> 23) & 0xff) - 126;
    bits = (bits & 0x007fffffu) | 0x3f000000u;  // mantissa in [0.5, 1)
    float m;
    memcpy(&m, &bits, 4);
    if (m < 0.707106781186547524f) { e -= 1; m = m + m; }
    float f = m - 1.0f;
    float z = f * f;
    float y = 7.0376836292e-2f;
    y = fmaf(y, f, -1.1514610310e-1f);
    y = fmaf(y, f, 1.1676998740e-1f);
    y = fmaf(y, f, -1.2420140846e-1f);
    y = fmaf(y, f, 1.4249322787e-1f);
    y = fmaf(y, f, -1.6668057665e-1f);
    y = fmaf(y, f, 2.0000714765e-1f);
    y = fmaf(y, f, -2.4999993993e-1f);
    y = fmaf(y, f, 3.3333331174e-1f);
    y = y * f;
    y = y * z;
    float fe = (float)e;
    y = fmaf(fe, -2.12194440e-4f, y);
    y = fmaf(z, -0.5f, y);
    float r = f + y;
    r = fmaf(fe, 0.693359375f, r);
    return r;
}
ORC_API float orc_det_sigmoid(float x) { return det_sigmoid(x); }
ORC_API float orc_det_log(float x) { return det_log(x); }
ORC_API float orc_u24(uint32_t r) { return u24(r); }
ORC_API float orc_u23_open(uint32_t r) { return u23_open(r); }

// ------------------------------------------------------------------------------------------------
// Model description and index compilation.
// ------------------------------------------------------------------------------------------------
struct Group {  // InteractionGroup, crates/thrml-core/src/interaction.rs:107-125
    std::vector<int64_t> head;
    std::vector<std::vector<int64_t>> tails;
    int n_spin = 0;
    int d1 = 1, d2 = 1;
    std::vector<float> w;  // [rows][d1][d2]
};
struct Table {  // one (block, group) entry of BlockSamplingProgram, program.rs:70-85
    int k = 0, wdim = 1, n_spin = 0, source_group = 0;
    std::vector<int32_t> rows;              // interaction_slices [n*k]
    std::vector<uint8_t> active;            // [n*k]
    std::vector<float> w;                   // [n*k*wdim]
    std::vector<std::vector<int32_t>> idx;  // per tail [n*k] global positions
    std::vector<int> tail_sd;               // class of each tail
};
struct Model {
    std::vector<int32_t> kinds;
    std::vector<int32_t> dtype_order;
    std::vector<std::vector<int64_t>> free_blocks, clamped_blocks;
    std::vector<int> superblock_of, sampler_of;
    std::vector<Group> groups;
    // compiled
    bool compiled = false;
    int n_classes = 0;
    std::vector<int> class_of_block;                              // over free ++ clamped
    std::vector<int64_t> block_offset;                            // start position in its class
    std::vector<int64_t> class_size;
    std::unordered_map<int64_t, std::pair<int, int64_t>> loc;      // node -> (sd index, position)
    std::vector<std::vector<int>> sampling_order;
    std::vector<std::vector<Table>> tables;                       // per free block
};

static int spec_of_kind(int kind) { return kind == 0 ? 0 : 1; }  // TensorSpec::for_spin (Bool) / for_categorical (U8), node.rs:60-73

ORC_API int orc_model_create(const int32_t* kinds, int64_t n, const int32_t* dtype_order, int32_t n_order, Model** out) {
    Model* m = new Model();
    m->kinds.assign(kinds, kinds + n);
    m->dtype_order.assign(dtype_order, dtype_order + n_order);
    *out = m;
    return 0;
}
ORC_API void orc_model_destroy(Model* m) { delete m; }

// Block::new — crates/thrml-core/src/block.rs:11-27
static int check_block(const Model* m, const int64_t* nodes, int64_t n) {
    if (n <= 0) return fail("Block cannot be empty");
    for (int64_t i = 0; i < n; i++)
        if (nodes[i] < 0 || nodes[i] >= (int64_t)m->kinds.size()) return fail("node id out of range");
    for (int64_t i = 1; i < n; i++)
        if (m->kinds[nodes[i]] != m->kinds[nodes[0]]) return fail("All nodes in a block must be of the same type");
    return 0;
}
ORC_API int orc_model_add_free_block(Model* m, const int64_t* nodes, int64_t n, int32_t superblock, int32_t sampler) {
    if (check_block(m, nodes, n)) return -1;
    m->free_blocks.emplace_back(nodes, nodes + n);
    m->superblock_of.push_back(superblock);
    m->sampler_of.push_back(sampler);
    return 0;
}
ORC_API int orc_model_add_clamped_block(Model* m, const int64_t* nodes, int64_t n) {
    if (check_block(m, nodes, n)) return -1;
    m->clamped_blocks.emplace_back(nodes, nodes + n);
    return 0;
}
// InteractionGroup::with_data — interaction.rs:148-181
ORC_API int orc_model_add_group(Model* m, const int64_t* head, int64_t rows, const int64_t* tails, int32_t n_tails,
                                int32_t n_spin, const float* w, int32_t d1, int32_t d2) {
    if (check_block(m, head, rows)) return -1;
    Group g;
    g.head.assign(head, head + rows);
    for (int t = 0; t < n_tails; t++) {
        if (check_block(m, tails + (int64_t)t * rows, rows)) return -1;
        g.tails.emplace_back(tails + (int64_t)t * rows, tails + (int64_t)(t + 1) * rows);
    }
    if (n_spin > n_tails) return fail("n_spin cannot exceed number of tail blocks");
    g.n_spin = n_spin;
    g.d1 = d1;
    g.d2 = d2;
    g.w.assign(w, w + rows * d1 * d2);
    m->groups.push_back(std::move(g));
    return 0;
}

// DiscreteEBMFactor::to_interaction_groups — crates/thrml-models/src/discrete_ebm.rs:379-510.
ORC_API int orc_model_add_discrete_factor(Model* m, const int64_t* spin_groups, int32_t n_spin, const int64_t* cat_groups,
                                          int32_t n_cat, int64_t rows, const float* w, int32_t d1, int32_t d2, int32_t* n_out) {
    // DiscreteEBMFactor::new validation — discrete_ebm.rs:301-355
    if (n_spin + n_cat == 0) return fail("At least one node group must be provided");
    for (int g = 0; g < n_spin; g++)
        if (check_block(m, spin_groups + (int64_t)g * rows, rows)) return -1;
    for (int g = 0; g < n_cat; g++)
        if (check_block(m, cat_groups + (int64_t)g * rows, rows)) return -1;
    int eff = 3;
    if (d2 == 1) { eff = 2; if (d1 == 1) eff = 1; }
    if (eff < 1 + n_cat) return fail("The shape of the weight tensor must be [b, x_1, ..., x_k]");
    int n_total = n_spin + n_cat, made = 0;
    int64_t wsz = rows * d1 * d2;
    if (n_spin > 0) {  // one merged group, every spin group takes a turn as head (:391-453)
        Group g;
        g.tails.resize(n_total - 1);
        for (int h = 0; h < n_spin; h++) {
            g.head.insert(g.head.end(), spin_groups + (int64_t)h * rows, spin_groups + (int64_t)(h + 1) * rows);
            int ti = 0;
            for (int o = 0; o < n_spin; o++) {
                if (o == h) continue;
                g.tails[ti].insert(g.tails[ti].end(), spin_groups + (int64_t)o * rows, spin_groups + (int64_t)(o + 1) * rows);
                ti++;
            }
            for (int j = 0; j < n_cat; j++)
                g.tails[n_spin - 1 + j].insert(g.tails[n_spin - 1 + j].end(), cat_groups + (int64_t)j * rows,
                                               cat_groups + (int64_t)(j + 1) * rows);
            g.w.insert(g.w.end(), w, w + wsz);  // weights tiled n_spin times (:428-438)
        }
        g.n_spin = n_spin - 1;  // :448
        g.d1 = d1;
        g.d2 = d2;
        m->groups.push_back(std::move(g));
        made++;
    }
    for (int h = 0; h < n_cat; h++) {  // one group per categorical head (:456-507)
        Group g;
        g.head.assign(cat_groups + (int64_t)h * rows, cat_groups + (int64_t)(h + 1) * rows);
        for (int s = 0; s < n_spin; s++) g.tails.emplace_back(spin_groups + (int64_t)s * rows, spin_groups + (int64_t)(s + 1) * rows);
        for (int o = 0; o < n_cat; o++)
            if (o != h) g.tails.emplace_back(cat_groups + (int64_t)o * rows, cat_groups + (int64_t)(o + 1) * rows);
        g.n_spin = n_spin;
        if (n_cat == 1 || h == 0) {  // :482-490, :534-537
            g.d1 = d1; g.d2 = d2;
            g.w.assign(w, w + wsz);
        } else {  // swap_dims(1,2), :538-541
            g.d1 = d2; g.d2 = d1;
            g.w.resize(wsz);
            for (int64_t r = 0; r < rows; r++)
                for (int a = 0; a < d1; a++)
                    for (int b = 0; b < d2; b++) g.w[(r * d2 + b) * d1 + a] = w[(r * d1 + a) * d2 + b];
        }
        m->groups.push_back(std::move(g));
        made++;
    }
    if (n_out) *n_out = made;
    return 0;
}

// IsingEBM::get_factors — crates/thrml-models/src/ising.rs:105-143 (bias factor, then edge factor; beta scales both).
ORC_API int orc_model_add_ising(Model* m, const int64_t* nodes, int64_t n_nodes, const float* b, const int64_t* edges,
                                int64_t n_edges, const float* J, float beta) {
    if (n_nodes > 0) {
        std::vector<float> w(n_nodes);
        for (int64_t i = 0; i < n_nodes; i++) w[i] = beta * b[i];
        if (orc_model_add_discrete_factor(m, nodes, 1, nullptr, 0, n_nodes, w.data(), 1, 1, nullptr)) return -1;
    }
    if (n_edges > 0) {
        std::vector<int64_t> sg(2 * n_edges);
        std::vector<float> w(n_edges);
        for (int64_t e = 0; e < n_edges; e++) {
            sg[e] = edges[2 * e];
            sg[n_edges + e] = edges[2 * e + 1];
            w[e] = beta * J[e];
        }
        if (orc_model_add_discrete_factor(m, sg.data(), 2, nullptr, 0, n_edges, w.data(), 1, 1, nullptr)) return -1;
    }
    return 0;
}

// BlockGibbsSpec::new (program.rs:28-64) + BlockSpec::new (blockspec.rs:15-66) + BlockSamplingProgram::new (program.rs:88-318)
ORC_API int orc_model_compile(Model* m) {
    // classes = unique TensorSpecs in node_shape_dtypes order (blockspec.rs:19-28)
    std::vector<int> sd_of_spec(2, -1);
    m->n_classes = 0;
    for (int kind : m->dtype_order) {
        int sp = spec_of_kind(kind);
        if (sd_of_spec[sp] < 0) sd_of_spec[sp] = m->n_classes++;
    }
    m->sampling_order.clear();
    int last_sb = -1;
    for (size_t i = 0; i < m->free_blocks.size(); i++) {
        if (m->sampling_order.empty() || m->superblock_of[i] != last_sb) m->sampling_order.emplace_back();
        m->sampling_order.back().push_back((int)i);
        last_sb = m->superblock_of[i];
    }
    std::vector<const std::vector<int64_t>*> all;
    for (auto& b : m->free_blocks) all.push_back(&b);
    for (auto& b : m->clamped_blocks) all.push_back(&b);
    m->class_size.assign(m->n_classes, 0);
    m->class_of_block.clear();
    m->block_offset.clear();
    m->loc.clear();
    for (auto* blk : all) {
        if (blk->empty()) return fail("Encountered an empty block in BlockSpec");
        int kind = m->kinds[(*blk)[0]];
        bool known = false;
        for (int k : m->dtype_order) known |= (k == kind);
        if (!known) return fail("Node type not found in node_shape_dtypes");
        int sd = sd_of_spec[spec_of_kind(kind)];
        int64_t start = m->class_size[sd];
        m->class_size[sd] += (int64_t)blk->size();
        m->class_of_block.push_back(sd);
        m->block_offset.push_back(start);
        for (size_t k = 0; k < blk->size(); k++) {
            if (m->loc.count((*blk)[k])) return fail("Node appears twice in blocks");
            m->loc[(*blk)[k]] = {sd, start + (int64_t)k};
        }
    }
    if (m->sampler_of.size() != m->free_blocks.size()) return fail("Number of samplers must match number of free blocks");
    // head_node_map (program.rs:101-108)
    std::unordered_map<int64_t, std::vector<std::pair<int, int64_t>>> head_map;
    for (size_t gi = 0; gi < m->groups.size(); gi++)
        for (size_t j = 0; j < m->groups[gi].head.size(); j++) head_map[m->groups[gi].head[j]].push_back({(int)gi, (int64_t)j});
    m->tables.clear();
    for (auto& block : m->free_blocks) {
        size_t n = block.size();
        std::vector<std::vector<std::vector<int64_t>>> info(m->groups.size(), std::vector<std::vector<int64_t>>(n));
        for (size_t j = 0; j < n; j++) {
            auto it = head_map.find(block[j]);
            if (it == head_map.end()) continue;
            for (auto& pr : it->second) info[pr.first][j].push_back(pr.second);
        }
        std::vector<Table> tabs;
        for (size_t gi = 0; gi < m->groups.size(); gi++) {
            size_t k = 0;
            for (auto& v : info[gi]) k = std::max(k, v.size());
            if (k == 0) continue;  // program.rs:166
            const Group& g = m->groups[gi];
            Table t;
            t.k = (int)k;
            t.wdim = g.d1 * g.d2;
            t.n_spin = g.n_spin;
            t.source_group = (int)gi;
            t.rows.assign(n * k, 0);
            t.active.assign(n * k, 0);
            t.idx.assign(g.tails.size(), std::vector<int32_t>(n * k, 0));
            for (auto& tail : g.tails) {  // get_node_locations(tail_block), program.rs:175-179
                for (int64_t nd : tail)
                    if (!m->loc.count(nd)) return fail("Node not found in global location map");
                t.tail_sd.push_back(sd_of_spec[spec_of_kind(m->kinds[tail[0]])]);
            }
            for (size_t i = 0; i < n; i++)
                for (size_t j = 0; j < info[gi][i].size(); j++) {
                    int64_t row = info[gi][i][j];
                    t.rows[i * k + j] = (int32_t)row;
                    t.active[i * k + j] = 1;
                    for (size_t tl = 0; tl < g.tails.size(); tl++) t.idx[tl][i * k + j] = (int32_t)m->loc[g.tails[tl][row]].second;
                }
            t.w.resize(n * k * t.wdim);  // select(0, flat_indices) + reshape, program.rs:216-235
            for (size_t s = 0; s < n * k; s++)
                for (int d = 0; d < t.wdim; d++) t.w[s * t.wdim + d] = g.w[(size_t)t.rows[s] * t.wdim + d];
            tabs.push_back(std::move(t));
        }
        m->tables.push_back(std::move(tabs));
    }
    m->compiled = true;
    return 0;
}

ORC_API int orc_model_counts(const Model* m, int32_t* n_free, int32_t* n_clamped, int32_t* n_groups, int32_t* n_classes) {
    if (n_free) *n_free = (int)m->free_blocks.size();
    if (n_clamped) *n_clamped = (int)m->clamped_blocks.size();
    if (n_groups) *n_groups = (int)m->groups.size();
    if (n_classes) *n_classes = m->n_classes;
    return 0;
}
ORC_API int orc_model_node_location(const Model* m, int64_t node, int32_t* sd, int64_t* pos) {
    auto it = m->loc.find(node);
    if (it == m->loc.end()) return fail("Node not found in global location map");
    *sd = it->second.first;
    *pos = it->second.second;
    return 0;
}
ORC_API int orc_model_group_shape(const Model* m, int32_t g, int64_t* rows, int32_t* n_tails, int32_t* n_spin, int32_t* d1, int32_t* d2) {
    if (g < 0 || g >= (int)m->groups.size()) return fail("group index out of range");
    const Group& G = m->groups[g];
    *rows = (int64_t)G.head.size(); *n_tails = (int)G.tails.size(); *n_spin = G.n_spin; *d1 = G.d1; *d2 = G.d2;
    return 0;
}
ORC_API int orc_model_group_data(const Model* m, int32_t g, int64_t* head, int64_t* tails, float* w) {
    const Group& G = m->groups[g];
    size_t rows = G.head.size();
    if (head) memcpy(head, G.head.data(), rows * 8);
    if (tails) for (size_t t = 0; t < G.tails.size(); t++) memcpy(tails + t * rows, G.tails[t].data(), rows * 8);
    if (w) memcpy(w, G.w.data(), G.w.size() * 4);
    return 0;
}
ORC_API int orc_model_block_tables(const Model* m, int32_t block, int32_t* n_tables, int64_t* n_nodes) {
    if (!m->compiled || block < 0 || block >= (int)m->tables.size()) return fail("block index out of range");
    *n_tables = (int)m->tables[block].size();
    *n_nodes = (int64_t)m->free_blocks[block].size();
    return 0;
}
ORC_API int orc_model_table_shape(const Model* m, int32_t block, int32_t t, int32_t* k, int32_t* wdim, int32_t* n_spin,
                                  int32_t* n_tails, int32_t* source_group) {
    const Table& T = m->tables[block][t];
    *k = T.k; *wdim = T.wdim; *n_spin = T.n_spin; *n_tails = (int)T.idx.size(); *source_group = T.source_group;
    return 0;
}
ORC_API int orc_model_table_data(const Model* m, int32_t block, int32_t t, int32_t* rows, uint8_t* active, float* w,
                                 int32_t* idx, int32_t* tail_sd) {
    const Table& T = m->tables[block][t];
    size_t nk = T.rows.size();
    if (rows) memcpy(rows, T.rows.data(), nk * 4);
    if (active) memcpy(active, T.active.data(), nk);
    if (w) memcpy(w, T.w.data(), T.w.size() * 4);
    if (idx) for (size_t tl = 0; tl < T.idx.size(); tl++) memcpy(idx + tl * nk, T.idx[tl].data(), nk * 4);
    if (tail_sd) for (size_t tl = 0; tl < T.tail_sd.size(); tl++) tail_sd[tl] = T.tail_sd[tl];
    return 0;
}

// ------------------------------------------------------------------------------------------------
// Small reference operators pinned by the reference's own known-answer tests.
// ------------------------------------------------------------------------------------------------
// spin_product — discrete_ebm.rs:54-77 (empty list -> [1.0]).  vals[n_lists][n] as 0/1.
ORC_API int64_t orc_spin_product(const uint8_t* vals, int32_t n_lists, int64_t n, float* out) {
    if (n_lists == 0) { out[0] = 1.0f; return 1; }
    for (int64_t i = 0; i < n; i++) {
        float p = 1.0f;
        for (int l = 0; l < n_lists; l++) p *= (float)vals[(int64_t)l * n + i] * 2.0f - 1.0f;
        out[i] = p;
    }
    return n;
}
// batch_gather — discrete_ebm.rs:98-193: out[b] = W[b, idx0[b], idx1[b], ...], strides from trailing dims.
ORC_API int orc_batch_gather(const float* w, int64_t batch, const int32_t* dims, int32_t n_dims, const int32_t* idx /*[n_dims][batch]*/, float* out) {
    int64_t bstride = 1;
    for (int d = 0; d < n_dims; d++) bstride *= dims[d];
    for (int64_t b = 0; b < batch; b++) {
        int64_t lin = b * bstride, stride = bstride;
        for (int d = 0; d < n_dims; d++) {
            stride /= dims[d];
            lin += (int64_t)idx[(int64_t)d * batch + b] * stride;
        }
        out[b] = w[lin];
    }
    return 0;
}
// batch_gather_fused with explicit strides — crates/thrml-kernels/src/batch_gather/kernel.rs:38-62,256-280:
// out[b] = W_flat[b*batch_stride + sum_i idx[b][i]*stride_i]; an index that leaves the tensor yields 0 here.
ORC_API int orc_batch_gather_strided(const float* w, int64_t w_len, int64_t batch, int32_t n_idx, const int32_t* idx /*[batch][n_idx]*/, const int64_t* strides,
                                     int64_t batch_stride, float* out) {
    for (int64_t b = 0; b < batch; b++) {
        int64_t lin = b * batch_stride;
        for (int i = 0; i < n_idx; i++) lin += (int64_t)idx[b * n_idx + i] * strides[i];
        out[b] = (lin >= 0 && lin < w_len) ? w[lin] : 0.0f;
    }
    return 0;
}
// make_nearest_neighbor_lattice — graph_utils.rs:177-243 (edge order canonicalised to ascending (min,max)).
ORC_API int orc_lattice_edges(int64_t side_len, int32_t torus, int64_t* side_out, int64_t* n_edges_out, int64_t* edges_out, int32_t* colour_out) {
    if (side_len <= 0) return fail("side_len must be positive");
    int64_t side = (side_len + 1) / 2 * 2;
    std::vector<std::pair<int64_t, int64_t>> es;
    for (int64_t idx = 0; idx < side * side; idx++) {
        int64_t i = idx / side, j = idx % side;
        const int64_t jumps[2][2] = {{1, 0}, {0, 1}};
        for (auto& d : jumps) {
            int64_t ti = i + d[0], tj = j + d[1];
            if (torus) { ti = ((ti % side) + side) % side; tj = ((tj % side) + side) % side; }
            else if (ti < 0 || ti >= side || tj < 0 || tj >= side) continue;
            int64_t t = ti * side + tj;
            es.push_back({std::min(idx, t), std::max(idx, t)});
        }
    }
    std::sort(es.begin(), es.end());
    es.erase(std::unique(es.begin(), es.end()), es.end());  // the reference's HashSet
    *side_out = side;
    *n_edges_out = (int64_t)es.size();
    if (edges_out) for (size_t e = 0; e < es.size(); e++) { edges_out[2 * e] = es[e].first; edges_out[2 * e + 1] = es[e].second; }
    if (colour_out) for (int64_t idx = 0; idx < side * side; idx++) colour_out[idx] = (int32_t)(((idx / side) + (idx % side)) % 2);
    return 0;
}
// greedy_coloring — crates/thrml-examples/src/lib.rs:114-147.
ORC_API int orc_greedy_coloring(int64_t n, int64_t n_edges, const int64_t* edges, int32_t* colour, int32_t* n_colours) {
    std::vector<std::vector<int64_t>> adj(n);
    for (int64_t e = 0; e < n_edges; e++) { adj[edges[2 * e]].push_back(edges[2 * e + 1]); adj[edges[2 * e + 1]].push_back(edges[2 * e]); }
    std::vector<int32_t> col(n, -1);
    int32_t mx = 0;
    for (int64_t v = 0; v < n; v++) {
        std::vector<int32_t> used;
        for (int64_t u : adj[v]) if (col[u] >= 0) used.push_back(col[u]);
        std::sort(used.begin(), used.end());
        int32_t c = 0;
        for (int32_t nc : used) { if (nc == c) c++; else if (nc > c) break; }
        col[v] = c;
        mx = std::max(mx, c + 1);
    }
    memcpy(colour, col.data(), n * 4);
    if (n_colours) *n_colours = mx;
    return 0;
}
// categorical_sample on given logits/uniforms — softmax.rs:60-97 with the tie rule of gumbel_argmax/kernel.rs:75-84.
ORC_API int orc_categorical_sample(const float* logits, const float* u, int64_t n, int32_t K, float* out, int32_t use_libm) {
    for (int64_t i = 0; i < n; i++) {
        float best = 0; int bi = 0;
        for (int c = 0; c < K; c++) {
            float uu = u[i * K + c];
            float g = use_libm ? -logf(-logf(uu)) : -det_log(-det_log(uu));
            float p = logits[i * K + c] + g;
            if (c == 0 || p > best) { best = p; bi = c; }
        }
        out[i] = (float)bi;
    }
    return 0;
}
// sigmoid-Bernoulli on given gamma/uniforms — spin_gibbs.rs:94-97 (inclusive=1: u <= p) / sigmoid_bernoulli/kernel.rs:46-54 (u < p).
ORC_API int orc_sigmoid_bernoulli(const float* gamma, const float* u, int64_t n, float* out, int32_t inclusive) {
    for (int64_t i = 0; i < n; i++) {
        float p = det_sigmoid(gamma[i] * 2.0f);
        out[i] = inclusive ? (u[i] <= p ? 1.0f : 0.0f) : (u[i] < p ? 1.0f : 0.0f);
    }
    return 0;
}

// ------------------------------------------------------------------------------------------------
// State and the sampling step.
// ------------------------------------------------------------------------------------------------
struct OState {
    Model* m;
    int64_t n_chains, chain_offset;
    int threads = 1;
    int spin_noise = 0;  // 0: one 32-bit word per (spin, chain); 1: the packed mapping of the implicit lattice engine
    int cat_noise = 0;   // 0: word k & 3 of Philox(n, c, k >> 2); 1: word c & 3 of Philox(n, c >> 2, k) (the implicit Potts engine's)
    std::vector<std::vector<std::vector<float>>> g;  // [chain][class][position], f32 as in the reference
};
ORC_API int orc_state_create(Model* m, int64_t n_chains, int64_t chain_offset, OState** out) {
    if (!m->compiled) return fail("model not compiled");
    OState* s = new OState();
    s->m = m; s->n_chains = n_chains; s->chain_offset = chain_offset;
    s->g.resize(n_chains);
    for (auto& c : s->g) { c.resize(m->n_classes); for (int k = 0; k < m->n_classes; k++) c[k].assign(m->class_size[k], 0.0f); }
    *out = s;
    return 0;
}
ORC_API void orc_state_destroy(OState* s) { delete s; }
ORC_API void orc_state_set_threads(OState* s, int32_t t) { s->threads = t < 1 ? 1 : t; }
// The reference never consumes its RngKey (spin_gibbs.rs:61,82-83), so the key -> noise mapping belongs to the engine under
// test.  Mapping 1 restates the implicit lattice engine's bit-sliced mapping: for spin n (index in its block) and global
// chain c, bit b of the draw's top byte is bit (n & 31) of word (b & 3) of Philox(n >> 5, c, 1 + (b >> 2), TAG_SPIN), and
// the low 24 bits are those of word (c & 3) of Philox(n, c >> 2, 3, TAG_SPIN); the uniform is the draw's top 24 bits, as
// for mapping 0.  Mapping 2 restates the dense (tensor-core) path's mapping: top 16 bits = half (n & 1) of word ((n >> 1) & 3) of
// Philox(n >> 3, c, 1, TAG_SPIN), low 16 bits = low half of word (c & 3) of Philox(n, c >> 2, 2, TAG_SPIN).
ORC_API void orc_state_set_spin_noise(OState* s, int32_t mapping) { s->spin_noise = mapping; }
// Categorical blocks: mapping 1 restates the implicit Potts engine's own mapping — the Gumbel uniform of (node n, chain c,
// category k) is word (c & 3) of Philox(n, c >> 2, k, TAG_CAT).
ORC_API void orc_state_set_cat_noise(OState* s, int32_t mapping) { s->cat_noise = mapping; }
static const std::vector<int64_t>& block_nodes(const Model* m, int b) {
    return b < (int)m->free_blocks.size() ? m->free_blocks[b] : m->clamped_blocks[b - m->free_blocks.size()];
}
ORC_API int orc_state_set_block(OState* s, int32_t block, const float* host /*[chain][node]*/) {
    const Model* m = s->m;
    int64_t n = (int64_t)block_nodes(m, block).size(), off = m->block_offset[block];
    int cls = m->class_of_block[block];
    for (int64_t c = 0; c < s->n_chains; c++) memcpy(&s->g[c][cls][off], host + c * n, n * 4);
    return 0;
}
ORC_API int orc_state_get_block(const OState* s, int32_t block, float* host) {
    const Model* m = s->m;
    int64_t n = (int64_t)block_nodes(m, block).size(), off = m->block_offset[block];
    int cls = m->class_of_block[block];
    for (int64_t c = 0; c < s->n_chains; c++) memcpy(host + c * n, &s->g[c][cls][off], n * 4);
    return 0;
}

template <class F>
static void par_chains(const OState* s, F f) {
    int T = (int)std::min<int64_t>(s->threads, s->n_chains);
    if (T <= 1) { for (int64_t c = 0; c < s->n_chains; c++) f(c); return; }
    std::atomic<int64_t> next(0);
    std::vector<std::thread> th;
    for (int t = 0; t < T; t++) th.emplace_back([&]() { for (;;) { int64_t c = next.fetch_add(1); if (c >= s->n_chains) break; f(c); } });
    for (auto& x : th) x.join();
}

// Oracle A — compute_parameters_cpu_f64, spin_gibbs.rs:384-505 (f64, inactive slots skipped).
static void spin_field_f64(const Model* m, const std::vector<std::vector<float>>& g, int block, std::vector<double>& gamma) {
    size_t n = m->free_blocks[block].size();
    gamma.assign(n, 0.0);
    for (const Table& T : m->tables[block]) {
        size_t n_tails = T.idx.size();
        for (size_t i = 0; i < n; i++)
            for (int j = 0; j < T.k; j++) {
                size_t flat = i * T.k + j;
                if (!T.active[flat]) continue;
                double sp = 1.0;
                for (int t = 0; t < T.n_spin; t++) sp *= std::fma(2.0, (double)g[T.tail_sd[t]][T.idx[t][flat]], -1.0);
                double wv;
                if ((int)n_tails == T.n_spin) wv = T.w[flat * T.wdim];
                else {
                    size_t cat = (size_t)g[T.tail_sd[T.n_spin]][T.idx[T.n_spin][flat]];
                    size_t wi = flat * T.wdim + cat;
                    wv = wi < T.w.size() ? T.w[wi] : 0.0;
                }
                gamma[i] += wv * 1.0 * sp;
            }
    }
}
// Oracle B — compute_parameters, spin_gibbs.rs:512-611 in f32, following the op sequence: gather neighbour states to
// [n,k] (program.rs:343-365), spin_prod = prod(2s-1) (:618-637), weights (squeeze or gather by first categorical tail,
// :552-578), contribution = W*active*spin_prod, sum over slots (left to right), gamma += sum.
static void spin_field_f32(const Model* m, const std::vector<std::vector<float>>& g, int block, std::vector<float>& gamma,
                           std::vector<float>& scratch) {
    size_t n = m->free_blocks[block].size();
    gamma.assign(n, 0.0f);
    for (const Table& T : m->tables[block]) {
        size_t n_tails = T.idx.size(), nk = n * T.k;
        scratch.resize(nk * (n_tails + 1));
        float* nb = scratch.data();            // materialised neighbour states [tail][n*k]
        float* contrib = nb + nk * n_tails;    // [n*k]
        for (size_t t = 0; t < n_tails; t++) {
            const std::vector<float>& src = g[T.tail_sd[t]];
            const int32_t* ix = T.idx[t].data();
            for (size_t f = 0; f < nk; f++) nb[t * nk + f] = src[ix[f]];
        }
        for (size_t f = 0; f < nk; f++) {
            float sp = 1.0f;
            for (int t = 0; t < T.n_spin; t++) sp *= nb[t * nk + f] * 2.0f - 1.0f;
            float wv = ((int)n_tails == T.n_spin) ? T.w[f * T.wdim] : T.w[f * T.wdim + (size_t)nb[(size_t)T.n_spin * nk + f]];
            contrib[f] = wv * (float)T.active[f] * sp;
        }
        for (size_t i = 0; i < n; i++) {
            float sum = 0.0f;
            for (int j = 0; j < T.k; j++) sum += contrib[i * T.k + j];
            gamma[i] = gamma[i] + sum;
        }
    }
}
// CategoricalGibbsConditional::compute_parameters — softmax.rs:586-709 (f32 path; W[n,k,own,neighbour], first categorical tail only).
static int cat_field_f32(const Model* m, const std::vector<std::vector<float>>& g, int block, int K, std::vector<float>& theta) {
    size_t n = m->free_blocks[block].size();
    theta.assign(n * K, 0.0f);
    for (const Table& T : m->tables[block]) {
        size_t n_tails = T.idx.size();
        bool has_cat = (int)n_tails > T.n_spin;
        if (T.wdim != (has_cat ? K * K : K)) return fail("categorical weights must be [n,k,K] or [n,k,K*K]");
        for (size_t i = 0; i < n; i++) {
            for (int c = 0; c < K; c++) {
                float sum = 0.0f;
                for (int j = 0; j < T.k; j++) {
                    size_t f = i * T.k + j;
                    float sp = 1.0f;
                    for (int t = 0; t < T.n_spin; t++) sp *= g[T.tail_sd[t]][T.idx[t][f]] * 2.0f - 1.0f;
                    float wv;
                    if (has_cat) {
                        int x = (int)g[T.tail_sd[T.n_spin]][T.idx[T.n_spin][f]];
                        wv = T.w[f * T.wdim + (size_t)c * K + x];
                    } else wv = T.w[f * T.wdim + c];
                    sum += sp * wv * (float)T.active[f];
                }
                theta[i * K + c] += sum;
            }
        }
    }
    return 0;
}

// SoftmaxConditional::compute_parameters — softmax.rs:147-222: theta = sum over the interactions whose weights carry one
// entry per category (dims[2] == n_categories, others are skipped, :183-187) of sum_slots W * active; neighbour states
// are not read.
static void softmax_field_f32(const Model* m, int block, int K, std::vector<float>& theta) {
    size_t n = m->free_blocks[block].size();
    theta.assign(n * K, 0.0f);
    for (const Table& T : m->tables[block]) {
        if (T.wdim != K) continue;
        for (size_t i = 0; i < n; i++)
            for (int c = 0; c < K; c++) {
                float sum = 0.0f;
                for (int j = 0; j < T.k; j++) {
                    size_t f = i * T.k + j;
                    sum += T.w[f * T.wdim + c] * (float)T.active[f];
                }
                theta[i * K + c] += sum;
            }
    }
}
static int cat_or_softmax_field(const Model* m, const std::vector<std::vector<float>>& g, int block, int K, std::vector<float>& theta) {
    if (m->sampler_of[block] == 2) { softmax_field_f32(m, block, K, theta); return 0; }
    return cat_field_f32(m, g, block, K, theta);
}

ORC_API int orc_fields(OState* s, int32_t block, double* out64, float* out32) {
    const Model* m = s->m;
    size_t n = m->free_blocks[block].size();
    int kind = m->kinds[m->free_blocks[block][0]];
    if (m->sampler_of[block] == 0) {
        for (int64_t c = 0; c < s->n_chains; c++) {
            std::vector<double> g64; std::vector<float> g32, scr;
            if (out64) { spin_field_f64(m, s->g[c], block, g64); memcpy(out64 + c * n, g64.data(), n * 8); }
            if (out32) { spin_field_f32(m, s->g[c], block, g32, scr); memcpy(out32 + c * n, g32.data(), n * 4); }
        }
    } else {
        for (int64_t c = 0; c < s->n_chains; c++) {
            std::vector<float> th;
            if (cat_or_softmax_field(m, s->g[c], block, kind, th)) return -1;
            if (out32) memcpy(out32 + c * n * kind, th.data(), n * kind * 4);
            if (out64) for (size_t i = 0; i < n * kind; i++) out64[c * n * kind + i] = th[i];
        }
    }
    return 0;
}

struct Noise { const float* u; int64_t len; int64_t pos; };

// One block update for all chains: program.rs:324-393 -> sampler.  new_state[chain][node].
static int update_block(OState* s, int block, uint64_t key, Noise* inj, std::vector<std::vector<float>>& new_state) {
    const Model* m = s->m;
    size_t n = m->free_blocks[block].size();
    int kind = m->kinds[m->free_blocks[block][0]];
    uint32_t k0 = (uint32_t)key, k1 = (uint32_t)(key >> 32);
    int64_t C = s->n_chains;
    new_state.assign(C, {});
    int err = 0;
    if (m->sampler_of[block] == 0) {
        if (kind != 0) return fail("spin sampler on a non-spin block");
        const float* u_inj = nullptr;
        if (inj) { if (inj->pos + (int64_t)n * C > inj->len) return fail("injected noise too short"); u_inj = inj->u + inj->pos; inj->pos += (int64_t)n * C; }
        par_chains(s, [&](int64_t c) {
            std::vector<float> gamma, scr;
            spin_field_f32(m, s->g[c], block, gamma, scr);
            uint64_t gc = (uint64_t)(s->chain_offset + c);
            std::vector<float>& out = new_state[c];
            out.resize(n);
            for (size_t i = 0; i < n; i++) {
                float u;
                if (u_inj) u = u_inj[i * C + c];
                else if (s->spin_noise == 1) {
                    uint32_t pl[8], lo[4];
                    philox4x32_10((uint32_t)(i >> 5), (uint32_t)gc, 1, TAG_SPIN, k0, k1, pl);
                    philox4x32_10((uint32_t)(i >> 5), (uint32_t)gc, 2, TAG_SPIN, k0, k1, pl + 4);
                    philox4x32_10((uint32_t)i, (uint32_t)(gc >> 2), 3, TAG_SPIN, k0, k1, lo);
                    uint32_t top = 0;
                    for (int b = 0; b < 8; b++) top |= ((pl[b] >> (i & 31)) & 1u) << b;
                    u = u24((top << 24) | (lo[gc & 3] & 0xffffffu));
                }
                else if (s->spin_noise == 2) {
                    uint32_t tp[4], lo[4];
                    philox4x32_10((uint32_t)(i >> 3), (uint32_t)gc, 1, TAG_SPIN, k0, k1, tp);
                    philox4x32_10((uint32_t)i, (uint32_t)(gc >> 2), 2, TAG_SPIN, k0, k1, lo);
                    uint32_t top = (tp[(i >> 1) & 3] >> (16 * (i & 1))) & 0xffffu;
                    u = u24((top << 16) | (lo[gc & 3] & 0xffffu));
                }
                else { uint32_t r[4]; philox4x32_10((uint32_t)i, (uint32_t)(gc >> 2), 0, TAG_SPIN, k0, k1, r); u = u24(r[gc & 3]); }
                float p = det_sigmoid(gamma[i] * 2.0f);  // spin_gibbs.rs:95
                out[i] = (u <= p) ? 1.0f : 0.0f;          // spin_gibbs.rs:97
            }
        });
    } else {
        int K = kind;
        if (K < 1) return fail("categorical sampler on a spin block");
        const float* u_inj = nullptr;
        if (inj) { if (inj->pos + (int64_t)n * K * C > inj->len) return fail("injected noise too short"); u_inj = inj->u + inj->pos; inj->pos += (int64_t)n * K * C; }
        std::atomic<int> bad(0);
        par_chains(s, [&](int64_t c) {
            std::vector<float> theta;
            if (cat_or_softmax_field(m, s->g[c], block, K, theta)) { bad = 1; return; }
            uint64_t gc = (uint64_t)(s->chain_offset + c);
            std::vector<float>& out = new_state[c];
            out.resize(n);
            for (size_t i = 0; i < n; i++) {
                float best = 0; int bi = 0; uint32_t r[4] = {0, 0, 0, 0};
                for (int k = 0; k < K; k++) {
                    float u;
                    if (u_inj) u = u_inj[(i * K + k) * C + c];
                    else if (s->cat_noise == 1) { philox4x32_10((uint32_t)i, (uint32_t)(gc >> 2), (uint32_t)k, TAG_CAT, k0, k1, r); u = u23_open(r[gc & 3]); }
                    else { if ((k & 3) == 0) philox4x32_10((uint32_t)i, (uint32_t)gc, (uint32_t)(k >> 2), TAG_CAT, k0, k1, r); u = u23_open(r[k & 3]); }
                    float gmb = -det_log(-det_log(u));  // softmax.rs:84
                    float p = theta[i * K + k] + gmb;
                    if (k == 0 || p > best) { best = p; bi = k; }  // first maximum wins, gumbel_argmax/kernel.rs:81-83
                }
                out[i] = (float)bi;
            }
        });
        err = bad;
    }
    return err ? -1 : 0;
}

// sample_blocks — sampling.rs:28-63
static int sample_blocks(OState* s, uint64_t key, Noise* inj) {
    const Model* m = s->m;
    size_t nb = m->free_blocks.size();
    std::vector<uint64_t> keys(nb);
    orc_rng_split(key, (int64_t)nb, keys.data());
    for (auto& group : m->sampling_order) {
        std::vector<std::vector<std::vector<float>>> upd(group.size());
        for (size_t gi = 0; gi < group.size(); gi++)
            if (update_block(s, group[gi], keys[group[gi]], inj, upd[gi])) return -1;
        for (size_t gi = 0; gi < group.size(); gi++) {  // written back together, sampling.rs:57-59
            int b = group[gi];
            int cls = m->class_of_block[b];
            int64_t off = m->block_offset[b];
            for (int64_t c = 0; c < s->n_chains; c++) memcpy(&s->g[c][cls][off], upd[gi][c].data(), upd[gi][c].size() * 4);
        }
    }
    return 0;
}
// run_blocks — sampling.rs:81-106
static int run_blocks(OState* s, uint64_t key, int64_t n_iters, Noise* inj) {
    if (n_iters <= 0) return 0;
    std::vector<uint64_t> keys(n_iters);
    orc_rng_split(key, n_iters, keys.data());
    for (uint64_t k : keys)
        if (sample_blocks(s, k, inj)) return -1;
    return 0;
}
// sample_single_block — program.rs:324-393: one free block, written back immediately.
ORC_API int orc_sample_single_block(OState* s, int32_t block, uint64_t key) {
    const Model* m = s->m;
    if (block < 0 || block >= (int)m->free_blocks.size()) return fail("block index out of range");
    std::vector<std::vector<float>> upd;
    if (update_block(s, block, key, nullptr, upd)) return -1;
    int cls = m->class_of_block[block];
    int64_t off = m->block_offset[block];
    for (int64_t c = 0; c < s->n_chains; c++) memcpy(&s->g[c][cls][off], upd[c].data(), upd[c].size() * 4);
    return 0;
}
ORC_API int orc_sample_blocks(OState* s, uint64_t key, const float* inj_u, int64_t inj_len) {
    Noise nz{inj_u, inj_len, 0};
    return sample_blocks(s, key, inj_u ? &nz : nullptr);
}
ORC_API int orc_run_blocks(OState* s, uint64_t key, int64_t n_iters, const float* inj_u, int64_t inj_len) {
    Noise nz{inj_u, inj_len, 0};
    return run_blocks(s, key, n_iters, inj_u ? &nz : nullptr);
}

// hinton_init — ising.rs:602-673: p = sigmoid(beta*b) (:650), s = (u <= p) (:667); keys = key.split(n_blocks) (:618, unused by the
// reference; here they key the engine's stream).  inj_u layout [block][chain][node].
ORC_API int orc_hinton_init(OState* s, const int32_t* blocks, int32_t n_blocks, const float* biases, float beta, uint64_t key, const float* inj_u) {
    const Model* m = s->m;
    std::vector<uint64_t> keys(n_blocks);
    orc_rng_split(key, n_blocks, keys.data());
    int64_t boff = 0, uoff = 0;
    for (int bi = 0; bi < n_blocks; bi++) {
        int b = blocks[bi];
        int64_t n = (int64_t)block_nodes(m, b).size(), off = m->block_offset[b];
        int cls = m->class_of_block[b];
        uint32_t k0 = (uint32_t)keys[bi], k1 = (uint32_t)(keys[bi] >> 32);
        for (int64_t c = 0; c < s->n_chains; c++) {
            uint64_t gc = (uint64_t)(s->chain_offset + c);
            for (int64_t i = 0; i < n; i++) {
                float p = det_sigmoid(biases[boff + i] * beta);
                float u;
                if (inj_u) u = inj_u[uoff + c * n + i];
                else { uint32_t r[4]; philox4x32_10((uint32_t)i, (uint32_t)(gc >> 2), 0, TAG_HINT, k0, k1, r); u = u24(r[gc & 3]); }
                s->g[c][cls][off + i] = (u <= p) ? 1.0f : 0.0f;
            }
        }
        boff += n;
        uoff += n * s->n_chains;
    }
    return 0;
}
// Uniform random start (engine convenience; no reference counterpart): spins = top bit, categories = floor(u*K).
ORC_API int orc_state_randomize(OState* s, uint64_t key) {
    const Model* m = s->m;
    size_t nb = m->free_blocks.size();
    std::vector<uint64_t> keys(nb);
    orc_rng_split(key, (int64_t)nb, keys.data());
    for (size_t b = 0; b < nb; b++) {
        int64_t n = (int64_t)m->free_blocks[b].size(), off = m->block_offset[b];
        int cls = m->class_of_block[b], kind = m->kinds[m->free_blocks[b][0]];
        uint32_t k0 = (uint32_t)keys[b], k1 = (uint32_t)(keys[b] >> 32);
        for (int64_t c = 0; c < s->n_chains; c++) {
            uint64_t gc = (uint64_t)(s->chain_offset + c);
            for (int64_t i = 0; i < n; i++) {
                uint32_t r[4];
                philox4x32_10((uint32_t)i, (uint32_t)(gc >> 2), 0, TAG_RAND, k0, k1, r);
                uint32_t x = r[gc & 3];
                s->g[c][cls][off + i] = kind == 0 ? (float)(x >> 31) : (float)(((uint64_t)(x >> 8) * (uint64_t)kind) >> 24);
            }
        }
    }
    return 0;
}

// ------------------------------------------------------------------------------------------------
// Observers.
// ------------------------------------------------------------------------------------------------
struct OMoments {  // MomentAccumulatorObserver, moment.rs:29-121
    Model* m;
    std::vector<int64_t> rows_per_type, row_ptr, members;
    std::vector<int32_t> mem_sd;
    std::vector<int64_t> mem_pos;
    bool spin_transform;
    std::vector<int64_t> sums;  // all types concatenated
    int64_t n_obs = 0;
};
ORC_API int orc_moments_create(Model* m, int32_t n_types, const int64_t* rows_per_type, const int64_t* row_ptr, const int64_t* members,
                               int32_t transform_to_spin, OMoments** out) {
    OMoments* o = new OMoments();
    o->m = m;
    o->rows_per_type.assign(rows_per_type, rows_per_type + n_types);
    int64_t rows = 0;
    for (int t = 0; t < n_types; t++) rows += rows_per_type[t];
    o->row_ptr.assign(row_ptr, row_ptr + rows + 1);
    o->members.assign(members, members + row_ptr[rows]);
    for (int64_t nd : o->members) {
        auto it = m->loc.find(nd);
        if (it == m->loc.end()) { delete o; return fail("Node not found in global location map"); }
        o->mem_sd.push_back(it->second.first);
        o->mem_pos.push_back(it->second.second);
    }
    o->spin_transform = transform_to_spin != 0;
    o->sums.assign(rows, 0);
    *out = o;
    return 0;
}
ORC_API void orc_moments_destroy(OMoments* o) { delete o; }
// observe — moment.rs:157-237: product of f(x) over each row's members, added to the running sums.
ORC_API int orc_moments_observe(OMoments* o, const OState* s) {
    size_t rows = o->sums.size();
    for (int64_t c = 0; c < s->n_chains; c++)
        for (size_t r = 0; r < rows; r++) {
            float prod = 1.0f;
            for (int64_t q = o->row_ptr[r]; q < o->row_ptr[r + 1]; q++) {
                float x = s->g[c][o->mem_sd[q]][o->mem_pos[q]];
                prod *= o->spin_transform ? x * 2.0f - 1.0f : x;
            }
            o->sums[r] += (int64_t)prod;
        }
    o->n_obs += s->n_chains;
    return 0;
}
ORC_API int orc_moments_read(const OMoments* o, int32_t type, int64_t* sums_out, int64_t* n_obs) {
    int64_t start = 0;
    for (int t = 0; t < type; t++) start += o->rows_per_type[t];
    memcpy(sums_out, o->sums.data() + start, o->rows_per_type[type] * 8);
    if (n_obs) *n_obs = o->n_obs;
    return 0;
}

static void observe_states(const OState* s, const int32_t* obs_blocks, int32_t n_obs_blocks, uint8_t* dst) {
    const Model* m = s->m;  // StateObserver::observe, state_observer.rs:25-47; layout [observed node][chain]
    int64_t row = 0;
    for (int b = 0; b < n_obs_blocks; b++) {
        int blk = obs_blocks[b];
        int64_t n = (int64_t)block_nodes(m, blk).size(), off = m->block_offset[blk];
        int cls = m->class_of_block[blk];
        for (int64_t i = 0; i < n; i++, row++)
            for (int64_t c = 0; c < s->n_chains; c++) dst[row * s->n_chains + c] = (uint8_t)s->g[c][cls][off + i];
    }
}
// sample_with_observation — sampling.rs:178-320.
ORC_API int orc_sample_with_observation(OState* s, uint64_t key, int64_t n_warmup, int64_t n_samples, int64_t steps_per_sample, OMoments* mom,
                                        const int32_t* obs_blocks, int32_t n_obs_blocks, uint8_t* obs_out, const float* inj_u, int64_t inj_len) {
    Noise nz{inj_u, inj_len, 0};
    Noise* inj = inj_u ? &nz : nullptr;
    uint64_t two[2];
    orc_rng_split(key, 2, two);  // split_two, sampling.rs:189
    if (run_blocks(s, two[0], n_warmup, inj)) return -1;
    int64_t obs_rows = 0;
    for (int b = 0; b < n_obs_blocks; b++) obs_rows += (int64_t)block_nodes(s->m, obs_blocks[b]).size();
    int64_t stride = obs_rows * s->n_chains;
    if (mom) orc_moments_observe(mom, s);
    if (obs_out) observe_states(s, obs_blocks, n_obs_blocks, obs_out);
    if (n_samples <= 1) return 0;  // sampling.rs:215-217, 249-257
    std::vector<uint64_t> keys(n_samples - 1);
    orc_rng_split(two[1], n_samples - 1, keys.data());
    for (int64_t i = 0; i < n_samples - 1; i++) {
        if (run_blocks(s, keys[i], steps_per_sample, inj)) return -1;
        if (mom) orc_moments_observe(mom, s);
        if (obs_out) observe_states(s, obs_blocks, n_obs_blocks, obs_out + (i + 1) * stride);
    }
    return 0;
}
