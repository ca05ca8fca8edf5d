// Device-side halves of the two steps that precede the sampling path: the slot tables of BlockSamplingProgram::new
// (crates/thrml-samplers/src/program.rs:88-318) and greedy_coloring (crates/thrml-examples/src/lib.rs:114-147).
//
// Tables.  The reference walks a HashMap from head node to the (group, row) pairs in which it is head.  Here one
// interaction group at a time is handled as a sort: rows are keyed by the head node's index among the free-block nodes
// (block-major), a stable radix sort brings the rows of one node together in row order (the slot order of
// program.rs:104-125), the slot of a row is its distance from the start of its run, the padded slot count of a block is
// the longest run among its nodes, and one scatter writes rows / active / tail positions into [n, k] tables that start
// zeroed (a padded slot points at row 0 and position 0, program.rs:187-235).  A gather then materialises the weights.
// The layout half (classes, sampling order, node positions, argument checks) is O(nodes) and stays on the host.
//
// Colouring.  The greedy colouring in node-index order is a dataflow over the edges directed from the lower to the
// higher index: colour(v) = the smallest colour no lower-indexed neighbour holds.  Each pass colours every node whose
// lower-indexed neighbours are all coloured, so the result equals the sequential one exactly and the number of passes is
// the longest index-increasing path of the graph.
#include <cub/device/device_radix_sort.cuh>
#include <cub/device/device_scan.cuh>

#include <algorithm>
#include <cstring>
#include <numeric>
#include <vector>

#include "ctx.h"
#include "devbuf.h"

using thrml::fail;

namespace {

constexpr uint32_t KEY_NONE = 0xFFFFFFFFu;
constexpr int TPB = 256;
inline unsigned blocks_for(int64_t n) { return static_cast<unsigned>(std::min<int64_t>((n + TPB - 1) / TPB, 1 << 20)); }

// key = index of the head node among the free-block nodes (KEY_NONE for a head outside every free block), value = row
__global__ void k_head_keys(const int64_t* __restrict__ head, const int32_t* __restrict__ node_fid, int64_t rows, uint32_t* __restrict__ key,
                            int32_t* __restrict__ val) {
    for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < rows; i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int32_t f = node_fid[head[i]];
        key[i] = f < 0 ? KEY_NONE : static_cast<uint32_t>(f);
        val[i] = static_cast<int32_t>(i);
    }
}
// start[i] = i where a run of equal keys begins, 0 elsewhere; an inclusive max-scan turns it into the run start of every i
__global__ void k_run_starts(const uint32_t* __restrict__ key, int64_t rows, int32_t* __restrict__ start) {
    for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < rows; i += static_cast<int64_t>(gridDim.x) * blockDim.x)
        start[i] = (i > 0 && key[i] != key[i - 1]) ? static_cast<int32_t>(i) : 0;
}
__global__ void k_block_kmax(const uint32_t* __restrict__ key, const int32_t* __restrict__ start, const int32_t* __restrict__ fid_blk, int64_t rows,
                             int32_t* __restrict__ kmax) {
    // the keys are sorted block-major, so the lanes of a warp mostly see one block: one atomic per warp and block
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t base = blockIdx.x * static_cast<int64_t>(blockDim.x); base < rows; base += stride) {  // uniform trip count over a warp
        const int64_t i = base + threadIdx.x;
        int32_t blk = -1, len = 0;
        if (i < rows && key[i] != KEY_NONE) {
            blk = fid_blk[key[i]];
            // only the last entry of a run carries the run's length
            if (i + 1 >= rows || key[i + 1] != key[i]) len = static_cast<int32_t>(i) - start[i] + 1;
        }
        const unsigned peers = __match_any_sync(0xffffffffu, blk);
        const int32_t longest = __reduce_max_sync(peers, len);
        if (blk >= 0 && longest > 0 && (threadIdx.x & 31) == __ffs(peers) - 1) atomicMax(&kmax[blk], longest);
    }
}
struct ScatterArgs {
    const uint32_t* key;
    const int32_t* row;
    const int32_t* start;
    const int32_t* fid_blk;
    const int64_t* blk_base;  // first free-node index of each block
    const int32_t* blk_k;     // padded slot count of each block for this group (0 = no table)
    const int64_t* blk_off;   // first element of each block's table inside the concatenated arrays
    const int64_t* tails;     // [n_tails][rows] node ids
    const int64_t* loc_pos;   // per node
    int64_t rows, total;
    int32_t n_tails;
    int32_t* out_rows;
    uint8_t* out_active;
    int32_t* out_idx;  // [n_tails][total]
};
__global__ void k_scatter_slots(ScatterArgs a) {
    for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < a.rows; i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const uint32_t f = a.key[i];
        if (f == KEY_NONE) continue;
        const int32_t blk = a.fid_blk[f];
        const int64_t j = static_cast<int64_t>(f) - a.blk_base[blk];
        const int64_t at = a.blk_off[blk] + j * a.blk_k[blk] + (static_cast<int32_t>(i) - a.start[i]);
        const int32_t row = a.row[i];
        a.out_rows[at] = row;
        a.out_active[at] = 1;
        for (int32_t t = 0; t < a.n_tails; ++t) a.out_idx[t * a.total + at] = static_cast<int32_t>(a.loc_pos[a.tails[t * a.rows + row]]);
    }
}
// every slot, padded ones included (they hold row 0), copies the weights of its row: program.rs:216-235
__global__ void k_gather_weights(const int32_t* __restrict__ rows, const float* __restrict__ gw, int64_t total, int32_t wdim, float* __restrict__ w) {
    const int64_t n = total * wdim;
    for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n; i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int64_t s = i / wdim;
        w[i] = gw[static_cast<int64_t>(rows[s]) * wdim + (i - s * wdim)];
    }
}

// ---- colouring ----
__global__ void k_lower_degree(const int64_t* __restrict__ edges, int64_t n_edges, int32_t* __restrict__ deg, uint32_t* __restrict__ key, int32_t* __restrict__ val) {
    for (int64_t e = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; e < n_edges; e += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int64_t a = edges[2 * e], b = edges[2 * e + 1];
        if (a == b) {  // a self-loop never constrains: the node is uncoloured while it is visited
            key[e] = KEY_NONE;
            val[e] = 0;
            continue;
        }
        const int64_t hi = a > b ? a : b, lo = a > b ? b : a;
        key[e] = static_cast<uint32_t>(hi);
        val[e] = static_cast<int32_t>(lo);
        atomicAdd(&deg[hi], 1);
    }
}
// One pass: every uncoloured node whose lower-indexed neighbours are all coloured takes the smallest colour none of them
// holds.  A colour is written once and never changes, so reading a neighbour coloured earlier in the same pass is harmless.
__global__ void k_colour_pass(const int32_t* __restrict__ ptr, const int32_t* __restrict__ lower, int64_t n_nodes, int32_t* colour,
                              unsigned long long* __restrict__ n_done, int32_t* __restrict__ n_colours) {
    for (int64_t v = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; v < n_nodes; v += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        if (reinterpret_cast<volatile int32_t*>(colour)[v] >= 0) continue;
        const int32_t q0 = ptr[v], q1 = ptr[v + 1];
        unsigned long long taken = 0;
        bool ready = true;
        for (int32_t q = q0; q < q1; ++q) {
            const int32_t c = reinterpret_cast<volatile int32_t*>(colour)[lower[q]];
            if (c < 0) { ready = false; break; }
            if (c < 64) taken |= 1ull << c;
        }
        if (!ready) continue;
        int32_t c = __ffsll(static_cast<long long>(~taken)) - 1;  // smallest clear bit; -1 when all 64 are set
        if (c < 0) {  // colours 0..63 are all taken by the neighbourhood: search upwards one colour at a time
            for (c = 64;; ++c) {
                bool used = false;
                for (int32_t q = q0; q < q1 && !used; ++q) used = reinterpret_cast<volatile int32_t*>(colour)[lower[q]] == c;
                if (!used) break;
            }
        }
        colour[v] = c;
        atomicAdd(n_done, 1ull);
        atomicMax(n_colours, c + 1);
    }
}

template <class T> int32_t upload(DevBuf& d, const T* src, size_t n, cudaStream_t s) {
    if (int32_t rc = d.reserve(std::max<size_t>(n, 1) * sizeof(T))) return rc;
    if (n) CU_TRY(cudaMemcpyAsync(d.p, src, n * sizeof(T), cudaMemcpyHostToDevice, s));
    return THRML_OK;
}

}  // namespace

extern "C" {

int32_t thrml_builder_compile_device(thrml_builder* b, thrml_ctx* ctx) {
    if (!ctx) return fail(THRML_ERR_INVALID_ARG, "null context");
    if (int32_t rc = thrml::compile_layout(b)) return rc;
    CU_TRY(cudaSetDevice(ctx->device));
    cudaStream_t s = ctx->stream;
    const int64_t n_nodes = static_cast<int64_t>(b->kinds.size());
    const int32_t n_blocks = static_cast<int32_t>(b->free_blocks.size());
    // free-node numbering: block-major, position inside the block minor
    std::vector<int32_t> node_fid(static_cast<size_t>(n_nodes), -1);
    std::vector<int64_t> blk_base(static_cast<size_t>(n_blocks) + 1, 0);
    for (int32_t bi = 0; bi < n_blocks; ++bi) blk_base[bi + 1] = blk_base[bi] + static_cast<int64_t>(b->free_blocks[bi].nodes.size());
    const int64_t n_free = blk_base[n_blocks];
    if (n_free >= 0x7fffffffLL) return fail(THRML_ERR_UNSUPPORTED, "more than 2^31-2 free nodes");
    std::vector<int32_t> fid_blk(static_cast<size_t>(n_free));
    for (int32_t bi = 0; bi < n_blocks; ++bi) {
        const auto& nodes = b->free_blocks[bi].nodes;
        for (size_t j = 0; j < nodes.size(); ++j) {
            node_fid[nodes[j]] = static_cast<int32_t>(blk_base[bi] + static_cast<int64_t>(j));
            fid_blk[blk_base[bi] + static_cast<int64_t>(j)] = bi;
        }
    }
    DevBuf d_node_fid, d_fid_blk, d_blk_base, d_loc_pos, d_blk_k, d_blk_off, d_kmax;
    if (int32_t rc = upload(d_node_fid, node_fid.data(), node_fid.size(), s)) return rc;
    if (int32_t rc = upload(d_fid_blk, fid_blk.data(), fid_blk.size(), s)) return rc;
    if (int32_t rc = upload(d_blk_base, blk_base.data(), blk_base.size(), s)) return rc;
    if (int32_t rc = upload(d_loc_pos, b->loc_pos.data(), b->loc_pos.size(), s)) return rc;
    if (int32_t rc = d_blk_k.alloc(sizeof(int32_t) * std::max(n_blocks, 1))) return rc;
    if (int32_t rc = d_blk_off.alloc(sizeof(int64_t) * std::max(n_blocks, 1))) return rc;
    if (int32_t rc = d_kmax.alloc(sizeof(int32_t) * std::max(n_blocks, 1))) return rc;

    b->tables.assign(static_cast<size_t>(n_blocks), {});
    DevBuf d_head, d_tails, d_gw, d_key, d_key2, d_val, d_val2, d_start, d_rows, d_active, d_idx, d_w, d_tmp;
    std::vector<int32_t> kmax(static_cast<size_t>(std::max(n_blocks, 1)));
    std::vector<int64_t> blk_off(static_cast<size_t>(std::max(n_blocks, 1)));
    std::vector<int32_t> h_rows, h_idx;
    std::vector<uint8_t> h_active;
    std::vector<float> h_w;
    for (size_t gi = 0; gi < b->groups.size(); ++gi) {
        const thrml::GroupDesc& g = b->groups[gi];
        const int64_t R = static_cast<int64_t>(g.head.size());
        if (R > 0x7fffffffLL) return fail(THRML_ERR_UNSUPPORTED, "interaction group with more than 2^31-1 rows");
        const int32_t T = static_cast<int32_t>(g.tails.size());
        const int32_t wdim = g.d1 * g.d2;
        if (int32_t rc = upload(d_head, g.head.data(), g.head.size(), s)) return rc;
        if (int32_t rc = d_tails.reserve(sizeof(int64_t) * std::max<int64_t>(R * T, 1))) return rc;
        for (int32_t t = 0; t < T; ++t)
            CU_TRY(cudaMemcpyAsync(d_tails.as<int64_t>() + static_cast<int64_t>(t) * R, g.tails[t].data(), sizeof(int64_t) * R, cudaMemcpyHostToDevice, s));
        if (int32_t rc = upload(d_gw, g.w.data(), g.w.size(), s)) return rc;
        for (DevBuf* d : {&d_key, &d_key2, &d_val, &d_val2, &d_start})
            if (int32_t rc = d->reserve(sizeof(int32_t) * R)) return rc;
        k_head_keys<<<blocks_for(R), TPB, 0, s>>>(d_head.as<int64_t>(), d_node_fid.as<int32_t>(), R, d_key.as<uint32_t>(), d_val.as<int32_t>());
        // stable sort: the rows of one head node stay in row order.  Heads outside the free blocks carry the all-ones key, so
        // the full 32 bits are sorted.
        size_t tmp_bytes = 0;
        CU_TRY(cub::DeviceRadixSort::SortPairs(nullptr, tmp_bytes, d_key.as<uint32_t>(), d_key2.as<uint32_t>(), d_val.as<int32_t>(), d_val2.as<int32_t>(),
                                               static_cast<int64_t>(R), 0, 32, s));
        size_t scan_bytes = 0;
        CU_TRY(cub::DeviceScan::InclusiveScan(nullptr, scan_bytes, d_start.as<int32_t>(), d_start.as<int32_t>(), cub::Max(), static_cast<int64_t>(R), s));
        if (int32_t rc = d_tmp.reserve(std::max<size_t>(std::max(tmp_bytes, scan_bytes), 16))) return rc;
        tmp_bytes = d_tmp.bytes;
        CU_TRY(cub::DeviceRadixSort::SortPairs(d_tmp.p, tmp_bytes, d_key.as<uint32_t>(), d_key2.as<uint32_t>(), d_val.as<int32_t>(), d_val2.as<int32_t>(),
                                               static_cast<int64_t>(R), 0, 32, s));
        k_run_starts<<<blocks_for(R), TPB, 0, s>>>(d_key2.as<uint32_t>(), R, d_start.as<int32_t>());
        scan_bytes = d_tmp.bytes;
        CU_TRY(cub::DeviceScan::InclusiveScan(d_tmp.p, scan_bytes, d_start.as<int32_t>(), d_start.as<int32_t>(), cub::Max(), static_cast<int64_t>(R), s));
        CU_TRY(cudaMemsetAsync(d_kmax.p, 0, sizeof(int32_t) * std::max(n_blocks, 1), s));
        k_block_kmax<<<blocks_for(R), TPB, 0, s>>>(d_key2.as<uint32_t>(), d_start.as<int32_t>(), d_fid_blk.as<int32_t>(), R, d_kmax.as<int32_t>());
        CU_TRY(cudaMemcpyAsync(kmax.data(), d_kmax.p, sizeof(int32_t) * std::max(n_blocks, 1), cudaMemcpyDeviceToHost, s));
        CU_TRY(cudaStreamSynchronize(s));
        int64_t total = 0;
        for (int32_t bi = 0; bi < n_blocks; ++bi) {
            blk_off[bi] = total;
            total += static_cast<int64_t>(b->free_blocks[bi].nodes.size()) * kmax[bi];
        }
        if (total == 0) continue;  // program.rs:166: no block has this group's heads
        CU_TRY(cudaMemcpyAsync(d_blk_k.p, kmax.data(), sizeof(int32_t) * n_blocks, cudaMemcpyHostToDevice, s));
        CU_TRY(cudaMemcpyAsync(d_blk_off.p, blk_off.data(), sizeof(int64_t) * n_blocks, cudaMemcpyHostToDevice, s));
        if (int32_t rc = d_rows.reserve(sizeof(int32_t) * total)) return rc;
        if (int32_t rc = d_active.reserve(total)) return rc;
        if (int32_t rc = d_idx.reserve(sizeof(int32_t) * std::max<int64_t>(total * T, 1))) return rc;
        if (int32_t rc = d_w.reserve(sizeof(float) * total * wdim)) return rc;
        CU_TRY(cudaMemsetAsync(d_rows.p, 0, sizeof(int32_t) * total, s));
        CU_TRY(cudaMemsetAsync(d_active.p, 0, total, s));
        if (T) CU_TRY(cudaMemsetAsync(d_idx.p, 0, sizeof(int32_t) * total * T, s));
        ScatterArgs a{d_key2.as<uint32_t>(), d_val2.as<int32_t>(), d_start.as<int32_t>(), d_fid_blk.as<int32_t>(), d_blk_base.as<int64_t>(),
                      d_blk_k.as<int32_t>(), d_blk_off.as<int64_t>(), d_tails.as<int64_t>(), d_loc_pos.as<int64_t>(), R, total, T,
                      d_rows.as<int32_t>(), d_active.as<uint8_t>(), d_idx.as<int32_t>()};
        k_scatter_slots<<<blocks_for(R), TPB, 0, s>>>(a);
        k_gather_weights<<<blocks_for(total * wdim), TPB, 0, s>>>(d_rows.as<int32_t>(), d_gw.as<float>(), total, wdim, d_w.as<float>());
        CU_TRY(cudaGetLastError());
        h_rows.resize(static_cast<size_t>(total));
        h_active.resize(static_cast<size_t>(total));
        h_idx.resize(static_cast<size_t>(total) * T);
        h_w.resize(static_cast<size_t>(total) * wdim);
        CU_TRY(cudaMemcpyAsync(h_rows.data(), d_rows.p, sizeof(int32_t) * total, cudaMemcpyDeviceToHost, s));
        CU_TRY(cudaMemcpyAsync(h_active.data(), d_active.p, total, cudaMemcpyDeviceToHost, s));
        if (T) CU_TRY(cudaMemcpyAsync(h_idx.data(), d_idx.p, sizeof(int32_t) * total * T, cudaMemcpyDeviceToHost, s));
        CU_TRY(cudaMemcpyAsync(h_w.data(), d_w.p, sizeof(float) * total * wdim, cudaMemcpyDeviceToHost, s));
        CU_TRY(cudaStreamSynchronize(s));
        for (int32_t bi = 0; bi < n_blocks; ++bi) {
            if (kmax[bi] == 0) continue;
            thrml::SlotTable t;
            t.k = kmax[bi];
            t.wdim = wdim;
            t.n_spin = g.n_spin;
            t.source_group = static_cast<int32_t>(gi);
            const size_t nk = b->free_blocks[bi].nodes.size() * static_cast<size_t>(t.k);
            const size_t o = static_cast<size_t>(blk_off[bi]);
            t.rows.assign(h_rows.begin() + o, h_rows.begin() + o + nk);
            t.active.assign(h_active.begin() + o, h_active.begin() + o + nk);
            t.w.assign(h_w.begin() + o * wdim, h_w.begin() + (o + nk) * wdim);
            for (int32_t tl = 0; tl < T; ++tl) {
                const size_t base = static_cast<size_t>(tl) * total + o;
                t.idx.emplace_back(h_idx.begin() + base, h_idx.begin() + base + nk);
                const int32_t kind = b->kinds[g.tails[tl][0]];
                t.tail_sd.push_back(kind == 0 ? b->sd_spin : b->sd_cat);
                t.tail_is_cat.push_back(kind != 0);
            }
            b->tables[bi].push_back(std::move(t));
        }
    }
    b->compiled = true;
    return THRML_OK;
}

int32_t thrml_greedy_coloring_device(thrml_ctx* ctx, int64_t n_nodes, int64_t n_edges, const int64_t* edges, int32_t* colour_out,
                                     int32_t* n_colours_out, int32_t* n_passes_out) {
    if (!ctx) return fail(THRML_ERR_INVALID_ARG, "null context");
    if (n_nodes < 0 || n_edges < 0 || !colour_out || (n_edges > 0 && !edges)) return fail(THRML_ERR_INVALID_ARG, "bad colouring arguments");
    if (n_nodes >= 0x7fffffffLL || n_edges >= 0x7fffffffLL) return fail(THRML_ERR_UNSUPPORTED, "more than 2^31-2 nodes or edges");
    for (int64_t e = 0; e < 2 * n_edges; ++e)
        if (edges[e] < 0 || edges[e] >= n_nodes) return fail(THRML_ERR_INVALID_ARG, "edge endpoint out of range");
    if (n_colours_out) *n_colours_out = 0;
    if (n_passes_out) *n_passes_out = 0;
    if (n_nodes == 0) return THRML_OK;
    CU_TRY(cudaSetDevice(ctx->device));
    cudaStream_t s = ctx->stream;
    DevBuf d_edges, d_deg, d_ptr, d_key, d_key2, d_val, d_val2, d_colour, d_count, d_tmp;
    if (int32_t rc = upload(d_edges, edges, static_cast<size_t>(2 * n_edges), s)) return rc;
    if (int32_t rc = d_deg.alloc(sizeof(int32_t) * (n_nodes + 1))) return rc;
    if (int32_t rc = d_ptr.alloc(sizeof(int32_t) * (n_nodes + 1))) return rc;
    for (DevBuf* d : {&d_key, &d_key2, &d_val, &d_val2})
        if (int32_t rc = d->alloc(sizeof(int32_t) * std::max<int64_t>(n_edges, 1))) return rc;
    if (int32_t rc = d_colour.alloc(sizeof(int32_t) * n_nodes)) return rc;
    if (int32_t rc = d_count.alloc(16)) return rc;
    CU_TRY(cudaMemsetAsync(d_deg.p, 0, sizeof(int32_t) * (n_nodes + 1), s));
    CU_TRY(cudaMemsetAsync(d_colour.p, 0xFF, sizeof(int32_t) * n_nodes, s));  // -1 = not coloured
    CU_TRY(cudaMemsetAsync(d_count.p, 0, 16, s));
    if (n_edges) k_lower_degree<<<blocks_for(n_edges), TPB, 0, s>>>(d_edges.as<int64_t>(), n_edges, d_deg.as<int32_t>(), d_key.as<uint32_t>(), d_val.as<int32_t>());
    size_t sort_bytes = 0, scan_bytes = 0;
    CU_TRY(cub::DeviceRadixSort::SortPairs(nullptr, sort_bytes, d_key.as<uint32_t>(), d_key2.as<uint32_t>(), d_val.as<int32_t>(), d_val2.as<int32_t>(), n_edges, 0,
                                           32, s));
    CU_TRY(cub::DeviceScan::ExclusiveSum(nullptr, scan_bytes, d_deg.as<int32_t>(), d_ptr.as<int32_t>(), n_nodes + 1, s));
    if (int32_t rc = d_tmp.alloc(std::max<size_t>(std::max(sort_bytes, scan_bytes), 16))) return rc;
    if (n_edges) {
        sort_bytes = d_tmp.bytes;
        CU_TRY(cub::DeviceRadixSort::SortPairs(d_tmp.p, sort_bytes, d_key.as<uint32_t>(), d_key2.as<uint32_t>(), d_val.as<int32_t>(), d_val2.as<int32_t>(), n_edges,
                                               0, 32, s));
    }
    scan_bytes = d_tmp.bytes;
    CU_TRY(cub::DeviceScan::ExclusiveSum(d_tmp.p, scan_bytes, d_deg.as<int32_t>(), d_ptr.as<int32_t>(), n_nodes + 1, s));
    // passes in batches; the host looks at the progress counter after each batch.  Every pass colours at least the lowest
    // uncoloured node, so n_nodes passes always suffice and the loop is bounded by that.
    unsigned long long done = 0;
    int64_t passes = 0;
    const int batch = 8;
    auto* d_done = d_count.as<unsigned long long>();
    auto* d_ncol = reinterpret_cast<int32_t*>(d_count.as<unsigned long long>() + 1);
    while (done < static_cast<unsigned long long>(n_nodes)) {
        if (passes > n_nodes + batch) return fail(THRML_ERR_CUDA, "colouring made no progress");
        for (int i = 0; i < batch; ++i)
            k_colour_pass<<<blocks_for(n_nodes), TPB, 0, s>>>(d_ptr.as<int32_t>(), d_val2.as<int32_t>(), n_nodes, d_colour.as<int32_t>(), d_done, d_ncol);
        passes += batch;
        CU_TRY(cudaMemcpyAsync(&done, d_done, sizeof(done), cudaMemcpyDeviceToHost, s));
        CU_TRY(cudaStreamSynchronize(s));
    }
    int32_t ncol = 0;
    CU_TRY(cudaMemcpyAsync(&ncol, d_ncol, sizeof(ncol), cudaMemcpyDeviceToHost, s));
    CU_TRY(cudaMemcpyAsync(colour_out, d_colour.p, sizeof(int32_t) * n_nodes, cudaMemcpyDeviceToHost, s));
    CU_TRY(cudaStreamSynchronize(s));
    if (n_colours_out) *n_colours_out = ncol;
    if (n_passes_out) *n_passes_out = static_cast<int32_t>(std::min<int64_t>(passes, 0x7fffffff));
    return THRML_OK;
}

}  // extern "C"
